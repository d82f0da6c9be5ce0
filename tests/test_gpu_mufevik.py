"""Mufevik on the GPU: replay through bin/trace_run against the plain implementation (whole
prompts, tails decoded token by token, portions down to two tokens, mixed batches in a pool so
small that pages and slots are used again), every new kernel alone against NumPy, keys planted far
away and at page borders for heads that exchange their weights, the recurrent states and the
convolutions' inputs across steps and slots used again, and greedy generation through the Python
entry point, the scheduler and the command line."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_mufevik as pm
import tiny_mufevik as tm
import trace_tools as tt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LENGTHS = {"MA": [1, 2, 19, 100, 65, 48, 33], "MB": [5, 41, 97, 230, 129, 64], "MC": [3, 70, 130, 17],
           "MD": [2, 150, 31, 16, 77], "ME": [1, 90, 33, 2, 64], "MF": [4, 120, 8, 57], "ML": [7, 150, 300, 64]}


@pytest.fixture(scope="module")
def cases(model_folders):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            folder = model_folders(name, dtype)
            rng = np.random.default_rng(900 + ord(name[1]))
            reqs = tt.make_requests(rng, tm.TINY[name]["config"]["vocab"], LENGTHS[name])
            cfg, w = pm.load_folder(folder)
            made[(name, dtype)] = (folder, reqs, {r: pm.logits_all(cfg, w, t) for r, t in reqs.items()})
        return made[(name, dtype)]
    return get


# In bfloat16 a router's choice between two experts whose choice scores differ by less than the
# rounding of its input is a toss-up, and states and keys carry the other expert's output on.  So in
# bfloat16 whole-model logits are compared in the bulk; the sharp checks of cache, state and batching
# are the 32-bit runs, which take the same way through the host's code, and the kernels' own tests.
# (At these widths of under a hundred the bulk itself sits near 1 to 2 %, on the FP32-core attention
# kernel and on the warp-level ones alike.)
def _compare(got, tb, plain, dtype, label, tol_rms=3e-5):
    errs = []
    for sid in sorted(tb.rows):
        want = tt.expected_rows(tb.rows[sid], plain)
        have = got[sid]
        assert have.shape == want.shape and np.isfinite(have).all(), (label, sid)
        errs.extend(np.sqrt(((have - want) ** 2).mean(axis=1)) / np.sqrt((want ** 2).mean(axis=1)))
    errs = np.sort(np.asarray(errs))
    print(f"{label} {dtype}: {len(errs)} rows, relative rms error median {np.median(errs):.2e}, "
          f"90 % {errs[int(0.9 * (len(errs) - 1))]:.2e}, worst {errs[-1]:.2e}")
    if dtype == "float32":
        assert errs[-1] <= tol_rms, (label, errs[-1])
    else:
        assert np.median(errs) <= 2.5e-2 and errs[int(0.9 * (len(errs) - 1))] <= 6e-2, label


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["MA", "MB", "MC", "MD", "ME", "MF"])
def test_alone_whole_tail_portions(name, dtype, cases, tmp_path):
    folder, reqs, plain = cases(name, dtype)
    ps = tm.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_whole(tb, reqs)
    tt.trace_tail_decode(tb, reqs)
    tt.trace_portions(tb, reqs, np.random.default_rng(7))
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    _compare(got, tb, plain, dtype, f"config {name}")
    if dtype == "float32":
        tt.compare_cuts([(got, tb)], dtype, f"config {name}", tol=3e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["MA", "MB", "MC", "MD", "ME", "MF"])
def test_mixed_with_page_and_slot_reuse(name, dtype, cases, tmp_path):
    folder, reqs, plain = cases(name, dtype)
    ps = tm.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_mixed(tb, reqs, np.random.default_rng(11), max_live=3)
    assert tb.pages_taken > tb.peak_tokens // ps, "the trace must make the pool hand pages out again"
    assert max(len(s["entries"]) for s in tb.steps) >= 3
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"),
                       extra_args=["--max-live", "3"])          # three slots for all requests
    _compare(got, tb, plain, dtype, f"config {name} mixed")


def test_long_decoding(cases, tmp_path):
    folder, reqs, plain = cases("MB", "float32")
    ps = tm.TINY["MB"]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_tail_decode(tb, {"r3": reqs["r3"]}, tail=200)
    got = tt.run_trace(folder, "float32", tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    _compare(got, tb, plain, "float32", "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_sizes_of_the_tensor_core_kernels(dtype, cases, tmp_path):
    folder, reqs, plain = cases("ML", dtype)
    ps = tm.TINY["ML"]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_whole(tb, reqs)
    tt.trace_tail_decode(tb, reqs, tail=40)
    tt.trace_portions(tb, reqs, np.random.default_rng(3))
    tt.trace_mixed(tb, reqs, np.random.default_rng(5))
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    _compare(got, tb, plain, dtype, "config ML", tol_rms=6e-5)
    if dtype == "float32":
        tt.compare_cuts([(got, tb)], dtype, "config ML", tol=6e-5)


# ------------------------------------------------------------------ kernels
@pytest.fixture(scope="module")
def K():
    from crane_b200.kernels import get_kernels
    return get_kernels()


def _dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).to(DEV)


def _i32(a):
    return _dev(a, torch.int32)


def _err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R, hidden", [(1, 48), (2, 96), (3, 68), (4, 1000), (8, 7)])
def test_streams_norm(K, dtype, R, hidden):
    """The first read (all streams start as the embedding output), an update with the next read in
    one kernel (from whole results and from partial sums), the plain sum for the last norm, and the
    last norm on chosen rows only, which must leave the streams as they are."""
    from crane_b200.kernels import Partials
    rng = np.random.default_rng(R * 100 + hidden)
    n, eps = 6, 1e-6
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    x0 = rng.standard_normal((n, hidden)) * 2
    inw, outw, mix = rng.standard_normal(R), rng.standard_normal(R), np.eye(R) + 0.3 * rng.standard_normal((R, R))
    g = np.array([1.3])
    streams = torch.full((R, n, hidden), 7.0, device=DEV)
    out = torch.empty(n, hidden, dtype=dtype, device=DEV)
    K.streams_norm(streams, _dev(x0), None, None, None, _dev(inw), _dev(g), eps, out)
    xs = np.repeat(x0.astype(np.float32).astype(np.float64)[None], R, axis=0)
    assert np.abs(streams.cpu().numpy() - xs).max() == 0
    want = pm.scalar_norm(pm.streams_read(xs, inw), g[0], eps)
    assert np.abs(out.double().cpu().numpy() - want).max() < tol * 4
    for form in ("whole", "parts"):
        if form == "whole":
            y = _dev(rng.standard_normal((n, hidden)), dtype)
            yn = y.double().cpu().numpy()
        else:
            parts = _dev(rng.standard_normal((3, n, hidden)))
            y = Partials(parts)
            yn = parts.sum(0).to(dtype).double().cpu().numpy()
        inw2 = rng.standard_normal(R)
        K.streams_norm(streams, None, y, _dev(mix), _dev(outw), _dev(inw2), _dev(g), eps, out)
        xs = pm.streams_write(xs, yn, mix, outw)
        assert np.abs(streams.cpu().numpy() - xs).max() < 1e-5 * np.abs(xs).max()
        want = pm.scalar_norm(pm.streams_read(xs, inw2), g[0], eps)
        assert np.abs(out.double().cpu().numpy() - want).max() < tol * 4, form
    # the model's last norm: the update, then the plain sum, on two rows; no stream is written
    y = _dev(rng.standard_normal((n, hidden)), dtype)
    rows = _i32([4, 1])
    out2 = torch.empty(2, hidden, dtype=dtype, device=DEV)
    before = streams.clone()
    K.streams_norm(streams, None, y, _dev(mix), _dev(outw), None, _dev(g), eps, out2, rows)
    new = pm.streams_write(xs, y.double().cpu().numpy(), mix, outw)
    want = pm.scalar_norm(new.sum(0), g[0], eps)[[4, 1]]
    assert np.abs(out2.double().cpu().numpy() - want).max() < tol * 4
    assert torch.equal(streams, before)


@pytest.mark.parametrize("experts, top, groups, keep", [(3, 3, 1, 1), (6, 2, 3, 2), (8, 3, 4, 2), (9, 4, 3, 3), (20, 5, 4, 3),
                                                        (64, 6, 8, 4), (12, 1, 12, 1), (40, 8, 5, 2), (128, 8, 1, 1)])
@pytest.mark.parametrize("gate", [False, True])
def test_route_grouped(K, experts, top, groups, keep, gate):
    rng = np.random.default_rng(experts * 10 + top)
    n = 37
    z = rng.standard_normal((n, experts + 3)).astype(np.float32) * 2       # wider rows than the router needs
    corr = (rng.standard_normal(experts) * 0.2).astype(np.float32)
    z[0, :experts] = 0.5                                  # all equal: the correction alone decides
    z[1, :experts] = 0.5
    z[2, :experts] = -30.0 * np.arange(experts)           # scores that vanish: choice scores of the correction alone
    route = torch.full((n, experts + (1 if gate else 0)), 5.0, device=DEV)
    for c in (corr, None, corr - 1.0):                    # the last: every choice score is negative
        K.route_grouped(_dev(z), None if c is None else _dev(c), route, experts, top, groups, keep, gate)
        got = route.cpu().numpy()
        for t in range(n):
            cc = np.zeros(experts) if c is None else c.astype(np.float64)
            idx, wt = pm.choose_experts(z[t, :experts].astype(np.float64), cc, top, groups, keep)
            want = np.zeros(experts)
            want[idx] = wt
            # (a choice between two scores closer than 32-bit rounding may go either way)
            s = pm.softmax(z[t, :experts].astype(np.float64)) + cc
            close = np.sort(s)[::-1]
            if (np.abs(np.diff(close)) < 1e-6).any() and t > 2:
                continue
            assert np.abs(got[t, :experts] - want).max() < 1e-6, (t, idx)
            assert (got[t, :experts] != 0).sum() <= top
            if gate:
                assert abs(got[t, experts] - pm.sigmoid(float(z[t, experts]))) < 1e-6
    # equal scores and no correction: the lowest indices of the lowest groups
    K.route_grouped(_dev(z), None, route, experts, top, groups, keep, gate)
    per = experts // groups
    allowed = [e for e in range(experts) if e // per < keep][:top]
    assert sorted(np.nonzero(route[0, :experts].cpu().numpy())[0].tolist()) == allowed


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("gate", [False, True])
def test_gated_activation(K, dtype, gate):
    from crane_b200.kernels import Partials
    rng = np.random.default_rng(5)
    n, E, F, Fs = 6, 3, 5, 4
    cols = E * F + Fs
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    route = rng.random((n, E + (1 if gate else 0))).astype(np.float32)
    route[:, 1] = 0.0
    for form in ("whole", "parts"):
        if form == "whole":
            gu = _dev(rng.standard_normal((n, 2 * cols)) * 2, dtype)
            gn = gu.double().cpu().numpy()
        else:
            parts = _dev(rng.standard_normal((2, n, 2 * cols)))
            gu = Partials(parts)
            gn = parts.sum(0).to(dtype).double().cpu().numpy()
        out = torch.empty(n, cols, dtype=dtype, device=DEV)
        K.gated_activation(gu, out, _dev(route), E, F, E * F, gate)
        want = pm.silu(gn[:, :cols]) * gn[:, cols:]
        want[:, :E * F] *= np.repeat(route[:, :E], F, axis=1)
        if gate:
            want[:, E * F:] *= route[:, E:]
        assert np.abs(out.double().cpu().numpy() - want).max() < tol * 8, form
        assert (out[:, F:2 * F] == 0).all()
    out = torch.empty(n, cols, dtype=dtype, device=DEV)              # no routing at all: a plain gated feed-forward
    gu = _dev(rng.standard_normal((n, 2 * cols)), dtype)
    K.gated_activation(gu, out)
    gn = gu.double().cpu().numpy()
    assert np.abs(out.double().cpu().numpy() - pm.silu(gn[:, :cols]) * gn[:, cols:]).max() < tol * 8


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [48, 68, 1000])
def test_pair_norm_mean(K, dtype, hidden):
    rng = np.random.default_rng(hidden)
    n, eps = 5, 1e-5
    a, b = _dev(rng.standard_normal((n, hidden)) * 0.01, dtype), _dev(rng.standard_normal((n, hidden)) * 30, dtype)
    wa, wb = 1 + 0.3 * rng.standard_normal(hidden), 1 + 0.3 * rng.standard_normal(hidden)
    out = torch.empty(n, hidden, dtype=dtype, device=DEV)
    K.pair_norm_mean(a, b, _dev(wa), _dev(wb), eps, out)
    want = 0.5 * (pm.unit_rms(a.double().cpu().numpy(), eps) * wa + pm.unit_rms(b.double().cpu().numpy(), eps) * wb)
    assert np.abs(out.double().cpu().numpy() - want).max() < (2e-5 if dtype == torch.float32 else 3e-2)


# ---------------------------------------------------------------- heads that exchange their weights
def _step_meta(lens, page_size, rng, extra_pages=2):
    """Block tables of requests of ``lens`` tokens, pages in random order."""
    blocks = [(t + page_size - 1) // page_size for t in lens]
    order = rng.permutation(sum(blocks) + extra_pages)
    table = -np.ones((len(lens), max(blocks)), dtype=np.int32)
    nxt = 0
    for e, b in enumerate(blocks):
        table[e, :b] = order[nxt:nxt + b]
        nxt += b
    return table, len(order)


def _plain_talking_row(q, k, v, scale, talk):
    """One query q [H, d] (temperature folded in) over k [T, G, d], v [T, G, m] in float64."""
    H, G = q.shape[0], k.shape[1]
    w = np.stack([pm.softmax(k[:, h // (H // G)] @ q[h] * scale) for h in range(H)])       # [H, T]
    mixed = talk @ w
    return np.stack([mixed[h] @ v[:, h // (H // G)] for h in range(H)])


@pytest.mark.parametrize("dtype, splits", [(torch.float32, 0), (torch.bfloat16, 0), (torch.bfloat16, 1), (torch.bfloat16, 3),
                                           (torch.bfloat16, 16)])
@pytest.mark.parametrize("H, G, d, m, rot, ps", [(4, 1, 64, 80, 32, 64), (6, 2, 16, 24, 8, 16), (3, 3, 24, 8, 0, 8),
                                                 (8, 2, 128, 128, 64, 32), (4, 2, 100, 128, 100, 16), (2, 2, 32, 16, 32, 16)])
def test_talking_attention_with_planted_keys(K, dtype, splits, H, G, d, m, rot, ps):
    """Rotation, temperature, cache write, attention and the exchange of weights over prompts and
    decoded tokens.  One key per request is made to stand out for head 0's last query in the part
    of the head that is not rotated (far back, at a page's last place with its opposite at the next
    page's first, the newest), so a key that is lost or one place off changes every head that
    hears head 0.  ``splits`` 0: the FP32-core kernel on rows as wide as they are; else the
    warp-level kernels on rows stored at a common head size, decoded tokens in that many slices."""
    from crane_b200.config.mufevik import _common_head_size
    D = Dv = 0
    if splits:
        D = Dv = _common_head_size(d, m)
        assert D and K.prefill_attention_supports(D, H, G) and K.decode_attention_supports(D, H, G)
    D, Dv = D or d, Dv or m
    rng = np.random.default_rng(H * 100 + d)
    lens = [700, 2 * ps + 1, 1, 37]
    scale, base = 0.4, 300.0
    temp = 0.5 + rng.random(H)
    talk = np.eye(H) * 0.6 + 0.4 * rng.standard_normal((H, H))
    planted = {0: 3, 1: ps - 1, 3: 36}
    cols = H * d + G * d + G * m
    qkv = [rng.standard_normal((n, cols)) for n in lens]
    free = slice(rot, d) if rot < d else slice(0, d)          # where a rotation does not turn the planted key away
    for e, key in planted.items():
        qkv[e][key, H * d + free.start:H * d + free.stop] *= 6.0
        qkv[e][-1, free] = qkv[e][key, H * d + free.start:H * d + free.stop] * 2
    qkv[1][ps, H * d:H * d + d] = -qkv[1][ps - 1, H * d:H * d + d]
    store = torch.float32 if dtype == torch.float32 else torch.bfloat16
    qkv_dev = [_dev(a, store) for a in qkv]
    qkv_r = [a.double().cpu().numpy() for a in qkv_dev]
    stored = lambda a: torch.as_tensor(a).to(store).double().numpy()
    pos_of = [np.arange(n) for n in lens]
    qn = [stored(pm.rotate_half(a[:, :H * d].reshape(-1, H, d), p, rot, base) * temp[None, :, None])
          for a, p in zip(qkv_r, pos_of)]
    kn = [stored(pm.rotate_half(a[:, H * d:H * d + G * d].reshape(-1, G, d), p, rot, base)) for a, p in zip(qkv_r, pos_of)]
    vn = [a[:, H * d + G * d:].reshape(-1, G, m) for a in qkv_r]
    cos = sin = None
    if rot:
        ang = np.arange(max(lens))[:, None] * (base ** (-2.0 * np.arange(rot // 2) / rot))[None, :]
        cos, sin = _dev(np.cos(ang)), _dev(np.sin(ang))
    err = _err()
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    full_table, n_pages = _step_meta(lens, ps, rng)
    k_pool = torch.randn(n_pages, G, ps, D, device=DEV).mul_(30).to(store)
    v_pool = torch.randn(n_pages, G, ps, Dv, device=DEV).mul_(30).to(store)
    # whole prompts but the last token of each longer request, then a step that decodes those
    for stage in (0, 1):
        if stage == 0:
            ents, q_lens, before = list(range(len(lens))), [max(1, n - 1) for n in lens], [0] * len(lens)
        else:
            ents = [e for e, n in enumerate(lens) if n > 1]
            q_lens, before = [1] * len(ents), [lens[e] - 1 for e in ents]
        table = _i32(full_table[ents])
        cu = _i32(np.concatenate([[0], np.cumsum(q_lens)]))
        pos = np.concatenate([np.arange(b, b + q) for b, q in zip(before, q_lens)]).astype(np.int32)
        ent = np.concatenate([np.full(q, i) for i, q in enumerate(q_lens)]).astype(np.int32)
        rows = torch.cat([qkv_dev[e][b:b + q] for e, b, q in zip(ents, before, q_lens)])
        n = rows.shape[0]
        q_out = torch.empty(n, H * D, dtype=store, device=DEV)
        K.projection_norm_cache(rows, cols, _i32(pos), _i32(ent), table, ps, None, None, 0.0, q_out, k_pool, v_pool,
                                H, G, d, m, err, cos=cos, sin=sin, rot_dims=rot, q_head_scale=_dev(temp))
        cross = torch.full((n, H * G * Dv), 7.0, device=DEV)
        if not splits:
            K.paged_attention_simt(q_out, None, k_pool, v_pool, _i32(pos), _i32(ent), table, ps, H, G, d, 0, scale, err,
                                   dv=m, v_stride=m, out_cross=cross)
        else:
            kv = _i32([b + q for b, q in zip(before, q_lens)])
            if stage == 0:
                tiles = sum((q + 63) // 64 for q in q_lens)
                K.paged_prefill_attention(q_out, cross, k_pool, v_pool, cu, kv, table, ps, tiles, H, G, D, 0, scale, err,
                                          cross=True)
            else:
                part_o = torch.empty(n * H * G * splits, D, device=DEV)
                part_ml = torch.empty(n * H * G * splits, 2, device=DEV)
                K.paged_decode_attention(q_out, cross, k_pool, v_pool, cu, kv, table, ps, H, G, D, 0, scale, splits,
                                         part_o, part_ml, err, cross=True)
        o = torch.full((n + 1, H * m), 5.0, dtype=store, device=DEV)
        K.head_talk_mix(cross, _dev(talk), _i32(ent), o[:n], H, G, Dv, m)
        assert (o[n] == 5.0).all()                                  # nothing is written behind the last head
        got = o[:n].double().cpu().numpy().reshape(n, H, m)
        for i in range(n):
            e, p = ents[ent[i]], pos[i]
            want = _plain_talking_row(qn[e][p], kn[e][:p + 1], vn[e][:p + 1], scale, talk)
            assert np.abs(got[i] - want).max() < tol * max(1.0, np.abs(want).max()), (stage, e, p)
        if stage == 1 and rot < d:
            for j, e in enumerate(ents):
                if e in planted:                                    # head 0's own weights sit on the planted key
                    w0 = pm.softmax(kn[e][:, 0] @ qn[e][-1, 0] * scale)
                    assert w0[planted[e]] > 0.9, (e, w0[planted[e]])
    assert int(err.item()) == 0


# ---------------------------------------------------------------- recurrences with a matrix state
def _steps_of(lens, plan):
    """``plan``: per step a list of (request, tokens taken, slot).  Yields per step the metadata of the
    kernels and, per entry, (request, first position, count)."""
    done = [0] * len(lens)
    for step in plan:
        ents = []
        for r, take, slot in step:
            ents.append((r, done[r], take, slot))
            done[r] += take
        q_lens = [t for _, _, t, _ in ents]
        ctx = SimpleNamespace(cu_q=_i32(np.concatenate([[0], np.cumsum(q_lens)])),
                              kv_len=_i32([b + t for _, b, t, _ in ents]), slots=_i32([s for _, _, _, s in ents]),
                              tok_entry=_i32(np.concatenate([np.full(t, i) for i, t in enumerate(q_lens)])))
        yield ctx, ents
    assert done == list(lens)


# three requests and a fourth that takes the second one's slot; portions, single tokens, a request left
# out of a step; slots in no order
PLAN = [[(0, 20, 2), (1, 1, 0), (2, 4, 1)], [(2, 5, 1), (0, 1, 2)], [(0, 1, 2)], [(0, 15, 2), (3, 2, 0)], [(3, 9, 0)]]
PLAN_LENS = [37, 1, 9, 11]


@pytest.mark.parametrize("delta", [False, True])
@pytest.mark.parametrize("H, G, dk, dv", [(2, 2, 16, 8), (4, 2, 24, 40), (1, 1, 64, 32), (6, 3, 48, 16), (2, 1, 128, 128),
                                          (1, 1, 300, 20), (2, 2, 32, 8), (3, 1, 32, 12), (2, 2, 256, 4)])
def test_matrix_state_scan(K, delta, H, G, dk, dv):
    """Both recurrences over portions, single tokens and a slot that is used again, from a state pool
    full of another request's numbers.  The decays stay near 1 and the first token's key and value
    are large, so a state that is lost or started anew shows at every later read-out."""
    rng = np.random.default_rng(dk + dv + delta)
    Hq = G if delta else H                                  # the decay per channel has its own q and k per head
    data = []
    for n in PLAN_LENS:
        q, k = rng.standard_normal((n, Hq, dk)), rng.standard_normal((n, Hq, dk))
        v = rng.standard_normal((n, H, dv))
        v[0] *= 8.0
        if delta:
            k, q = pm.unit_vector(k), pm.unit_vector(q)
            w, beta = 0.9 + 0.1 * rng.random((n, H)), rng.random((n, H))
            want = pm.gated_delta_scan(q, k, v, beta, w)[0]
            row = np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), w, beta], axis=1)
        else:
            k[0] *= 3.0
            w = 0.93 + 0.07 * rng.random((n, H, dk))
            want = pm.gated_linear_scan(q, k, v, w)[0]
            row = np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), w.reshape(n, -1)], axis=1)
        data.append((row.astype(np.float32), want))
    qk, hv = Hq * dk, H * dv
    offs = (0, qk, 2 * qk, 2 * qk + hv, 2 * qk + hv + H) if delta else (0, qk, 2 * qk, 2 * qk + hv, 0)
    rows_, lanes = K.matrix_state_plan(dk)
    floats = H * rows_ * lanes * dv
    state = torch.full((4, floats + 5), 1e3, device=DEV)          # another request's numbers; 5 floats that stay
    err = _err()
    for ctx, ents in _steps_of(PLAN_LENS, PLAN):
        aux = torch.cat([_dev(data[r][0][b:b + t]) for r, b, t, _ in ents])
        n = aux.shape[0]
        o = torch.full((n + 1, hv), 5.0, device=DEV)
        K.matrix_state_scan(aux, offs, not delta, delta, H // Hq, ctx, state, o[:n], H, dk, dv, err)
        got = o[:n].double().cpu().numpy().reshape(n, H, dv)
        assert (o[n] == 5.0).all()
        at = 0
        for r, b, t, _ in ents:
            want = data[r][1][b:b + t]
            assert np.abs(got[at:at + t] - want).max() < 3e-5 * max(1.0, np.abs(want).max()), (r, b, t)
            at += t
    assert (state[:, floats:] == 1e3).all() and (state[3] == 1e3).all()      # nothing behind the state, no other slot
    assert int(err.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, d, dv, taps", [(4, 2, 16, 24, 3), (5, 1, 16, 16, 1), (1, 1, 64, 32, 5), (3, 3, 8, 8, 2),
                                               (2, 2, 40, 12, 16)])
def test_conv_delta_prep(K, dtype, H, G, d, dv, taps):
    """The short convolutions with their inputs carried in the slot, silu, unit vectors, decay and beta,
    over the same plan of steps: a portion shorter than the taps, single tokens, a slot used again."""
    rng = np.random.default_rng(H * 10 + taps)
    C = 2 * G * d + H * dv
    cols = C + H * dv + 2 * H
    conv_w = rng.standard_normal((C, taps))
    a_log, dt_bias = rng.standard_normal(H) * 0.5, rng.standard_normal(H)
    proj = [_dev(rng.standard_normal((n, cols)), dtype) for n in PLAN_LENS]
    wants = []
    for p in proj:
        x = p.double().cpu().numpy()
        n = x.shape[0]
        y = pm.silu(pm.short_convolution(x[:, :C], conv_w)[0])
        q = pm.unit_vector(y[:, :G * d].reshape(n, G, d)) * d ** -0.5
        k = pm.unit_vector(y[:, G * d:2 * G * d].reshape(n, G, d))
        b, a = x[:, C + H * dv:C + H * dv + H], x[:, C + H * dv + H:]
        w = np.exp(-np.exp(a_log) * pm.softplus(a + dt_bias))
        wants.append(np.concatenate([q.reshape(n, -1), k.reshape(n, -1), y[:, 2 * G * d:], w, pm.sigmoid(b)], axis=1))
    off = 7
    state = torch.full((4, off + (taps - 1) * C + 3), 1e3, device=DEV)
    err = _err()
    for ctx, ents in _steps_of(PLAN_LENS, PLAN):
        rows = torch.cat([proj[r][b:b + t] for r, b, t, _ in ents])
        n = rows.shape[0]
        aux = torch.full((n, C + 2 * H), 5.0, device=DEV)
        K.conv_delta_prep(rows, cols, ctx, state, off, _dev(conv_w), taps, _dev(a_log), _dev(dt_bias), aux, H, G, d, dv,
                          1e-6, d ** -0.5, err, dtype)
        got = aux.double().cpu().numpy()
        at = 0
        for r, b, t, _ in ents:
            assert np.abs(got[at:at + t] - wants[r][b:b + t]).max() < 2e-5, (r, b, t)
            at += t
    assert (state[:, :off] == 1e3).all() and (state[:, off + (taps - 1) * C:] == 1e3).all() and (state[3] == 1e3).all()
    assert int(err.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, d, dv, rank, tau", [(3, 16, 8, 5, 4.0), (1, 24, 40, 3, 1.0), (5, 8, 16, 2, 2.5), (2, 64, 128, 32, 16.0)])
def test_decay_gate_prep(K, dtype, H, d, dv, rank, tau):
    rng = np.random.default_rng(rank)
    n, hd, hv = 23, H * d, H * dv
    cols = 2 * hd + 2 * hv + rank
    proj = _dev(rng.standard_normal((n, cols)) * 2, dtype)
    a2t, bias = rng.standard_normal((rank, hd)), rng.standard_normal(hd) * 2
    ent = np.zeros(n, dtype=np.int32)
    ent[5] = -1                                                    # a row of no entry stays as it is
    aux = torch.full((n, 3 * hd + hv), 5.0, device=DEV)
    K.decay_gate_prep(proj, cols, _i32(ent), _dev(a2t), _dev(bias), 1.0 / tau, d ** -0.5, aux, H, d, dv, dtype)
    x = proj.double().cpu().numpy()
    w = pm.sigmoid(x[:, 2 * hd + 2 * hv:] @ a2t + bias) ** (1.0 / tau)
    want = np.concatenate([x[:, :hd] * d ** -0.5, x[:, hd:2 * hd], x[:, 2 * hd:2 * hd + hv], w], axis=1)
    want[5] = 5.0
    assert np.abs(aux.double().cpu().numpy() - want).max() < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, dv", [(3, 8), (1, 40), (4, 128), (2, 100)])
def test_head_norm_gate(K, dtype, H, dv):
    rng = np.random.default_rng(dv)
    n, eps, gate_off = 19, 1e-3, 11
    cols = gate_off + H * dv + 3
    o_raw = rng.standard_normal((n, H, dv)) * 0.02                 # small, so that eps counts
    proj = _dev(rng.standard_normal((n, cols)), dtype)
    norm_w = rng.standard_normal(dv)
    out = torch.empty(n, H * dv, dtype=dtype, device=DEV)
    K.head_norm_gate(_dev(o_raw.reshape(n, -1)), proj, cols, gate_off, _i32(np.zeros(n)), _dev(norm_w), eps, out, H, dv)
    gate = proj.double().cpu().numpy()[:, gate_off:gate_off + H * dv].reshape(n, H, dv)
    want = pm.unit_rms(o_raw, eps) * norm_w * pm.silu(gate)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(out.double().cpu().numpy().reshape(n, H, dv) - want).max() < tol * max(1.0, np.abs(want).max())


# ---------------------------------------------------------------- generation
def _load(folder, dtype, **opts):
    from crane_b200.generation import ModelForCausalLM
    return ModelForCausalLM.from_pretrained(folder, dtype, **opts)


def _greedy(n):
    from crane_b200.generation import GenerationConfig
    return GenerationConfig(max_new_tokens=n, temperature=None, eos_token_id=-1)


@pytest.mark.parametrize("name", ["MA", "MB", "MC", "MD", "ME", "MF"])
def test_greedy_generation_float32_equals_plain(name, model_folders):
    folder = model_folders(name, "float32")
    cfg, w = pm.load_folder(folder)
    m = _load(folder, "fp32", page_size=tm.TINY[name]["page_size"], num_pages=24, max_concurrent=3,
              max_batched_tokens=64, max_seq_len=256)
    rng = np.random.default_rng(3)
    for n in (1, 5, 17):
        prompt = rng.integers(0, cfg["vocab"], n).tolist()
        assert m.generate(prompt, _greedy(8)) == pm.greedy_generate(cfg, w, prompt, 8)
    m.runner.table.check()
    assert m.runner.table.live() == 0


@pytest.mark.parametrize("name", ["MA", "ML"])
def test_greedy_batch_bfloat16_through_the_scheduler(name, model_folders):
    """Six prompts, three slots, portions of at most 16 tokens: requests wait, slots and pages are
    used again, and decode steps replay graphs with the recurrent states in them."""
    folder = model_folders(name, "bfloat16")
    cfg, w = pm.load_folder(folder)
    m = _load(folder, "bf16", page_size=16, num_pages=40, max_concurrent=3, max_batched_tokens=48, chunk_size=16,
              max_seq_len=256)
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (12, 3, 40, 1, 25, 7)]
    outs = m.generate_batch(prompts, _greedy(20))
    ok = 0
    for prompt, toks in zip(prompts, outs):
        assert len(toks) == len(prompt) + 20 and toks[:len(prompt)] == prompt
        logits = pm.logits_all(cfg, w, toks[:-1])
        for i in range(len(prompt), len(toks)):
            row = logits[i - 1]
            # (a token that another rounding would not have chosen does not end the comparison: every later
            # one is checked against the plain logits of the sequence as it was generated)
            ok += bool(row[toks[i]] >= row.max() - 3e-2 * np.abs(row).max())
    assert ok >= 0.95 * 20 * len(prompts), ok
    m.runner.table.check()
    assert m.runner.table.live() == 0
    assert m.runner.graph_replays > 0


def test_command_line(model_folders):
    """bin/crane picks the model class from config.json."""
    import os
    import subprocess
    import sys
    folder = model_folders("MD", "float32")
    cfg, w = pm.load_folder(folder)
    crane = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "crane")
    cmd = [sys.executable, crane, "-m", folder, "--dtype", "fp32", "--prompt-ids", "5,6,7", "--max-new-tokens", "6",
           "--eos-token-id", "-1", "--page-size", "16", "--num-pages", "8", "-c", "2", "--max-batched-tokens", "32",
           "--max-seq-len", "64"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.strip().splitlines()[-1] == ",".join(map(str, pm.greedy_generate(cfg, w, [5, 6, 7], 6)[3:]))
