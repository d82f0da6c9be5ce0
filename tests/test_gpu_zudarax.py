"""Zudarax on the GPU: replay through bin/trace_run against the plain implementation (whole prompts,
tails decoded token by token, portions down to two tokens, mixed batches in a pool so small that pages
and slots are used again), every new kernel alone against NumPy, keys planted far away, at page borders
and just inside and just outside a block of visible positions for every kind of weights (on the
FP32-core kernel and on the warp-level kernels with 1, 3 and 16 key slices), the convolutions' inputs
across steps and slots used again, and greedy generation through the Python entry point, the scheduler
and the command line."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_zudarax as pz
import tiny_zudarax as tz
import trace_tools as tt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LENGTHS = {"ZA": [1, 2, 19, 100, 65, 48, 33], "ZB": [5, 41, 97, 230, 129, 64], "ZC": [3, 70, 130, 17],
           "ZD": [2, 150, 31, 16, 77], "ZL": [7, 150, 300, 64]}


@pytest.fixture(scope="module")
def cases(model_folders):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            folder = model_folders(name, dtype)
            rng = np.random.default_rng(700 + ord(name[1]))
            reqs = tt.make_requests(rng, tz.TINY[name]["config"]["vocab"], LENGTHS[name])
            cfg, w = pz.load_folder(folder)
            made[(name, dtype)] = (folder, reqs, {r: pz.logits_all(cfg, w, t) for r, t in reqs.items()})
        return made[(name, dtype)]
    return get


def _compare(got, tb, plain, dtype, label, tol_rms=3e-5):
    """Every wanted row against the plain logits: root-mean-square error relative to the row's own size."""
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
        assert np.median(errs) <= 1.2e-2 and errs[-1] <= 4e-2, (label, np.median(errs), errs[-1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["ZA", "ZB", "ZC", "ZD"])
def test_alone_whole_tail_portions(name, dtype, cases, tmp_path):
    folder, reqs, plain = cases(name, dtype)
    ps = tz.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_whole(tb, reqs)
    tt.trace_tail_decode(tb, reqs)
    tt.trace_portions(tb, reqs, np.random.default_rng(7))
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    _compare(got, tb, plain, dtype, f"config {name}")
    tt.compare_cuts([(got, tb)], dtype, f"config {name}", tol=1e-6 if dtype == "float32" else 2.5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["ZA", "ZB", "ZC", "ZD"])
def test_mixed_with_page_and_slot_reuse(name, dtype, cases, tmp_path):
    folder, reqs, plain = cases(name, dtype)
    ps = tz.TINY[name]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_mixed(tb, reqs, np.random.default_rng(11), max_live=3)
    assert tb.pages_taken > tb.peak_tokens // ps, "the trace must make the pool hand pages out again"
    assert max(len(s["entries"]) for s in tb.steps) >= 3
    # three slots for all requests; single tokens beside portions take the split-KV kernel from the first key on
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"),
                       extra_args=["--max-live", "3", "--mixed-decode-min-keys", "1"])
    _compare(got, tb, plain, dtype, f"config {name} mixed")


def test_long_decoding(cases, tmp_path):
    """200 tokens decoded one by one: across blocks of 7 positions and pages of 8."""
    folder, reqs, plain = cases("ZB", "float32")
    ps = tz.TINY["ZB"]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_tail_decode(tb, {"r3": reqs["r3"]}, tail=200)
    got = tt.run_trace(folder, "float32", tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    _compare(got, tb, plain, "float32", "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_sizes_of_the_tensor_core_kernels(dtype, cases, tmp_path):
    folder, reqs, plain = cases("ZL", dtype)
    ps = tz.TINY["ZL"]["page_size"]
    tb = tt.TraceBuilder(ps)
    tt.trace_whole(tb, reqs)
    tt.trace_tail_decode(tb, reqs, tail=40)
    tt.trace_portions(tb, reqs, np.random.default_rng(3))
    tt.trace_mixed(tb, reqs, np.random.default_rng(5))
    got = tt.run_trace(folder, dtype, tb.steps, tb.peak_tokens, ps, str(tmp_path / "out"))
    _compare(got, tb, plain, dtype, "config ZL", tol_rms=6e-5)
    if dtype == "float32":
        tt.compare_cuts([(got, tb)], dtype, "config ZL", tol=6e-5)


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
@pytest.mark.parametrize("width, groups", [(48, 1), (96, 3), (68, 4), (1000, 2), (64, 16), (2048, 8), (15, 15)])
def test_add_group_rmsnorm(K, dtype, width, groups):
    """Nothing pending, one result, two results (whole and as partial sums), and chosen rows only, which
    must leave the stream as it is."""
    from crane_b200.kernels import Partials
    rng = np.random.default_rng(width + groups)
    n, eps = 6, 1e-5
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    x = _dev(rng.standard_normal((n, width)) * 3)
    w = 1 + 0.3 * rng.standard_normal(width)
    xs = x.double().cpu().numpy()
    out = torch.empty(n, width, dtype=dtype, device=DEV)
    K.add_group_rmsnorm(x, None, None, _dev(w), groups, eps, out)
    assert np.abs(out.double().cpu().numpy() - pz.group_norm(xs, w, groups, eps)).max() < tol * 4
    assert np.array_equal(x.double().cpu().numpy(), xs)
    a = _dev(rng.standard_normal((n, width)), dtype)
    parts = _dev(rng.standard_normal((3, n, width)))
    f = Partials(parts)
    fn = parts.sum(0).to(dtype).double().cpu().numpy()
    for first, second in ((a, None), (None, f), (a, f)):
        add = (first.double().cpu().numpy() if first is not None else 0.0) + (fn if second is not None else 0.0)
        K.add_group_rmsnorm(x, first, second, _dev(w), groups, eps, out)
        xs = xs + add
        assert np.abs(x.double().cpu().numpy() - xs).max() < 1e-5 * np.abs(xs).max()
        assert np.abs(out.double().cpu().numpy() - pz.group_norm(xs, w, groups, eps)).max() < tol * 4
    rows = _i32([4, 1])
    out2 = torch.empty(2, width, dtype=dtype, device=DEV)
    before = x.clone()
    K.add_group_rmsnorm(x, a, f, _dev(w), groups, eps, out2, rows)
    want = pz.group_norm(xs + a.double().cpu().numpy() + fn, w, groups, eps)[[4, 1]]
    assert np.abs(out2.double().cpu().numpy() - want).max() < tol * 4
    assert torch.equal(x, before)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("F", [40, 33, 1024, 3001])
def test_poly_norm(K, dtype, F):
    from crane_b200.kernels import Partials
    rng = np.random.default_rng(F)
    n, eps = 5, 1e-6
    coef = np.array([0.7, -0.4, 0.2, 0.1])
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for form in ("whole", "parts"):
        if form == "whole":
            up = _dev(rng.standard_normal((n, F)) * 1.5, dtype)
            un = up.double().cpu().numpy()
        else:
            parts = _dev(rng.standard_normal((2, n, F)))
            up = Partials(parts)
            un = parts.sum(0).to(dtype).double().cpu().numpy()
        out = torch.full((n + 1, F), 5.0, dtype=dtype, device=DEV)
        K.poly_norm(up, _dev(coef), eps, out[:n])
        want = pz.poly_norm(un, coef, eps)
        assert np.abs(out[:n].double().cpu().numpy() - want).max() < tol * max(1.0, np.abs(want).max()), form
        assert (out[n] == 5.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, maps, dv, dv_in, dv_out, norm, gated", [(3, 2, 24, 24, 24, True, True), (1, 2, 40, 64, 40, True, False),
                                                                     (4, 1, 8, 8, 16, False, True), (2, 1, 100, 128, 100, True, True)])
def test_head_finish(K, dtype, H, maps, dv, dv_in, dv_out, norm, gated):
    rng = np.random.default_rng(H * dv)
    n, eps, lam, scale = 9, 1e-3, 0.37, 0.6
    a = rng.standard_normal((n, H, maps, dv_in)) * 0.05          # small, so that eps counts
    gate = rng.random((n, H))
    ent = np.zeros(n, dtype=np.int32)
    ent[3] = -1                                                    # a row of no entry stays as it is
    out = torch.full((n, H * dv_out), 5.0, dtype=dtype, device=DEV)
    K.head_finish(_dev(a.reshape(n, -1)), _i32(ent), _dev(gate) if gated else None, out, H, maps, dv, lam, norm, scale, eps)
    o = a[:, :, 0, :dv] - (lam * a[:, :, 1, :dv] if maps == 2 else 0.0)
    if norm:
        o = pz.unit_rms(o, eps) * scale
    if gated:
        o = o * gate[:, :, None]
    want = np.zeros((n, H, dv_out))
    want[:, :, :dv] = o
    want[3] = 5.0
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(out.double().cpu().numpy().reshape(n, H, dv_out) - want).max() < tol * max(1.0, np.abs(want).max())


# ---------------------------------------------------------------- preparation and attention
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


def _steps_of(lens, plan):
    """``plan``: per step a list of (request, tokens taken, slot).  Yields per step (request, first
    position, count, slot) of every entry."""
    done = [0] * len(lens)
    for step in plan:
        ents = []
        for r, take, slot in step:
            ents.append((r, done[r], take, slot))
            done[r] += take
        yield ents
    assert done == list(lens)


def _ctx(ents):
    q_lens = [t for _, _, t, _ in ents]
    return SimpleNamespace(cu_q=_i32(np.concatenate([[0], np.cumsum(q_lens)])),
                           kv_len=_i32([b + t for _, b, t, _ in ents]), slots=_i32([s for _, _, _, s in ents]),
                           tok_entry=_i32(np.concatenate([np.full(t, i) for i, t in enumerate(q_lens)])),
                           positions=_i32(np.concatenate([np.arange(b, b + t) for _, b, t, _ in ents])))


# three requests and a fourth that takes the second one's slot; portions (one shorter than the taps), single
# tokens, a request left out of a step; slots in no order
PLAN = [[(0, 20, 2), (1, 1, 0), (2, 4, 1)], [(2, 5, 1), (0, 1, 2)], [(0, 1, 2)], [(0, 15, 2), (3, 2, 0)], [(3, 9, 0)]]
PLAN_LENS = [37, 1, 9, 11]


def _plain_prep(x, H, G, maps, d, m, conv_w, qw, kw, eps, rot, base, scaling, gated):
    """Rows x [n, cols] of one request -> q [n, H maps, d], k [n, G maps, d], v [n, G, m], gate [n, H]."""
    n = x.shape[0]
    cq, ck, cv = H * maps * d, G * maps * d, G * m
    y = x[:, :cq + ck + cv]
    if conv_w is not None:
        y = pz.short_convolution(y, conv_w)[0]
    q, k, v = y[:, :cq], y[:, cq:cq + ck], y[:, cq + ck:]
    if qw is not None:
        q, k = pz.unit_rms(q, eps) * qw, pz.unit_rms(k, eps) * kw
    pos = np.arange(n)
    q = pz.rotate_half(q.reshape(n, H * maps, d), pos, rot, base, scaling)
    k = pz.rotate_half(k.reshape(n, G * maps, d), pos, rot, base, scaling)
    gate = pz.sigmoid(x[:, cq + ck + cv:cq + ck + cv + H]) if gated else None
    return q, k, v.reshape(n, G, m), gate


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, maps, d, m, taps, norm, rot, dk_store, dpad, dv_store, gated", [
    (4, 2, 1, 16, 24, 3, True, 8, 16, 16, 24, False), (5, 1, 1, 16, 16, 1, False, 0, 32, 32, 32, False),
    (2, 1, 2, 12, 40, 0, False, 4, 64, 32, 64, True), (3, 3, 1, 8, 8, 2, True, 8, 8, 8, 8, True),
    (2, 2, 2, 40, 12, 16, True, 16, 80, 40, 12, True), (1, 1, 1, 64, 32, 5, False, 64, 64, 64, 48, False)])
def test_scored_prep(K, dtype, H, G, maps, d, m, taps, norm, rot, dk_store, dpad, dv_store, gated):
    """Convolutions with their inputs carried in the slot, norms over the whole rows, rotation of each map,
    the cache write (also into rows wider than the heads) and the gate, over a plan of steps: a portion
    shorter than the taps, single tokens, a request left out of a step, a slot used again."""
    rng = np.random.default_rng(H * 10 + taps + d)
    cq, ck, cv = H * maps * d, G * maps * d, G * m
    C = cq + ck + cv
    cols = C + (H if gated else 0) + 3
    ps, eps, base = 8, 1e-5, 300.0
    scaling = {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 0.5} if rot >= 8 else None
    conv_w = rng.standard_normal((C, taps)) if taps else None
    qw, kw = (1 + 0.3 * rng.standard_normal(cq), 1 + 0.3 * rng.standard_normal(ck)) if norm else (None, None)
    proj = [_dev(rng.standard_normal((n, cols)), dtype) for n in PLAN_LENS]
    wants = [_plain_prep(p.double().cpu().numpy(), H, G, maps, d, m, conv_w, qw, kw, eps, rot, base, scaling, gated)
             for p in proj]
    cos = sin = None
    if rot:
        f, mag = pz.rotary_frequencies(rot, base, scaling)
        ang = np.arange(max(PLAN_LENS))[:, None] * f[None, :]
        cos, sin = _dev(np.cos(ang) * mag), _dev(np.sin(ang) * mag)
    full_table, n_pages = _step_meta(PLAN_LENS, ps, rng)
    k_pool = torch.full((n_pages, G, ps, dk_store), 9.0, dtype=dtype, device=DEV)
    v_pool = torch.full((n_pages, G, ps, dv_store), 9.0, dtype=dtype, device=DEV)
    tails = torch.full((4, max(taps - 1, 0) * C + 3), 1e3, device=DEV) if taps > 1 else None
    err = _err()
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for ents in _steps_of(PLAN_LENS, PLAN):
        ctx = _ctx(ents)
        rows = torch.cat([proj[r][b:b + t] for r, b, t, _ in ents])
        n = rows.shape[0]
        table = _i32(full_table[[r for r, _, _, _ in ents]])
        q_out = torch.full((n + 1, H * dk_store), 5.0, dtype=dtype, device=DEV)
        gate = torch.full((n, H), 5.0, device=DEV) if gated else None
        K.scored_prep(rows, cols, ctx, table, tails, None if conv_w is None else _dev(conv_w.T.copy()), max(taps, 1), ps,
                      None if qw is None else _dev(qw), None if kw is None else _dev(kw), eps, q_out[:n], k_pool, v_pool,
                      H, G, maps, d, m, dpad, cos, sin, rot, gate, C, err)
        assert (q_out[n] == 5.0).all()
        got_q = q_out[:n].double().cpu().numpy().reshape(n, H, dk_store)
        at = 0
        for r, b, t, _ in ents:
            wq, wk, wv, wg = wants[r]
            for i in range(t):
                for mp in range(maps):
                    have = got_q[at + i, :, mp * dpad:mp * dpad + d]
                    want = wq[b + i].reshape(H, maps, d)[:, mp]
                    assert np.abs(have - want).max() < tol * max(1.0, np.abs(want).max()), ("q", r, b + i, mp)
                    assert (got_q[at + i, :, mp * dpad + d:(mp + 1) * dpad] == 0).all()
                page, place = full_table[r][(b + i) // ps], (b + i) % ps
                have_k = k_pool[page, :, place].double().cpu().numpy()
                for mp in range(maps):
                    want = wk[b + i].reshape(G, maps, d)[:, mp]
                    assert np.abs(have_k[:, mp * dpad:mp * dpad + d] - want).max() < tol * max(1.0, np.abs(want).max())
                    assert (have_k[:, mp * dpad + d:(mp + 1) * dpad] == 0).all()
                assert (have_k[:, maps * dpad:] == 0).all()
                have_v = v_pool[page, :, place].double().cpu().numpy()
                assert np.abs(have_v[:, :m] - wv[b + i]).max() < tol * max(1.0, np.abs(wv).max())
                assert (have_v[:, m:] == 0).all()
                if gated:
                    assert np.abs(gate[at + i].double().cpu().numpy() - wg[b + i]).max() < 1e-5
            at += t
    if tails is not None:
        assert (tails[:, (taps - 1) * C:] == 1e3).all() and (tails[3] == 1e3).all()     # nothing behind, no other slot
    assert int(err.item()) == 0


def _plain_head(kind, q, k, v, pos, scale, cap, block, bias, lam, norm_scale, eps):
    """One query position ``pos`` of one head: q [maps, d], k [T, maps, d], v [T, m]."""
    keys = np.arange(k.shape[0])
    if kind == "sig":
        return pz.attention_weights(q[:1], k[:, 0], [pos], keys, scale, cap, block, "sigmoid", bias)[0] @ v
    a = [pz.attention_weights(q[i:i + 1], k[:, i], [pos], keys, scale, cap, block)[0] @ v for i in range(q.shape[0])]
    if kind == "soft":
        return a[0]
    return pz.unit_rms(a[0] - lam * a[1], eps) * norm_scale


@pytest.mark.parametrize("dtype, splits", [(torch.float32, 0), (torch.bfloat16, 0), (torch.bfloat16, 1), (torch.bfloat16, 3),
                                           (torch.bfloat16, 16)])
@pytest.mark.parametrize("kind, H, G, d, m, rot, ps, block, cap, taps", [
    ("soft", 4, 1, 64, 80, 32, 64, 100, 8.0, 3), ("soft", 6, 2, 16, 24, 8, 16, 24, 0.0, 0), ("soft", 2, 2, 100, 128, 100, 16, 0, 30.0, 2),
    ("sig", 3, 3, 24, 8, 0, 8, 0, 0.0, 2), ("sig", 8, 2, 128, 128, 64, 32, 0, 0.0, 4), ("sig", 5, 1, 48, 40, 16, 16, 50, 4.0, 0),
    ("diff", 6, 2, 32, 48, 16, 16, 0, 0.0, 0), ("diff", 2, 2, 12, 40, 4, 16, 0, 0.0, 0), ("diff", 16, 2, 64, 128, 64, 32, 0, 0.0, 0),
    ("diff", 3, 1, 16, 16, 16, 8, 20, 6.0, 3)])
def test_scored_attention_with_planted_keys(K, dtype, splits, kind, H, G, d, m, rot, ps, block, cap, taps):
    """Preparation, cache write and attention over prompts and decoded tokens for every kind of weights.
    One key per request is made to stand out for the last query of head 0 in the part of the head that is
    not rotated: far back, at a page's last place with its opposite at the next page's first, the newest,
    and with blocks the block's first position, with a still larger key at the position before it, which
    must stay unseen.  ``splits`` 0: the FP32-core kernel on rows as wide as they are; else the warp-level
    kernels on rows stored at a common head size, decoded tokens in that many slices."""
    from crane_b200.config.zudarax import _stored_head
    maps = 2 if kind == "diff" else 1
    D, dpad = (_stored_head(maps, d, m) if splits else (0, 0))
    if splits:
        assert D and K.scored_attention_supports(D, H, G, maps)
    Dk, Dv, dpad = D or maps * d, D or m, dpad or d
    rng = np.random.default_rng(H * 100 + d)
    lens = [700, 2 * ps + 1, 1, 37]
    scale, base, eps, lam, norm_scale = 0.4, 300.0, 1e-6, 0.45, 0.55
    gated = kind == "diff"
    bias = rng.standard_normal(H) if kind == "sig" else None
    cq, ck, cv = H * maps * d, G * maps * d, G * m
    C = cq + ck + cv
    cols = C + (H if gated else 0)
    conv_w = None
    if taps:
        conv_w = 0.1 * rng.standard_normal((C, taps))
        conv_w[:, -1] = 1.0 + 0.1 * rng.standard_normal(C)          # mostly the token itself, so that planted keys stay
    qkv = [rng.standard_normal((n, cols)) for n in lens]
    free = slice(rot, d) if rot < d else slice(0, d)
    first_seen = lambda p: p // block * block if block else 0
    planted = {0: first_seen(699) if block else 3, 1: ps - 1 if not block or first_seen(2 * ps) <= ps - 1 else 2 * ps, 3: 36}
    for e, key in planted.items():
        qkv[e][key, cq + free.start:cq + free.stop] *= 6.0
        qkv[e][-1, free] = qkv[e][key, cq + free.start:cq + free.stop] * 2
    if block and planted[0] > 0:
        qkv[0][planted[0] - 1, cq:cq + d] = qkv[0][planted[0], cq:cq + d] * 2      # just outside the block
    qkv[1][ps, cq:cq + d] = -qkv[1][ps - 1, cq:cq + d]
    store = torch.float32 if dtype == torch.float32 else torch.bfloat16
    qkv_dev = [_dev(a, store) for a in qkv]
    stored = lambda a: torch.as_tensor(a).to(store).double().numpy()
    prep = [_plain_prep(a.double().cpu().numpy(), H, G, maps, d, m, conv_w, None, None, eps, rot, base, None, gated)
            for a in qkv_dev]
    cos = sin = None
    if rot:
        ang = np.arange(max(lens))[:, None] * (base ** (-2.0 * np.arange(rot // 2) / rot))[None, :]
        cos, sin = _dev(np.cos(ang)), _dev(np.sin(ang))
    err = _err()
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    full_table, n_pages = _step_meta(lens, ps, rng)
    k_pool = torch.randn(n_pages, G, ps, Dk, device=DEV).mul_(30).to(store)
    v_pool = torch.randn(n_pages, G, ps, Dv, device=DEV).mul_(30).to(store)
    tails = torch.full((len(lens), max(taps - 1, 0) * C), 1e3, device=DEV) if taps > 1 else None
    finish = kind == "diff"
    mod = K.ScoreMod(softcap=cap, chunk=block, sigmoid=kind == "sig", head_bias=None if bias is None else _dev(bias),
                     maps=maps, lam=lam, head_norm=finish, norm_scale=norm_scale, eps=eps, dv=m, compact=finish)
    # whole prompts but the last token of each longer request, then a step that decodes those
    for stage in (0, 1):
        if stage == 0:
            ents = [(e, 0, max(1, n - 1), e) for e, n in enumerate(lens)]
        else:
            ents = [(e, n - 1, 1, e) for e, n in enumerate(lens) if n > 1]
        ctx = _ctx(ents)
        table = _i32(full_table[[e for e, _, _, _ in ents]])
        rows = torch.cat([qkv_dev[e][b:b + t] for e, b, t, _ in ents])
        n = rows.shape[0]
        q_out = torch.empty(n, H * Dk, dtype=store, device=DEV)
        gate = torch.empty(n, H, device=DEV) if gated else None
        K.scored_prep(rows, cols, ctx, table, tails, None if conv_w is None else _dev(conv_w.T.copy()), max(taps, 1), ps, None, None,
                      eps, q_out, k_pool, v_pool, H, G, maps, d, m, dpad, cos, sin, rot, gate, C, err)
        if not splits:
            raw = torch.full((n, H * maps * m), 7.0, device=DEV) if finish else None
            o = torch.full((n + 1, H * m), 5.0, dtype=store, device=DEV)
            K.scored_attention_simt(q_out, None if finish else o[:n], k_pool, v_pool, ctx.positions, ctx.tok_entry, table, ps,
                                    H, G, d, m, 0, scale, err, softcap=cap, chunk=block, sigmoid=kind == "sig",
                                    head_bias=mod.head_bias, maps=maps, d_row=maps * d, d_map=d, out_f32=raw)
            if finish:
                K.head_finish(raw, ctx.tok_entry, gate, o[:n], H, maps, m, lam, True, norm_scale, eps)
            got = o[:n].double().cpu().numpy().reshape(n, H, m)
        else:
            mod.gate = gate
            width = m if finish else D
            o = torch.full((n + 1, H * width), 5.0, dtype=store, device=DEV)
            if stage == 0:
                tiles = sum((t + 63) // 64 for _, _, t, _ in ents)
                K.scored_prefill_attention(q_out, o[:n], k_pool, v_pool, ctx.cu_q, ctx.kv_len, table, ps, tiles, H, G, D, 0,
                                           scale, mod, err)
            else:
                part_o = torch.empty(n * H * maps * splits, D, device=DEV)
                part_ml = torch.empty(n * H * maps * splits, 2, device=DEV)
                K.scored_decode_attention(q_out, o[:n], k_pool, v_pool, ctx.cu_q, ctx.kv_len, table, ps, H, G, D, 0, scale,
                                          splits, part_o, part_ml, mod, err)
            got = o[:n].double().cpu().numpy().reshape(n, H, width)[:, :, :m]
        assert (o[n] == 5.0).all()                                  # nothing is written behind the last head
        at = 0
        for e, b, t, _ in ents:
            wq, wk, wv, wg = prep[e]
            wq, wk, wv = stored(wq), stored(wk), stored(wv)
            for i in range(t):
                p = b + i
                for h in range(H):
                    g = h // (H // G)
                    want = _plain_head(kind, wq[p].reshape(H, maps, d)[h], wk[:p + 1].reshape(p + 1, G, maps, d)[:, g],
                                       wv[:p + 1, g], p, scale, cap, block, 0.0 if bias is None else bias[h], lam,
                                       norm_scale, eps)
                    if gated:
                        want = want * wg[p, h]
                    assert np.abs(got[at + i, h] - want).max() < tol * max(1.0, np.abs(want).max()), (stage, e, p, h)
            at += t
        if stage == 1 and rot < d and kind == "soft" and not cap and not taps:
            for e, b, _, _ in ents:
                if e in planted:                                    # head 0's weights sit on the planted key
                    wq, wk = stored(prep[e][0]), stored(prep[e][1])
                    w0 = pz.attention_weights(wq[b].reshape(H, maps, d)[0, :1], wk[:b + 1].reshape(b + 1, G, maps, d)[:, 0, 0],
                                              [b], np.arange(b + 1), scale, cap, block)[0]
                    assert w0[planted[e]] > 0.9, (e, w0[planted[e]])
    assert int(err.item()) == 0


# ---------------------------------------------------------------- generation
def _load(folder, dtype, **opts):
    from crane_b200.generation import ModelForCausalLM
    return ModelForCausalLM.from_pretrained(folder, dtype, **opts)


def _greedy(n):
    from crane_b200.generation import GenerationConfig
    return GenerationConfig(max_new_tokens=n, temperature=None, eos_token_id=-1)


@pytest.mark.parametrize("name", ["ZA", "ZB", "ZC", "ZD"])
def test_greedy_generation_float32_equals_plain(name, model_folders):
    folder = model_folders(name, "float32")
    cfg, w = pz.load_folder(folder)
    m = _load(folder, "fp32", page_size=tz.TINY[name]["page_size"], num_pages=24, max_concurrent=3,
              max_batched_tokens=64, max_seq_len=256)
    rng = np.random.default_rng(3)
    for n in (1, 5, 17):
        prompt = rng.integers(0, cfg["vocab"], n).tolist()
        assert m.generate(prompt, _greedy(8)) == pz.greedy_generate(cfg, w, prompt, 8)
    m.runner.table.check()
    assert m.runner.table.live() == 0


@pytest.mark.parametrize("name", ["ZA", "ZL"])
def test_greedy_batch_bfloat16_through_the_scheduler(name, model_folders):
    """Six prompts, three slots, portions of at most 16 tokens: requests wait, slots and pages are used
    again, and decode steps replay graphs with the convolutions' inputs in them."""
    folder = model_folders(name, "bfloat16")
    cfg, w = pz.load_folder(folder)
    m = _load(folder, "bf16", page_size=16, num_pages=40, max_concurrent=3, max_batched_tokens=48, chunk_size=16,
              max_seq_len=256)
    # the warp-level kernels serve, at the head sizes the heads are stored at
    assert all(b.mixer.store > 0 for b in m.runner.model.blocks)
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (12, 3, 40, 1, 25, 7)]
    outs = m.generate_batch(prompts, _greedy(20))
    ok = 0
    for prompt, toks in zip(prompts, outs):
        assert len(toks) == len(prompt) + 20 and toks[:len(prompt)] == prompt
        logits = pz.logits_all(cfg, w, toks[:-1])
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
    folder = model_folders("ZD", "float32")
    cfg, w = pz.load_folder(folder)
    crane = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "crane")
    cmd = [sys.executable, crane, "-m", folder, "--dtype", "fp32", "--prompt-ids", "5,6,7", "--max-new-tokens", "6",
           "--eos-token-id", "-1", "--page-size", "16", "--num-pages", "8", "-c", "2", "--max-batched-tokens", "32",
           "--max-seq-len", "64"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.strip().splitlines()[-1] == ",".join(map(str, pz.greedy_generate(cfg, w, [5, 6, 7], 6)[3:]))
