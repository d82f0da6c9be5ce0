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
           "MD": [2, 150, 31, 16, 77], "ML": [7, 150, 300, 64]}


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
        assert np.median(errs) <= 1.2e-2 and errs[int(0.9 * (len(errs) - 1))] <= 4e-2, label


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["MA", "MB", "MC", "MD"])
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
@pytest.mark.parametrize("name", ["MA", "MB", "MC", "MD"])
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
