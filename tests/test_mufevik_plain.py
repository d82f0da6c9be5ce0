"""Mufevik on the host: configuration errors, the manifest, and the plain implementation's own
mechanisms against hand arithmetic and against their continuation from a carried state."""
import copy
import math

import numpy as np
import pytest

import plain_mufevik as pm
import tiny_mufevik as tm
from crane_b200.config import ConfigError, resolve
from crane_b200.parts import model_manifest


def _spec(config):
    arch = resolve(config)
    return arch, arch.build_spec(arch.config_from_dict(config))


def test_registered_by_its_name():
    arch, spec = _spec(tm.MA)
    assert arch.name == "Mufevik" and spec.architecture == "Mufevik"
    assert [l.block for l in spec.layers] == ["hyper_connections"] * 4
    assert [l.parts["mixer"].name for l in spec.layers] == ["parallel_pair", "gated_delta", "gated_delta", "parallel_pair"]
    assert "ffn" not in spec.layers[1].parts and "connect2" not in spec.layers[1].parts
    assert spec.layers[0].parts["ffn"].name == "grouped_experts"
    pair = spec.layers[0].parts["mixer"].params
    assert pair["left"].name == "talking_attention" and pair["right"].name == "gated_linear_attention"
    assert [s.layer for s in spec.schedule] == [0, 1, 2, 3]


def test_manifest_names_and_shapes():
    _, spec = _spec(tm.MA)
    m = model_manifest(spec)
    assert m["embed"].shape == (211, 96) and m["head"].shape == (211, 96) and m["final.norm"].shape == ()
    assert m["l0.norm1"].shape == () and m["l0.hc1.in"].shape == (2,) and m["l0.hc2.mix"].shape == (2, 2)
    assert m["l0.mix.left.q"].shape == (144, 96) and m["l0.mix.left.k"].shape == (48, 96)
    assert m["l0.mix.left.v"].shape == (64, 96) and m["l0.mix.left.o"].shape == (96, 192)
    assert m["l0.mix.left.talk"].shape == (6, 6) and m["l0.mix.left.temp"].shape == (6,)
    assert m["l0.mix.right.q"].shape == (48, 96) and m["l0.mix.right.v"].shape == (24, 96)
    assert m["l0.mix.right.a1"].shape == (5, 96) and m["l0.mix.right.a2"].shape == (48, 5)
    assert m["l0.mix.right.a2.b"].shape == (48,) and m["l0.mix.right.norm"].shape == (8,)
    assert m["l0.mix.left.out"].shape == (96,) and m["l0.mix.right.out"].shape == (96,)
    assert m["l1.mix.q"].shape == (32, 96) and m["l1.mix.v"].shape == (96, 96) and m["l1.mix.q.conv"].shape == (32, 3)
    assert m["l1.mix.v.conv"].shape == (96, 3) and m["l1.mix.b"].shape == (4, 96) and m["l1.mix.A_log"].shape == (4,)
    assert m["l1.mix.dt_bias"].shape == (4,) and m["l1.mix.norm"].shape == (24,) and m["l1.mix.o"].shape == (96, 96)
    assert "l1.norm2" not in m and "l1.hc2.in" not in m and "l1.mlp.router" not in m
    assert m["l0.mlp.router"].shape == (6, 96) and m["l0.mlp.correction"].shape == (6,)
    assert m["l0.mlp.e5.gate"].shape == (24, 96) and m["l0.mlp.e0.down"].shape == (96, 24)
    assert m["l0.mlp.shared.up"].shape == (40, 96) and m["l0.mlp.shared.sg"].shape == (1, 96)
    assert "l2.mlp.shared.gate" not in m and "l2.mlp.shared.sg" not in m
    # without a streams entry there is nothing stored for the connections
    m = model_manifest(_spec(tm.MB)[1])
    assert not any(".hc" in name for name in m)
    assert model_manifest(_spec(tm.MD)[1])["l1.hc2.mix"].shape == (1, 1)


def test_the_decay_rank_of_a_stored_model_is_read_from_its_tensors():
    cfg = copy.deepcopy(tm.MC)
    del cfg["layers"][1]["mixer"]["right"]["decay_rank"]
    m = model_manifest(_spec(cfg)[1])
    assert m["l1.mix.right.a1"].shape == (-1, 68) and m["l1.mix.right.a2"].shape == (40, -1)


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="windowed"), "no mixer"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "fewer experts than top"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=26), "at most dim"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(conv=0), "taps"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(tau=0.0), "tau"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "feed-forward kind"),
])
def test_configuration_errors(edit, text):
    cfg = copy.deepcopy(tm.MA)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        _spec(cfg)


# ------------------------------------------------------------------ mechanisms by hand
def test_rotation_pairs_element_i_with_i_plus_half_of_the_rotated_part():
    x = np.arange(1.0, 7.0).reshape(1, 1, 6)                     # rotate the leading 4 of 6
    y = pm.rotate_half(x, [3], 4, 100.0)
    a0, a1 = 3 * 1.0, 3 * 100.0 ** -0.5
    assert np.allclose(y[0, 0], [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                                 3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5.0, 6.0])
    assert np.array_equal(pm.rotate_half(x, [0], 4, 100.0), x)   # position 0 turns nothing
    assert np.array_equal(pm.rotate_half(x, [9], 0, 100.0), x)   # nothing rotated at all


def test_talking_attention_by_hand():
    rng = np.random.default_rng(0)
    n, H, G, d, m = 5, 4, 2, 3, 2
    q, k, v = rng.standard_normal((n, H, d)), rng.standard_normal((n, G, d)), rng.standard_normal((n, G, m))
    temp = np.array([1.0, 0.5, 2.0, 1.5])
    plain = pm.talking_attention(q, k, v, 0.7, temp, np.eye(H))
    for h in range(H):                                            # the identity: ordinary grouped attention
        for i in range(n):
            s = np.array([q[i, h] @ k[j, h // 2] for j in range(i + 1)]) * 0.7 * temp[h]
            p = np.exp(s) / np.exp(s).sum()
            assert np.allclose(plain[i, h], p @ v[:i + 1, h // 2])
    # head 0 takes head 3's weights and applies them to its OWN key/value head's values
    talk = np.eye(H)
    talk[0] = [0, 0, 0, 1]
    out = pm.talking_attention(q, k, v, 0.7, temp, talk)
    for i in range(n):
        s = np.array([q[i, 3] @ k[j, 1] for j in range(i + 1)]) * 0.7 * temp[3]
        p = np.exp(s) / np.exp(s).sum()
        assert np.allclose(out[i, 0], p @ v[:i + 1, 0])
    assert np.allclose(out[:, 1:], plain[:, 1:])
    assert np.allclose(out[0, 0], v[0, 0])                        # the first token sees itself alone


def test_gated_linear_scan_by_hand():
    q = np.array([[[1.0, 2.0]], [[0.5, -1.0]]])
    k = np.array([[[1.0, 0.0]], [[2.0, 1.0]]])
    v = np.array([[[3.0]], [[-1.0]]])
    alpha = np.array([[[0.5, 0.25]], [[0.5, 0.25]]])
    o, S = pm.gated_linear_scan(q, k, v, alpha)
    # S1 = k1 v1^T = [[3], [0]]; o1 = 3;  S2 = diag(.5, .25) S1 + k2 v2^T = [[1.5 - 2], [0 - 1]]
    assert np.allclose(o[:, 0, 0], [3.0, 0.5 * -0.5 + -1.0 * -1.0])
    assert np.allclose(S[0], [[-0.5], [-1.0]])
    o2, S2 = pm.gated_linear_scan(q[1:], k[1:], v[1:], alpha[1:], pm.gated_linear_scan(q[:1], k[:1], v[:1], alpha[:1])[1])
    assert np.allclose(o2[0], o[1]) and np.allclose(S2, S)


def test_gated_delta_scan_by_hand():
    k = np.array([[[1.0, 0.0]], [[1.0, 0.0]]])
    q = np.array([[[1.0, 0.0]], [[1.0, 1.0]]])
    v = np.array([[[2.0, 4.0]], [[10.0, 0.0]]])
    beta, decay = np.array([[1.0], [0.5]]), np.array([[0.3], [0.5]])
    o, S = pm.gated_delta_scan(q, k, v, beta, decay)
    # token 1: S = 0 decays to 0; u = v; S = k u^T = [[2, 4], [0, 0]]; o = S^T q = [2, 4] (sees its own write)
    assert np.allclose(o[0, 0], [2.0, 4.0])
    # token 2: S <- .5 S = [[1, 2], [0, 0]]; S^T k = [1, 2]; u = .5 ([10, 0] - [1, 2]) = [4.5, -1]; S = [[5.5, 1], [0, 0]]
    assert np.allclose(S[0], [[5.5, 1.0], [0.0, 0.0]]) and np.allclose(o[1, 0], [5.5, 1.0])
    # two heads on one query/key head
    v2 = np.concatenate([v, 2 * v], axis=1)
    o2, _ = pm.gated_delta_scan(q, k, v2, np.repeat(beta, 2, 1), np.repeat(decay, 2, 1))
    assert np.allclose(o2[:, 1], 2 * o[:, 0])


def test_short_convolution_by_hand():
    x = np.array([[1.0], [2.0], [3.0], [4.0]])
    w = np.array([[100.0, 10.0, 1.0]])                             # the last column is the current token's
    y, last = pm.short_convolution(x, w)
    assert np.allclose(y[:, 0], [1.0, 12.0, 123.0, 234.0]) and np.allclose(last[:, 0], [3.0, 4.0])
    y2, last2 = pm.short_convolution(x[1:], w, pm.short_convolution(x[:1], w)[1])
    assert np.allclose(y2, y[1:]) and np.allclose(last2, last)
    y1, none = pm.short_convolution(x, np.array([[2.0]]))          # one tap keeps nothing
    assert np.allclose(y1, 2 * x) and none.shape == (0, 1)


def test_choice_of_experts_by_hand():
    z = np.log(np.array([0.30, 0.05, 0.20, 0.15, 0.05, 0.25]))     # scores are these themselves
    none = np.zeros(6)
    idx, wt = pm.choose_experts(z, none, 2, 1, 1)
    assert idx == [0, 5] and np.allclose(wt, [0.30, 0.25])         # not renormalised
    # three groups of two, the best two kept: (0, 1) scores .30, (2, 3) .20, (4, 5) .25 -> expert 2 cannot be chosen
    idx, wt = pm.choose_experts(z, none, 3, 3, 2)
    assert idx == [0, 5, 1] or idx == [0, 5, 4]
    assert idx == [0, 5, 1]                                        # .05 against .05: the lower index
    # the correction moves the choice, not the weight
    corr = np.array([0.0, 0.0, 0.2, 0.0, 0.0, 0.0])
    idx, wt = pm.choose_experts(z, corr, 2, 3, 2)
    assert idx == [2, 0] and np.allclose(wt, [0.20, 0.30])
    # choice scores may all be negative: experts outside the kept groups count as minus infinity, not 0
    corr = np.full(6, -1.0)
    idx, _ = pm.choose_experts(z, corr, 3, 3, 1)
    assert idx[:2] == [0, 1] and len(idx) == 2                     # only the best group's two experts exist


def test_streams_by_hand():
    xs = np.array([[[1.0, 2.0]], [[10.0, 20.0]]])                   # two streams, one token, width 2
    assert np.allclose(pm.streams_read(xs, np.array([2.0, 0.5])), [[7.0, 14.0]])
    mix = np.array([[1.0, 3.0], [0.0, 1.0]])                       # [from, to]: stream 0 also feeds stream 1
    out = pm.streams_write(xs, np.array([[100.0, 200.0]]), mix, np.array([0.0, 1.0]))
    assert np.allclose(out[0], [[1.0, 2.0]]) and np.allclose(out[1], [[3 + 10 + 100.0, 6 + 20 + 200.0]])


def test_scalar_norm_and_unit_vector():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(pm.scalar_norm(x, 2.0, 0.5), x / math.sqrt(12.5 + 0.5) * 2.0)
    assert np.allclose(pm.unit_vector(x, 0.0), [[0.6, 0.8]])
    assert np.allclose(pm.unit_vector(np.zeros((1, 2))), 0.0)      # the epsilon keeps a zero vector finite


# ------------------------------------------------------------------ the whole model
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from crane_b200.weights.random_init import write_model_folder
    made = {}

    def get(name):
        if name not in made:
            spec = tm.TINY[name]
            d = tmp_path_factory.mktemp(name)
            write_model_folder(str(d), spec["config"], spec["seed"], "float32", std=spec["std"], norm_std=spec["norm_std"])
            made[name] = pm.load_folder(str(d))
        return made[name]
    return get


@pytest.mark.parametrize("name", ["MA", "MB", "MC", "MD", "ME", "MF"])
def test_cut_anywhere_the_logits_stay(name, folders):
    cfg, w = folders(name)
    rng = np.random.default_rng(1)
    toks = rng.integers(0, cfg["vocab"], 23).tolist()
    whole, sums, _ = pm.forward(cfg, w, toks)
    assert whole.shape == (23, cfg["vocab"]) and sums.shape == (len(cfg["layers"]), 23, cfg["width"])
    got, state, pos = [], None, 0
    for n in (1, 2, 7, 1, 12):
        part, _, state = pm.forward(cfg, w, toks[pos:pos + n], state, start=pos)
        got.append(part)
        pos += n
    assert np.abs(np.concatenate(got) - whole).max() < 1e-10
    # causal: what comes later changes nothing before it
    other = toks[:10] + rng.integers(0, cfg["vocab"], 13).tolist()
    assert np.abs(pm.logits_all(cfg, w, other)[:10] - whole[:10]).max() < 1e-12


def test_streams_that_start_equal_and_a_single_stream_is_the_residual_sum(folders):
    cfg, w = folders("MB")                                         # no streams entry: x <- x + sublayer(norm(x))
    toks = [3, 1, 4, 1, 5]
    eps = cfg["norm"]["eps"]
    x = w["embed"][toks]
    state = [None] * 3
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = pm.scalar_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "delta":
            y, _ = pm.delta_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            y, _ = pm.parallel_mixer(h, w, p + "mix.", layer["mixer"], eps, np.arange(5))
        x = x + y
        if layer["mlp"] is not None:
            x = x + pm.moe(pm.scalar_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
    logits = pm.scalar_norm(x, w["final.norm"], eps) @ w["head"].T
    assert np.abs(pm.logits_all(cfg, w, toks) - logits).max() < 1e-12
