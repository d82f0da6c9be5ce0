"""Zudarax on the host: configuration errors, the manifest, and the plain implementation's own
mechanisms against hand arithmetic and against their continuation from what an earlier call left."""
import copy
import math

import numpy as np
import pytest

import plain_zudarax as pz
import tiny_zudarax as tz
from crane_b200.config import ConfigError, resolve
from crane_b200.config.zudarax import _stored_head
from crane_b200.parts import model_manifest


def _spec(config):
    arch = resolve(config)
    return arch, arch.build_spec(arch.config_from_dict(config))


def test_registered_by_its_name():
    arch, spec = _spec(tz.ZA)
    assert arch.name == "Zudarax" and spec.architecture == "Zudarax"
    assert [l.block for l in spec.layers] == ["parallel_shared_norm"] * 4
    assert all(l.parts["mixer"].name == "scored_attention" for l in spec.layers)
    assert "ffn" not in spec.layers[1].parts and spec.layers[0].parts["ffn"].name == "poly_norm_mlp"
    assert spec.layers[0].parts["norm1"].name == "group_rms_norm" and spec.layers[0].parts["norm1"].params["groups"] == 3
    assert spec.final_norm.name == "group_rms_norm" and "norm2" not in spec.layers[0].parts
    a, d, s = (spec.layers[i].parts["mixer"].params for i in (0, 1, 2))
    assert a["bias"] and a["qk_norm"] and a["conv"] == 3 and a["softcap"] == 12.0 and a["chunk"] == 24
    assert a["maps"] == 1 and a["weighting"] == "softmax" and not a["gate"] and not a["head_norm"]
    assert a["rotary_dim"] == 8 and a["position"].params["scaling"] is None
    assert d["maps"] == 2 and d["gate"] and d["head_norm"] and d["diff"] == 0.3 and not d["bias"] and not d["conv"]
    assert s["weighting"] == "sigmoid" and s["head_bias"] and s["conv"] == 2 and not s["qk_norm"]
    assert s["position"].params["scaling"] == {"factor": 4.0, "original": 64.0, "fast": 8.0, "slow": 1.0}
    assert [st.layer for st in spec.schedule] == [0, 1, 2, 3]


def test_manifest_names_and_shapes():
    m = model_manifest(_spec(tz.ZA)[1])
    assert m["embed"].shape == (211, 96) and m["head"].shape == (211, 96) and m["final.norm"].shape == (96,)
    assert m["l0.norm1"].shape == (96,) and "l0.norm2" not in m
    assert m["l0.mix.q"].shape == (144, 96) and m["l0.mix.k"].shape == (48, 96) and m["l0.mix.v"].shape == (64, 96)
    assert m["l0.mix.q.b"].shape == (144,) and m["l0.mix.k.b"].shape == (48,) and m["l0.mix.v.b"].shape == (64,)
    assert m["l0.mix.q.conv"].shape == (144, 3) and m["l0.mix.v.conv"].shape == (64, 3)
    assert m["l0.mix.q.norm"].shape == (144,) and m["l0.mix.k.norm"].shape == (48,) and m["l0.mix.o"].shape == (96, 192)
    assert m["l0.mlp.up"].shape == (40, 96) and m["l0.mlp.down"].shape == (96, 40) and m["l0.mlp.act"].shape == (4,)
    # two maps: twice the rows in q and k
    assert m["l1.mix.q"].shape == (128, 96) and m["l1.mix.k"].shape == (64, 96) and m["l1.mix.v"].shape == (48, 96)
    assert m["l1.mix.lq1"].shape == (16,) and m["l1.mix.lk2"].shape == (16,) and m["l1.mix.g"].shape == (4, 96)
    assert m["l1.mix.o"].shape == (96, 96) and "l1.mix.q.b" not in m and "l1.mix.q.conv" not in m
    assert "l1.mlp.up" not in m and "l1.mix.pb" not in m
    assert m["l2.mix.pb"].shape == (2,) and m["l2.mix.k.conv"].shape == (48, 2) and "l2.mix.q.norm" not in m
    assert model_manifest(_spec(tz.ZB)[1])["l0.mix.q.conv"].shape == (80, 1)


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="attention_4"), "no mixer"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "at most dim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "lacks 'diff'"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"), "lacks 'fast'"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "no feed-forward kind"),
    (lambda c: c["norm"].update(groups=5), "must divide"),
    (lambda c: c.pop("width"), "lacks 'width'"),
    (lambda c: c["norm"].pop("eps"), "lacks 'eps'"),
])
def test_configuration_errors(edit, text):
    cfg = copy.deepcopy(tz.ZA)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        _spec(cfg)


def test_options_a_mixer_entry_does_not_name_are_absent():
    cfg = copy.deepcopy(tz.ZA)
    m = cfg["layers"][0]["mixer"]
    for key in ("conv", "rot", "softcap", "mask"):
        m.pop(key)
    _, spec = _spec(cfg)
    a = spec.layers[0].parts["mixer"].params
    assert not a["conv"] and not a["rotary_dim"] and a["position"] is None and not a["softcap"] and not a["chunk"]
    assert "l0.mix.q.conv" not in model_manifest(spec)
    del cfg["norm"]["groups"]
    assert _spec(cfg)[1].final_norm.params["groups"] == 1


def test_the_head_size_heads_are_stored_at():
    assert _stored_head(1, 24, 32) == (32, 32) and _stored_head(1, 100, 8) == (112, 112)
    assert _stored_head(2, 16, 24) == (32, 16) and _stored_head(2, 12, 40) == (64, 32)
    assert _stored_head(2, 64, 128) == (128, 64) and _stored_head(2, 32, 16) == (64, 32)
    assert _stored_head(1, 300, 8) == (0, 0)


# ------------------------------------------------------------------ mechanisms against hand arithmetic
def test_group_norm():
    x = np.array([[3.0, 4.0, 0.0, 1.0, 1.0, 1.0]])
    w = np.array([1.0, 2.0, 1.0, 1.0, 1.0, 0.5])
    got = pz.group_norm(x, w, 2, 0.0)
    r1, r2 = math.sqrt(25.0 / 3), 1.0
    assert np.allclose(got, [[3 / r1, 8 / r1, 0.0, 1.0, 1.0, 0.5]])
    assert np.allclose(pz.group_norm(x, w, 1, 0.0), x / math.sqrt(28.0 / 6) * w)
    assert np.allclose(pz.group_norm(np.zeros((1, 6)), w, 3, 1e-6), 0.0)


def test_poly_norm():
    z = np.array([[1.0, -2.0]])
    a, b, c, e = 0.5, -1.0, 2.0, 0.25
    n1, n2, n3 = math.sqrt(2.5), math.sqrt(8.5), math.sqrt(32.5)
    want = [a * 1 / n1 + b * 1 / n2 + c * 1 / n3 + e, a * -2 / n1 + b * 4 / n2 + c * -8 / n3 + e]
    assert np.allclose(pz.poly_norm(z, [a, b, c, e], 0.0), [want])


def test_short_convolution_and_its_continuation():
    rng = np.random.default_rng(0)
    u, w = rng.standard_normal((9, 3)), rng.standard_normal((3, 4))
    y, tail = pz.short_convolution(u, w)
    assert np.allclose(y[0], w[:, 3] * u[0]) and np.allclose(y[1], w[:, 3] * u[1] + w[:, 2] * u[0])
    assert np.allclose(y[5], sum(w[:, j] * u[5 - 3 + j] for j in range(4))) and np.allclose(tail, u[6:])
    for cut in (1, 2, 5, 8):
        y1, t1 = pz.short_convolution(u[:cut], w)
        y2, t2 = pz.short_convolution(u[cut:], w, t1)
        assert np.allclose(np.concatenate([y1, y2]), y) and np.allclose(t2, tail)
    y1, t1 = pz.short_convolution(u, w[:, :1])
    assert np.allclose(y1, u * w[:, 0]) and t1.shape == (0, 3)


def test_rotation_and_yarn():
    f, mag = pz.rotary_frequencies(8, 100.0)
    assert np.allclose(f, [1.0, 100 ** -0.25, 0.1, 100 ** -0.75]) and mag == 1.0
    x = np.zeros((1, 1, 6))
    x[0, 0] = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]
    got = pz.rotate_half(x, [2], 4, 100.0)[0, 0]
    a0, a1 = 2.0, 2.0 * 0.1
    assert np.allclose(got, [math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                             3 * math.cos(a0) + math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5.0, 6.0])
    # YaRN: fast turns keep their frequency, slow ones are divided by the factor, between them a ramp
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    f0, _ = pz.rotary_frequencies(32, 2000.0)
    f, mag = pz.rotary_frequencies(32, 2000.0, sc)
    where = lambda t: 32 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(2000.0))
    lo, hi = max(math.floor(where(8.0)), 0), min(math.ceil(where(1.0)), 31)
    assert lo == 0 and hi == 5
    assert np.allclose(f[0], f0[0]) and np.allclose(f[5:], f0[5:] / 4.0) and np.allclose(f[2], f0[2] * (0.6 + 0.4 / 4))
    assert math.isclose(mag, 0.1 * math.log(4.0) + 1.0)
    from crane_b200.config.spec import PartSpec
    from crane_b200.parts.base import build_part
    part = build_part(PartSpec("position", "yarn_rope", {"dims": 32, "base": 2000.0, "scaling": sc, "max_positions": 64}))
    fe, me = part.frequencies()
    assert np.allclose(fe, f, rtol=1e-14) and math.isclose(me, mag)


def test_weights_blocks_squashing_sigmoid():
    rng = np.random.default_rng(1)
    q, k = rng.standard_normal((6, 4)), rng.standard_normal((6, 4))
    pos = np.arange(6)
    w = pz.attention_weights(q, k, pos, pos, 0.5)
    assert np.allclose(w.sum(1), 1.0) and np.allclose(np.triu(w, 1), 0.0) and w[0, 0] == 1.0
    w = pz.attention_weights(q, k, pos, pos, 0.5, block=4)
    assert w[4, 4] == 1.0 and np.allclose(w[5, :4], 0.0) and np.allclose(w[3, :4].sum(), 1.0)
    # from a later start: blocks are counted from position 0, not from the first row given
    w2 = pz.attention_weights(q[3:], k, pos[3:], pos, 0.5, block=4)
    assert np.allclose(w2, w[3:])
    s = q @ k.T * 0.5
    w = pz.attention_weights(q, k, pos, pos, 0.5, softcap=0.7)
    capped = 0.7 * np.tanh(s / 0.7)
    assert np.allclose(w[5], pz.softmax(capped[5]))
    w = pz.attention_weights(q, k, pos, pos, 0.5, weighting="sigmoid", bias=-1.0)
    assert np.allclose(w[2, :3], pz.sigmoid(s[2, :3] - 1.0)) and np.allclose(w[2, 3:], 0.0)


def _weights(config, seed=0):
    import torch
    from crane_b200.weights.random_init import model_manifest_for, random_tensors
    t = random_tensors(model_manifest_for(config), seed, torch.float32, "cpu", 0.1, 0.05)
    return {k: v.double().numpy() for k, v in t.items()}


def test_two_maps_lambda_norm_and_gate():
    cfg = tz.ZA
    w = _weights(cfg)
    m = cfg["layers"][1]["mixer"]
    rng = np.random.default_rng(2)
    h = rng.standard_normal((5, 96))
    out, st = pz.attention_mixer("attention_2", h, w, "l1.mix.", m, 1e-6, np.arange(5))
    H, G, d, vd = 4, 2, 16, 24
    q = pz.rotate_half((h @ w["l1.mix.q"].T).reshape(5, H * 2, d), np.arange(5), 16, 10000.0)
    k = pz.rotate_half((h @ w["l1.mix.k"].T).reshape(5, G * 2, d), np.arange(5), 16, 10000.0)
    v = (h @ w["l1.mix.v"].T).reshape(5, G, vd)
    lam = math.exp(w["l1.mix.lq1"] @ w["l1.mix.lk1"]) - math.exp(w["l1.mix.lq2"] @ w["l1.mix.lk2"]) + 0.3
    t, hd = 4, 3                                    # the last token, the last head: key/value head 1
    a = []
    for i in range(2):
        s = k[:t + 1, 2 * 1 + i] @ q[t, 2 * hd + i] * 0.25
        a.append(pz.softmax(s) @ v[:t + 1, 1])
    o = a[0] - lam * a[1]
    o = o / math.sqrt((o * o).mean() + 1e-6) * 0.7 * pz.sigmoid(h[t] @ w["l1.mix.g"][hd])
    # the function itself with every other head's columns of the output projection set to zero
    only = {**w, "l1.mix.o": np.concatenate([np.zeros((96, hd * vd)), w["l1.mix.o"][:, hd * vd:]], axis=1)}
    got = pz.attention_mixer("attention_2", h, only, "l1.mix.", m, 1e-6, np.arange(5))[0][t]
    assert np.allclose(got, o @ w["l1.mix.o"][:, hd * vd:].T)


@pytest.mark.parametrize("name", ["ZA", "ZB", "ZC", "ZD"])
def test_the_plain_model_cut_anywhere_agrees_with_itself(name):
    cfg = tz.TINY[name]["config"]
    w = _weights(cfg, 3)
    rng = np.random.default_rng(4)
    toks = rng.integers(0, cfg["vocab"], 41).tolist()
    whole = pz.logits_all(cfg, w, toks)
    assert np.isfinite(whole).all() and np.abs(whole).max() > 1e-3
    for cuts in ([1, 40], [7, 1, 1, 30, 2], [24, 17], [33, 8]):
        past, at, rows = None, 0, []
        for n in cuts:
            lg, past = pz.forward(cfg, w, toks[at:at + n], past, at)
            rows.append(lg)
            at += n
        assert np.allclose(np.concatenate(rows), whole, atol=1e-9), cuts
    # a key outside the query's block changes nothing; one inside does
    if name == "ZB":
        only = copy.deepcopy(cfg)
        only["layers"] = only["layers"][1:2]                          # blocks of 7 positions, a convolution of 5 taps
        w1 = {k.replace("l1.", "l0."): v for k, v in w.items() if not k.startswith(("l0.", "l2."))}
        base = pz.logits_all(only, w1, toks[:21])
        other = list(toks[:21])
        other[9] = (other[9] + 1) % cfg["vocab"]                      # position 9: block 1; the taps reach 13
        changed = pz.logits_all(only, w1, other)
        assert np.allclose(changed[14:], base[14:], atol=1e-12) and not np.allclose(changed[13], base[13])
        assert np.allclose(changed[:9], base[:9], atol=1e-12)


def test_greedy_generation_continues_the_prompt():
    cfg = tz.ZD
    w = _weights(cfg, 5)
    prompt = [3, 9, 27, 1]
    out = pz.greedy_generate(cfg, w, prompt, 5)
    assert len(out) == 9 and out[:4] == prompt
    assert out[5] == int(np.argmax(pz.logits_all(cfg, w, out[:5])[-1]))
