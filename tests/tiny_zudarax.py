"""Tiny Zudarax configurations for tests.  They differ from one another in every size, and each sets
apart what a model may happen to make equal or 1: key and value widths, query and key/value head counts,
the rotated part of a head and the head, the norm's groups, the taps of the convolutions, the block of
visible positions against the page, the squashing constant, lambda's constant."""


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _soft(heads, kv_heads, dim, vdim, scale, conv=0, rot=None, softcap=0.0, block=0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if rot:
        m["rot"] = rot
    if softcap:
        m["softcap"] = softcap
    if block:
        m["mask"] = {"size": block}
    return m


def _diff(heads, kv_heads, dim, vdim, scale, diff, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if rot:
        m["rot"] = rot
    return m


def _ff(n):
    return {"kind": "dense", "ff": n} if n else None


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": _ff(ff)}


# three groups; values wider than keys; a third of each head rotated; blocks of 24 positions over pages
# of 16; a layer without feed-forward; a whole head rotated; YaRN over a rotated part; a layer whose
# query heads are its key/value heads
ZA = {
    "architecture": "Zudarax", "vocab": 211, "width": 96, "norm": {"eps": 1e-6, "groups": 3},
    "layers": [
        _layer("attention", _soft(6, 2, 24, 32, 0.3, conv=3, rot=_rot(8, 500.0), softcap=12.0, block=24), 40),
        _layer("attention_2", _diff(4, 2, 16, 24, 0.25, 0.3, rot=_rot(16, 10000.0)), 0),
        _layer("attention_3", _soft(2, 1, 48, 16, 0.15, conv=2, rot=_rot(32, 2000.0, (4.0, 64, 8.0, 1.0))), 64),
        _layer("attention_2", _diff(3, 3, 8, 8, 0.4, 0.8), 56),
    ],
}

# one group (a plain RMS norm); one key/value head for five and for three query heads; convolutions of one
# tap and of five; no rotation, no squashing, blocks of 7 positions; squashing without blocks
ZB = {
    "architecture": "Zudarax", "vocab": 131, "width": 80, "norm": {"eps": 1e-5, "groups": 1},
    "layers": [
        _layer("attention_3", _soft(5, 1, 16, 16, 0.25, conv=1), 48),
        _layer("attention", _soft(3, 1, 16, 24, 0.3, conv=5, block=7), 32),
        _layer("attention", _soft(4, 4, 8, 8, 0.5, conv=2, rot=_rot(4, 100.0), softcap=5.0), 0),
    ],
}

# a width that is no multiple of 8 in four groups of 17; maps of 12 elements (no multiple of 16) with
# values of 40; a head rotated wholly with YaRN; blocks of 33 positions over pages of 32; keys much wider
# than values
ZC = {
    "architecture": "Zudarax", "vocab": 97, "width": 68, "norm": {"eps": 2e-6, "groups": 4},
    "layers": [
        _layer("attention_2", _diff(2, 1, 12, 40, 0.3, 0.5, rot=_rot(4, 50.0)), 24),
        _layer("attention_3", _soft(3, 3, 20, 12, 0.2, conv=4, rot=_rot(20, 300.0, (1.5, 40, 4.0, 0.5))), 100),
        _layer("attention", _soft(2, 2, 40, 8, 0.12, conv=3, rot=_rot(16, 1000.0), softcap=50.0, block=33), 36),
    ],
}

# single heads everywhere; sixteen groups; every layer of another kind than its neighbour; no feed-forward in
# the last layer; a block shorter than the convolution
ZD = {
    "architecture": "Zudarax", "vocab": 64, "width": 64, "norm": {"eps": 1e-4, "groups": 16},
    "layers": [
        _layer("attention_2", _diff(1, 1, 32, 16, 0.2, 0.1, rot=_rot(32, 20.0)), 16),
        _layer("attention", _soft(1, 1, 56, 56, 0.1, conv=4, rot=_rot(2, 7.0), softcap=3.0, block=3), 72),
        _layer("attention_3", _soft(1, 1, 8, 72, 0.35, conv=3), 0),
    ],
}

# layer sizes at which the tensor-core kernels of the products are taken; heads stored at 128, 128 and 64
ZL = {
    "architecture": "Zudarax", "vocab": 512, "width": 512, "norm": {"eps": 1e-5, "groups": 8},
    "layers": [
        _layer("attention", _soft(8, 2, 128, 128, 0.09, conv=4, rot=_rot(64, 10000.0), softcap=20.0, block=96), 1024),
        _layer("attention_2", _diff(8, 4, 64, 128, 0.125, 0.4, rot=_rot(32, 10000.0)), 1024),
        _layer("attention_3", _soft(16, 2, 64, 64, 0.125, conv=4, rot=_rot(64, 100000.0, (2.0, 128, 16.0, 1.0))), 768),
    ],
}

TINY = {
    "ZA": {"config": ZA, "seed": 41, "std": 0.08, "norm_std": 0.05, "page_size": 16},
    "ZB": {"config": ZB, "seed": 42, "std": 0.1, "norm_std": 0.05, "page_size": 8},
    "ZC": {"config": ZC, "seed": 43, "std": 0.1, "norm_std": 0.05, "page_size": 32},
    "ZD": {"config": ZD, "seed": 44, "std": 0.12, "norm_std": 0.05, "page_size": 16},
    "ZL": {"config": ZL, "seed": 45, "std": 0.03, "norm_std": 0.05, "page_size": 64},
}
