"""Tiny Mufevik configurations for tests.  They differ from one another in every size, and each sets
apart what a model may happen to make equal or 1: key and value widths, query and key/value head
counts, the rotated part of a head and the head, the experts chosen, kept and there, the number of
residual streams, the convolution's taps, the logit scale."""


def _left(heads, kv_heads, dim, vdim, scale, rot_dims, base):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return m


def _right(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(experts, top, count, keep, ff, shared):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if count:
        m["router"]["groups"] = {"count": count, "keep": keep}
    if shared:
        m["shared"] = {"ff": shared}
    return m


# two streams; a third of each head rotated; values wider than keys on the left and narrower on the
# right; two query/key heads for four heads of the delta rule; a layer without feed-forward; two of
# three groups kept
MA = {
    "architecture": "Mufevik", "vocab": 211, "width": 96, "norm": {"eps": 1e-6}, "streams": 2, "logit_scale": 1.5,
    "layers": [
        {"type": "parallel", "mixer": {"left": _left(6, 2, 24, 32, 0.3, 8, 500.0), "right": _right(3, 16, 8, 4.0, 5)},
         "mlp": _moe(6, 2, 3, 2, 24, 40)},
        {"type": "delta", "mixer": _delta(4, 2, 16, 24, 3), "mlp": None},
        {"type": "delta", "mixer": _delta(2, 2, 48, 16, 4), "mlp": _moe(4, 1, 2, 1, 16, 0)},
        {"type": "parallel", "mixer": {"left": _left(2, 2, 32, 16, 0.2, 32, 10000.0), "right": _right(1, 24, 40, 1.0, 3)},
         "mlp": _moe(6, 2, 3, 2, 24, 40)},
    ],
}

# no streams entry at all (the plain residual sum), no logit scale, no groups, all experts chosen;
# one key/value head for three query heads; no rotation in one layer; a convolution of one tap
MB = {
    "architecture": "Mufevik", "vocab": 131, "width": 80, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "delta", "mixer": _delta(5, 1, 16, 16, 1), "mlp": _moe(3, 3, 0, 0, 32, 24)},
        {"type": "parallel", "mixer": {"left": _left(3, 1, 16, 24, 0.25, 0, 0.0), "right": _right(2, 32, 32, 8.0, 4)},
         "mlp": _moe(8, 3, 4, 2, 8, 16)},
        {"type": "parallel", "mixer": {"left": _left(4, 4, 8, 8, 0.5, 4, 100.0), "right": _right(5, 8, 16, 2.5, 2)},
         "mlp": None},
    ],
}

# four streams; a width that is no multiple of 8; one head of the delta rule; one group of all
# experts is the same as none; a convolution of five taps
MC = {
    "architecture": "Mufevik", "vocab": 97, "width": 68, "norm": {"eps": 1e-5}, "streams": 4, "logit_scale": 0.5,
    "layers": [
        {"type": "delta", "mixer": _delta(1, 1, 64, 32, 5), "mlp": _moe(4, 2, 1, 1, 20, 12)},
        {"type": "parallel", "mixer": {"left": _left(4, 2, 12, 20, 0.4, 12, 50.0), "right": _right(2, 20, 12, 16.0, 6)},
         "mlp": _moe(9, 4, 3, 3, 12, 0)},
    ],
}

# one stream named outright (its three tensors are stored, each a single number); one of two groups kept
MD = {
    "architecture": "Mufevik", "vocab": 61, "width": 48, "norm": {"eps": 1e-6}, "streams": 1,
    "layers": [
        {"type": "parallel", "mixer": {"left": _left(2, 1, 16, 16, 0.25, 16, 7.0), "right": _right(2, 8, 8, 3.0, 2)},
         "mlp": _moe(4, 2, 2, 1, 16, 8)},
        {"type": "delta", "mixer": _delta(3, 3, 8, 8, 2), "mlp": _moe(4, 2, 2, 1, 16, 8)},
    ],
}

# layers of the delta rule only (no layer asks for pages); one query/key head per head and one for all
ME = {
    "architecture": "Mufevik", "vocab": 83, "width": 56, "norm": {"eps": 1e-5}, "streams": 2, "logit_scale": 3.0,
    "layers": [
        {"type": "delta", "mixer": _delta(2, 2, 32, 12, 2), "mlp": _moe(5, 2, 0, 0, 12, 8)},
        {"type": "delta", "mixer": _delta(3, 1, 24, 16, 3), "mlp": None},
    ],
}

# pairs only; as many key/value heads as query heads, the whole head rotated, keys as wide as values;
# a single attention head in the second layer
MF = {
    "architecture": "Mufevik", "vocab": 150, "width": 72, "norm": {"eps": 1e-6}, "streams": 3,
    "layers": [
        {"type": "parallel", "mixer": {"left": _left(3, 3, 16, 16, 0.25, 16, 3000.0), "right": _right(1, 16, 16, 5.0, 4)},
         "mlp": _moe(6, 3, 2, 2, 16, 24)},
        {"type": "parallel", "mixer": {"left": _left(1, 1, 48, 48, 0.15, 48, 3000.0), "right": _right(3, 8, 24, 1.5, 3)},
         "mlp": None},
    ],
}

# layer sizes at which the tensor-core kernels are taken
ML = {
    "architecture": "Mufevik", "vocab": 512, "width": 512, "norm": {"eps": 1e-5}, "streams": 3, "logit_scale": 0.75,
    "layers": [
        {"type": "delta", "mixer": _delta(8, 4, 64, 64, 4), "mlp": _moe(8, 2, 4, 2, 256, 512)},
        {"type": "parallel", "mixer": {"left": _left(8, 2, 128, 128, 0.09, 64, 10000.0), "right": _right(4, 64, 128, 16.0, 32)},
         "mlp": _moe(8, 2, 2, 1, 256, 0)},
        {"type": "delta", "mixer": _delta(4, 4, 128, 128, 4), "mlp": _moe(16, 3, 4, 2, 128, 256)},
    ],
}

TINY = {
    "MA": {"config": MA, "seed": 31, "std": 0.08, "norm_std": 0.05, "page_size": 16},
    "MB": {"config": MB, "seed": 32, "std": 0.1, "norm_std": 0.05, "page_size": 8},
    "MC": {"config": MC, "seed": 33, "std": 0.1, "norm_std": 0.05, "page_size": 32},
    "MD": {"config": MD, "seed": 34, "std": 0.12, "norm_std": 0.05, "page_size": 16},
    "ME": {"config": ME, "seed": 36, "std": 0.12, "norm_std": 0.05, "page_size": 16},
    "MF": {"config": MF, "seed": 37, "std": 0.1, "norm_std": 0.05, "page_size": 8},
    "ML": {"config": ML, "seed": 35, "std": 0.03, "norm_std": 0.05, "page_size": 64},
}
