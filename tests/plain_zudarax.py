"""A plain, slow restatement of Zudarax in NumPy float64, one function per mechanism, written from
the design's equations and sharing nothing with the engine.

Notation: n tokens, W width, H query heads, G key/value heads, d query/key size, m value size.
Weights are a dictionary name -> float64 array; a matrix is stored [out, in] and applied as
``x @ M.T`` to rows x.  Functions over time take what came before the rows they are given (the
convolutions' last inputs, the keys and values of earlier positions) and hand the new one back, so a
sequence can be run in one call or continued from where another call stopped.

The design.  Per layer ``h = groupnorm(x); x <- x + (mixer(h) + ff(h))``: one norm, both sublayers
read it.  groupnorm: the vector in ``groups`` equal consecutive parts, each over the root of its own
mean square (+ eps), the whole times w.  Three mixers, all grouped-query attention over every earlier
position of the request:

* ``attention``: q, k, v with biases; a causal convolution of a few taps over time on every channel of
  q, k and v; RMS norm of q and of k over their whole rows with plain weights; rotation of the leading
  ``rot.dims`` elements of each head (element i with i + dims / 2); scores ``q.k * scale`` squashed to
  ``cap * tanh(s / cap)``; a position sees the earlier positions of its own block of ``mask.size``
  positions only (blocks counted from position 0); softmax.
* ``attention_2`` (differential): every head has two maps of queries and keys, rows [map 1 | map 2], each a
  softmax attention of its own over the same values; ``o = a1 - lam a2`` with ``lam = exp(lq1.lk1) -
  exp(lq2.lk2) + diff``; o over the root of its mean square per head, times ``1 - diff``; times
  ``sigmoid(W_g h)`` per head.
* ``attention_3``: convolutions as above, rotation with YaRN-scaled frequencies, and instead of a
  softmax the weight ``sigmoid(s + pb[h])`` for every visible key, not normalised.

Feed-forward: ``down(act(up h))`` with ``act(z) = a N(z) + b N(z^2) + c N(z^3) + e``, N dividing a
token's vector by the root of its mean square.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import numpy as np
import torch

from crane_b200.weights.safetensors_io import TensorSource, model_files


def load_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    src = TensorSource(model_files(folder))
    w = {}
    for name in src.names():
        t = src.tensor(name)
        w[name] = t.to(torch.float64).numpy() if t.dtype.is_floating_point else t.numpy()
    return cfg, w


# ------------------------------------------------------------------ small functions
def sigmoid(z):
    return 0.5 * (1.0 + np.tanh(0.5 * np.asarray(z, dtype=np.float64)))


def unit_rms(x, eps):
    """x over the root of its mean square, eps under the root."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def group_norm(x, w, groups: int, eps: float):
    """Rows x [n, W] in ``groups`` equal consecutive parts, each over its own root mean square; times w."""
    n, width = x.shape
    parts = x.reshape(n, groups, width // groups)
    return unit_rms(parts, eps).reshape(n, width) * w


def poly_norm(z, coef, eps: float):
    """a N(z) + b N(z^2) + c N(z^3) + e over a token's row."""
    a, b, c, e = (float(v) for v in coef)
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def softmax(z, axis=-1):
    e = np.exp(z - z.max(axis=axis, keepdims=True))
    return e / e.sum(axis=axis, keepdims=True)


# ------------------------------------------------------------------ convolution over time
def short_convolution(u, taps_w, before=None):
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j) per channel; ``before`` [taps - 1, C] are the inputs
    ahead of u's first row (zeros at a sequence's start).  Returns (y, the last taps - 1 inputs)."""
    n, C = u.shape
    taps = taps_w.shape[1]
    if before is None:
        before = np.zeros((taps - 1, C))
    full = np.concatenate([before, u], axis=0)
    y = np.zeros((n, C))
    for j in range(taps):
        y += full[j:j + n] * taps_w[:, j]
    return y, full[full.shape[0] - (taps - 1):]


# ------------------------------------------------------------------ rotation
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict] = None):
    """(frequencies [dims / 2], the factor on cos and sin).  ``scaling`` (YaRN): factor, original, fast, slow."""
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, dims: int, base: float, scaling: Optional[dict] = None):
    """x [n, heads, d]: the leading ``dims`` elements of every head turn, element i with i + dims / 2."""
    if not dims:
        return x
    f, mag = rotary_frequencies(dims, base, scaling)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------ attention weights
def visible(pos_q, pos_k, block: int = 0):
    """[nq, nk] booleans: key j is seen from position i when j <= i and, with ``block``, both lie in the
    same block of that many positions counted from 0."""
    i, j = np.asarray(pos_q)[:, None], np.asarray(pos_k)[None, :]
    ok = j <= i
    if block:
        ok &= (i // block) == (j // block)
    return ok


def attention_weights(q, k, pos_q, pos_k, scale: float, softcap: float = 0.0, block: int = 0,
                      weighting: str = "softmax", bias: float = 0.0):
    """One head: q [nq, d], k [nk, d] -> weights [nq, nk]."""
    s = (q @ k.T) * scale
    if softcap:
        s = softcap * np.tanh(s / softcap)
    ok = visible(pos_q, pos_k, block)
    if weighting == "sigmoid":
        return np.where(ok, sigmoid(s + bias), 0.0)
    s = np.where(ok, s, -np.inf)
    return softmax(s, axis=-1)


# ------------------------------------------------------------------ the three mixers
def _heads(x, n_heads):
    return x.reshape(x.shape[0], n_heads, -1)


def _grow(past, key, new):
    out = new if past is None or past.get(key) is None else np.concatenate([past[key], new], axis=0)
    return out


def _project_conv(h, w, p, names, m, past, state):
    """q, k, v: projection (+ bias where the model has one), then the convolution where it has one."""
    out = []
    for nm in names:
        u = h @ w[p + nm].T
        if p + nm + ".b" in w:
            u = u + w[p + nm + ".b"]
        if m.get("conv"):
            u, state["conv_" + nm] = short_convolution(u, w[p + nm + ".conv"], None if past is None else past["conv_" + nm])
        out.append(u)
    return out


def attention_mixer(kind: str, h, w, p: str, m: dict, eps: float, positions, past: Optional[dict] = None):
    """One of ``attention``, ``attention_2``, ``attention_3`` on rows h at ``positions``; ``past``: what an
    earlier call returned for the positions before.  Returns (result [n, W], what the next call needs)."""
    H, G, d, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    maps = 2 if kind == "attention_2" else 1
    state: dict = {}
    q, k, v = _project_conv(h, w, p, ("q", "k", "v"), m, past, state)
    if p + "q.norm" in w:
        q = unit_rms(q, eps) * w[p + "q.norm"]
        k = unit_rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    # a head's maps turn like heads of their own
    q = rotate_half(_heads(q, H * maps), positions, dims, float(rot.get("base") or 1.0), rot.get("scaling"))
    k = rotate_half(_heads(k, G * maps), positions, dims, float(rot.get("base") or 1.0), rot.get("scaling"))
    v = _heads(v, G)
    state["k"], state["v"] = _grow(past, "k", k), _grow(past, "v", v)
    state["pos"] = _grow(past, "pos", np.asarray(positions))
    K, V, pos_k = state["k"], state["v"], state["pos"]
    n = h.shape[0]
    out = np.zeros((n, H, vd))
    block = int((m.get("mask") or {}).get("size") or 0)
    cap = float(m.get("softcap") or 0.0)
    scale = float(m["scale"])
    rep = H // G
    for hd in range(H):
        g = hd // rep
        if kind == "attention_2":
            diff = float(m["diff"])
            lam = math.exp(float(w[p + "lq1"] @ w[p + "lk1"])) - math.exp(float(w[p + "lq2"] @ w[p + "lk2"])) + diff
            a = [attention_weights(q[:, 2 * hd + i], K[:, 2 * g + i], positions, pos_k, scale, cap, block) @ V[:, g]
                 for i in range(2)]
            o = unit_rms(a[0] - lam * a[1], eps) * (1.0 - diff)
        elif kind == "attention_3":
            o = attention_weights(q[:, hd], K[:, g], positions, pos_k, scale, cap, block, "sigmoid",
                                  float(w[p + "pb"][hd])) @ V[:, g]
        else:
            o = attention_weights(q[:, hd], K[:, g], positions, pos_k, scale, cap, block) @ V[:, g]
        out[:, hd] = o
    if p + "g" in w:
        out = out * sigmoid(h @ w[p + "g"].T)[:, :, None]
    return out.reshape(n, H * vd) @ w[p + "o"].T, state


def feed_forward(h, w, p: str, eps: float):
    return poly_norm(h @ w[p + "up"].T, w[p + "act"], eps) @ w[p + "down"].T


# ------------------------------------------------------------------ the model
def forward(cfg: dict, w: Dict[str, np.ndarray], tokens, past: Optional[list] = None, start: int = 0,
            layers_out: Optional[list] = None):
    """Logits [n, vocab] of ``tokens`` at positions start ..; ``past``: per layer what an earlier call
    returned.  Returns (logits, past for the next call).  ``layers_out``: the stream after every layer."""
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups") or 1)
    x = w["embed"][np.asarray(tokens)]
    positions = np.arange(start, start + len(tokens))
    new_past = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = group_norm(x, w[p + "norm1"], groups, eps)
        a, st = attention_mixer(layer["type"], h, w, p + "mix.", layer["mixer"], eps, positions,
                                None if past is None else past[i])
        new_past.append(st)
        f = feed_forward(h, w, p + "mlp.", eps) if layer.get("mlp") else 0.0
        x = x + (a + f)
        if layers_out is not None:
            layers_out.append(x.copy())
    h = group_norm(x, w["final.norm"], groups, eps)
    return h @ w["head"].T, new_past


def logits_all(cfg: dict, w: Dict[str, np.ndarray], tokens) -> np.ndarray:
    return forward(cfg, w, tokens)[0]


def greedy_generate(cfg: dict, w: Dict[str, np.ndarray], prompt: List[int], new_tokens: int) -> List[int]:
    """The prompt and ``new_tokens`` more, each the largest logit's (ties to the lower index)."""
    logits, past = forward(cfg, w, prompt)
    out, pos = list(prompt), len(prompt)
    for _ in range(new_tokens):
        tok = int(np.argmax(logits[-1]))
        out.append(tok)
        logits, past = forward(cfg, w, [tok], past, pos)
        pos += 1
    return out
