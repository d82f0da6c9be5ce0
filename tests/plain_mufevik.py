"""A plain, slow restatement of Mufevik in NumPy float64, one function per mechanism, written
from the design's equations and sharing nothing with the engine.

Notation: n tokens, W width, H heads, G key/value heads, d key size, m value size, E experts,
R residual streams.  Weights are dictionaries name -> float64 array.  Every matrix is stored
[out, in] and applied as ``x @ M.T`` to rows x.  Recurrent functions take and return their state,
so a sequence can be run in one call or continued from where another call stopped.
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
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def unit_rms(x, eps):
    """x over the root of its mean square, eps under the root."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def scalar_norm(x, g, eps):
    """The layer norm of this design: one number g for all coordinates."""
    return unit_rms(x, eps) * float(g)


def softmax(z, axis=-1):
    e = np.exp(z - z.max(axis=axis, keepdims=True))
    return e / e.sum(axis=axis, keepdims=True)


# ------------------------------------------------------------------ rotary positions
def rotate_half(x, positions, dims: int, base: float):
    """x [n, heads, d]: the leading ``dims`` elements of every head are rotated, element i with
    element i + dims / 2, by the angle p * base^(-2 i / dims)."""
    out = x.copy()
    half = dims // 2
    if half == 0:
        return out
    f = base ** (-2.0 * np.arange(half) / dims)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------ attention whose heads talk
def talking_attention(q, k, v, scale: float, temp, talk):
    """q [n, H, d], k [n, G, d], v [n, G, m] of one sequence (positions 0 .. n - 1, already rotated).
    Scores of head h: q_h . k_(h // (H / G)) * scale * temp[h], causal softmax; the heads' weights
    are then mixed, w'_h = sum_g talk[h, g] w_g, and head h applies w'_h to the values of its own
    key/value head.  Returns [n, H, m]."""
    n, H, d = q.shape
    G = k.shape[1]
    rep = H // G
    causal = np.tril(np.ones((n, n), dtype=bool))
    weights = np.zeros((H, n, n))
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].T) * scale * float(temp[h])
        s = np.where(causal, s, -np.inf)
        weights[h] = softmax(s, axis=-1)
    mixed = np.einsum("hg,gij->hij", np.asarray(talk, dtype=np.float64), weights)
    out = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        out[:, h] = mixed[h] @ v[:, h // rep]
    return out


# ------------------------------------------------------------------ recurrences with a matrix state
def gated_linear_scan(q, k, v, alpha, state=None):
    """Per head S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t.  q, k, alpha [n, H, d], v [n, H, m];
    ``state`` [H, d, m] or None (zeros).  Returns (o [n, H, m], state)."""
    n, H, d = q.shape
    m = v.shape[2]
    S = np.zeros((H, d, m)) if state is None else state.copy()
    o = np.zeros((n, H, m))
    for t in range(n):
        for h in range(H):
            S[h] = alpha[t, h][:, None] * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


def gated_delta_scan(q, k, v, beta, decay, state=None):
    """Per head: S <- decay_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t.
    q, k [n, G, d] (head h reads q/k head h // (H / G)), v [n, H, m], beta, decay [n, H];
    ``state`` [H, d, m] or None.  Returns (o [n, H, m], state)."""
    n, H, m = v.shape
    G, d = q.shape[1], q.shape[2]
    rep = H // G
    S = np.zeros((H, d, m)) if state is None else state.copy()
    o = np.zeros((n, H, m))
    for t in range(n):
        for h in range(H):
            kk, qq = k[t, h // rep], q[t, h // rep]
            S[h] = decay[t, h] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ kk)
            S[h] = S[h] + np.outer(kk, u)
            o[t, h] = S[h].T @ qq
    return o, S


def short_convolution(x, taps_w, before=None):
    """A causal convolution over time per channel: y_t[c] = sum_j w[c, j] x_(t - (T - 1) + j)[c], the
    last column of w is the current token's, zeros before the start.  x [n, C], taps_w [C, T],
    ``before`` [T - 1, C]: the inputs just before x (None: the start of a sequence).  Returns
    (y [n, C], the last T - 1 inputs)."""
    n, C = x.shape
    T = taps_w.shape[1]
    past = np.zeros((T - 1, C)) if before is None else before
    ext = np.concatenate([past, x], axis=0)
    y = np.zeros((n, C))
    for t in range(n):
        y[t] = (ext[t:t + T] * taps_w.T).sum(axis=0)
    return y, ext[ext.shape[0] - (T - 1):].copy()


def unit_vector(x, eps=1e-6):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + eps)


# ------------------------------------------------------------------ the mixers
def parallel_left(h, w, p: str, m: dict, positions):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(n, H, d)
    k = (h @ w[p + "k"].T).reshape(n, G, d)
    v = (h @ w[p + "v"].T).reshape(n, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, positions, int(rot["dims"]), float(rot["base"]))
        k = rotate_half(k, positions, int(rot["dims"]), float(rot["base"]))
    o = talking_attention(q, k, v, float(m["scale"]), w[p + "temp"], w[p + "talk"])
    return o.reshape(n, H * dv) @ w[p + "o"].T


def parallel_right(h, w, p: str, m: dict, eps: float, state=None):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(n, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).reshape(n, H, d)
    v = (h @ w[p + "v"].T).reshape(n, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / float(m["tau"]))).reshape(n, H, d)
    o, state = gated_linear_scan(q, k, v, alpha, state)
    o = unit_rms(o, eps) * w[p + "norm"]
    o = o.reshape(n, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T, state


def parallel_mixer(h, w, p: str, m: dict, eps: float, positions, state=None):
    """Two mixers on the same input; each result is RMS-normed over the width with a plain weight,
    and the mixer's result is half their sum."""
    a = parallel_left(h, w, p + "left.", m["left"], positions)
    b, state = parallel_right(h, w, p + "right.", m["right"], eps, state)
    return 0.5 * (unit_rms(a, eps) * w[p + "left.out"] + unit_rms(b, eps) * w[p + "right.out"]), state


def delta_mixer(h, w, p: str, m: dict, eps: float, state=None):
    """``state``: (S [H, d, m], the last taps - 1 inputs of the q, k and v convolutions) or None."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    S, cq, ck, cv = state if state is not None else (None, None, None, None)
    q, cq = short_convolution(h @ w[p + "q"].T, w[p + "q.conv"], cq)
    k, ck = short_convolution(h @ w[p + "k"].T, w[p + "k.conv"], ck)
    v, cv = short_convolution(h @ w[p + "v"].T, w[p + "v.conv"], cv)
    q = unit_vector(silu(q).reshape(n, G, d)) * d ** -0.5
    k = unit_vector(silu(k).reshape(n, G, d))
    v = silu(v).reshape(n, H, dv)
    beta = sigmoid(h @ w[p + "b"].T)
    decay = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o, S = gated_delta_scan(q, k, v, beta, decay, S)
    o = unit_rms(o, eps) * w[p + "norm"]
    o = o.reshape(n, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T, (S, cq, ck, cv)


# ------------------------------------------------------------------ feed-forward
def choose_experts(z, correction, top: int, groups: int, keep: int):
    """One token's router logits z [E]: scores = softmax(z); an expert's choice score is its score
    plus its correction; experts come in ``groups`` equal groups of neighbours, a group's score is
    its largest choice score, and only experts of the ``keep`` best groups can be chosen; the
    ``top`` largest choice scores among those are chosen (ties to the lower index).  Returns
    (chosen indices, their scores without the correction)."""
    s = softmax(z)
    c = s + correction
    E = z.shape[0]
    per = E // groups
    gs = c.reshape(groups, per).max(axis=1)
    best = sorted(range(groups), key=lambda g: (-gs[g], g))[:keep]
    allowed = np.zeros(E, dtype=bool)
    for g in best:
        allowed[g * per:(g + 1) * per] = True
    order = sorted((e for e in range(E) if allowed[e]), key=lambda e: (-c[e], e))[:top]
    return order, s[order]


def gated_expert(h, w, p: str):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def moe(h, w, p: str, mlp: dict):
    r = mlp["router"]
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    corr = w.get(p + "correction")
    corr = np.zeros(E) if corr is None else corr
    z = h @ w[p + "router"].T
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        idx, wt = choose_experts(z[t], corr, top, int(groups["count"]), int(groups["keep"]))
        for e, a in zip(idx, wt):
            out[t] += a * gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out += gated_expert(h, w, p + "shared.") * sigmoid(h @ w[p + "shared.sg"].T)
    return out


# ------------------------------------------------------------------ several residual streams
def streams_read(xs, w_in):
    """xs [R, n, W]: what a sublayer reads, sum_r w_in[r] x_r."""
    return np.einsum("r,rnw->nw", w_in, xs)


def streams_write(xs, y, w_mix, w_out):
    """All streams at once from the old ones: x_t <- sum_r w_mix[r, t] x_r + w_out[t] y."""
    return np.einsum("rt,rnw->tnw", w_mix, xs) + w_out[:, None, None] * y[None]


# ------------------------------------------------------------------ the model
def forward(cfg: dict, w: Dict[str, np.ndarray], tokens, state: Optional[list] = None, start: int = 0):
    """One sequence's tokens at positions start .. start + n - 1, continued from ``state`` (a list per
    layer; None: the start).  Attention layers keep their rotated keys and values in it.  Returns
    (logits [n, V], the sum of the streams after every layer [L, n, W], state)."""
    eps = float(cfg["norm"]["eps"])
    R = int(cfg.get("streams") or 1)
    n = len(tokens)
    positions = np.arange(start, start + n)
    x0 = w["embed"][np.asarray(tokens)]
    xs = np.repeat(x0[None], R, axis=0)
    state = [None] * len(cfg["layers"]) if state is None else list(state)
    sums = []
    ones = (np.ones(1), np.ones((1, 1)), np.ones(1))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        hc = lambda q: (w[f"{p}hc{q}.in"], w[f"{p}hc{q}.mix"], w[f"{p}hc{q}.out"]) if R > 1 or f"{p}hc{q}.in" in w else ones
        w_in, w_mix, w_out = hc(1)
        h = scalar_norm(streams_read(xs, w_in), w[p + "norm1"], eps)
        if layer["type"] == "parallel":
            st = state[i] or {}
            left = layer["mixer"]["left"]
            # the left mixer over the whole sequence so far: earlier inputs are kept
            hs = h if "h" not in st else np.concatenate([st["h"], h], axis=0)
            a_all = parallel_left(hs, w, p + "mix.left.", left, np.arange(hs.shape[0]))
            a = a_all[hs.shape[0] - n:]
            b, S = parallel_right(h, w, p + "mix.right.", layer["mixer"]["right"], eps, st.get("S"))
            y = 0.5 * (unit_rms(a, eps) * w[p + "mix.left.out"] + unit_rms(b, eps) * w[p + "mix.right.out"])
            state[i] = {"h": hs, "S": S}
        elif layer["type"] == "delta":
            y, state[i] = delta_mixer(h, w, p + "mix.", layer["mixer"], eps, state[i])
        else:
            raise ValueError(f"no mixer '{layer['type']}'")
        xs = streams_write(xs, y, w_mix, w_out)
        if layer.get("mlp") is not None:
            w_in, w_mix, w_out = hc(2)
            h = scalar_norm(streams_read(xs, w_in), w[p + "norm2"], eps)
            xs = streams_write(xs, moe(h, w, p + "mlp.", layer["mlp"]), w_mix, w_out)
        sums.append(xs.sum(axis=0))
    x = scalar_norm(xs.sum(axis=0), w["final.norm"], eps)
    logits = (x @ w["head"].T) * float(cfg.get("logit_scale") or 1.0)
    return logits, np.stack(sums), state


def logits_all(cfg: dict, w: Dict[str, np.ndarray], tokens) -> np.ndarray:
    """Logits at every position of one sequence, [n, V]."""
    return forward(cfg, w, list(tokens))[0]


def greedy_generate(cfg: dict, w: Dict[str, np.ndarray], prompt: List[int], new_tokens: int) -> List[int]:
    """The prompt and ``new_tokens`` more, each the largest logit's index (ties to the lower index);
    the prompt in one call, then token by token from the carried state."""
    toks = list(prompt)
    logits, _, state = forward(cfg, w, toks)
    for _ in range(new_tokens):
        toks.append(int(np.argmax(logits[-1])))
        logits, _, state = forward(cfg, w, toks[-1:], state, start=len(toks) - 1)
    return toks
