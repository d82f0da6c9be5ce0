"""Mixers whose memory is one matrix S [dim, vdim] per head and request, walked token by token:

    S <- diag(w_t) S;   u = beta_t (v_t - S^T k_t)  or  u = v_t;   S <- S + k_t u^T;   o_t = S^T q_t

``gated_linear_attention``: no correction (u = v), a decay per key channel
w = sigmoid(W_a2 (W_a1 x) + b)^(1 / tau), q scaled by dim^(-1/2).

``gated_delta``: the delta rule's correction with beta = sigmoid(W_b x) and one decay per head,
w = exp(-exp(A_log) softplus(W_a x + dt_bias)); q, k and v first pass a short causal convolution
over time and silu, q and k are scaled to unit length per head (q also by dim^(-1/2)); head h reads
q/k head h // (heads / kv_heads).  The convolutions' last taps - 1 inputs are state too.

Both norm each head's read-out over vdim (a plain weight shared by the heads), multiply by
silu(W_g x) and project.  State and everything between the projections and the output projection
are 32-bit.  One kernel walks the recurrence for both (``matrix_state_scan``), prompts, portions
and single tokens alike, so a state does not depend on how the tokens were cut.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import CacheNeed, Part, register_part


def _state_floats(rt, heads: int, dim: int, vdim: int, where: str) -> int:
    rows, lanes = rt.kernels.matrix_state_plan(dim)
    if rows == 0:
        raise ValueError(f"{where}: keys of {dim} elements are wider than the recurrence kernel takes")
    return heads * rows * lanes * vdim


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Part):
    """params: ``hidden_size``, ``heads``, ``dim``, ``vdim``, ``tau``, ``norm_eps`` (of the head norm),
    ``decay_rank`` (inner size of the decay's two products; None: read from the stored tensor),
    ``names``.  Tensors: q, k [H dim, hidden], v, g [H vdim, hidden], o [hidden, H vdim],
    a1 [rank, hidden], a2 [H dim, rank], and in 32-bit a2_bias [H dim], norm [vdim]."""
    kind = "mixer"
    state_graph_safe = True      # the kernels read the step's metadata on the device, skip rows of no
                                 # entry and touch no slot for an entry without rows
    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "a1": "a1", "a2": "a2", "a2_bias": "a2.b", "norm": "norm"}

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        w, H, d, m = int(a["hidden_size"]), int(a["heads"]), int(a["dim"]), int(a["vdim"])
        nm = dict(cls.NAMES, **(a.get("names") or {}))
        rank = a.get("decay_rank")
        rank, free = (-1, 16) if rank is None else (int(rank), 0)
        return {p + nm["q"]: TensorSpec((H * d, w)), p + nm["k"]: TensorSpec((H * d, w)),
                p + nm["v"]: TensorSpec((H * m, w)), p + nm["g"]: TensorSpec((H * m, w)),
                p + nm["o"]: TensorSpec((w, H * m)), p + nm["a1"]: TensorSpec((rank, w), free=free),
                p + nm["a2"]: TensorSpec((H * d, rank), "float32", "unit", free=free),
                p + nm["a2_bias"]: TensorSpec((H * d,), "float32", "unit"),
                p + nm["norm"]: TensorSpec((m,), "float32", "scale")}

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.H, self.d, self.m = int(a["heads"]), int(a["dim"]), int(a["vdim"])
        nm = dict(self.NAMES, **(a.get("names") or {}))
        self.tau = float(a["tau"])
        self.eps = float(a.get("norm_eps") or 0.0)
        # one product for everything that reads the block's input: [q | k | v | g | a1]
        self.w_in = torch.cat([weights.pop(p + nm[n]) for n in ("q", "k", "v", "g", "a1")], dim=0).contiguous()
        self.cols = self.w_in.shape[0]
        self.a2t = weights.pop(p + nm["a2"]).t().contiguous()          # [rank, H dim]: channels side by side
        if self.a2t.shape[0] != self.cols - 2 * self.H * (self.d + self.m):
            raise ValueError(f"{p}: the decay's two matrices do not share their inner size")
        self.bias, self.norm_w, self.o_w = weights[p + nm["a2_bias"]], weights[p + nm["norm"]], weights[p + nm["o"]]
        self.floats = _state_floats(rt, self.H, self.d, self.m, p)

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", state_shape=(self.floats,), state_dtype=torch.float32)

    def forward(self, h, ctx, cache, rt, hold: bool = False):
        n, k = h.shape[0], rt.kernels
        hd, hv = self.H * self.d, self.H * self.m
        proj = rt.linear(h, self.w_in, None, "gla_proj")
        aux = rt.ws.get("gla_aux", n, 3 * hd + hv, torch.float32)
        k.decay_gate_prep(proj, self.cols, ctx.tok_entry, self.a2t, self.bias, 1.0 / self.tau, self.d ** -0.5, aux,
                          self.H, self.d, self.m, rt.dtype)
        o_raw = rt.ws.get("gla_o_raw", n, hv, torch.float32)
        k.matrix_state_scan(aux, (0, hd, 2 * hd, 2 * hd + hv, 0), True, False, 1, ctx, cache.state, o_raw,
                            self.H, self.d, self.m, rt.err)
        o = rt.ws.get("gla_o", n, hv, rt.dtype)
        k.head_norm_gate(o_raw, proj, self.cols, 2 * hd + hv, ctx.tok_entry, self.norm_w, self.eps, o, self.H, self.m)
        rt.launches += 3
        return rt.linear(o, self.o_w, None, "gla_out", hold=hold)


@register_part("mixer", "gated_delta")
class GatedDelta(Part):
    """params: ``hidden_size``, ``heads``, ``kv_heads`` (q/k heads), ``dim``, ``vdim``, ``conv`` (taps),
    ``norm_eps`` (of the head norm), ``key_eps`` (under the root of the unit vectors; default 1e-6),
    ``names``.  Tensors: q, k [G dim, hidden], v, g [H vdim, hidden], b, a [H, hidden],
    o [hidden, H vdim], and in 32-bit q_conv, k_conv [G dim, taps], v_conv [H vdim, taps], A_log,
    dt_bias [H], norm [vdim]."""
    kind = "mixer"
    state_graph_safe = True
    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "b": "b", "a": "a", "o": "o", "q_conv": "q.conv",
             "k_conv": "k.conv", "v_conv": "v.conv", "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm"}

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        w, H, G, d, m, T = (int(a[k]) for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim", "conv"))
        nm = dict(cls.NAMES, **(a.get("names") or {}))
        return {p + nm["q"]: TensorSpec((G * d, w)), p + nm["k"]: TensorSpec((G * d, w)),
                p + nm["v"]: TensorSpec((H * m, w)), p + nm["g"]: TensorSpec((H * m, w)),
                p + nm["b"]: TensorSpec((H, w)), p + nm["a"]: TensorSpec((H, w)),
                p + nm["o"]: TensorSpec((w, H * m)),
                p + nm["q_conv"]: TensorSpec((G * d, T), "float32", "unit"),
                p + nm["k_conv"]: TensorSpec((G * d, T), "float32", "unit"),
                p + nm["v_conv"]: TensorSpec((H * m, T), "float32", "unit"),
                p + nm["A_log"]: TensorSpec((H,), "float32", "offset"),
                p + nm["dt_bias"]: TensorSpec((H,), "float32", "offset"),
                p + nm["norm"]: TensorSpec((m,), "float32", "scale")}

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.H, self.G, self.d, self.m, self.taps = (int(a[k]) for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
        if self.H % self.G:
            raise ValueError(f"{p}: {self.H} heads are not a multiple of {self.G} query/key heads")
        nm = dict(self.NAMES, **(a.get("names") or {}))
        self.eps = float(a.get("norm_eps") or 0.0)
        self.key_eps = float(a["key_eps"]) if a.get("key_eps") is not None else 1e-6
        # one product for everything that reads the block's input: [q | k | v | g | b | a]
        self.w_in = torch.cat([weights.pop(p + nm[n]) for n in ("q", "k", "v", "g", "b", "a")], dim=0).contiguous()
        self.cols = self.w_in.shape[0]
        self.conv_w = torch.cat([weights.pop(p + nm[n]) for n in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.a_log, self.dt_bias = weights[p + nm["A_log"]], weights[p + nm["dt_bias"]]
        self.norm_w, self.o_w = weights[p + nm["norm"]], weights[p + nm["o"]]
        self.channels = 2 * self.G * self.d + self.H * self.m
        self.conv_off = _state_floats(rt, self.H, self.d, self.m, p)
        self.floats = self.conv_off + (self.taps - 1) * self.channels

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", state_shape=(self.floats,), state_dtype=torch.float32)

    def forward(self, h, ctx, cache, rt):
        n, k = h.shape[0], rt.kernels
        gd, hv, H = self.G * self.d, self.H * self.m, self.H
        proj = rt.linear(h, self.w_in, None, "delta_proj")
        aux = rt.ws.get("gated_delta_aux", n, self.channels + 2 * H, torch.float32)
        k.conv_delta_prep(proj, self.cols, ctx, cache.state, self.conv_off, self.conv_w, self.taps, self.a_log,
                          self.dt_bias, aux, H, self.G, self.d, self.m, self.key_eps, self.d ** -0.5, rt.err, rt.dtype)
        o_raw = rt.ws.get("gated_delta_o_raw", n, hv, torch.float32)
        k.matrix_state_scan(aux, (0, gd, 2 * gd, self.channels, self.channels + H), False, True, H // self.G, ctx,
                            cache.state, o_raw, H, self.d, self.m, rt.err)
        o = rt.ws.get("gated_delta_o", n, hv, rt.dtype)
        k.head_norm_gate(o_raw, proj, self.cols, self.channels, ctx.tok_entry, self.norm_w, self.eps, o, H, self.m)
        rt.launches += 4 if self.taps > 1 else 3
        return rt.linear(o, self.o_w, None, "delta_out")
