"""Grouped-query attention over the paged cache whose scores are worked on before they become
weights, with what may stand before and behind it.  Every step is an option of its own:

* biases on q, k, v (added in the merged projection);
* a causal convolution of ``conv`` taps over time on every channel of q, k and v, straight after the
  projection: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before a request's first position; the last
  taps - 1 projected rows of a request live in its state slot;
* RMS norm of q and of k over their whole rows (all heads at once), plain weights;
* rotation of the leading ``rotary_dim`` elements of every head, element i with i + rotary_dim / 2, by
  the tables of a ``position`` part (YaRN scaling is that part's business);
* score = q . k * scale, then ``softcap`` * tanh(score / ``softcap``);
* visibility: every earlier position, the last ``window``, and/or the query's own block of ``chunk``
  positions (blocks counted from position 0 of the request, wherever a prompt was cut);
* weights: softmax over the visible keys, or ``sigmoid(score + head_bias[h])`` for every visible key
  without any normalisation over the keys;
* ``maps`` = 2 (differential attention): a head's query and key rows hold two maps, each a softmax
  attention of its own over the same values, o = a1 - lambda a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2)
  + ``diff``;
* ``head_norm``: o over the root of its mean square per head (no weight), times 1 - ``diff``;
* ``gate``: head h's result times sigmoid(W_g x)_h, one number per head, from the mixer's input.

Scores, weights, norms, angles and the gate are 32-bit on both paths.
"""
from __future__ import annotations

import math
import os

import torch

from ..weights.loader import TensorSpec
from .base import CacheNeed, Part, build_part, query_tiles, register_part


@register_part("mixer", "scored_attention")
class ScoredAttention(Part):
    """params: ``hidden_size``, ``heads``, ``kv_heads``, ``dim`` (of one map of a query/key head), ``vdim``,
    ``scale``, ``bias``, ``conv`` (taps; 0: none), ``qk_norm`` + ``norm_eps``, ``rotary_dim`` + ``position``
    (a PartSpec of kind position whose tables have rotary_dim / 2 columns), ``softcap`` (0: none), ``window``,
    ``chunk`` (0: none), ``weighting`` ("softmax" | "sigmoid"), ``head_bias`` (sigmoid: a number per head added
    to the score), ``maps`` (1 | 2), ``diff``, ``head_norm``, ``gate``, ``head_dim`` / ``map_stride`` (bfloat16:
    the head size keys and values are stored at and where a head's second map starts; 0: as wide as they
    are), ``names``.
    Tensors: q [H maps dim, hidden], k [G maps dim, hidden], v [G vdim, hidden], o [hidden, H vdim]; with
    ``bias`` q.b, k.b, v.b; with ``conv`` q.conv, k.conv, v.conv [channels, taps]; with ``qk_norm`` q.norm,
    k.norm; with ``head_bias`` pb [H]; with ``maps`` 2 lq1, lk1, lq2, lk2 [dim]; with ``gate`` g [H, hidden]."""
    kind = "mixer"
    state_graph_safe = True
    decode_bucket_safe = True
    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
             "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "q_norm": "q.norm", "k_norm": "k.norm",
             "head_bias": "pb", "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2", "gate": "g"}

    @classmethod
    def _sizes(cls, a):
        return (int(a["hidden_size"]), int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"]),
                int(a.get("maps") or 1), int(a.get("conv") or 0))

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        w, H, G, d, m, maps, taps = cls._sizes(a)
        nm = dict(cls.NAMES, **(a.get("names") or {}))
        cq, ck, cv = H * maps * d, G * maps * d, G * m
        out = {p + nm["q"]: TensorSpec((cq, w)), p + nm["k"]: TensorSpec((ck, w)), p + nm["v"]: TensorSpec((cv, w)),
               p + nm["o"]: TensorSpec((w, H * m))}
        if a.get("bias"):
            for n, c in (("q_bias", cq), ("k_bias", ck), ("v_bias", cv)):
                out[p + nm[n]] = TensorSpec((c,), "float32", "offset")
        if taps >= 1:
            for n, c in (("q_conv", cq), ("k_conv", ck), ("v_conv", cv)):
                out[p + nm[n]] = TensorSpec((c, taps), "float32", "unit")
        if a.get("qk_norm"):
            out[p + nm["q_norm"]] = TensorSpec((cq,), "float32", "scale")
            out[p + nm["k_norm"]] = TensorSpec((ck,), "float32", "scale")
        if a.get("head_bias"):
            out[p + nm["head_bias"]] = TensorSpec((H,), "float32", "offset")
        if maps == 2:
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[p + nm[n]] = TensorSpec((d,), "float32", "unit")
        if a.get("gate"):
            out[p + nm["gate"]] = TensorSpec((H, w))
        return out

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.w, self.H, self.G, self.d, self.m, self.maps, self.taps = self._sizes(a)
        nm = dict(self.NAMES, **(a.get("names") or {}))
        H, G, d, m, maps = self.H, self.G, self.d, self.m, self.maps
        if H % G:
            raise ValueError(f"{p}: {H} query heads are not a multiple of {G} key/value heads")
        if maps not in (1, 2):
            raise ValueError(f"{p}: a head has one map or two, not {maps}")
        if d > 1024 or m > 512:
            raise ValueError(f"{p}: heads of {d} / {m} elements are wider than the attention kernels take (1024 / 512)")
        self.scale = float(a["scale"])
        self.softcap = float(a.get("softcap") or 0.0)
        self.window, self.chunk = int(a.get("window") or 0), int(a.get("chunk") or 0)
        self.sigmoid = (a.get("weighting") or "softmax") == "sigmoid"
        if (a.get("weighting") or "softmax") not in ("softmax", "sigmoid"):
            raise ValueError(f"{p}: weighting is 'softmax' or 'sigmoid', got {a.get('weighting')!r}")
        if self.sigmoid and maps != 1:
            raise ValueError(f"{p}: two maps are two softmax attentions; sigmoid weights take one map")
        self.eps = float(a.get("norm_eps") or 0.0)
        self.diff = float(a.get("diff") or 0.0)
        self.head_norm = bool(a.get("head_norm"))
        self.rot = int(a.get("rotary_dim") or 0)
        if self.rot % 2 or self.rot > d:
            raise ValueError(f"{p}: rotary_dim {self.rot} must be even and at most dim {d}")
        self.position = build_part(a["position"]) if self.rot and a.get("position") is not None else None
        if self.rot and self.position is None:
            raise ValueError(f"{p}: rotary_dim {self.rot} needs a position part")
        if self.position is not None:
            self.position.load(weights, rt)
        self.cq, self.ck, self.cv = H * maps * d, G * maps * d, G * m
        self.channels = self.cq + self.ck + self.cv
        # one product for everything that reads the mixer's input: [q | k | v | gate]
        mats = [weights.pop(p + nm[n]) for n in ("q", "k", "v")]
        self.has_gate = bool(a.get("gate"))
        if self.has_gate:
            mats.append(weights.pop(p + nm["gate"]))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.cols = self.w_in.shape[0]
        self.b_in = None
        if a.get("bias"):
            bias = [weights.pop(p + nm[n]) for n in ("q_bias", "k_bias", "v_bias")]
            if self.has_gate:
                bias.append(torch.zeros(H, dtype=torch.float32, device=bias[0].device))
            self.b_in = torch.cat(bias).contiguous()
        self.conv_w = None
        if self.taps >= 1:
            # [taps, channels]: a tap's weights of neighbouring channels side by side, as the kernel's lanes read them
            self.conv_w = torch.cat([weights.pop(p + nm[n]) for n in ("q_conv", "k_conv", "v_conv")], dim=0).t().contiguous()
        norm = bool(a.get("qk_norm"))
        self.q_norm = weights[p + nm["q_norm"]] if norm else None
        self.k_norm = weights[p + nm["k_norm"]] if norm else None
        self.head_bias = weights[p + nm["head_bias"]] if a.get("head_bias") else None
        self.lam = 0.0
        if maps == 2:
            lq1, lk1, lq2, lk2 = (weights[p + nm[n]].double() for n in ("lq1", "lk1", "lq2", "lk2"))
            self.lam = math.exp(float(lq1 @ lk1)) - math.exp(float(lq2 @ lk2)) + self.diff
        self.o_w = weights[p + nm["o"]]
        # Whether the heads' results pass through `head_finish` (float results of the maps in, the
        # output projection's rows out) or go to the output projection as the attention kernel wrote them.
        self.finish = maps == 2 or self.head_norm or self.has_gate
        # bfloat16: keys and values at one common head size that the warp-level kernels are compiled for
        # (zero-filled columns add nothing to a score; value columns beyond vdim are never read back)
        self.store = int(a.get("head_dim") or 0) if not rt.exact else 0
        self.dpad = int(a.get("map_stride") or 0) if self.store else d
        if os.environ.get("CRANE_SCORED_ATTENTION", "mma") == "simt":        # the FP32-core kernel in bfloat16 too
            self.store, self.dpad = 0, d
        if self.store and not rt.kernels.scored_attention_supports(self.store, H, G, maps):
            self.store, self.dpad = 0, d
        if self.store and not self.finish and self.store != m:
            wide = torch.zeros((self.w, H, self.store), dtype=self.o_w.dtype, device=self.o_w.device)
            wide[:, :, :m] = self.o_w.view(self.w, H, m)
            self.o_w = wide.view(self.w, H * self.store).contiguous()
        self.max_splits = int(os.environ.get("CRANE_DECODE_SPLITS", "64"))

    def cache_need(self) -> CacheNeed:
        if self.store:
            kv = CacheNeed("kv", kv_heads=self.G, head_dim=self.store, window=self.window)
        else:
            kv = CacheNeed("kv", kv_heads=self.G, head_dim=self.maps * self.d, window=self.window, v_head_dim=self.m)
        if self.taps <= 1:
            return kv
        tails = CacheNeed("state", state_shape=((self.taps - 1) * self.channels,), state_dtype=torch.float32)
        return CacheNeed("multi", parts=(kv, tails))

    def forward(self, h, ctx, cache, rt, hold: bool = False):
        n, k = h.shape[0], rt.kernels
        H, G, d, m, maps = self.H, self.G, self.d, self.m, self.maps
        kv, tails = (cache.parts[0], cache.parts[1].state) if self.taps > 1 else (cache, None)
        proj = rt.linear(h, self.w_in, self.b_in, "attn_qkv")
        table = ctx.block_tables[kv.group]
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.tables(rt, ctx.max_positions)
            if cos.shape[1] * 2 != self.rot:
                raise ValueError(f"{self.prefix}: the position encoding gives tables for a rotated width of "
                                 f"{cos.shape[1] * 2}, the mixer rotates {self.rot}")
        Dk = self.store or maps * d
        Dv = self.store or m
        q = rt.ws.get("attn_q", n, H * Dk, rt.dtype)
        gate = rt.ws.get("attn_gate", n, H, torch.float32) if self.has_gate else None
        k.scored_prep(proj, self.cols, ctx, table, tails, self.conv_w, max(self.taps, 1), kv.page_size, self.q_norm,
                      self.k_norm, self.eps, q, kv.k, kv.v, H, G, maps, d, m, self.dpad, cos, sin, self.rot, gate,
                      self.channels, rt.err)
        rt.launches += 2 if self.taps > 1 else 1
        norm_scale = 1.0 - self.diff if self.head_norm else 1.0
        if not self.store:
            # the FP32-core kernel: the true 32-bit path, and head sizes that the warp-level kernels lack
            o = rt.ws.get("attn_o", n, H * m, rt.dtype)
            raw = rt.ws.get("attn_maps", n, H * maps * m, torch.float32) if self.finish else None
            k.scored_attention_simt(q, None if self.finish else o, kv.k, kv.v, ctx.positions, ctx.tok_entry, table,
                                    kv.page_size, H, G, d, m, self.window, self.scale, rt.err, softcap=self.softcap,
                                    chunk=self.chunk, sigmoid=self.sigmoid, head_bias=self.head_bias, maps=maps,
                                    d_row=maps * d, d_map=d, out_f32=raw)
            rt.launches += 1
            if self.finish:
                k.head_finish(raw, ctx.tok_entry, gate, o, H, maps, m, self.lam, self.head_norm, norm_scale, self.eps)
                rt.launches += 1
            return rt.linear(o, self.o_w, None, "attn_out", hold=hold)
        # the warp-level kernels at the stored head size: the weights of both maps, lambda, the head norm
        # and the gate are finished inside them (or in the merge of a single token's key slices)
        o = rt.ws.get("attn_o", n, H * (m if self.finish else Dv), rt.dtype)
        mod = k.ScoreMod(softcap=self.softcap, chunk=self.chunk, sigmoid=self.sigmoid, head_bias=self.head_bias,
                         maps=maps, lam=self.lam, head_norm=self.head_norm, norm_scale=norm_scale, eps=self.eps,
                         gate=gate, dv=m, compact=self.finish)
        rt.launches += scored_attention_kernels(k, rt, ctx, q, o, kv, table, H, G, self.store, self.window, self.scale,
                                                mod, self.max_splits)
        return rt.linear(o, self.o_w, None, "attn_out", hold=hold)


def scored_attention_kernels(k, rt, ctx, q, o, cache, table, H, G, D, window, scale, mod, max_splits) -> int:
    """Attention of q [n, H, D] over pools of head size D with the warp-level kernels for worked-on
    scores: entries of one token through the split-KV kernel where that pays, the others through the
    kernel for portions.  Returns the launches."""
    n = q.shape[0]
    split_kv = H // G <= 16                  # the query heads of a key/value head are the rows of one MMA tile
    decode = split_kv and ctx.max_q_len == 1 and n == ctx.n_entries
    singles = getattr(ctx, "single_entries", 0) if split_kv and not decode else 0
    launches = 0
    if decode or singles:
        if decode:
            # enough slices for two CTAs an SM (three with two maps, whose CTAs hold two tile stages a warp)
            per_sm = 3 if mod.maps == 2 else 2
            splits = max(1, min(32, (per_sm * rt.num_sms) // max(1, ctx.n_entries * G)))
        else:
            splits = min(8, k.decode_splits(singles, G, rt.num_sms, max_splits))
        rows = rt.max_decode_rows * H * mod.maps * 32
        part_o = rt.ws.get("attn_part_o", rows, D, torch.float32, cap=rows)
        part_ml = rt.ws.get("attn_part_ml", rows, 2, torch.float32, cap=rows)
        k.scored_decode_attention(q, o, cache.k, cache.v, ctx.cu_q, ctx.kv_len, table, cache.page_size, H, G, D,
                                  window, scale, splits, part_o, part_ml, mod, rt.err)
        launches += 2
        if decode:
            return launches
    tiles = query_tiles(ctx, 64, skip_single=bool(singles))
    k.scored_prefill_attention(q, o, cache.k, cache.v, ctx.cu_q, ctx.kv_len, table, cache.page_size, tiles, H, G, D,
                               window, scale, mod, rt.err, skip_single=bool(singles))
    return launches + 1
