"""Grouped-query attention over the paged cache.

One product for q, k and v (the three matrices merged, as in the reference,
crane-core/src/models/hunyuan_dense/modeling.rs:349-365, 516-528); rotary
encoding of q and k, THEN per-head RMSNorm of q and k with one [d] weight each
(modeling.rs:541-555); the post-rotary, post-norm k and the raw v go to the
cache (modeling.rs:557); scores q k^T / sqrt(d), causal, softmax, times v;
query head h reads kv head h // (nq / nkv) (modeling.rs:572-636); output
projection (modeling.rs:638-645).  A layer without keys and values of its own
computes q only and reads the cache it is given (modeling.rs:501-514).
"""
from __future__ import annotations

import math
import os

import torch

from ..weights.loader import TensorSpec
from .base import CacheNeed, Part, build_part, query_tiles, register_part


@register_part("mixer", "gqa_attention")
class GqaAttention(Part):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``bias`` (q/k/v/o biases), ``qk_norm`` + ``qk_norm_eps``, ``window`` (0: all
    earlier positions), ``own_kv`` (False: reads another layer's cache),
    ``position`` (a PartSpec of kind position, or None), ``scale`` (default
    1/sqrt(head_dim)); and how heads are rotated and normalised, whose defaults
    are the reference's: ``rotary_dim`` (the leading elements of a head that
    are rotated; default all), ``rope_pairing`` ("half": element i with
    i + rotary_dim/2, or "interleaved": 2i with 2i + 1), ``qk_norm_order``
    ("after_rope" or "before_rope"), ``qk_norm_offset`` (the norms multiply by
    offset + w: 0, or 1 for weights stored as w - 1).
    Tensors: ``<prefix>{q,k,v,o}_proj.weight`` (+ ``.bias``),
    ``<prefix>query_layernorm.weight`` / ``key_layernorm.weight`` [head_dim]."""
    kind = "mixer"

    @classmethod
    def manifest(cls, spec):
        a = spec.params
        h, nq, nkv, d = a["hidden_size"], a["num_heads"], a["num_kv_heads"], a["head_dim"]
        p = spec.prefix
        own = a.get("own_kv", True)
        m = {p + "q_proj.weight": TensorSpec((nq * d, h)), p + "o_proj.weight": TensorSpec((h, nq * d))}
        if own:
            m[p + "k_proj.weight"] = TensorSpec((nkv * d, h))
            m[p + "v_proj.weight"] = TensorSpec((nkv * d, h))
        if a.get("bias"):
            m[p + "q_proj.bias"] = TensorSpec((nq * d,), "float32")
            m[p + "o_proj.bias"] = TensorSpec((h,), "float32")
            if own:
                m[p + "k_proj.bias"] = TensorSpec((nkv * d,), "float32")
                m[p + "v_proj.bias"] = TensorSpec((nkv * d,), "float32")
        if a.get("qk_norm"):
            m[p + "query_layernorm.weight"] = TensorSpec((d,), "float32")
            if own:
                m[p + "key_layernorm.weight"] = TensorSpec((d,), "float32")
        return m

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.nq, self.nkv, self.d = int(a["num_heads"]), int(a["num_kv_heads"]), int(a["head_dim"])
        self.own_kv = bool(a.get("own_kv", True))
        self.window = int(a.get("window") or 0)
        self.scale = float(a.get("scale") or 1.0 / math.sqrt(self.d))
        self.eps = float(a.get("qk_norm_eps") or 0.0)
        if self.nq % self.nkv:
            raise ValueError(f"{p}: {self.nq} query heads are not a multiple of {self.nkv} kv heads")
        if self.d % 2 or self.d > 256:
            raise ValueError(f"{p}: head_dim {self.d} is not supported by the attention kernels "
                             "(even sizes up to 256)")
        names = ["q_proj"] + (["k_proj", "v_proj"] if self.own_kv else [])
        ws = [weights.pop(p + n + ".weight") for n in names]
        self.qkv_w = torch.cat(ws, dim=0).contiguous() if len(ws) > 1 else ws[0]
        self.qkv_b = (torch.cat([weights.pop(p + n + ".bias") for n in names]).contiguous()
                      if a.get("bias") else None)
        self.o_w = weights[p + "o_proj.weight"]
        self.o_b = weights.get(p + "o_proj.bias") if a.get("bias") else None
        self.q_norm = weights.get(p + "query_layernorm.weight") if a.get("qk_norm") else None
        self.k_norm = weights.get(p + "key_layernorm.weight") if a.get("qk_norm") and self.own_kv else None
        self.position = build_part(a["position"]) if a.get("position") is not None else None
        if self.position is not None:
            self.position.load(weights, rt)          # a position encoding may have tensors of its own
        self.qkv_cols = self.qkv_w.shape[0]
        rotary_dim = int(a.get("rotary_dim") or self.d)
        pairing, order = a.get("rope_pairing") or "half", a.get("qk_norm_order") or "after_rope"
        if rotary_dim % 2 or not 0 < rotary_dim <= self.d:
            raise ValueError(f"{p}: rotary_dim {rotary_dim} must be even and at most head_dim {self.d}")
        if pairing not in ("half", "interleaved") or order not in ("after_rope", "before_rope"):
            raise ValueError(f"{p}: rope_pairing is 'half' or 'interleaved', qk_norm_order 'after_rope' or "
                             f"'before_rope'; got {pairing!r}, {order!r}")
        # (rotated width, interleaved pairs, norm before the rotation, offset added to the norm weights)
        self.rope = (rotary_dim, pairing == "interleaved", order == "before_rope",
                     float(a.get("qk_norm_offset") or 0.0))
        self.max_splits = int(os.environ.get("CRANE_DECODE_SPLITS", "64"))

    def cache_need(self) -> CacheNeed:
        if not self.own_kv:
            return CacheNeed("none")
        return CacheNeed("kv", kv_heads=self.nkv, head_dim=self.d, window=self.window)

    def forward(self, h, ctx, cache, rt):
        n = h.shape[0]
        k = rt.kernels
        # (keys and values of more than a few MB stream through L2 between this product and the output
        # projection: asking for that one's weights now would only fetch them twice)
        kv_bytes = int(ctx.h_kv_len[:ctx.n_entries].sum()) * self.nkv * self.d * 4
        qkv = rt.linear(h, self.qkv_w, self.qkv_b, "attn_qkv", hint_next=kv_bytes < (8 << 20))
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.tables(rt, ctx.max_positions)
            if cos.shape[1] * 2 != self.rope[0]:
                raise ValueError(f"{self.prefix}: the position encoding gives tables for a rotated width of "
                                 f"{cos.shape[1] * 2}, the mixer rotates {self.rope[0]}")
        table = ctx.block_tables[cache.group]
        o = rt.ws.get("attn_o", n, self.nq * self.d, rt.dtype)
        decode = (not rt.exact and ctx.max_q_len == 1 and n == ctx.n_entries
                  and k.decode_attention_supports(self.d, self.nq, self.nkv))
        if decode and self.d % 4 == 0:
            # single decoded tokens: rotary encoding, head norms, the cache write, attention over
            # key slices (enough of them to fill the device) in one kernel, their merge in a second
            splits = k.decode_splits(ctx.n_entries, self.nkv, rt.num_sms, self.max_splits,
                                     max_keys=ctx.max_kv_len)
            # slices x entries never exceed two CTAs per SM, or the slices are 4 at most: that bounds
            # the slices' scratch rows
            rows = self.nq * max(2 * rt.num_sms // self.nkv + 1, 4 * rt.max_decode_rows)
            part_o = rt.ws.get("attn_part_o", rows, self.d, torch.float32, cap=rows)
            part_ml = rt.ws.get("attn_part_ml", rows, 2, torch.float32, cap=rows)
            k.paged_decode_attention_fused(qkv, self.qkv_cols, self.own_kv, cos, sin, self.q_norm,
                                           self.k_norm, self.eps, o, cache.k, cache.v, ctx.cu_q,
                                           ctx.kv_len, table, cache.page_size, self.nq, self.nkv,
                                           self.d, self.window, self.scale, splits, part_o, part_ml,
                                           rt.err, rope=self.rope)
            rt.launches += 1 if splits <= 8 else 2     # the merge is a launch of its own above 8 slices
            return rt.linear(o, self.o_w, self.o_b, "attn_out")
        q = rt.ws.get("attn_q", n, self.nq * self.d, rt.dtype)
        k.rope_norm_cache(qkv, self.qkv_cols, rt.dtype, ctx.positions, ctx.tok_entry, table, cos,
                          sin, self.q_norm, self.k_norm, self.eps, q, cache.k, cache.v,
                          cache.page_size, self.nq, self.nkv, self.d, self.own_kv,
                          self.position is not None, rt.err, rope=self.rope)
        use_mma = not rt.exact and k.prefill_attention_supports(self.d, self.nq, self.nkv)
        # Whole prompts of at most 64 tokens take the warp-level kernel (64-row tiles, several CTAs per
        # SM) also at head size 128.  Measured at 16 / 4 heads, tcgen05 against warp-level: 256 prompts of
        # 8 tokens 244 / 144 us, 64 of 32: 44 / 28 us, 32 of 64: 22 / 19 us; 21 of 96: 22 / 23 us, 16 of 128:
        # 16 / 21 us; 16 portions of 32 behind 2,000 cached keys 50 / 94 us.
        short = bool(getattr(ctx, "short_prompts", False)) and use_mma
        use_tc = (not rt.exact and rt.use_tc_attention and not short
                  and k.prefill_attention_tc_supports(self.d, self.nq, self.nkv, cache.page_size))
        # Decoded tokens beside prompt portions: the entries of one token go to the split-KV decode
        # kernel (which skips the others), the prompt portions to the prefill kernel (which skips them).
        singles = getattr(ctx, "single_entries", 0) if (use_tc or use_mma) and not decode else 0
        if singles and not k.decode_attention_supports(self.d, self.nq, self.nkv):
            singles = 0
        if decode or singles:
            if decode:
                splits = max(1, min(32, (2 * rt.num_sms) // max(1, ctx.n_entries * self.nkv)))
            else:
                # at most 8 slices: at head size 128 they merge inside a cluster without scratch
                splits = min(8, k.decode_splits(singles, self.nkv, rt.num_sms, self.max_splits))
            part_o = part_ml = None
            if splits > 1:
                rows = rt.max_decode_rows * self.nq * 32
                part_o = rt.ws.get("attn_part_o", rows, self.d, torch.float32, cap=rows)
                part_ml = rt.ws.get("attn_part_ml", rows, 2, torch.float32, cap=rows)
            k.paged_decode_attention(q, o, cache.k, cache.v, ctx.cu_q, ctx.kv_len, table,
                                     cache.page_size, self.nq, self.nkv, self.d, self.window,
                                     self.scale, splits, part_o, part_ml, rt.err)
            rt.launches += 3 if splits > 1 else 2
            if decode:
                return rt.linear(o, self.o_w, self.o_b, "attn_out")
            rt.launches -= 1                      # the rotary kernel is counted once, below
        if use_tc:
            tiles = query_tiles(ctx, 128, skip_single=bool(singles))
            k.prefill_attention_tc(q, o, cache.k, cache.v, ctx.cu_q, ctx.kv_len, table, cache.page_size,
                                   tiles, self.nq, self.nkv, self.d, self.window, self.scale, rt.err,
                                   skip_single=bool(singles))
            rt.launches += 2
        elif use_mma:
            tiles = query_tiles(ctx, 64, skip_single=bool(singles))
            k.paged_prefill_attention(q, o, cache.k, cache.v, ctx.cu_q, ctx.kv_len, table,
                                      cache.page_size, tiles, self.nq, self.nkv, self.d, self.window,
                                      self.scale, rt.err, skip_single=bool(singles))
            rt.launches += 2
        else:
            k.paged_attention_simt(q, o, cache.k, cache.v, ctx.positions, ctx.tok_entry, table,
                                   cache.page_size, self.nq, self.nkv, self.d, self.window,
                                   self.scale, rt.err)
            rt.launches += 2
        return rt.linear(o, self.o_w, self.o_b, "attn_out")


@register_part("mixer", "sink_attention")
class SinkAttention(Part):
    """Grouped-query attention without positions, whose queries and keys are RMS-normed over
    their whole projections (all heads at once, plain weights), whose values may be wider or
    narrower than its keys, and whose softmax may have a sink: one more candidate of score 0
    that has no value, p_j = exp(s_j) / (1 + sum_i exp(s_i)).
    params: ``hidden_size``, ``heads``, ``kv_heads``, ``dim`` (query/key head), ``vdim`` (value
    head), ``scale``, ``sink`` (default True), ``qk_norm`` (default True) + ``norm_eps``,
    ``window`` (0: every earlier position), ``names`` (tensor names behind the prefix for q, k,
    v, o, q_norm, k_norm).  Tensors: q [H dim, hidden], k [G dim, hidden], v [G vdim, hidden],
    o [hidden, H vdim], q_norm [H dim], k_norm [G dim] (float)."""
    kind = "mixer"
    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}

    @classmethod
    def _sizes(cls, a):
        return (int(a["hidden_size"]), int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"]))

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        w, H, G, d, m = cls._sizes(a)
        nm = dict(cls.NAMES, **(a.get("names") or {}))
        out = {p + nm["q"]: TensorSpec((H * d, w)), p + nm["k"]: TensorSpec((G * d, w)),
               p + nm["v"]: TensorSpec((G * m, w)), p + nm["o"]: TensorSpec((w, H * m))}
        if a.get("qk_norm", True):
            out[p + nm["q_norm"]] = TensorSpec((H * d,), "float32", "scale")
            out[p + nm["k_norm"]] = TensorSpec((G * d,), "float32", "scale")
        return out

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.w, self.H, self.G, self.d, self.m = self._sizes(a)
        nm = dict(self.NAMES, **(a.get("names") or {}))
        if self.H % self.G:
            raise ValueError(f"{p}: {self.H} query heads are not a multiple of {self.G} key/value heads")
        if self.d > 1024 or self.m > 512:
            raise ValueError(f"{p}: heads of {self.d} / {self.m} elements are wider than the attention kernels "
                             "take (1024 / 512)")
        self.scale = float(a["scale"])
        self.sink = bool(a.get("sink", True))
        self.window = int(a.get("window") or 0)
        self.eps = float(a.get("norm_eps") or 0.0)
        self.qkv_w = torch.cat([weights.pop(p + nm[n]) for n in ("q", "k", "v")], dim=0).contiguous()
        self.cols = self.qkv_w.shape[0]
        self.o_w = weights[p + nm["o"]]
        norm = bool(a.get("qk_norm", True))
        self.q_norm = weights[p + nm["q_norm"]] if norm else None
        self.k_norm = weights[p + nm["k_norm"]] if norm else None
        # On the bfloat16 path keys and values are stored at one common head size that the warp-level
        # attention kernels are compiled for (zero-filled columns add nothing to a score, and the
        # value columns beyond vdim are never read back); the 32-bit path stores them as wide as they are.
        self.store = int(a.get("head_dim") or 0) if not rt.exact else 0
        if os.environ.get("CRANE_TALKING_ATTENTION", "mma") == "simt":       # the FP32-core kernel in bfloat16 too
            self.store = 0
        if self.store and not (rt.kernels.prefill_attention_supports(self.store, self.H, self.G)
                               and rt.kernels.decode_attention_supports(self.store, self.H, self.G)):
            self.store = 0
        if self.sink and not getattr(rt.kernels, "mma_attention_takes_sink", False):
            self.store = 0
        if self.store and self.store != self.m:
            wide = torch.zeros((self.w, self.H, self.store), dtype=self.o_w.dtype, device=self.o_w.device)
            wide[:, :, :self.m] = self.o_w.view(self.w, self.H, self.m)
            self.o_w = wide.view(self.w, self.H * self.store).contiguous()
        self.max_splits = int(os.environ.get("CRANE_DECODE_SPLITS", "64"))

    @staticmethod
    def common_head_size(dim: int, vdim: int, sizes) -> int:
        """The smallest head size of ``sizes`` that holds both a key and a value row (0: none)."""
        fit = [s for s in sorted(sizes) if s >= max(dim, vdim)]
        return fit[0] if fit else 0

    def cache_need(self) -> CacheNeed:
        if self.store:
            return CacheNeed("kv", kv_heads=self.G, head_dim=self.store, window=self.window)
        return CacheNeed("kv", kv_heads=self.G, head_dim=self.d, window=self.window, v_head_dim=self.m)

    def forward(self, h, ctx, cache, rt):
        n = h.shape[0]
        k = rt.kernels
        H, G, d, m = self.H, self.G, self.d, self.m
        qkv = rt.linear(h, self.qkv_w, None, "attn_qkv")
        table = ctx.block_tables[cache.group]
        D = self.store or d
        q = rt.ws.get("attn_q", n, H * D, rt.dtype)
        k.projection_norm_cache(qkv, self.cols, ctx.positions, ctx.tok_entry, table, cache.page_size, self.q_norm,
                                self.k_norm, self.eps, q, cache.k, cache.v, H, G, d, m, rt.err)
        rt.launches += 1
        if not self.store:
            o = rt.ws.get("attn_o", n, H * m, rt.dtype)
            k.paged_attention_simt(q, o, cache.k, cache.v, ctx.positions, ctx.tok_entry, table, cache.page_size,
                                   H, G, d, self.window, self.scale, rt.err, dv=m, v_stride=m, sink=self.sink)
            rt.launches += 1
            return rt.linear(o, self.o_w, None, "attn_out")
        # the warp-level kernels at the common head size; the output projection's matrix has zero
        # columns where a stored head is wider than vdim
        o = rt.ws.get("attn_o", n, H * D, rt.dtype)
        rt.launches += sink_attention_kernels(k, rt, ctx, q, o, cache, table, H, G, D, self.window, self.scale,
                                              self.sink, self.max_splits)
        return rt.linear(o, self.o_w, None, "attn_out")


def sink_attention_kernels(k, rt, ctx, q, o, cache, table, H, G, D, window, scale, sink, max_splits,
                           cross: bool = False) -> int:
    """Attention of q [n, H, D] over pools of head size D with the warp-level kernels: entries of
    one token through the split-KV decode kernel where that pays, the others through the prefill
    kernel.  ``cross``: ``o`` is float [n, H, G, D], every query head's weights applied to the values
    of every key/value head (a CTA per pair of key/value heads where there was one per head).
    Returns the launches."""
    n = q.shape[0]
    decode = ctx.max_q_len == 1 and n == ctx.n_entries
    singles = 0 if decode else getattr(ctx, "single_entries", 0)
    launches = 0
    if decode or singles:
        if decode:
            splits = max(1, min(32, (2 * rt.num_sms) // max(1, ctx.n_entries * G * (G if cross else 1))))
        else:
            splits = min(8, k.decode_splits(singles, G * (G if cross else 1), rt.num_sms, max_splits))
        part_o = part_ml = None
        if splits > 1 or cross:
            rows = rt.max_decode_rows * H * (G if cross else 1) * 32
            part_o = rt.ws.get("attn_part_o", rows, D, torch.float32, cap=rows)
            part_ml = rt.ws.get("attn_part_ml", rows, 2, torch.float32, cap=rows)
        k.paged_decode_attention(q, o, cache.k, cache.v, ctx.cu_q, ctx.kv_len, table, cache.page_size, H, G, D,
                                 window, scale, splits, part_o, part_ml, rt.err, sink=sink, cross=cross)
        launches += 2 if splits > 1 or cross else 1
        if decode:
            return launches
    tiles = query_tiles(ctx, 64, skip_single=bool(singles))
    k.paged_prefill_attention(q, o, cache.k, cache.v, ctx.cu_q, ctx.kv_len, table, cache.page_size, tiles, H, G, D,
                              window, scale, rt.err, skip_single=bool(singles), sink=sink, cross=cross)
    return launches + 1


@register_part("mixer", "talking_attention")
class TalkingAttention(Part):
    """Grouped-query attention whose heads exchange their softmax weights: scores of head h are
    q_h . k_(h // (H / G)) * scale * temp[h], causal softmax, then w'_h = sum_g talk[h, g] w_g, and head h
    applies w'_h to the values of its own key/value head.  Rotary positions on the leading
    ``rotary_dim`` elements of every query and key head (element i with i + rotary_dim / 2).

    The mixed weights are never formed.  o_h = sum_g talk[h, g] (w_g V_(kv of h)): every query head's own
    weights are applied to the values of EVERY key/value head (H x G results per token, 32-bit), and a
    small kernel mixes those with ``talk``.  The softmax itself stays an ordinary one per head.

    params: ``hidden_size``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rotary_dim`` (0: none),
    ``position`` (a PartSpec of kind position whose tables have rotary_dim / 2 columns, or None),
    ``window`` (0: every earlier position), ``head_dim`` (bfloat16: the common head size keys and values are
    stored at; 0: as wide as they are), ``names``.  Tensors: q [H dim, hidden], k [G dim, hidden],
    v [G vdim, hidden], o [hidden, H vdim], and in 32-bit talk [H, H], temp [H]."""
    kind = "mixer"
    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "talk": "talk", "temp": "temp"}

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        w, H, G, d, m = (int(a[k]) for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim"))
        nm = dict(cls.NAMES, **(a.get("names") or {}))
        return {p + nm["q"]: TensorSpec((H * d, w)), p + nm["k"]: TensorSpec((G * d, w)),
                p + nm["v"]: TensorSpec((G * m, w)), p + nm["o"]: TensorSpec((w, H * m)),
                p + nm["talk"]: TensorSpec((H, H), "float32", "eye"), p + nm["temp"]: TensorSpec((H,), "float32", "scale")}

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.w, self.H, self.G, self.d, self.m = (int(a[k]) for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim"))
        nm = dict(self.NAMES, **(a.get("names") or {}))
        if self.H % self.G:
            raise ValueError(f"{p}: {self.H} query heads are not a multiple of {self.G} key/value heads")
        if self.d > 1024 or self.m > 512:
            raise ValueError(f"{p}: heads of {self.d} / {self.m} elements are wider than the attention kernels "
                             "take (1024 / 512)")
        self.scale = float(a["scale"])
        self.window = int(a.get("window") or 0)
        self.rot = int(a.get("rotary_dim") or 0)
        self.position = build_part(a["position"]) if self.rot and a.get("position") is not None else None
        if self.rot and self.position is None:
            raise ValueError(f"{p}: rotary_dim {self.rot} needs a position part")
        if self.position is not None:
            self.position.load(weights, rt)
        self.qkv_w = torch.cat([weights.pop(p + nm[n]) for n in ("q", "k", "v")], dim=0).contiguous()
        self.cols = self.qkv_w.shape[0]
        self.o_w = weights[p + nm["o"]]
        self.talk, self.temp = weights[p + nm["talk"]], weights[p + nm["temp"]]
        # bfloat16: keys and values at one common head size that the warp-level kernels are compiled for
        # (zero-filled columns add nothing to a score; value columns beyond vdim are never read back)
        self.store = int(a.get("head_dim") or 0) if not rt.exact else 0
        if os.environ.get("CRANE_TALKING_ATTENTION", "mma") == "simt":       # the FP32-core kernel in bfloat16 too
            self.store = 0
        if self.store and not (rt.kernels.prefill_attention_supports(self.store, self.H, self.G)
                               and rt.kernels.decode_attention_supports(self.store, self.H, self.G)):
            self.store = 0
        self.max_splits = int(os.environ.get("CRANE_DECODE_SPLITS", "64"))

    def cache_need(self) -> CacheNeed:
        if self.store:
            return CacheNeed("kv", kv_heads=self.G, head_dim=self.store, window=self.window)
        return CacheNeed("kv", kv_heads=self.G, head_dim=self.d, window=self.window, v_head_dim=self.m)

    def forward(self, h, ctx, cache, rt, hold: bool = False):
        n, k = h.shape[0], rt.kernels
        H, G, d, m = self.H, self.G, self.d, self.m
        qkv = rt.linear(h, self.qkv_w, None, "attn_qkv")
        table = ctx.block_tables[cache.group]
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.tables(rt, ctx.max_positions)
            if cos.shape[1] * 2 != self.rot:
                raise ValueError(f"{self.prefix}: the position encoding gives tables for a rotated width of "
                                 f"{cos.shape[1] * 2}, the mixer rotates {self.rot}")
        D = self.store or d
        q = rt.ws.get("attn_q", n, H * D, rt.dtype)
        k.projection_norm_cache(qkv, self.cols, ctx.positions, ctx.tok_entry, table, cache.page_size, None, None, 0.0,
                                q, cache.k, cache.v, H, G, d, m, rt.err, cos=cos, sin=sin, rot_dims=self.rot,
                                q_head_scale=self.temp)
        Dv = self.store or m
        cross = rt.ws.get("attn_cross", n, H * G * Dv, torch.float32)
        if not self.store:
            k.paged_attention_simt(q, None, cache.k, cache.v, ctx.positions, ctx.tok_entry, table, cache.page_size,
                                   H, G, d, self.window, self.scale, rt.err, dv=m, v_stride=m, out_cross=cross)
            rt.launches += 1
        else:
            rt.launches += sink_attention_kernels(k, rt, ctx, q, cross, cache, table, H, G, D, self.window, self.scale,
                                                  False, self.max_splits, cross=True)
        o = rt.ws.get("attn_o", n, H * m, rt.dtype)
        k.head_talk_mix(cross, self.talk, ctx.tok_entry, o, H, G, Dv, m)
        rt.launches += 2
        return rt.linear(o, self.o_w, None, "attn_out", hold=hold)
