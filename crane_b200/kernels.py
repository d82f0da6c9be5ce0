"""Python face of the CUDA library: one method per kernel, tensors in, tensors out.

Every method launches on torch's current stream of the tensor's device and
checks the launch status.  There is no other implementation behind these
methods: if the library cannot be built or loaded, constructing ``Kernels``
raises.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Union

import torch

from .csrc import build

P, I, L, F = c_void_p, c_int, c_longlong, c_float

_SIGNATURES = {
    "crane_embed_gather": [I, P, P, P, I, I, I, P, I, P, P],
    "crane_add_rmsnorm": [I, P, P, P, I, L, P, P, P, I, I, F, P],
    "crane_rope_norm_cache": [I, P, P, I, L, I, P, P, P, I, P, P, I, P, P, F, P, P, P, I, I, I, I,
                              I, I, I, I, I, I, I, F, P, P],
    "crane_silu_mul": [I, P, P, I, L, P, I, I, I, P],
    "crane_to_float": [I, P, P, L, P],
    "crane_sum_parts": [P, I, L, L, P, L, I, I, P],
    "crane_gemm_simt": [I, I, P, P, P, P, I, I, I, L, L, L, P],
    "crane_gemm_bf16_tcgen05": [P, P, P, P, I, I, I, L, L, L, I, I, I, I, I, L, I, P, L, P, P],
    "crane_gemm_bf16_pair": [P, P, P, P, I, I, I, L, L, L, I, I, I, P, P],
    "crane_paged_attention_simt": [I, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P, P, P],
    "crane_paged_decode_attention_supports": [I, I, I],
    "crane_paged_decode_attention": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, I, P, P],
    "crane_paged_prefill_attention_supports": [I, I, I],
    "crane_paged_prefill_attention": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, I, P, P, P],
    "crane_paged_decode_attention_fused": [P, P, I, L, I, I, I, P, P, I, P, P, F, P, P, P, P, P, P, P, P,
                                           I, I, I, I, I, I, I, I, F, I, I, I, I, F, P, P],
    "crane_prefill_attention_tc_supports": [I, I, I, I],
    "crane_prefill_attention_tc": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P, P],
    "crane_embed_bigram": [I, P, P, P, P, I, I, I, I, L, L, P, P, P, P, P, I, P, I, P, P],
    "crane_combine_layernorm": [I, P, P, L, I, P, P, I, L, P, P, I, L, P, P, P, P, P, P, P, P, I, I, F, P],
    "crane_xielu": [I, P, P, I, L, P, L, P, P],
    "crane_latent_prep": [I, P, P, I, L, I, I, I, I, I, I, I, I, P, P, I, P, P, P, I, I, I, P, P, F, P, I, P, P],
    "crane_head_linear": [I, P, P, I, L, I, I, I, P, I, I, P, P, I, L, I, I, P, P, I, I, I, I, P],
    "crane_latent_attention_mma_supports": [I, I],
    "crane_latent_attention_mma": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, P, P],
    "crane_embed_sinusoid": [I, P, P, P, P, P, P, I, I, I, P, I, P, P],
    "crane_stream_enter": [P, P, P, I, I, P],
    "crane_add_normed_norm": [I, P, P, P, I, L, P, P, P, P, I, I, F, F, P],
    "crane_token_gate": [I, P, P, I, L, P, P, I, I, I, P, I, I, P, I, P, P],
    "crane_ffn_activation": [I, P, P, I, L, P, I, I, I, P, I, I, I, P],
    "crane_route_topk": [P, P, P, P, I, I, I, P],
    "crane_projection_norm_cache": [I, P, P, I, L, I, P, P, P, I, I, I, P, P, F, P, P, P, I, I, I, I, I, I, I,
                                    P, P, I, I, P, P, P],
    "crane_streams_norm": [I, P, L, I, P, P, P, I, L, P, P, P, P, P, P, I, I, F, P],
    "crane_route_grouped": [P, I, P, P, I, I, I, I, I, I, P],
    "crane_gated_activation": [I, P, P, I, L, P, I, I, P, I, I, I, I, P],
    "crane_conv_delta_prep": [I, P, P, I, L, I, P, P, P, P, I, P, L, L, P, I, P, P, P, I, I, I, I, I, I, I, F, F, P, P],
    "crane_decay_gate_prep": [I, P, P, I, L, I, P, P, P, I, F, F, P, I, I, I, I, I, P],
    "crane_matrix_state_plan": [I, P, P],
    "crane_matrix_state_scan": [P, I, I, I, I, I, I, I, I, I, P, P, P, I, P, L, P, I, I, I, I, P, P],
    "crane_head_norm_gate": [I, P, P, P, I, L, I, I, P, P, F, P, I, I, I, P],
    "crane_head_talk_mix": [I, P, P, P, P, I, I, I, I, I, P],
    "crane_pair_norm_mean": [I, P, P, I, L, P, P, I, L, P, P, F, P, I, I, P],
    "crane_delta_rule_prep": [I, P, P, I, L, I, P, P, P, P, P, I, I, I, I, F, F, P],
    "crane_delta_rule_scan": [I, P, P, I, L, I, P, P, P, P, I, P, P, F, P, P, P, I, I, I, I, I, P, P],
    "crane_add_group_rmsnorm": [I, P, P, P, I, L, P, P, I, L, P, P, P, I, I, I, F, P],
    "crane_poly_norm": [I, P, P, I, L, P, P, I, I, F, P],
    "crane_scored_prep": [I, P, P, I, L, I, P, P, P, P, P, I, P, L, P, I, P, I, I, I, P, P, F, P, P, P, I, I, I, I,
                          I, I, I, I, I, I, P, P, I, I, P, I, P, P],
    "crane_head_finish": [I, P, P, P, P, I, I, I, I, I, I, F, I, F, F, P],
    "crane_scored_attention_simt": [I, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, F, I, I, P, I, I, I,
                                    P, P, P],
    "crane_scored_attention_supports": [I, I, I, I],
    "crane_scored_attention": [I, I, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, I, F, I, I, P, F, I,
                               F, F, P, I, I, P, P],
    "crane_repetition_penalty": [P, L, I, I, P, I, P, P, P],
    "crane_sample": [P, L, I, I, P, P, P, P, P, P, P],
}


class KernelError(RuntimeError):
    pass


class Partials:
    """A matrix product left as ``n`` float partial sums [n, rows, cols] (split
    along the inner dimension); the consumer adds them up in order."""

    def __init__(self, parts: torch.Tensor):
        self.parts = parts

    @property
    def shape(self):
        return self.parts.shape[1:]

    def sum(self, dtype=None):
        """The product itself: the slices added up in order (rounded once to ``dtype``)."""
        total = self.parts.sum(dim=0)
        return total if dtype is None else total.to(dtype)


Act = Union[torch.Tensor, Partials]


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dt(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 storage, got {dtype}")


def _split(a: Act):
    """(whole ptr, parts ptr, n_parts, part_stride) of a product result."""
    if isinstance(a, Partials):
        p = a.parts
        return None, p.data_ptr(), p.shape[0], p.stride(0)
    return a.data_ptr(), None, 0, 0


class Kernels:
    def __init__(self, head_sizes=()) -> None:
        self.head_sizes: set = set()      # head sizes whose warp-level attention kernels the loaded library holds
        self._bind(build.load_kernels([d for d in head_sizes if d in build.ATTENTION_HEAD_SIZES]))

    def _bind(self, lib) -> None:
        self.lib = lib
        for name, sig in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.argtypes = sig
            fn.restype = c_int
        # kernels of a step overlap their start with the end of the kernel before them
        self.lib.crane_set_pdl.argtypes = [c_int]
        self.lib.crane_set_pdl.restype = None
        self.pdl_default = 0 if os.environ.get("CRANE_PDL", "1") == "0" else 1
        self.lib.crane_set_pdl(self.pdl_default)
        self.head_sizes = {d for d in build.ATTENTION_HEAD_SIZES
                           if self.lib.crane_paged_decode_attention_supports(d, 1, 1)}

    def require_head_size(self, d: int) -> None:
        """Makes sure the loaded library holds the warp-level attention kernels of
        head size ``d`` (if there are any for it): a first call for a model
        compiles what that model needs, a model with another head size adds its
        two files.  The library that was loaded before stays loaded (graphs that
        were recorded with it keep working)."""
        if d in self.head_sizes or d not in build.ATTENTION_HEAD_SIZES:
            return
        self._bind(build.load_kernels(sorted(self.head_sizes | {d})))

    # While a model runs a step, every launch goes to the stream that was current when the step
    # began (looked up once, not per launch); outside a step the current stream is asked for.
    pinned_stream: Optional[int] = None

    def _stream(self, t: torch.Tensor) -> int:
        if self.pinned_stream is not None:
            return self.pinned_stream
        return torch.cuda.current_stream(t.device).cuda_stream

    @staticmethod
    def _check(code: int, what: str) -> None:
        if code != 0:
            raise KernelError(f"{what}: CUDA error {code}")

    # ---- elementwise ---------------------------------------------------
    def embed_gather(self, tokens, table, x, err, deferred=None) -> None:
        """``deferred`` int32 [R]: a token id <= -2 is read from its row -id - 2."""
        n, hidden = x.shape
        self._check(self.lib.crane_embed_gather(_dt(table.dtype), tokens.data_ptr(), table.data_ptr(),
                                                x.data_ptr(), n, hidden, table.shape[0],
                                                deferred.data_ptr() if deferred is not None else None,
                                                deferred.numel() if deferred is not None else 0,
                                                err.data_ptr(), self._stream(x)), "embed_gather")

    def add_rmsnorm(self, x, delta: Optional[Act], weight, eps: float, out, rows=None) -> None:
        """x += delta (if given); out = rmsnorm(x) * weight.  With ``rows`` only
        those rows of x are read (and x is not written)."""
        whole, parts, n_parts, stride = (None, None, 0, 0) if delta is None else _split(delta)
        n_rows = out.shape[0]
        self._check(self.lib.crane_add_rmsnorm(_dt(out.dtype), x.data_ptr(), whole, parts, n_parts,
                                               stride, weight.data_ptr(), _ptr(rows), out.data_ptr(),
                                               n_rows, x.shape[1], float(eps), self._stream(x)),
                    "add_rmsnorm")

    def rope_norm_cache(self, qkv: Act, qkv_cols: int, dtype, positions, tok_entry, block_table,
                        cos, sin, q_norm_w, k_norm_w, eps, q_out, k_pool, v_pool, page_size, nq,
                        nkv, d, has_kv: bool, rotary: bool, err, rope=None) -> None:
        """``rope``: (rotary_dim, interleaved pairs, norm before the rotation,
        norm weight offset); None: the whole head, contiguous halves, norm after,
        plain weights.  cos/sin are [positions, rotary_dim / 2]."""
        rd, inter, first, off = rope or (d, False, False, 0.0)
        whole, parts, n_parts, stride = _split(qkv)
        n_tokens = q_out.shape[0]
        num_pages = k_pool.shape[0] if k_pool is not None else 0
        max_blocks = block_table.shape[1] if block_table is not None else 0
        self._check(self.lib.crane_rope_norm_cache(
            _dt(dtype), whole, parts, n_parts, stride, qkv_cols, positions.data_ptr(),
            _ptr(tok_entry), _ptr(block_table), max_blocks, _ptr(cos), _ptr(sin),
            cos.shape[0] if cos is not None else 0, _ptr(q_norm_w), _ptr(k_norm_w), float(eps),
            q_out.data_ptr(), _ptr(k_pool), _ptr(v_pool), num_pages, page_size, n_tokens, nq, nkv,
            d, 1 if has_kv else 0, 1 if rotary else 0, int(rd), 1 if inter else 0, 1 if first else 0,
            float(off), err.data_ptr(), self._stream(q_out)), "rope_norm_cache")

    def silu_mul(self, gu: Act, out, blocked: bool = False) -> None:
        """out = silu(gate) * up.  ``gu`` rows are [gate | up], or, ``blocked``,
        16 gate columns then the 16 up columns of the same features, and so on."""
        whole, parts, n_parts, stride = _split(gu)
        self._check(self.lib.crane_silu_mul(_dt(out.dtype), whole, parts, n_parts, stride,
                                            out.data_ptr(), out.shape[0], out.shape[1],
                                            1 if blocked else 0, self._stream(out)), "silu_mul")

    def sum_parts(self, parts: "Partials", out) -> None:
        """out[rows, cols] (float) = the partial sums added up in slice order."""
        p = parts.parts
        assert p.dtype == torch.float32 and out.dtype == torch.float32 and out.shape == p.shape[1:]
        assert p.stride(2) == 1 and out.stride(1) == 1
        self._check(self.lib.crane_sum_parts(p.data_ptr(), p.shape[0], p.stride(0), p.stride(1),
                                             out.data_ptr(), out.stride(0), p.shape[1], p.shape[2],
                                             self._stream(out)), "sum_parts")

    def to_float(self, t, out) -> None:
        self._check(self.lib.crane_to_float(_dt(t.dtype), t.data_ptr(), out.data_ptr(), t.numel(),
                                            self._stream(t)), "to_float")

    # ---- parts of other layer designs ------------------------------------
    def embed_bigram(self, tokens, table, bigram, x, buckets, mul_prev, mul_cur, positions, tok_entry,
                     cu_q, slots, last_token, err, deferred=None) -> None:
        """x[t] = table[token] + bigram[(previous * mul_prev + token * mul_cur) mod buckets];
        a sequence's first token takes row ``buckets``.  ``last_token`` int32 [slots]: the
        token before each request's next one, read and replaced here.  ``bigram`` None:
        the plain embedding."""
        n, hidden = x.shape
        self._check(self.lib.crane_embed_bigram(
            _dt(table.dtype), tokens.data_ptr(), table.data_ptr(), _ptr(bigram), x.data_ptr(), n, hidden,
            table.shape[0], int(buckets), int(mul_prev), int(mul_cur), positions.data_ptr(),
            tok_entry.data_ptr(), cu_q.data_ptr(), slots.data_ptr(), last_token.data_ptr(),
            last_token.numel(), _ptr(deferred), deferred.numel() if deferred is not None else 0,
            err.data_ptr(), self._stream(x)), "embed_bigram")

    def combine_layernorm(self, x, hist, n_hist, a: Optional[Act], f: Optional[Act], dwa, rows,
                          w1, b1, out1, w2, b2, out2, eps: float) -> None:
        """X = x + (a + f); hist[n_hist - 1] = X; x = sum_j dwa[j] hist[j] (``dwa`` None: x = X);
        out1 / out2 = the layer norms (w1, b1) / (w2, b2) of the new x.  ``hist`` float
        [slots, rows, hidden] or None.  With ``rows`` only those rows are read and
        nothing but out1 / out2 is written."""
        aw, ap, an, astr = (None, None, 0, 0) if a is None else _split(a)
        fw, fp, fn, fstr = (None, None, 0, 0) if f is None else _split(f)
        n_rows = out1.shape[0]
        self._check(self.lib.crane_combine_layernorm(
            _dt(out1.dtype), x.data_ptr(), _ptr(hist), hist.stride(0) if hist is not None else 0,
            int(n_hist), aw, ap, an, astr, fw, fp, fn, fstr, _ptr(dwa), _ptr(rows), w1.data_ptr(),
            b1.data_ptr(), out1.data_ptr(), _ptr(w2), _ptr(b2), _ptr(out2), n_rows, x.shape[1],
            float(eps), self._stream(x)), "combine_layernorm")

    def xielu(self, up: Act, out, pq) -> None:
        """out = xIELU(up) with the two float numbers ``pq`` (p, q) on the device."""
        whole, parts, n_parts, stride = _split(up)
        self._check(self.lib.crane_xielu(_dt(out.dtype), whole, parts, n_parts, stride, out.data_ptr(),
                                         out.numel(), pq.data_ptr(), self._stream(out)), "xielu")

    def latent_prep(self, proj: Act, cols, q_off, dkv_off, heads, dim, rot, rank, rot_dims, cos, sin,
                    positions, tok_entry, block_table, pool, page_size, norm_w, eps, q_abs, err) -> None:
        """Latent attention's cache write and query rotation; ``dkv_off`` < 0: the
        layer writes no cache.  ``pool`` [pages, 1, page_size, rank + rot]."""
        whole, parts, n_parts, stride = _split(proj)
        self._check(self.lib.crane_latent_prep(
            _dt(q_abs.dtype), whole, parts, n_parts, stride, int(cols), int(q_off), int(dkv_off), heads, dim,
            rot, rank, rot_dims, cos.data_ptr(), sin.data_ptr(), cos.shape[0], positions.data_ptr(),
            tok_entry.data_ptr(), block_table.data_ptr(), block_table.shape[1], pool.shape[0], page_size,
            pool.data_ptr(), _ptr(norm_w), float(eps), q_abs.data_ptr(), q_abs.shape[0], err.data_ptr(),
            self._stream(q_abs)), "latent_prep")

    def head_linear(self, x: Act, x_cols, x_off, x_head, w, n_in, n_out, out, out_pitch, out_head,
                    heads, tok_entry=None, gate: Optional[Act] = None, g_cols=0, g_off=0) -> None:
        """out[t, h, :n_out] = w[h] (as [n_in, n_out]) applied to x[t, x_off + h * x_head : + n_in],
        times sigmoid(gate[t, g_off + h * n_out : ...]) if a gate is given."""
        xw, xp, xn, xs = _split(x)
        gw, gp, gn, gs = (None, None, 0, 0) if gate is None else _split(gate)
        n_tokens = out.shape[0]
        self._check(self.lib.crane_head_linear(
            _dt(out.dtype), xw, xp, xn, xs, int(x_cols), int(x_off), int(x_head), w.data_ptr(), int(n_in),
            int(n_out), gw, gp, gn, gs, int(g_cols), int(g_off), _ptr(tok_entry), out.data_ptr(),
            int(out_pitch), int(out_head), n_tokens, int(heads), self._stream(out)), "head_linear")

    def latent_attention_mma_supports(self, dk: int, dv: int) -> bool:
        return bool(self.lib.crane_latent_attention_mma_supports(int(dk), int(dv)))

    def latent_attention_mma(self, q, out, pool, cu_q, kv_len, block_table, page_size, tiles, splits,
                             small: bool, heads, dk, dv, scale, part_o, part_ml, err) -> None:
        """Attention over cache rows [dk] whose values are their leading ``dv`` columns,
        ``heads`` query heads per token (bfloat16).  One launch takes the entries of at
        most 16 rows (tokens x heads) in tiles of 16 (``small``) or the others in tiles
        of 64; ``tiles``: at least how many there are.  ``splits`` > 1 cuts every tile's
        keys into slices that a second kernel merges (scratch: ``part_o``, ``part_ml``)."""
        self._check(self.lib.crane_latent_attention_mma(
            q.data_ptr(), out.data_ptr(), _ptr(part_o), _ptr(part_ml), pool.data_ptr(), cu_q.data_ptr(),
            kv_len.data_ptr(), block_table.data_ptr(), block_table.shape[1], pool.shape[0], page_size,
            kv_len.shape[0], int(tiles), int(splits), 1 if small else 0, heads, dk, dv, float(scale),
            err.data_ptr(), self._stream(q)), "latent_attention_mma")

    # ---- the stream of layers that norm what they add, routed feed-forwards ----
    def embed_sinusoid(self, tokens, positions, table, freq, x, keep, err, deferred=None) -> None:
        """x[t] = table[token] + the sinusoid of the position (``freq`` float64 [ceil(hidden / 2)]:
        column 2i gets sin(p freq[i]), 2i + 1 the cosine); ``keep``: a second copy of the rows."""
        n, hidden = x.shape
        self._check(self.lib.crane_embed_sinusoid(
            _dt(table.dtype), tokens.data_ptr(), positions.data_ptr(), table.data_ptr(), freq.data_ptr(),
            x.data_ptr(), _ptr(keep), n, hidden, table.shape[0], _ptr(deferred),
            deferred.numel() if deferred is not None else 0, err.data_ptr(), self._stream(x)), "embed_sinusoid")

    def stream_enter(self, x, kept, vec) -> None:
        """x += kept (float rows like x, or None) + vec (float [hidden])."""
        self._check(self.lib.crane_stream_enter(x.data_ptr(), _ptr(kept), vec.data_ptr(), x.shape[0], x.shape[1],
                                                self._stream(x)), "stream_enter")

    def add_normed_norm(self, x, delta: Act, w_delta, eps_delta: float, w_out=None, eps_out: float = 0.0,
                        out=None, raw=None) -> None:
        """x += delta / rms(delta) * w_delta; then, if given, out = x / rms(x) * w_out and
        raw = x in the model dtype.  rms(v) = sqrt(mean(v^2) + eps)."""
        whole, parts, n_parts, stride = _split(delta)
        dt = out.dtype if out is not None else raw.dtype if raw is not None else (
            delta.dtype if not isinstance(delta, Partials) else torch.bfloat16)
        self._check(self.lib.crane_add_normed_norm(
            _dt(dt), x.data_ptr(), whole, parts, n_parts, stride, w_delta.data_ptr(), _ptr(w_out), _ptr(out),
            _ptr(raw), x.shape[0], x.shape[1], float(eps_delta), float(eps_out), self._stream(x)), "add_normed_norm")

    def token_gate(self, z: Act, tokens, side, offset: int, out, err, deferred=None) -> None:
        """out[t] = gelu_tanh(z[t]) * side[token[t], offset : offset + dim]."""
        whole, parts, n_parts, stride = _split(z)
        n, dim = out.shape
        self._check(self.lib.crane_token_gate(
            _dt(out.dtype), whole, parts, n_parts, stride, tokens.data_ptr(), side.data_ptr(), side.shape[1],
            int(offset), dim, out.data_ptr(), n, side.shape[0], _ptr(deferred),
            deferred.numel() if deferred is not None else 0, err.data_ptr(), self._stream(out)), "token_gate")

    ACTIVATIONS = {"relu2": 0, "gelu": 1, "gelu_tanh": 2}
    mma_attention_takes_sink = True      # the warp-level attention kernels (prompt portions and decoded tokens) have the option

    def ffn_activation(self, up: Act, out, kind: str, route=None, per_expert: int = 0, routed_cols: int = 0) -> None:
        """out = act(up), times ``route[t, c // per_expert]`` (float [rows, experts]) for the leading
        ``routed_cols`` columns if routing weights are given."""
        whole, parts, n_parts, stride = _split(up)
        self._check(self.lib.crane_ffn_activation(
            _dt(out.dtype), whole, parts, n_parts, stride, out.data_ptr(), out.shape[0], out.shape[1],
            self.ACTIVATIONS[kind], _ptr(route), route.shape[1] if route is not None else 0, int(per_expert),
            int(routed_cols), self._stream(out)), "ffn_activation")

    def route_topk(self, logits, route, idx, wt) -> None:
        """Per row of float ``logits`` [n, experts]: the ``top`` (= idx.shape[1]) largest, softmax over
        them; ``route`` [n, experts] gets the weights (zero elsewhere), ``idx`` / ``wt`` the lists."""
        assert logits.dtype == torch.float32 and logits.is_contiguous()
        self._check(self.lib.crane_route_topk(logits.data_ptr(), route.data_ptr(), idx.data_ptr(), wt.data_ptr(),
                                              logits.shape[0], logits.shape[1], idx.shape[1],
                                              self._stream(logits)), "route_topk")

    def projection_norm_cache(self, qkv: Act, cols, positions, tok_entry, block_table, page_size, q_norm_w,
                              k_norm_w, eps, q_out, k_pool, v_pool, nq, nkv, d, dv, err, cos=None, sin=None,
                              rot_dims: int = 0, q_head_scale=None) -> None:
        """Rows [q | k | v] of a merged projection: q and k RMS-normed over all their heads at once
        (weights [nq d], [nkv d] or None), q written to ``q_out`` [n, nq, D], k and v into the
        token's place in the pools [pages, nkv, page_size, D / Dv], zero-filled where the pools'
        rows are wider than d / dv.  ``cos`` / ``sin`` float [positions, rot_dims / 2]: the leading
        ``rot_dims`` elements of every query and key head are rotated by the token's position, element
        i with i + rot_dims / 2; ``q_head_scale`` float [nq]: one factor per query head."""
        whole, parts, n_parts, stride = _split(qkv)
        self._check(self.lib.crane_projection_norm_cache(
            _dt(q_out.dtype), whole, parts, n_parts, stride, int(cols), positions.data_ptr(), tok_entry.data_ptr(),
            block_table.data_ptr(), block_table.shape[1], k_pool.shape[0], page_size, _ptr(q_norm_w),
            _ptr(k_norm_w), float(eps), q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), q_out.shape[0],
            nq, nkv, d, dv, k_pool.shape[3], v_pool.shape[3], _ptr(cos), _ptr(sin),
            cos.shape[0] if cos is not None else 0, int(rot_dims) if cos is not None else 0, _ptr(q_head_scale),
            err.data_ptr(), self._stream(q_out)), "projection_norm_cache")

    def delta_rule_max_dim(self) -> int:
        self.lib.crane_delta_rule_max_dim.restype = c_int
        return int(self.lib.crane_delta_rule_max_dim())

    def delta_rule_prep(self, proj: Act, cols, tok_entry, w2t, w0, ab, aux, heads, d, decay_scale, key_eps,
                        dtype) -> None:
        """aux [n, 3, heads d] (float) = decay, removal rate x unit key, unit key of every token, from
        rows [r | k | v | g | a | low (rank)] of the merged projection.  ``w2t`` [rank, heads d]: the
        decay's second matrix turned over."""
        whole, parts, n_parts, stride = _split(proj)
        self._check(self.lib.crane_delta_rule_prep(
            _dt(dtype), whole, parts, n_parts, stride, int(cols), tok_entry.data_ptr(), w2t.data_ptr(), w0.data_ptr(),
            ab.data_ptr(), aux.data_ptr(), aux.shape[0], heads, d, w2t.shape[0], float(decay_scale), float(key_eps),
            self._stream(aux)), "delta_rule_prep")

    def delta_rule_scan(self, proj: Act, cols, aux, cu_q, kv_len, slots, state, norm_w, norm_eps, out, heads, d,
                        err, col_blocks: int = 1, o_raw=None, tok_entry=None) -> None:
        """The recurrence over every entry's tokens, from and to ``state`` [slots, heads, d, d] (float;
        an entry whose tokens open its request starts from zero), with the head norm and the gate:
        ``out`` [n, heads d] in the model dtype.  ``col_blocks`` > 1 (with ``o_raw`` float [n, heads d]
        and ``tok_entry``): for few, long entries a head's columns are cut into that many blocks, a CTA
        each, and a second kernel norms and gates; the kernel falls back to one CTA a head where the
        head size does not allow it."""
        whole, parts, n_parts, stride = _split(proj)
        self._check(self.lib.crane_delta_rule_scan(
            _dt(out.dtype), whole, parts, n_parts, stride, int(cols), aux.data_ptr(), cu_q.data_ptr(),
            kv_len.data_ptr(), slots.data_ptr(), state.shape[0], state.data_ptr(), norm_w.data_ptr(),
            float(norm_eps), out.data_ptr(), _ptr(o_raw), _ptr(tok_entry), out.shape[0],
            int(col_blocks) if o_raw is not None and tok_entry is not None else 1, kv_len.shape[0], heads, d,
            err.data_ptr(), self._stream(out)), "delta_rule_scan")

    # ---- several residual streams, grouped routing, gated experts ----------
    def streams_norm(self, streams, x_first, y: Optional[Act], mix, outw, inw, g, eps: float, out, rows=None) -> None:
        """``streams`` float [R, n, hidden].  With ``y`` (a sublayer's result): x_t <- sum_s mix[s, t] x_s
        + outw[t] y for all t at once.  ``x_first`` float [n, hidden]: every stream starts as it (the
        embedding output) instead.  Then out = u / rms(u) * g[0] with u = sum_t inw[t] x_t (``inw`` None:
        the plain sum).  With ``rows`` only those rows are read and no stream is written."""
        whole, parts, n_parts, stride = (None, None, 0, 0) if y is None else _split(y)
        self._check(self.lib.crane_streams_norm(
            _dt(out.dtype), streams.data_ptr(), streams.stride(0), streams.shape[0], _ptr(x_first), whole, parts,
            n_parts, stride, _ptr(mix), _ptr(outw), _ptr(inw), g.data_ptr(), _ptr(rows), out.data_ptr(),
            out.shape[0], streams.shape[2], float(eps), self._stream(out)), "streams_norm")

    def route_grouped(self, z, correction, route, experts: int, top: int, groups: int, keep: int,
                      shared_gate: bool) -> None:
        """Per row of float ``z`` [n, >= experts (+ 1)]: scores = softmax over the experts; the ``top`` largest
        of score + correction among the experts of the ``keep`` best of ``groups`` groups are chosen;
        ``route`` [n, experts (+ 1)] gets their scores (zero elsewhere) and, ``shared_gate``, the
        sigmoid of column ``experts`` behind them."""
        assert z.dtype == torch.float32 and z.stride(1) == 1 and route.is_contiguous()
        self._check(self.lib.crane_route_grouped(
            z.data_ptr(), z.stride(0), _ptr(correction), route.data_ptr(), z.shape[0], int(experts), int(top),
            int(groups), int(keep), 1 if shared_gate else 0, self._stream(z)), "route_grouped")

    def gated_activation(self, gu: Act, out, route=None, experts: int = 0, per_expert: int = 0,
                         routed_cols: int = 0, shared_gate: bool = False) -> None:
        """out[t, c] = silu(gu[t, c]) * gu[t, cols + c], times the column's routing weight:
        ``route[t, c // per_expert]`` for c < routed_cols, behind them ``route[t, experts]``
        (``shared_gate``) or 1."""
        whole, parts, n_parts, stride = _split(gu)
        self._check(self.lib.crane_gated_activation(
            _dt(out.dtype), whole, parts, n_parts, stride, out.data_ptr(), out.shape[0], out.shape[1], _ptr(route),
            int(experts), int(per_expert), int(routed_cols), 1 if shared_gate else 0, self._stream(out)),
            "gated_activation")

    # ---- recurrences with a matrix state per head -----------------------
    def matrix_state_plan(self, dk: int):
        """(rows per lane, lanes per column) of the scan for keys of ``dk`` elements; the state of a head
        takes rows * lanes * dv floats.  (0, 0): wider than the kernel takes."""
        from ctypes import byref
        r, l = c_int(0), c_int(0)
        self.lib.crane_matrix_state_plan(int(dk), byref(r), byref(l))
        return r.value, l.value

    def conv_delta_prep(self, proj: Act, cols, ctx, state, conv_off, conv_w, taps, a_log, dt_bias, aux, H, G, d, dv,
                        key_eps, q_scale, err, dtype) -> None:
        """Rows [q | k | v | gate | b | a] of a merged projection -> ``aux`` rows [q | k | v | w | beta] in
        32-bit: q, k, v through their short convolutions (weights ``conv_w`` [channels, taps]) and silu,
        q and k to unit length per head (q times ``q_scale``), w = exp(-exp(a_log) softplus(a + dt_bias)),
        beta = sigmoid(b).  The convolutions' last taps - 1 inputs live in ``state`` [slots, floats] at
        ``conv_off`` and are replaced by a second kernel."""
        whole, parts, n_parts, stride = _split(proj)
        self._check(self.lib.crane_conv_delta_prep(
            _dt(dtype), whole, parts, n_parts, stride, int(cols), ctx.tok_entry.data_ptr(), ctx.cu_q.data_ptr(),
            ctx.kv_len.data_ptr(), ctx.slots.data_ptr(), state.shape[0], state.data_ptr(), state.stride(0),
            int(conv_off), conv_w.data_ptr(), int(taps), a_log.data_ptr(), dt_bias.data_ptr(), aux.data_ptr(),
            aux.shape[1], aux.shape[0], ctx.kv_len.shape[0], H, G, d, dv, float(key_eps), float(q_scale),
            err.data_ptr(), self._stream(aux)), "conv_delta_prep")

    def decay_gate_prep(self, proj: Act, cols, tok_entry, a2t, bias, inv_tau, q_scale, aux, H, d, dv, dtype) -> None:
        """Rows [q | k | v | gate | low] -> ``aux`` rows [q * q_scale | k | v | w] in 32-bit with
        w = sigmoid(low a2t + bias)^inv_tau per key channel."""
        whole, parts, n_parts, stride = _split(proj)
        self._check(self.lib.crane_decay_gate_prep(
            _dt(dtype), whole, parts, n_parts, stride, int(cols), tok_entry.data_ptr(), a2t.data_ptr(),
            bias.data_ptr(), a2t.shape[0], float(inv_tau), float(q_scale), aux.data_ptr(), aux.shape[1],
            aux.shape[0], H, d, dv, self._stream(aux)), "decay_gate_prep")

    def matrix_state_scan(self, aux, offs, w_vec: bool, delta: bool, qk_rep: int, ctx, state, o_raw, H, dk, dv,
                          err) -> None:
        """The recurrence S <- diag(w) S; u = beta (v - S^T k) (``delta``) or v; S <- S + k u^T; o = S^T q
        over every entry's tokens, from and to ``state`` [slots, floats] (its leading H * rows * lanes * dv
        floats).  ``offs``: columns of q, k, v, w, beta in ``aux``; ``o_raw`` float [n, H dv]."""
        self._check(self.lib.crane_matrix_state_scan(
            aux.data_ptr(), aux.shape[1], *[int(o) for o in offs], 1 if w_vec else 0, 1 if delta else 0, int(qk_rep),
            ctx.cu_q.data_ptr(), ctx.kv_len.data_ptr(), ctx.slots.data_ptr(), state.shape[0], state.data_ptr(),
            state.stride(0), o_raw.data_ptr(), ctx.kv_len.shape[0], H, dk, dv, err.data_ptr(),
            self._stream(o_raw)), "matrix_state_scan")

    def head_norm_gate(self, o_raw, proj: Act, cols, gate_off, tok_entry, norm_w, eps, out, H, dv) -> None:
        """out = o_raw / rms(o_raw per head) * norm_w * silu(gate columns of ``proj``)."""
        whole, parts, n_parts, stride = _split(proj)
        self._check(self.lib.crane_head_norm_gate(
            _dt(out.dtype), o_raw.data_ptr(), whole, parts, n_parts, stride, int(cols), int(gate_off),
            tok_entry.data_ptr(), norm_w.data_ptr(), float(eps), out.data_ptr(), out.shape[0], H, dv,
            self._stream(out)), "head_norm_gate")

    def head_talk_mix(self, cross, talk, tok_entry, out, H, G, dv, out_head) -> None:
        """out[t, h] = sum_g talk[h, g] cross[t, g, h // (H / G)]; heads ``out_head`` apart in ``out``."""
        self._check(self.lib.crane_head_talk_mix(
            _dt(out.dtype), cross.data_ptr(), talk.data_ptr(), tok_entry.data_ptr(), out.data_ptr(), out.shape[0],
            H, G, dv, int(out_head), self._stream(out)), "head_talk_mix")

    def pair_norm_mean(self, a: Act, b: Act, wa, wb, eps, out) -> None:
        """out = (a / rms(a) * wa + b / rms(b) * wb) / 2 per row."""
        aw, ap, an, astr = _split(a)
        bw, bp, bn, bstr = _split(b)
        self._check(self.lib.crane_pair_norm_mean(
            _dt(out.dtype), aw, ap, an, astr, bw, bp, bn, bstr, wa.data_ptr(), wb.data_ptr(), float(eps),
            out.data_ptr(), out.shape[0], out.shape[1], self._stream(out)), "pair_norm_mean")

    # ---- matrix product on the FP32 cores ------------------------------
    def gemm_simt(self, a, w, bias, out) -> None:
        """out[M,N] = a[M,K] @ w[N,K]^T (+ bias); rows may be strided."""
        M, K = a.shape
        N = w.shape[0]
        assert w.shape[1] == K and out.shape == (M, N)
        assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
        self._check(self.lib.crane_gemm_simt(_dt(a.dtype), _dt(out.dtype), a.data_ptr(),
                                             w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K,
                                             a.stride(0), w.stride(0), out.stride(0),
                                             self._stream(a)), "gemm_simt")

    # ---- matrix product on the tensor cores (bfloat16) -------------------
    @staticmethod
    def tcgen05_takes(x, w) -> bool:
        """Whether the tensor-core kernel takes these operands: bfloat16, inner
        dimension and row pitches multiples of 8 elements, 16-byte aligned."""
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    @staticmethod
    def split_plan(k: int, want: int):
        """(k-blocks of the shortest slice, slices) for a requested number of
        slices: at most one slice per 64-wide k-block."""
        num_kb = (k + 63) // 64
        slices = max(1, min(want, num_kb))
        return num_kb // slices, slices

    @staticmethod
    def slices_for(tiles: int, k: int, sms: int, max_waves: int = 3) -> int:
        """How many slices of the inner dimension make ``tiles`` output tiles fill
        the device's SMs best: the fewest slices among those whose last wave of
        CTAs is (nearly) as full as it gets."""
        num_kb = (k + 63) // 64
        best, best_eff = 1, 0.0
        for s in range(1, min(num_kb, max(1, (max_waves * sms) // max(1, tiles))) + 1):
            ctas = tiles * s
            eff = ctas / (-(-ctas // sms) * sms)
            if eff > best_eff + 0.02:
                best, best_eff = s, eff
        return best

    PAIR_TILES = (256, 224, 192, 128)

    def gemm_pair(self, x, w, bias, out, err, bn: int = 256, silu_mul: bool = False,
                  tile_rows: int = 256) -> None:
        """out[M,N] (bf16) = x[M,K] @ w[N,K]^T (+ bias) for many tokens, every
        256 x ``bn`` tile computed by two SMs together (tcgen05 cta_group::2).
        ``silu_mul`` as in ``gemm_tcgen05``.  ``tile_rows`` 512: tiles of 512
        tokens x ``bn`` (192, 224 or 256) features, two accumulators per SM."""
        M, K = x.shape
        N = w.shape[0]
        assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and bn in self.PAIR_TILES
        assert tuple(out.shape) == ((M, N // 2) if silu_mul else (M, N))
        self._check(self.lib.crane_gemm_bf16_pair(
            x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, x.stride(0), w.stride(0),
            out.stride(0), bn, tile_rows, 1 if silu_mul else 0, err.data_ptr(), self._stream(x)), "gemm_pair")

    WIDE_TILES = (256, 224, 192, 160, 128)

    @classmethod
    def tile_width_for(cls, m: int, n: int, sms: int) -> int:
        """The width of the 128 x width output tiles of a many-token product that
        takes the fewest rounds of tiles over the SMs, times the width (plus a
        little per tile); the widest among equals."""
        best, best_cost = 256, None
        for bn in cls.WIDE_TILES:
            tiles = -(-m // 128) * -(-n // bn)
            cost = -(-tiles // sms) * (bn + 16)
            if best_cost is None or cost < best_cost:
                best, best_cost = bn, cost
        return best

    TALL_TILES = (256, 192)

    @classmethod
    def tall_width_for(cls, m: int, n: int, sms: int) -> int:
        """The width of 256 x width tiles on one SM where they beat the 128-row
        tiles of ``tile_width_for``, else 0: a product whose 128-row tiles need a
        second, partly empty round over the SMs and whose 256-row tiles need one
        (measured at 2048 x 3072 x 2048: 27.9 -> 25.1 us in 256 x 192 tiles; the
        factor below is that measurement)."""
        if m <= 128:
            return 0
        bn1 = cls.tile_width_for(m, n, sms)
        best, best_cost = 0, -(-(-(-m // 128) * -(-n // bn1)) // sms) * (bn1 + 16)
        for bn in cls.TALL_TILES:
            tiles = -(-m // 256) * -(-n // bn)
            cost = -(-tiles // sms) * 2 * (bn + 16) * 0.92
            if cost < best_cost:
                best, best_cost = bn, cost
        return best

    PAIR_MIN_FLOPS = 4e10      # below this the pair kernel's set-up outweighs its better feeding

    @classmethod
    def pair_width_for(cls, m: int, n: int, k: int, sms: int) -> int:
        """The tile width for ``gemm_pair``, or 0 where the single-SM kernel is the
        better choice (small products, fewer than 256 rows)."""
        if m < 256 or 2.0 * m * n * k < cls.PAIR_MIN_FLOPS:
            return 0
        best, best_cost = 0, None
        for bn in cls.PAIR_TILES:
            tiles = -(-m // 256) * -(-n // bn)
            cost = -(-tiles // (sms // 2)) * (bn + 16)
            if best_cost is None or cost < best_cost:
                best, best_cost = bn, cost
        return best

    TALL_PAIR_TILES = (256, 224, 192)

    @classmethod
    def pair_plan(cls, m: int, n: int, k: int, sms: int, silu_mul: bool = False):
        """(tile width, tile rows) for ``gemm_pair``, (0, 0) where the single-SM
        kernel is the better choice.

        A model of the time of one round of tiles, in microseconds, fitted to
        measurements of 13 shapes (2048 .. 8192 tokens, inner dimensions 2048 ..
        14336): the operand bytes a CTA moves through its shared memory ((256 +
        width) x 128 bytes per 64-wide k-block for its 128 rows of a 256-row
        tile, (512 + width) x 128 for its 256 rows of a 512-row tile) cost 1.2e-5
        us each, and 128 rows x width x 16 are multiplied in width / 2 clocks;
        the two overlap, not perfectly (a 3-norm).  Tiles of 512 rows move the
        least bytes per product but have no second accumulator to work into while
        the epilogue reads the first, so their epilogue adds to every round: they
        win with a long inner dimension (2048 x 3072 x 8192: 86.6 -> 74.6 us,
        8192^3: 807 -> 740 us) and lose with a short one and with the silu
        epilogue.  Among near-equal costs the wider 256-row tile is taken (it
        runs a little better than the model says)."""
        if not cls.pair_width_for(m, n, k, sms):
            return 0, 0
        pairs = sms // 2

        def norm3(a, b):
            return (a ** 3 + b ** 3) ** (1.0 / 3.0)

        cands = []
        for bn in cls.PAIR_TILES:
            rounds = -(-(-(-m // 256) * -(-n // bn)) // pairs)
            cands.append((rounds * norm3((256 + bn) * k * 1.2e-5, k * bn / 56000.0), bn, 256))
        for bn in cls.TALL_PAIR_TILES:
            rounds = -(-(-(-m // 512) * -(-n // bn)) // pairs)
            epilogue = bn * (0.024 if silu_mul else 0.018)
            cands.append((rounds * (norm3((512 + bn) * k * 1.2e-5, k * bn / 28000.0) + epilogue), bn, 512))
        least = min(c[0] for c in cands)
        near = [c for c in cands if c[0] <= 1.03 * least]
        _, bn, rows = min(near, key=lambda c: (c[2], -c[1]))
        return bn, rows

    def gemm_tcgen05(self, x, w, bias, out, err, split_k: int = 1, swap: bool = False,
                     bn: int = 128, silu_mul: bool = False, prefetch=None, tile_rows: int = 128) -> None:
        """out[M,N] = x[M,K] @ w[N,K]^T (+ bias).  ``swap``: the weight fills the
        128-row side of the MMA and ``bn`` (16..64) covers the tokens.  With
        ``split_k`` > 1 ``out`` is float [slices, M, N] of partial sums.
        ``silu_mul``: w's rows come as 16 gate rows then the 16 up rows of the same
        features, and out[M, N/2] = silu(gate) * up.  ``prefetch``: (address,
        bytes) of what the step's next product will stream, asked into L2 by the
        narrow-tile kernel while it runs (a hint; ignored by the other kernels).
        ``tile_rows`` 256: tiles of 256 tokens x ``bn`` (128, 192 or 256) features
        (bf16 output, no slices, no swap, no silu)."""
        M, K = x.shape
        N = w.shape[0]
        if silu_mul:
            assert out.shape == (M, N // 2) and out.stride(1) == 1 and split_k == 1 and not swap
            ld, stride = out.stride(0), 0
        elif split_k > 1:
            assert out.dtype == torch.float32 and out.dim() == 3 and out.shape[1:] == (M, N)
            ld, stride = out.stride(1), out.stride(0)
        else:
            assert out.shape == (M, N) and out.stride(1) == 1
            ld, stride = out.stride(0), 0
        a, b = (w, x) if swap else (x, w)
        self._check(self.lib.crane_gemm_bf16_tcgen05(
            a.data_ptr(), b.data_ptr(), _ptr(bias), out.data_ptr(), a.shape[0], b.shape[0], K,
            a.stride(0), b.stride(0), ld, bn, tile_rows, 1 if out.dtype == torch.float32 else 0,
            1 if swap else 0, split_k, stride, 1 if silu_mul else 0,
            prefetch[0] if prefetch else None, prefetch[1] if prefetch else 0, err.data_ptr(),
            self._stream(x)), "gemm_tcgen05")

    # ---- attention ------------------------------------------------------
    def paged_attention_simt(self, q, out, k_pool, v_pool, positions, tok_entry, block_table,
                             page_size, nq, nkv, d, window, scale, err, dv=None, v_stride=None,
                             sink: bool = False, out_cross=None) -> None:
        """``dv``: width of a value row (default: the keys'), ``v_stride``: elements
        between value rows (default ``dv``).  With ``v_pool`` the key pool itself and
        ``v_stride == d`` the values are the leading ``dv`` columns of the key rows.
        ``sink``: the softmax has one more candidate of score 0 that has no value.
        ``out_cross`` float [n, nq, nkv, dv]: every query head's weights are applied to the values
        of EVERY key/value head (its scores still come from its own group's keys) and written there
        instead of ``out`` (which may be None), for attention whose heads exchange their weights."""
        dv = d if dv is None else int(dv)
        v_stride = dv if v_stride is None else int(v_stride)
        self._check(self.lib.crane_paged_attention_simt(
            _dt(q.dtype), q.data_ptr(), _ptr(out), k_pool.data_ptr(), v_pool.data_ptr(),
            positions.data_ptr(), tok_entry.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], k_pool.shape[0], page_size, q.shape[0], nq, nkv, d, dv, v_stride,
            int(window), float(scale), 1 if sink else 0, _ptr(out_cross), err.data_ptr(), self._stream(q)),
            "paged_attention_simt")

    # ---- attention whose scores are worked on, and the block around it
    @dataclass
    class ScoreMod:
        """What happens to a score before it becomes a weight, and to a head's weighted sums afterwards
        (the arguments of the warp-level kernels for worked-on scores)."""
        softcap: float = 0.0
        chunk: int = 0
        sigmoid: bool = False
        head_bias: Optional[torch.Tensor] = None     # float [heads]
        maps: int = 1
        lam: float = 0.0
        head_norm: bool = False
        norm_scale: float = 1.0
        eps: float = 0.0
        gate: Optional[torch.Tensor] = None          # float [rows, heads]
        dv: int = 0                                   # the real width of a value row (0: the stored one)
        compact: bool = False                         # out rows are [heads, dv] instead of [heads, stored]

    def scored_attention_supports(self, d: int, nq: int, nkv: int, maps: int = 1) -> bool:
        """Whether the warp-level kernels for worked-on scores take heads stored at ``d`` elements."""
        self.require_head_size(d)
        return bool(self.lib.crane_scored_attention_supports(int(d), int(nq), int(nkv), int(maps)))

    def _scored(self, decode, q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len, table, page_size, tiles, nq,
                nkv, d, window, scale, splits, skip_single, mod, err) -> None:
        self._check(self.lib.crane_scored_attention(
            1 if decode else 0, int(mod.maps), q.data_ptr(), out.data_ptr(), _ptr(part_o), _ptr(part_ml),
            k_pool.data_ptr(), v_pool.data_ptr(), cu_q.data_ptr(), kv_len.data_ptr(), table.data_ptr(),
            table.shape[1], k_pool.shape[0], page_size, kv_len.shape[0], int(tiles), nq, nkv, d, int(window),
            float(scale), int(splits), 1 if skip_single else 0, float(mod.softcap), int(mod.chunk),
            1 if mod.sigmoid else 0, _ptr(mod.head_bias), float(mod.lam), 1 if mod.head_norm else 0,
            float(mod.norm_scale), float(mod.eps), _ptr(mod.gate), int(mod.dv or d), 1 if mod.compact else 0,
            err.data_ptr(), self._stream(q)), "scored_attention")

    def scored_prefill_attention(self, q, out, k_pool, v_pool, cu_q, kv_len, table, page_size, tiles, nq, nkv, d,
                                 window, scale, mod, err, skip_single: bool = False) -> None:
        """bf16 attention with worked-on scores (``mod``) of q [rows, nq, d] over pools of head size d, for
        every entry of the step (``skip_single``: but those of exactly one token).  ``tiles``: the query
        tiles of 64 rows the entries have, or an upper bound."""
        self._scored(False, q, out, None, None, k_pool, v_pool, cu_q, kv_len, table, page_size, tiles, nq, nkv, d,
                     window, scale, 1, skip_single, mod, err)

    def scored_decode_attention(self, q, out, k_pool, v_pool, cu_q, kv_len, table, page_size, nq, nkv, d, window,
                                scale, splits, part_o, part_ml, mod, err) -> None:
        """The same for the entries of exactly one token, the keys in ``splits`` slices; ``part_o`` float
        [entries * nq * maps * splits, d] and ``part_ml`` [.., 2] hold the slices' sums for the merge."""
        self._scored(True, q, out, part_o, part_ml, k_pool, v_pool, cu_q, kv_len, table, page_size, 0, nq, nkv, d,
                     window, scale, splits, False, mod, err)

    def add_group_rmsnorm(self, x, a: Optional[Act], f: Optional[Act], weight, groups: int, eps: float, out,
                          rows=None) -> None:
        """x += (a + f) (either may be None), then RMS norm in ``groups`` equal consecutive parts of the
        row, times ``weight``.  With ``rows`` only those rows of x are read (and x is not written)."""
        aw, ap, an, as_ = (None, None, 0, 0) if a is None else _split(a)
        fw, fp, fn, fs = (None, None, 0, 0) if f is None else _split(f)
        self._check(self.lib.crane_add_group_rmsnorm(
            _dt(out.dtype), x.data_ptr(), aw, ap, an, as_, fw, fp, fn, fs, weight.data_ptr(), _ptr(rows),
            out.data_ptr(), out.shape[0], x.shape[1], int(groups), float(eps), self._stream(x)), "add_group_rmsnorm")

    def poly_norm(self, up: Act, coef, eps: float, out) -> None:
        """out = a N(z) + b N(z^2) + c N(z^3) + e per row z of ``up``; ``coef`` float [4] = (a, b, c, e)."""
        whole, parts, n_parts, stride = _split(up)
        self._check(self.lib.crane_poly_norm(_dt(out.dtype), whole, parts, n_parts, stride, coef.data_ptr(),
                                             out.data_ptr(), out.shape[0], out.shape[1], float(eps),
                                             self._stream(out)), "poly_norm")

    def scored_prep(self, proj: Act, cols, ctx, table, tails, conv_w, taps, page_size, q_norm_w, k_norm_w, eps, q_out,
                    k_pool, v_pool, H, G, maps, dim, dv, dpad, cos, sin, rot_dims, gate_out, gate_col, err) -> None:
        """Rows [q | k | v | gate] of a merged projection -> ``q_out`` [n, H, Dk], the token's rows in the
        pools [pages, G, page_size, Dk / Dv] (zero-filled where wider than the heads), ``gate_out`` float
        [n, H] = sigmoid(gate).  ``tails`` float [slots, taps - 1, channels] with ``conv_w`` [taps, channels]:
        a causal convolution over time on every channel first, the slot's last inputs replaced afterwards.
        A head holds ``maps`` maps of ``dim`` elements, map i stored at i * ``dpad``."""
        whole, parts, n_parts, stride = _split(proj)
        self._check(self.lib.crane_scored_prep(
            _dt(q_out.dtype), whole, parts, n_parts, stride, int(cols), ctx.positions.data_ptr(),
            ctx.tok_entry.data_ptr(), ctx.cu_q.data_ptr(), ctx.kv_len.data_ptr(), ctx.slots.data_ptr(),
            tails.shape[0] if tails is not None else 0, _ptr(tails), tails.stride(0) if tails is not None else 0,
            _ptr(conv_w), int(taps), table.data_ptr(), table.shape[1], k_pool.shape[0], page_size, _ptr(q_norm_w),
            _ptr(k_norm_w), float(eps), q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), q_out.shape[0],
            ctx.kv_len.shape[0], H, G, maps, dim, dv, k_pool.shape[3], dpad, v_pool.shape[3], _ptr(cos), _ptr(sin),
            cos.shape[0] if cos is not None else 0, int(rot_dims) if cos is not None else 0, _ptr(gate_out),
            int(gate_col), err.data_ptr(), self._stream(q_out)), "scored_prep")

    def head_finish(self, a, tok_entry, gate, out, H, maps, dv, lam, norm: bool, norm_scale, eps) -> None:
        """``a`` float [n, H, maps, dv_in] -> out [n, H, dv_out]: o = a1 - lam a2 for two maps, over the root of
        its mean square times ``norm_scale`` (``norm``), times ``gate`` float [n, H] (or None)."""
        n = out.shape[0]
        self._check(self.lib.crane_head_finish(
            _dt(out.dtype), a.data_ptr(), tok_entry.data_ptr(), _ptr(gate), out.data_ptr(), n, H, maps, dv,
            a.shape[1] // (H * maps), out.shape[1] // H, float(lam), 1 if norm else 0, float(norm_scale), float(eps),
            self._stream(out)), "head_finish")

    def scored_attention_simt(self, q, out, k_pool, v_pool, positions, tok_entry, block_table, page_size, nq, nkv, d,
                              dv, window, scale, err, softcap=0.0, chunk=0, sigmoid=False, head_bias=None, maps=1,
                              d_row=None, d_map=None, out_f32=None) -> None:
        """``paged_attention_simt`` with the scores worked on: squashed to softcap tanh(s / softcap), keys
        seen within the query's block of ``chunk`` positions only, weights sigmoid(s + head_bias[h]) without
        normalisation, ``maps`` maps of ``d`` elements per head (rows of ``d_row``, map i at i * ``d_map``),
        results in float [n, nq, maps, dv] (``out_f32``) or in ``out``."""
        d_row = int(d_row or maps * d)
        self._check(self.lib.crane_scored_attention_simt(
            _dt(q.dtype), q.data_ptr(), _ptr(out), k_pool.data_ptr(), v_pool.data_ptr(), positions.data_ptr(),
            tok_entry.data_ptr(), block_table.data_ptr(), block_table.shape[1], k_pool.shape[0], page_size,
            q.shape[0], nq, nkv, d, dv, v_pool.shape[3], int(window), float(scale), float(softcap), int(chunk),
            1 if sigmoid else 0, _ptr(head_bias), int(maps), d_row, int(d_map or d), _ptr(out_f32), err.data_ptr(),
            self._stream(q)), "scored_attention_simt")

    @staticmethod
    def decode_splits(entries: int, nkv: int, sms: int, cap: int = 64, max_keys: int = 1 << 30) -> int:
        """Key slices per (request, kv head) of the fused decode attention: enough CTAs to fill
        the device twice over (two fit on an SM), at most ``cap`` (the merge kernel takes 64);
        beyond that, the number of slices that fills the rounds over the SMs best.
        Measured in whole decode steps: 9 to 11 slices lose to 8, which merge themselves in a
        cluster without a second kernel; 33 to 40 lose to 32."""
        ctas, slots = max(1, entries * nkv), 2 * sms
        if ctas > slots:
            # More CTAs than fit at once.  The rounds over the SMs that are full run at the memory's
            # rate; a last round of few CTAs does not (about half the places have to be taken for
            # that), and it is as long as a full one.  Slices make the rounds shorter and the last one
            # fuller; they cost a little themselves (measured: 2 slices 2 %, 4 slices 7 %; 3, a
            # cluster of three, more).  The estimate below follows the measurements at a context of
            # 8,192 and 4 kv heads (ms per step with 1 / 2 / 4 slices): 80 requests 10.9 / 9.3 / 8.7,
            # 96 requests 11.1 / 9.7 / 10.1, 128 requests 12.2 / 12.2 / 13.0, 160 requests 16.7 / 15.6 /
            # 16.1, 192 requests 18.0 / - / 18.9.
            best, best_cost = 1, None
            for s, over in ((1, 1.0), (2, 1.02), (4, 1.07)):
                if s > cap:
                    break
                full, last = divmod(ctas * s, slots)
                cost = (full * slots + (max(last, slots // 2) if last else 0)) / s * over
                if best_cost is None or cost < best_cost:
                    best, best_cost = s, cost
            return best
        splits = max(1, min(cap, 64, slots // ctas))
        if splits > 8 and max_keys <= 2048:
            # few keys: 8 slices, which merge in their cluster, beat more slices and the merge kernel
            # (one request at a context of 256 / 1,024: 1.366 -> 1.284 / 1.380 -> 1.313 ms per step; four
            # requests: 1.440 -> 1.329 / 1.434 -> 1.387 ms; at 4,096 keys more slices win again)
            return 8
        while splits < 8 and splits & (splits - 1) and ctas * splits > 0.85 * slots:
            # 2 to 8 slices are a thread-block cluster, which has to find its places in one GPC: clusters
            # of 3 (5, 6, 7) that would take nearly every place do not all fit at once (24 requests of 4
            # kv heads at a context of 8,192: 288 CTAs in clusters of 3 4.74 ms per step, 192 in clusters
            # of 2 3.57 ms; 20 requests: 240 CTAs in clusters of 3 3.09 ms, 160 in clusters of 2 3.60 ms)
            splits -= 1
        if 8 < splits <= 11:
            return 8
        if 32 < splits <= 40:
            return 32
        return splits

    def decode_attention_supports(self, d: int, nq: int, nkv: int) -> bool:
        self.require_head_size(d)
        return bool(self.lib.crane_paged_decode_attention_supports(d, nq, nkv))

    def paged_decode_attention(self, q, out, k_pool, v_pool, cu_q, kv_len, block_table, page_size,
                               nq, nkv, d, window, scale, n_splits, part_o, part_ml, err, sink: bool = False,
                               cross: bool = False) -> None:
        """The entries of exactly one token (bfloat16); entries with more or no
        rows are skipped.  ``part_o`` [entries * nq * n_splits * d] and ``part_ml``
        [entries * nq * n_splits * 2] floats are scratch for n_splits > 1.  ``sink``: the
        softmax has one more candidate of score 0 that has no value.  ``cross``: ``out`` is float
        [n, nq, nkv, d], every query head's weights applied to the values of EVERY key/value head
        (for heads that exchange their weights); the scratch is always used and nkv times as large."""
        assert not cross or (out.dtype == torch.float32 and part_o is not None)
        n_entries = kv_len.shape[0]
        self.require_head_size(d)
        self._check(self.lib.crane_paged_decode_attention(
            q.data_ptr(), out.data_ptr(), _ptr(part_o), _ptr(part_ml), k_pool.data_ptr(),
            v_pool.data_ptr(), cu_q.data_ptr(), kv_len.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], k_pool.shape[0], page_size, n_entries, nq, nkv, d, int(window),
            float(scale), int(n_splits), 1 if sink else 0, 1 if cross else 0, err.data_ptr(), self._stream(q)),
            "paged_decode_attention")

    def prefill_attention_supports(self, d: int, nq: int, nkv: int) -> bool:
        self.require_head_size(d)
        return bool(self.lib.crane_paged_prefill_attention_supports(d, nq, nkv))

    def paged_prefill_attention(self, q, out, k_pool, v_pool, cu_q, kv_len, block_table, page_size,
                                total_q_tiles, nq, nkv, d, window, scale, err, skip_single=False,
                                sink: bool = False, cross: bool = False) -> None:
        """Any mix of portions and single tokens (bfloat16).  ``total_q_tiles``:
        the sum over the entries of ceil(tokens / 64), or more.  ``skip_single``:
        entries of exactly one token are left to the decode kernel.  ``sink`` and ``cross`` as in
        ``paged_decode_attention``."""
        assert not cross or out.dtype == torch.float32
        self.require_head_size(d)
        self._check(self.lib.crane_paged_prefill_attention(
            q.data_ptr(), out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), cu_q.data_ptr(),
            kv_len.data_ptr(), block_table.data_ptr(), block_table.shape[1], k_pool.shape[0],
            page_size, kv_len.shape[0], int(total_q_tiles), nq, nkv, d, int(window), float(scale),
            1 if skip_single else 0, 1 if sink else 0, out.data_ptr() if cross else None, err.data_ptr(),
            self._stream(q)), "paged_prefill_attention")

    def prefill_attention_tc_supports(self, d: int, nq: int, nkv: int, page_size: int) -> bool:
        return bool(self.lib.crane_prefill_attention_tc_supports(d, nq, nkv, page_size))

    def prefill_attention_tc(self, q, out, k_pool, v_pool, cu_q, kv_len, block_table, page_size,
                             total_q_tiles, nq, nkv, d, window, scale, err, skip_single=False) -> None:
        """Flash attention on tcgen05 (head size 128).  ``total_q_tiles``: the sum
        over the entries of ceil(tokens / 128), or more.  ``skip_single`` as in
        ``paged_prefill_attention``."""
        self._check(self.lib.crane_prefill_attention_tc(
            q.data_ptr(), out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), cu_q.data_ptr(),
            kv_len.data_ptr(), block_table.data_ptr(), block_table.shape[1], k_pool.shape[0],
            page_size, kv_len.shape[0], q.shape[0], int(total_q_tiles), nq, nkv, d, int(window),
            float(scale), 1 if skip_single else 0, err.data_ptr(), self._stream(q)), "prefill_attention_tc")

    def paged_decode_attention_fused(self, qkv: Act, qkv_cols, has_kv, cos, sin, q_norm_w, k_norm_w,
                                     eps, out, k_pool, v_pool, cu_q, kv_len, block_table, page_size,
                                     nq, nkv, d, window, scale, n_splits, part_o, part_ml, err,
                                     rope=None) -> None:
        """One token per entry, straight from the q/k/v product: rotary encoding,
        per-head norm, cache write and attention in one kernel, then the merge of
        the key slices.  ``rope`` as in ``rope_norm_cache``."""
        rd, inter, first, off = rope or (d, False, False, 0.0)
        whole, parts, n_parts, stride = _split(qkv)
        n_entries = kv_len.shape[0]
        self.require_head_size(d)
        self._check(self.lib.crane_paged_decode_attention_fused(
            whole, parts, n_parts, stride, qkv_cols, 1 if has_kv else 0, 1 if cos is not None else 0,
            _ptr(cos), _ptr(sin), cos.shape[0] if cos is not None else 0, _ptr(q_norm_w),
            _ptr(k_norm_w), float(eps), out.data_ptr(), _ptr(part_o), _ptr(part_ml),
            k_pool.data_ptr(), v_pool.data_ptr(), cu_q.data_ptr(), kv_len.data_ptr(),
            block_table.data_ptr(), block_table.shape[1], k_pool.shape[0], page_size, n_entries, nq,
            nkv, d, int(window), float(scale), int(n_splits), int(rd), 1 if inter else 0,
            1 if first else 0, float(off), err.data_ptr(), self._stream(out)),
            "paged_decode_attention_fused")

    # ---- sampling -------------------------------------------------------
    def repetition_penalty(self, logits, context, ctx_len, penalty) -> None:
        rows, vocab = logits.shape
        self._check(self.lib.crane_repetition_penalty(
            logits.data_ptr(), logits.stride(0), rows, vocab, context.data_ptr(), context.stride(0),
            ctx_len.data_ptr(), penalty.data_ptr(), self._stream(logits)), "repetition_penalty")

    def sample(self, logits, out, temperature=None, top_k=None, top_p=None, seed=None,
               counter=None) -> None:
        rows, vocab = logits.shape
        if temperature is not None and (seed is None or counter is None):
            raise KernelError("sampling with a temperature needs seed and counter per row")
        self._check(self.lib.crane_sample(
            logits.data_ptr(), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(top_k),
            _ptr(top_p), _ptr(seed), _ptr(counter), out.data_ptr(), self._stream(logits)), "sample")


_kernels: Optional[Kernels] = None


def get_kernels(head_sizes=()) -> Kernels:
    """The process's kernels.  ``head_sizes``: head sizes that will be needed (a
    model's), so that a library compiled at this first call holds them at once."""
    global _kernels
    if _kernels is None:
        _kernels = Kernels(head_sizes)
    else:
        for d in head_sizes:
            _kernels.require_head_size(d)
    return _kernels
