"""Token embedding and the output head.

x0 = E[token] without scaling (crane-core/src/models/hunyuan_dense/
modeling.rs:831-835, 998); logits = h W^T without bias, W the embedding table
when tied, else the top-level tensor ``lm_head.weight`` (modeling.rs:846-854).
Logits leave the head as float.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part, register_part


@register_part("embed", "token_embedding")
class TokenEmbedding(Part):
    """params: ``vocab_size``, ``hidden_size``, ``table`` (tensor name behind the prefix; default
    "weight").  Tensor [V,H]."""
    kind = "embed"

    @classmethod
    def manifest(cls, spec):
        return {spec.prefix + (spec.params.get("table") or "weight"): TensorSpec((spec.params["vocab_size"],
                                                                                  spec.params["hidden_size"]))}

    def load(self, weights, rt):
        self.table = weights[self.prefix + (self.params.get("table") or "weight")]

    def forward(self, tokens, x, rt, deferred=None):
        """Writes the float residual rows ``x`` [N,H] for int32 ``tokens`` [N].
        A token id <= -2 names row ``-id - 2`` of ``deferred`` (int32, on the
        device): a token sampled by an earlier launch that the host has not read."""
        rt.kernels.embed_gather(tokens, self.table, x, rt.err, deferred)
        rt.launches += 1


@register_part("head", "lm_head")
class LMHead(Part):
    """params: ``vocab_size``, ``hidden_size``, ``tied_to`` (name of the tensor
    it shares, or None), ``tensor`` (its own tensor's name behind the prefix; default
    "weight").  Tensor when untied [V,H]."""
    kind = "head"

    @classmethod
    def manifest(cls, spec):
        if spec.params.get("tied_to"):
            return {}
        return {spec.prefix + (spec.params.get("tensor") or "weight"): TensorSpec((spec.params["vocab_size"],
                                                                                   spec.params["hidden_size"]))}

    def load(self, weights, rt):
        tied = self.params.get("tied_to")
        self.weight = weights[tied] if tied else weights[self.prefix + (self.params.get("tensor") or "weight")]

    def forward(self, h, rt):
        # wanted rows are few when serving; the buffer grows if a caller wants more
        return rt.linear(h, self.weight, None, "logits", out_dtype=torch.float32, cap=64)


@register_part("embed", "bigram_embedding")
class BigramEmbedding(Part):
    """x0 = E[token] + B[(previous * mul_prev + token * mul_cur) mod buckets]; a sequence's
    first token takes B's last row (number ``buckets``).  params: ``vocab_size``,
    ``hidden_size``, ``table`` (tensor name), ``bigram``: None or ``{table, buckets, mul_prev,
    mul_cur}``.  Tensors: E [V,H], B [buckets + 1, H].

    The token before a portion's first one is the request's state: one int32 in the
    request's slot, kept by the cache manager like a mixer's state, read and replaced on
    the device by the embedding kernel (the token may be one that the host has not seen
    yet).  The kernel leaves rows of no entry and entries without rows alone, so steps
    padded for graph replay are safe."""
    kind = "embed"
    needs_context = True
    state_graph_safe = True

    @classmethod
    def manifest(cls, spec):
        a = spec.params
        m = {spec.prefix + a["table"]: TensorSpec((a["vocab_size"], a["hidden_size"]))}
        if a.get("bigram"):
            m[spec.prefix + a["bigram"]["table"]] = TensorSpec((a["bigram"]["buckets"] + 1, a["hidden_size"]))
        return m

    def load(self, weights, rt):
        a = self.params
        self.table = weights[self.prefix + a["table"]]
        bg = a.get("bigram")
        self.bigram = weights[self.prefix + bg["table"]] if bg else None
        self.buckets, self.mul_prev, self.mul_cur = ((int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))
                                                     if bg else (0, 0, 0))

    def cache_need(self):
        from .base import CacheNeed
        if self.bigram is None:
            return CacheNeed("none")
        return CacheNeed("state", state_shape=(1,), state_dtype=torch.int32)

    def forward(self, tokens, x, rt, deferred=None, ctx=None, cache=None):
        state = cache.state if cache is not None and cache.state is not None else None
        if self.bigram is None or state is None:
            rt.kernels.embed_gather(tokens, self.table, x, rt.err, deferred)
        else:
            rt.kernels.embed_bigram(tokens, self.table, self.bigram, x, self.buckets, self.mul_prev,
                                    self.mul_cur, ctx.positions, ctx.tok_entry, ctx.cu_q, ctx.slots, state,
                                    rt.err, deferred)
        rt.launches += 1


@register_part("embed", "sinusoid_embedding")
class SinusoidEmbedding(Part):
    """x0 = E[token] + s(position): column 2i of s is sin(p f_i), column 2i + 1 is cos(p f_i),
    f_i = base^(-2i / hidden).  params: ``vocab_size``, ``hidden_size``, ``table`` (tensor name),
    ``base`` (default 10000), ``keep_copy`` (the rows are also written to the workspace buffer
    "embedding_output", for a model that adds the embedding output again later).  Tensor E [V,H].
    The f_i are formed in 64-bit on the host and the angle p f_i in 64-bit on the device."""
    kind = "embed"
    needs_context = True          # it reads the tokens' positions
    KEPT = "embedding_output"

    @classmethod
    def manifest(cls, spec):
        a = spec.params
        return {spec.prefix + a.get("table", "weight"): TensorSpec((a["vocab_size"], a["hidden_size"]))}

    def load(self, weights, rt):
        a = self.params
        self.table = weights[self.prefix + a.get("table", "weight")]
        self.hidden = int(a["hidden_size"])
        base = float(a.get("base") or 10000.0)
        half = (self.hidden + 1) // 2
        self.freq = torch.tensor([base ** (-2.0 * i / self.hidden) for i in range(half)], dtype=torch.float64,
                                 device=rt.device)
        self.keep_copy = bool(a.get("keep_copy"))

    def forward(self, tokens, x, rt, deferred=None, ctx=None, cache=None):
        keep = rt.ws.get(self.KEPT, x.shape[0], self.hidden, torch.float32) if self.keep_copy else None
        rt.kernels.embed_sinusoid(tokens, ctx.positions, self.table, self.freq, x, keep, rt.err, deferred)
        rt.launches += 1
