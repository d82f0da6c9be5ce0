"""Arrangements of parts in a layer.

``prenorm_residual``: h = norm1(x); x += mixer(h); h = norm2(x); x += ffn(h)
(crane-core/src/models/hunyuan_dense/modeling.rs:792-810).  Each addition is
fused into the norm that follows it, so a block hands its last output on
unadded ("pending") and receives the one of the block before it.

``sandwich_residual``: every sublayer's result is normed before it is added,
x += norm1b(mixer(norm1(x))); x += norm2b(ffn(norm2(x))); then an optional per-layer
token input joins the stream.

``parallel_depth_average``: both branches read norms of the same x, their sum
is added once, and what the next layer reads is a weighted sum of all layer
results so far.

``parallel_shared_norm``: ONE norm that both sublayers read, h = norm1(x);
x <- x + (mixer(h) + ffn(h)).

``hyper_connections``: R residual streams, all equal to the embedding output at the
start; a sublayer reads u = sum_s in[s] x_s through its norm, and its result y joins
all streams at once, x_t <- sum_s mix[s][t] x_s + out[t] y.  The model's last norm
reads the plain sum of the streams.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part, build_part, register_block, register_part
from .norm import BranchSum, StreamUpdate, add_normed, combine_and_norm


@register_block("prenorm_residual")
class PreNormResidualBlock:
    """parts: ``norm1``, ``mixer``, ``norm2``, ``ffn``."""

    def __init__(self, layer_spec):
        self.norm1 = build_part(layer_spec.parts["norm1"])
        self.mixer = build_part(layer_spec.parts["mixer"])
        self.norm2 = build_part(layer_spec.parts["norm2"])
        self.ffn = build_part(layer_spec.parts["ffn"])

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def forward(self, x, pending, ctx, cache, rt):
        h = self.norm1.forward(x, pending, rt)
        a = self.mixer.forward(h, ctx, cache, rt)
        h = self.norm2.forward(x, a, rt)
        return self.ffn.forward(h, ctx, rt)


@register_part("combine", "depth_average")
class DepthAverage(Part):
    """After layer ``index`` the stream is sum_j w[j] X_j over j = 0 .. index + 1, X_0 the
    embedding output and X_(j+1) the result of layer j (its input stream plus its branches).
    params: ``index``, ``slots`` (layers + 1), ``size``, ``weight`` (tensor name behind the
    prefix).  Tensor [index + 2], kept float.  The X_j of a step live in one float buffer
    [slots, rows, size] that all layers' parts share; the kernel that adds a block's
    branches writes X_(index+1) there and reads the others."""
    kind = "combine"

    @classmethod
    def manifest(cls, spec):
        return {spec.prefix + spec.params.get("weight", "weight"):
                TensorSpec((spec.params["index"] + 2,), "float32", "mix")}

    def load(self, weights, rt):
        self.weights = weights[self.prefix + self.params.get("weight", "weight")]
        self.index, self.slots, self.size = (int(self.params[k]) for k in ("index", "slots", "size"))

    def history(self, rt, rows: int):
        buf = rt.ws.get("layer_history", self.slots * rows, self.size, torch.float32,
                        cap=self.slots * rt.ws.max_rows)
        return buf.view(self.slots, rows, self.size)


@register_block("parallel_depth_average")
class ParallelDepthAverageBlock:
    """x <- x + (mixer(norm1(x)) + ffn(norm2(x))), both branches of the same x, then the
    depth-weighted average of ``combine``.  parts: ``norm1``, ``mixer``, ``combine`` and,
    unless the layer has no feed-forward, ``norm2`` and ``ffn``.  The additions, the
    average and the next reader's norms are one kernel (``norm.combine_and_norm``), so
    the block hands its branches on as a ``BranchSum``."""

    def __init__(self, layer_spec):
        p = layer_spec.parts
        self.norm1 = build_part(p["norm1"])
        self.mixer = build_part(p["mixer"])
        self.combine = build_part(p["combine"]) if "combine" in p else None
        self.ffn = build_part(p["ffn"]) if "ffn" in p else None
        self.norm2 = build_part(p["norm2"]) if self.ffn is not None else None
        self.norm1.history_of = self.combine

    def parts(self):
        return [q for q in (self.norm1, self.mixer, self.norm2, self.ffn, self.combine) if q is not None]

    def forward(self, x, pending, ctx, cache, rt):
        h1, h2 = combine_and_norm(x, pending, self.norm1, self.norm2, rt)
        a = self.mixer.forward(h1, ctx, cache, rt)
        f = self.ffn.forward(h2, ctx, rt) if self.ffn is not None else None
        return BranchSum(a, f, self.combine)


@register_block("parallel_shared_norm")
class ParallelSharedNormBlock:
    """h = norm1(x); x <- x + (mixer(h) + ffn(h)): the two sublayers read the same normed rows.  parts:
    ``norm1``, ``mixer`` and, unless the layer has no feed-forward, ``ffn``.  The block hands its two
    results on as a ``BranchSum``; the norm that reads the stream next adds them in its own kernel."""

    def __init__(self, layer_spec):
        p = layer_spec.parts
        self.norm1 = build_part(p["norm1"])
        self.mixer = build_part(p["mixer"])
        self.ffn = build_part(p["ffn"]) if "ffn" in p else None

    def parts(self):
        return [q for q in (self.norm1, self.mixer, self.ffn) if q is not None]

    def forward(self, x, pending, ctx, cache, rt):
        h = self.norm1.forward(x, pending, rt)
        # the mixer's result is read only after the feed-forward's products have run
        a = self.mixer.forward(h, ctx, cache, rt, hold=self.ffn is not None)
        f = self.ffn.forward(h, ctx, rt) if self.ffn is not None else None
        return BranchSum(a, f)


@register_part("entry", "pass_entry")
class PassEntry(Part):
    """What joins the stream where a pass over repeated layers begins: row ``row`` of a
    [times, size] tensor and, ``add_embedding``, the embedding output that the embedding part
    kept (workspace buffer "embedding_output").  params: ``size``, ``times``, ``tensor`` (name).
    The tensor is kept float: it is added to the float stream."""
    kind = "entry"

    @classmethod
    def manifest(cls, spec):
        a = spec.params
        return {spec.prefix + a["tensor"]: TensorSpec((a["times"], a["size"]), "float32", "offset")}

    def load(self, weights, rt):
        self.rows = weights[self.prefix + self.params["tensor"]]
        self.size = int(self.params["size"])

    def forward(self, x, pending, ctx, rt, row: int, add_embedding: bool = False):
        if pending is not None:
            raise ValueError("a pass begins behind a block that has not added its last result to the stream")
        kept = rt.ws.get("embedding_output", x.shape[0], self.size, torch.float32) if add_embedding else None
        rt.kernels.stream_enter(x, kept, self.rows[row])
        rt.launches += 1
        return None


@register_part("side", "token_side_input")
class TokenSideInput(Part):
    """A per-layer input from the token itself: e = table[token, offset : offset + dim];
    g = gelu_tanh(W_gate x) * e; y = W_proj g; x += y / rms(y) * w (a plain weight).
    params: ``hidden_size``, ``dim``, ``offset``, ``table_cols``, ``vocab_size``, ``eps``, ``table``
    (the table's full tensor name: all layers share it), tensors behind the prefix: ``gate``
    [dim, hidden], ``proj`` [hidden, dim], ``norm`` [hidden] (float)."""
    kind = "side"

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        return {a["table"]: TensorSpec((a["vocab_size"], a["table_cols"])),
                p + "gate": TensorSpec((a["dim"], a["hidden_size"])),
                p + "proj": TensorSpec((a["hidden_size"], a["dim"])),
                p + "norm": TensorSpec((a["hidden_size"],), "float32", "scale")}

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.table = weights[a["table"]]
        self.gate, self.proj, self.weight = weights[p + "gate"], weights[p + "proj"], weights[p + "norm"]
        self.dim, self.offset, self.eps, self.size = int(a["dim"]), int(a["offset"]), float(a["eps"]), int(a["hidden_size"])

    def forward(self, x, x_model, ctx, rt):
        """``x_model``: the stream in the model dtype (what the gate's product reads)."""
        z = rt.linear(x_model, self.gate, None, "side_gate")
        g = rt.ws.get("side_gated", x.shape[0], self.dim, rt.dtype)
        rt.kernels.token_gate(z, ctx.tokens, self.table, self.offset, g, rt.err, getattr(ctx, "deferred_tokens", None))
        rt.launches += 1
        y = rt.linear(g, self.proj, None, "side_out")
        add_normed(x, y, self, rt)


@register_block("sandwich_residual")
class SandwichResidualBlock:
    """parts: ``norm1``, ``mixer``, ``norm1b``; unless the layer has no feed-forward ``norm2``,
    ``ffn``, ``norm2b``; optionally ``side`` (a ``token_side_input``).  Each addition of a normed
    result is one kernel with the norm that reads the stream next.  The block leaves nothing
    pending: its last addition needs the result's own norm first."""

    def __init__(self, layer_spec):
        p = layer_spec.parts
        self.norm1, self.mixer, self.norm1b = (build_part(p[k]) for k in ("norm1", "mixer", "norm1b"))
        self.ffn = build_part(p["ffn"]) if "ffn" in p else None
        self.norm2 = build_part(p["norm2"]) if self.ffn is not None else None
        self.norm2b = build_part(p["norm2b"]) if self.ffn is not None else None
        self.side = build_part(p["side"]) if "side" in p else None

    def parts(self):
        return [q for q in (self.norm1, self.mixer, self.norm1b, self.norm2, self.ffn, self.norm2b, self.side)
                if q is not None]

    def forward(self, x, pending, ctx, cache, rt):
        h = self.norm1.forward(x, pending, rt)
        a = self.mixer.forward(h, ctx, cache, rt)
        raw_name = "stream_model" if self.side is not None else None
        if self.ffn is None:
            _, raw = add_normed(x, a, self.norm1b, rt, raw_name=raw_name)
        else:
            h2, _ = add_normed(x, a, self.norm1b, rt, then=self.norm2, name="normed2")
            f = self.ffn.forward(h2, ctx, rt)
            _, raw = add_normed(x, f, self.norm2b, rt, raw_name=raw_name)
        if self.side is not None:
            self.side.forward(x, raw, ctx, rt)
        return None


@register_part("connect", "stream_connection")
class StreamConnection(Part):
    """How one sublayer reads and writes ``streams`` residual streams: ``in`` [R] (what it reads),
    ``mix`` [R, R] indexed [from, to] and ``out`` [R] (how its result joins).  params: ``streams``,
    ``stored`` (False: one stream and the plain residual sum, in = mix = out = 1, no tensors),
    ``names``.  Tensors kept float."""
    kind = "connect"
    NAMES = {"in": "in", "mix": "mix", "out": "out"}

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        if not a.get("stored", True):
            return {}
        r = int(a["streams"])
        nm = dict(cls.NAMES, **(a.get("names") or {}))
        return {p + nm["in"]: TensorSpec((r,), "float32", "mix"), p + nm["out"]: TensorSpec((r,), "float32", "scale"),
                p + nm["mix"]: TensorSpec((r, r), "float32", "eye")}

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.streams = int(a["streams"])
        if not a.get("stored", True):
            if self.streams != 1:
                raise ValueError(f"{p}: {self.streams} streams need their tensors")
            one = torch.ones(1, dtype=torch.float32, device=rt.device)
            self.inw, self.mix, self.out = one, one.clone(), one.clone()
            return
        nm = dict(self.NAMES, **(a.get("names") or {}))
        self.inw, self.mix, self.out = weights[p + nm["in"]], weights[p + nm["mix"]], weights[p + nm["out"]]


@register_block("hyper_connections")
class HyperConnectionBlock:
    """parts: ``norm1`` (a ``scalar_rms_norm``), ``mixer``, ``connect1``; unless the layer has no
    feed-forward ``norm2``, ``ffn``, ``connect2``.  Every update of the streams is one kernel with the
    norm that reads them next, so the block hands its last result on as a ``StreamUpdate``."""

    def __init__(self, layer_spec):
        p = layer_spec.parts
        self.norm1, self.mixer, self.connect1 = (build_part(p[k]) for k in ("norm1", "mixer", "connect1"))
        self.ffn = build_part(p["ffn"]) if "ffn" in p else None
        self.norm2 = build_part(p["norm2"]) if self.ffn is not None else None
        self.connect2 = build_part(p["connect2"]) if self.ffn is not None else None

    def parts(self):
        return [q for q in (self.norm1, self.mixer, self.connect1, self.norm2, self.ffn, self.connect2)
                if q is not None]

    def forward(self, x, pending, ctx, cache, rt):
        h = self.norm1.forward(x, pending, rt, connect=self.connect1)
        a = self.mixer.forward(h, ctx, cache, rt)
        if self.ffn is None:
            return StreamUpdate(a, self.connect1)
        h2 = self.norm2.forward(x, StreamUpdate(a, self.connect1), rt, name="normed2", connect=self.connect2)
        return StreamUpdate(self.ffn.forward(h2, ctx, rt), self.connect2)
