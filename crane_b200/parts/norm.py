"""RMSNorm fused with the residual addition that precedes it.

y = x * rsqrt(mean(x^2) + eps) * w, weight applied after normalising, sums in
32-bit (crane-core/kernels/fused_ops.cu:45-51, 183-232; the reference's fused
add+norm kernel exists but is never launched, fused_ops/cuda_impl.rs:241-260).
"""
from __future__ import annotations

from ..weights.loader import TensorSpec
from .base import Part, register_part


@register_part("norm", "rms_norm")
class RMSNorm(Part):
    """params: ``size``, ``eps``; ``weight`` (tensor name behind the prefix, default "weight");
    ``weight_offset`` (the norm multiplies by offset + w: 0, or 1 for weights stored around
    zero; folded into the weight when it is loaded).  Tensor [size], kept float."""
    kind = "norm"

    @classmethod
    def manifest(cls, spec):
        offset = float(spec.params.get("weight_offset") or 0.0)
        return {spec.prefix + spec.params.get("weight", "weight"):
                TensorSpec((spec.params["size"],), "float32", "offset" if offset else "scale" if
                           "weight" in spec.params else "")}

    def load(self, weights, rt):
        self.weight = weights[self.prefix + self.params.get("weight", "weight")]
        offset = float(self.params.get("weight_offset") or 0.0)
        if offset:
            self.weight = (self.weight + offset).contiguous()
        self.eps = float(self.params["eps"])
        self.size = int(self.params["size"])

    def forward(self, x, delta, rt, rows=None, name="normed"):
        """``x`` [N, size] float residual, updated in place by ``delta``;
        returns the normalised rows in the model dtype.  ``rows`` (int32 index
        tensor): normalise only x[rows] + delta[rows] and leave x alone."""
        n = x.shape[0] if rows is None else rows.shape[0]
        out = rt.ws.get(name, n, self.size, rt.dtype)
        rt.kernels.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        rt.launches += 1
        return out


@register_part("norm", "group_rms_norm")
class GroupRMSNorm(Part):
    """RMS norm in groups: the row in ``groups`` equal consecutive parts, each over the root of its own
    mean square (+ eps), the whole times w.  What is pending is added to the float stream first, in the
    same kernel: a product's result, or the ``BranchSum`` of a block whose two sublayers read one norm
    (their results are added to one another, then to the stream).  params: ``size``, ``eps``, ``groups``
    (default 1), ``weight`` (tensor name behind the prefix, default "weight").  Tensor [size], kept float."""
    kind = "norm"

    @classmethod
    def manifest(cls, spec):
        return {spec.prefix + spec.params.get("weight", "weight"): TensorSpec((spec.params["size"],), "float32", "scale")}

    def load(self, weights, rt):
        self.weight = weights[self.prefix + self.params.get("weight", "weight")]
        self.eps, self.size = float(self.params["eps"]), int(self.params["size"])
        self.groups = int(self.params.get("groups") or 1)
        if self.size % self.groups:
            raise ValueError(f"{self.prefix}: {self.groups} groups do not divide a row of {self.size}")

    def forward(self, x, pending, rt, rows=None, name="normed"):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = rt.ws.get(name, n, self.size, rt.dtype)
        a, f = (pending.a, pending.f) if isinstance(pending, BranchSum) else (pending, None)
        if isinstance(pending, BranchSum) and pending.combine is not None:
            raise TypeError("group_rms_norm adds a block's two results as they are; it mixes no layer history")
        rt.kernels.add_group_rmsnorm(x, a, f, self.weight, self.groups, self.eps, out, rows)
        rt.launches += 1
        return out


def add_normed(x, delta, norm, rt, then=None, name="normed", raw_name=None):
    """x += norm(delta) (an ``rms_norm`` part applied to a sublayer's result before it joins the
    float stream) and, in the same kernel, ``then`` (another ``rms_norm`` part) of the new stream
    and/or the stream itself in the model dtype (``raw_name``).  Returns (normed, raw)."""
    n = x.shape[0]
    out = rt.ws.get(name, n, norm.size, rt.dtype) if then is not None else None
    raw = rt.ws.get(raw_name, n, norm.size, rt.dtype) if raw_name is not None else None
    rt.kernels.add_normed_norm(x, delta, norm.weight, norm.eps, then.weight if then is not None else None,
                               then.eps if then is not None else 0.0, out, raw)
    rt.launches += 1
    return out, raw


class BranchSum:
    """What a parallel block hands on instead of adding it: the outputs of its two
    branches (either may be None) and the part that mixes the sum into the stream
    (``combine``: a ``depth_average`` part, or None for a plain residual addition).
    The norm that reads the stream next does the additions in its own kernel."""

    def __init__(self, a, f, combine=None):
        self.a, self.f, self.combine = a, f, combine


def combine_and_norm(x, pending, norm_a, norm_b, rt, rows=None, names=("normed", "normed2")):
    """Adds what is pending to the float stream ``x`` (a ``BranchSum``, a plain
    product result or None), lets a ``BranchSum``'s ``combine`` part mix the
    new layer result with the earlier ones, and returns LayerNorm_a and
    (``norm_b`` given) LayerNorm_b of the new stream: one kernel.  ``rows``: only
    x[rows] is read and nothing of the stream is written."""
    n = x.shape[0] if rows is None else rows.shape[0]
    out_a = rt.ws.get(names[0], n, norm_a.size, rt.dtype)
    out_b = rt.ws.get(names[1], n, norm_b.size, rt.dtype) if norm_b is not None else None
    a = f = combine = None
    if isinstance(pending, BranchSum):
        a, f, combine = pending.a, pending.f, pending.combine
    else:
        a = pending
    hist, n_hist, dwa = None, 1, None
    if combine is not None:
        hist, n_hist, dwa = combine.history(rt, x.shape[0]), combine.index + 2, combine.weights
    elif norm_a.history_of is not None and pending is None:
        # the stream as the embedding leaves it is the first entry of the layers' history
        hist = norm_a.history_of.history(rt, x.shape[0])
    rt.kernels.combine_layernorm(x, hist, n_hist, a, f, dwa, rows, norm_a.weight, norm_a.bias, out_a,
                                 norm_b.weight if norm_b is not None else None,
                                 norm_b.bias if norm_b is not None else None, out_b, norm_a.eps)
    rt.launches += 1
    return out_a, out_b


@register_part("norm", "layer_norm")
class LayerNorm(Part):
    """y = (x - mean) / sqrt(var + eps) * w + b with var the mean of the squared deviations,
    all in 32-bit, fused with the additions that precede it.  params: ``size``, ``eps``,
    ``weight`` / ``bias`` (tensor names behind the prefix; default "weight" / "bias").
    Both tensors [size], kept float."""
    kind = "norm"
    history_of = None        # set by a block whose layer results are kept: its ``depth_average`` part

    @classmethod
    def _names(cls, spec):
        return (spec.prefix + spec.params.get("weight", "weight"), spec.prefix + spec.params.get("bias", "bias"))

    @classmethod
    def manifest(cls, spec):
        w, b = cls._names(spec)
        size = (spec.params["size"],)
        return {w: TensorSpec(size, "float32", "scale"), b: TensorSpec(size, "float32", "offset")}

    def load(self, weights, rt):
        w, b = self._names(self.spec)
        self.weight, self.bias = weights[w], weights[b]
        self.eps = float(self.params["eps"])
        self.size = int(self.params["size"])

    def forward(self, x, delta, rt, rows=None, name="normed"):
        """As ``RMSNorm.forward``; ``delta`` may also be a ``BranchSum``."""
        return combine_and_norm(x, delta, self, None, rt, rows, (name, name + "2"))[0]


class StreamUpdate:
    """What a block of several residual streams hands on instead of adding it: a sublayer's result
    ``y`` and the ``stream_connection`` part that says how it joins the streams.  The norm that
    reads the streams next does the update in its own kernel."""

    def __init__(self, y, connect):
        self.y, self.connect = y, connect


def residual_streams(rt, n: int, size: int, streams: int):
    """The step's residual streams, float [streams, n, size], in the workspace."""
    import torch
    buf = rt.ws.get("residual_streams", streams * n, size, torch.float32, cap=streams * rt.ws.max_rows)
    return buf.view(streams, n, size)


@register_part("norm", "scalar_rms_norm")
class ScalarRMSNorm(Part):
    """RMS norm with ONE learnt number for all coordinates, reading ``streams`` residual streams:
    u = sum_t in[t] x_t (``connect`` given: the reading sublayer's weights; else the plain sum),
    y = u / sqrt(mean(u^2) + eps) * g.  An update of the streams that is still pending (a
    ``StreamUpdate``) is applied first, in the same kernel.  params: ``size``, ``eps``, ``weight``
    (tensor name behind the prefix), ``streams``, ``gain`` (a constant folded into g: a model's
    logit scale, for its last norm).  Tensor [] (a single number), kept float."""
    kind = "norm"

    @classmethod
    def manifest(cls, spec):
        return {spec.prefix + spec.params.get("weight", "weight"): TensorSpec((), "float32", "scale")}

    def load(self, weights, rt):
        g = weights[self.prefix + self.params.get("weight", "weight")].reshape(1)
        self.g = (g * float(self.params.get("gain") or 1.0)).contiguous()
        self.eps = float(self.params["eps"])
        self.size = int(self.params["size"])
        self.streams = int(self.params.get("streams") or 1)

    def forward(self, x, pending, rt, rows=None, name="normed", connect=None):
        """``x`` [n, size]: the embedding output, which every stream starts as when nothing is pending
        and no layer has run (``pending`` None).  Returns the normed rows in the model dtype."""
        n = x.shape[0] if rows is None else rows.shape[0]
        out = rt.ws.get(name, n, self.size, rt.dtype)
        streams = residual_streams(rt, x.shape[0], self.size, self.streams)
        y = mix = outw = None
        if isinstance(pending, StreamUpdate):
            y, mix, outw = pending.y, pending.connect.mix, pending.connect.out
        elif pending is not None:
            raise TypeError("scalar_rms_norm reads residual streams; what is pending must be a StreamUpdate")
        rt.kernels.streams_norm(streams, x if pending is None else None, y, mix, outw,
                                connect.inw if connect is not None else None, self.g, self.eps, out, rows)
        rt.launches += 1
        return out
