"""Two mixers side by side on the same input: each result is RMS-normed over the model width with a
plain weight of its own, and the pair's result is half their sum.  Each keeps what it needs between
steps (pages for one, a state for the other): the pair's cache need is the two together.
"""
from __future__ import annotations

from ..weights.loader import TensorSpec
from .base import CacheNeed, Part, build_part, part_class, register_part


@register_part("mixer", "parallel_pair")
class ParallelPair(Part):
    """params: ``hidden_size``, ``eps``, ``left`` / ``right`` (PartSpecs of kind mixer), ``left_norm`` /
    ``right_norm`` (tensor names behind the prefix, [hidden], kept float)."""
    kind = "mixer"

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        m = {p + a["left_norm"]: TensorSpec((int(a["hidden_size"]),), "float32", "scale"),
             p + a["right_norm"]: TensorSpec((int(a["hidden_size"]),), "float32", "scale")}
        for side in ("left", "right"):
            m.update(part_class(a[side]).manifest(a[side]))
        return m

    def __init__(self, spec):
        super().__init__(spec)
        self.left, self.right = build_part(spec.params["left"]), build_part(spec.params["right"])

    @property
    def capturable(self):
        return getattr(self.left, "capturable", True) and getattr(self.right, "capturable", True)

    @property
    def state_graph_safe(self):
        keeps = [m for m in (self.left, self.right) if any(f.kind == "state" for f in m.cache_need().flat())]
        return all(getattr(m, "state_graph_safe", False) for m in keeps)

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        self.left.load(weights, rt)
        self.right.load(weights, rt)
        self.w_left, self.w_right = weights[p + a["left_norm"]], weights[p + a["right_norm"]]
        self.eps, self.size = float(a["eps"]), int(a["hidden_size"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed("multi", parts=(self.left.cache_need(), self.right.cache_need()))

    def forward(self, h, ctx, cache, rt):
        # the first result is read only after the second mixer's products have run
        a = self.left.forward(h, ctx, cache.parts[0], rt, hold=True)
        b = self.right.forward(h, ctx, cache.parts[1], rt)
        out = rt.ws.get("pair_out", h.shape[0], self.size, rt.dtype)
        rt.kernels.pair_norm_mean(a, b, self.w_left, self.w_right, self.eps, out)
        rt.launches += 1
        return out
