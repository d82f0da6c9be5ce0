"""SiLU-gated feed-forward: down( silu(gate(h)) * up(h) ), no biases.

The gate and up matrices are merged into one [2I, H] product, as the reference
does (crane-core/src/models/hunyuan_dense/modeling.rs:667-694, 711-732);
silu(x) = x / (1 + exp(-x)) in 32-bit (crane-core/kernels/fused_ops.cu:39-42,
112-130).
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part, register_part


@register_part("ffn", "swiglu")
class SwiGLU(Part):
    """params: ``hidden_size``, ``intermediate_size``.  Tensors:
    ``<prefix>gate_proj.weight`` [I,H], ``up_proj.weight`` [I,H], ``down_proj.weight`` [H,I]."""
    kind = "ffn"

    @classmethod
    def manifest(cls, spec):
        h, i = spec.params["hidden_size"], spec.params["intermediate_size"]
        p = spec.prefix
        return {p + "gate_proj.weight": TensorSpec((i, h)), p + "up_proj.weight": TensorSpec((i, h)),
                p + "down_proj.weight": TensorSpec((h, i))}

    def load(self, weights, rt):
        p = self.prefix
        self.inter = int(self.params["intermediate_size"])
        gate, up = weights.pop(p + "gate_proj.weight"), weights.pop(p + "up_proj.weight")
        # On the tensor-core path the merged matrix holds 16 gate rows, then the 16 up rows of
        # the same features, and so on: a tile of the product then has both halves of a
        # feature side by side and its epilogue can apply silu(gate) * up itself.
        self.blocked = (not rt.exact) and self.inter % 16 == 0
        if self.blocked:
            h = gate.shape[1]
            self.gate_up = torch.stack([gate.view(-1, 16, h), up.view(-1, 16, h)], dim=1).reshape(
                2 * self.inter, h).contiguous()
        else:
            self.gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.down = weights[p + "down_proj.weight"]

    def forward(self, h, ctx, rt):
        act = rt.ws.get("ffn_act", h.shape[0], self.inter, rt.dtype)
        if self.blocked and rt.linear_silu_mul(h, self.gate_up, act):
            return rt.linear(act, self.down, None, "ffn_down")
        gu = rt.linear(h, self.gate_up, None, "ffn_gate_up")
        rt.kernels.silu_mul(gu, act, self.blocked)
        rt.launches += 1
        return rt.linear(act, self.down, None, "ffn_down")


@register_part("ffn", "xielu_mlp")
class XieluMlp(Part):
    """down(act(up(h))), no biases, act = xIELU with two learnt numbers (p, q):
    z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2, in 32-bit.
    params: ``hidden_size``, ``intermediate_size``.  Tensors: ``<prefix>up`` [I,H],
    ``<prefix>down`` [H,I], ``<prefix>act`` [2] (kept float)."""
    kind = "ffn"

    @classmethod
    def manifest(cls, spec):
        h, i = spec.params["hidden_size"], spec.params["intermediate_size"]
        p = spec.prefix
        return {p + "up": TensorSpec((i, h)), p + "down": TensorSpec((h, i)), p + "act": TensorSpec((2,), "float32", "unit")}

    def load(self, weights, rt):
        p = self.prefix
        self.inter = int(self.params["intermediate_size"])
        self.up, self.down, self.pq = weights[p + "up"], weights[p + "down"], weights[p + "act"]

    def forward(self, h, ctx, rt):
        up = rt.linear(h, self.up, None, "ffn_up")
        act = rt.ws.get("ffn_act", h.shape[0], self.inter, rt.dtype)
        rt.kernels.xielu(up, act, self.pq)
        rt.launches += 1
        return rt.linear(act, self.down, None, "ffn_down")


@register_part("ffn", "poly_norm_mlp")
class PolyNormMlp(Part):
    """down(act(up(h))), no biases, act = PolyNorm with four learnt numbers (a, b, c, e):
    a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N dividing a token's row by the root of
    its mean square (+ eps), in 32-bit.  params: ``hidden_size``, ``intermediate_size``, ``eps``, ``names``
    (up, down, act).  Tensors: up [I,H], down [H,I], act [4] (kept float)."""
    kind = "ffn"
    NAMES = {"up": "up", "down": "down", "act": "act"}

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        nm = dict(cls.NAMES, **(a.get("names") or {}))
        h, i = a["hidden_size"], a["intermediate_size"]
        return {p + nm["up"]: TensorSpec((i, h)), p + nm["down"]: TensorSpec((h, i)),
                p + nm["act"]: TensorSpec((4,), "float32", "unit")}

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        nm = dict(self.NAMES, **(a.get("names") or {}))
        self.inter, self.eps = int(a["intermediate_size"]), float(a["eps"])
        self.up, self.down, self.coef = weights[p + nm["up"]], weights[p + nm["down"]], weights[p + nm["act"]]

    def forward(self, h, ctx, rt):
        up = rt.linear(h, self.up, None, "ffn_up")
        act = rt.ws.get("ffn_act", h.shape[0], self.inter, rt.dtype)
        rt.kernels.poly_norm(up, self.coef, self.eps, act)
        rt.launches += 1
        return rt.linear(act, self.down, None, "ffn_down")


@register_part("ffn", "act_mlp")
class ActMlp(Part):
    """down(act(up(h))), no biases.  params: ``hidden_size``, ``intermediate_size``, ``act``
    ("relu2": the square of relu, "gelu": the erf form, "gelu_tanh"), ``names`` (up, down).
    Tensors: up [I,H], down [H,I]."""
    kind = "ffn"

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        nm = dict({"up": "up", "down": "down"}, **(a.get("names") or {}))
        h, i = a["hidden_size"], a["intermediate_size"]
        return {p + nm["up"]: TensorSpec((i, h)), p + nm["down"]: TensorSpec((h, i))}

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        nm = dict({"up": "up", "down": "down"}, **(a.get("names") or {}))
        self.inter, self.act = int(a["intermediate_size"]), str(a["act"])
        if self.act not in rt.kernels.ACTIVATIONS:
            raise ValueError(f"{p}: no activation '{self.act}'; there are: {', '.join(rt.kernels.ACTIVATIONS)}")
        self.up, self.down = weights[p + nm["up"]], weights[p + nm["down"]]

    def forward(self, h, ctx, rt):
        up = rt.linear(h, self.up, None, "ffn_up")
        act = rt.ws.get("ffn_act", h.shape[0], self.inter, rt.dtype)
        rt.kernels.ffn_activation(up, act, self.act)
        rt.launches += 1
        return rt.linear(act, self.down, None, "ffn_down")


@register_part("ffn", "routed_experts")
class RoutedExperts(Part):
    """A mixture of small feed-forwards down_e(act(up_e(h))): the router's logits z = W_r h are
    formed in 32-bit, the ``top`` largest choose a token's experts (ties to the lower index), and
    their weights are the softmax over the chosen logits alone.  An optional shared expert of the
    same form runs for every token and is added.
    params: ``hidden_size``, ``experts``, ``top``, ``expert_size``, ``shared_size`` (0: none), ``act``,
    ``names`` (router, expert: a pattern with {e}, shared, up, down).
    Tensors: router [E,H]; per expert up [F,H], down [H,F]; shared up [Fs,H], down [H,Fs].

    All experts' up matrices (and the shared one's) are one matrix, and so are the down matrices:
    a step is two products with the activation between them, which multiplies every expert's
    columns by the token's routing weight (zero for experts that it did not choose).  The result
    of a token does not depend on what else is in the batch."""
    kind = "ffn"
    NAMES = {"router": "router", "expert": "e{e}.", "shared": "shared.", "up": "up", "down": "down"}

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        nm = dict(cls.NAMES, **(a.get("names") or {}))
        h, E, F, Fs = int(a["hidden_size"]), int(a["experts"]), int(a["expert_size"]), int(a.get("shared_size") or 0)
        m = {p + nm["router"]: TensorSpec((E, h))}
        for e in range(E):
            q = p + nm["expert"].format(e=e)
            m[q + nm["up"]] = TensorSpec((F, h))
            m[q + nm["down"]] = TensorSpec((h, F))
        if Fs:
            m[p + nm["shared"] + nm["up"]] = TensorSpec((Fs, h))
            m[p + nm["shared"] + nm["down"]] = TensorSpec((h, Fs))
        return m

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        nm = dict(self.NAMES, **(a.get("names") or {}))
        self.E, self.top, self.F = int(a["experts"]), int(a["top"]), int(a["expert_size"])
        self.Fs, self.act = int(a.get("shared_size") or 0), str(a["act"])
        if not 0 < self.top <= self.E:
            raise ValueError(f"{p}: {self.top} of {self.E} experts cannot be chosen")
        if self.act not in rt.kernels.ACTIVATIONS:
            raise ValueError(f"{p}: no activation '{self.act}'; there are: {', '.join(rt.kernels.ACTIVATIONS)}")
        self.router = weights[p + nm["router"]]
        ups = [weights.pop(p + nm["expert"].format(e=e) + nm["up"]) for e in range(self.E)]
        downs = [weights.pop(p + nm["expert"].format(e=e) + nm["down"]) for e in range(self.E)]
        if self.Fs:
            ups.append(weights.pop(p + nm["shared"] + nm["up"]))
            downs.append(weights.pop(p + nm["shared"] + nm["down"]))
        self.up = torch.cat(ups, dim=0).contiguous()                 # [E F + Fs, H]
        self.down = torch.cat(downs, dim=1).contiguous()             # [H, E F + Fs]
        self.inter = self.up.shape[0]

    def forward(self, h, ctx, rt):
        n = h.shape[0]
        k = rt.kernels
        logits = rt.linear(h, self.router, None, "router_logits", out_dtype=torch.float32)
        route = rt.ws.get("route_weights", n, self.E, torch.float32)
        idx = rt.ws.get("route_idx", n, self.top, torch.int32)
        wt = rt.ws.get("route_wt", n, self.top, torch.float32)
        k.route_topk(logits, route, idx, wt)
        up = rt.linear(h, self.up, None, "experts_up")
        act = rt.ws.get("experts_act", n, self.inter, rt.dtype)
        k.ffn_activation(up, act, self.act, route, self.F, self.E * self.F)
        rt.launches += 2
        return rt.linear(act, self.down, None, "experts_down")


@register_part("ffn", "grouped_experts")
class GroupedExperts(Part):
    """A mixture of gated feed-forwards down_e(silu(gate_e(h)) * up_e(h)).  The router's logits
    z = W_r h are formed in 32-bit; scores s = softmax(z) over ALL experts; an expert's choice score
    is s plus a learnt correction; experts come in ``groups`` equal groups of neighbours, a group
    counts as much as its best choice score, and only experts of the ``keep`` best groups can be
    chosen; the ``top`` largest choice scores among those are chosen (ties to the lower index) and
    weighted by their scores s, without the correction and without renormalising.  An optional shared
    expert of the same form runs for every token and is added, times sigmoid(w_sg . h) if it has a gate.
    params: ``hidden_size``, ``experts``, ``top``, ``groups``, ``keep``, ``expert_size``, ``shared_size``
    (0: none), ``correction`` (tensor name or None), ``shared_gate`` (tensor name or None), ``names``.
    Tensors: router [E,H]; correction [E] (float); per expert gate, up [F,H], down [H,F]; shared gate,
    up [Fs,H], down [H,Fs]; shared_gate [1,H].

    All experts' gate matrices (and the shared one's), then all up matrices, are ONE matrix, and so are
    the down matrices: a step is two products with the activation between them, which multiplies
    every expert's columns by the token's routing weight (zero for experts that it did not choose).
    The router's matrix carries the shared gate's row behind the experts'.  The result of a token does
    not depend on what else is in the batch."""
    kind = "ffn"
    NAMES = {"router": "router", "expert": "e{e}.", "shared": "shared.", "gate": "gate", "up": "up", "down": "down"}

    @classmethod
    def _sizes(cls, a):
        return (int(a["hidden_size"]), int(a["experts"]), int(a["expert_size"]), int(a.get("shared_size") or 0))

    @classmethod
    def manifest(cls, spec):
        a, p = spec.params, spec.prefix
        nm = dict(cls.NAMES, **(a.get("names") or {}))
        h, E, F, Fs = cls._sizes(a)
        m = {p + nm["router"]: TensorSpec((E, h))}
        if a.get("correction"):
            m[p + a["correction"]] = TensorSpec((E,), "float32", "offset")
        for e in range(E):
            q = p + nm["expert"].format(e=e)
            m[q + nm["gate"]] = TensorSpec((F, h))
            m[q + nm["up"]] = TensorSpec((F, h))
            m[q + nm["down"]] = TensorSpec((h, F))
        if Fs:
            q = p + nm["shared"]
            m[q + nm["gate"]] = TensorSpec((Fs, h))
            m[q + nm["up"]] = TensorSpec((Fs, h))
            m[q + nm["down"]] = TensorSpec((h, Fs))
            if a.get("shared_gate"):
                m[p + a["shared_gate"]] = TensorSpec((1, h))
        return m

    def load(self, weights, rt):
        a, p = self.params, self.prefix
        nm = dict(self.NAMES, **(a.get("names") or {}))
        _, self.E, self.F, self.Fs = self._sizes(a)
        self.top, self.groups = int(a["top"]), int(a.get("groups") or 1)
        self.keep = int(a.get("keep") or self.groups)
        if not 0 < self.top <= self.E or self.E % self.groups or not 0 < self.keep <= self.groups:
            raise ValueError(f"{p}: {self.top} of {self.E} experts in {self.groups} groups ({self.keep} kept) cannot be chosen")
        self.correction = weights[p + a["correction"]] if a.get("correction") else None
        self.shared_gate = bool(self.Fs and a.get("shared_gate"))
        router = [weights.pop(p + nm["router"])]
        if self.shared_gate:
            router.append(weights.pop(p + a["shared_gate"]).reshape(1, -1))
        self.router = torch.cat(router, dim=0).contiguous()           # [E (+ 1), H]
        names = [p + nm["expert"].format(e=e) for e in range(self.E)] + ([p + nm["shared"]] if self.Fs else [])
        gates = [weights.pop(q + nm["gate"]) for q in names]
        ups = [weights.pop(q + nm["up"]) for q in names]
        downs = [weights.pop(q + nm["down"]) for q in names]
        self.gate_up = torch.cat(gates + ups, dim=0).contiguous()      # [2 (E F + Fs), H]: gates, then ups
        self.down = torch.cat(downs, dim=1).contiguous()               # [H, E F + Fs]
        self.inter = self.down.shape[1]

    def forward(self, h, ctx, rt):
        n, k = h.shape[0], rt.kernels
        z = rt.linear(h, self.router, None, "router_logits", out_dtype=torch.float32)
        route = rt.ws.get("route_weights", n, self.E + (1 if self.shared_gate else 0), torch.float32)
        k.route_grouped(z, self.correction, route, self.E, self.top, self.groups, self.keep, self.shared_gate)
        gu = rt.linear(h, self.gate_up, None, "experts_gate_up")
        act = rt.ws.get("experts_act", n, self.inter, rt.dtype)
        k.gated_activation(gu, act, route, self.E, self.F, self.E * self.F, self.shared_gate)
        rt.launches += 2
        return rt.linear(act, self.down, None, "experts_down")
