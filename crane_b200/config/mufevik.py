"""Typed configuration of Mufevik, read from the keys of its config.json.

A Mufevik model keeps several residual streams (hyper-connections): every sublayer reads a
weighted sum of the streams through an RMS norm with a single gain, and its result joins all
streams at once through a small mixing matrix.  Two mixers: ``parallel`` (attention whose
heads exchange their softmax weights, with rotary positions on part of each head and a
temperature per head, beside gated linear attention with a decay per key channel; both
results normed over the width and averaged) and ``delta`` (the gated delta rule behind short
causal convolutions).  The feed-forward is a mixture of gated experts whose router chooses
within the best groups of experts, plus a shared expert behind a sigmoid gate.  The logits
are scaled by a constant.

config.json: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``streams`` (optional: absent
means the plain residual sum), ``logit_scale`` (optional) and ``layers``, a list of ``{"type",
"mixer": {...}, "mlp": {...} | null}``.  Every size and constant that a model states is read
from there; the decay's inner size is read from the stored tensors.  The design has no
position limit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .hunyuan_dense import ConfigError

ARCHITECTURE = "Mufevik"
ALIASES = ("mufevik",)
# the design has no limit on positions; the engine's own (``EngineConfig.max_seq_len``) is capped here
MAX_POSITIONS = 1 << 17
# the constant that the design fixes: what is added under the root where q and k become unit vectors
UNIT_KEY_EPS = 1e-6
MAX_STREAMS = 8
# head sizes that the warp-level attention kernels are compiled for
ATTENTION_HEAD_SIZES = (16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 256)


@dataclass(frozen=True)
class TalkingConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class LinearConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: Optional[int] = None      # only random weights need it; a stored model's tensors say it


@dataclass(frozen=True)
class ParallelConfig:
    left: TalkingConfig
    right: LinearConfig


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    groups: int
    keep: int
    expert_ff: int
    shared_ff: int


@dataclass(frozen=True)
class MufevikLayer:
    type: str
    mixer: Any
    mlp: Optional[MoeConfig]


@dataclass(frozen=True)
class MufevikConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[MufevikLayer, ...]
    streams: Optional[int] = None         # None: one stream and the plain residual sum (no tensors for it)
    logit_scale: float = 1.0
    eos_token_id: Optional[Tuple[int, ...]] = None

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "MufevikConfig":
        def need(obj, key, where):
            if not isinstance(obj, dict) or obj.get(key) is None:
                raise ConfigError(f"config.json lacks '{key}' in {where}")
            return obj[key]

        layers: List[MufevikLayer] = []
        for i, ld in enumerate(need(d, "layers", "the top level")):
            where = f"layers[{i}]"
            kind = str(need(ld, "type", where))
            m = need(ld, "mixer", where)
            if kind == "parallel":
                lt, rt = need(m, "left", where + ".mixer"), need(m, "right", where + ".mixer")
                heads, dim = int(need(lt, "heads", where + ".mixer.left")), int(need(lt, "dim", where + ".mixer.left"))
                rot = lt.get("rot") or {}
                left = TalkingConfig(heads=heads, kv_heads=int(lt.get("kv_heads") or heads), dim=dim,
                                     vdim=int(lt.get("vdim") or dim),
                                     scale=float(lt["scale"]) if lt.get("scale") is not None else dim ** -0.5,
                                     rot_dims=int(rot.get("dims") or 0), rot_base=float(rot.get("base") or 10000.0))
                rdim = int(need(rt, "dim", where + ".mixer.right"))
                rank = rt.get("decay_rank")
                right = LinearConfig(heads=int(need(rt, "heads", where + ".mixer.right")), dim=rdim,
                                     vdim=int(rt.get("vdim") or rdim), tau=float(need(rt, "tau", where + ".mixer.right")),
                                     decay_rank=None if rank is None else int(rank))
                mixer: Any = ParallelConfig(left, right)
            elif kind == "delta":
                heads, dim = int(need(m, "heads", where + ".mixer")), int(need(m, "dim", where + ".mixer"))
                mixer = DeltaConfig(heads=heads, kv_heads=int(m.get("kv_heads") or heads), dim=dim,
                                    vdim=int(m.get("vdim") or dim), conv=int(need(m, "conv", where + ".mixer")))
            else:
                raise ConfigError(f"{where}: no mixer '{kind}'; this design has: parallel, delta")
            md = ld.get("mlp")
            mlp = None
            if md is not None:
                mk = str(md.get("kind") or "moe")
                if mk != "moe":
                    raise ConfigError(f"{where}.mlp: no feed-forward kind '{mk}'; this design has: moe")
                router = need(md, "router", where + ".mlp")
                groups = router.get("groups") or {}
                shared = md.get("shared")
                count = int(groups.get("count") or 1)
                mlp = MoeConfig(experts=int(need(router, "experts", where + ".mlp.router")),
                                top=int(need(router, "top", where + ".mlp.router")), groups=count,
                                keep=int(groups.get("keep") or count),
                                expert_ff=int(need(need(md, "expert", where + ".mlp"), "ff", where + ".mlp.expert")),
                                shared_ff=int(need(shared, "ff", where + ".mlp.shared")) if shared else 0)
            layers.append(MufevikLayer(kind, mixer, mlp))
        eos = d.get("eos_token_id")
        eos = (int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos) if eos else None
        cfg = MufevikConfig(vocab=int(need(d, "vocab", "the top level")), width=int(need(d, "width", "the top level")),
                            eps=float(need(need(d, "norm", "the top level"), "eps", "norm")), layers=tuple(layers),
                            streams=int(d["streams"]) if d.get("streams") is not None else None,
                            logit_scale=float(d["logit_scale"]) if d.get("logit_scale") is not None else 1.0,
                            eos_token_id=eos)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be > 0, got {self.eps}")
        if self.streams is not None and not 1 <= self.streams <= MAX_STREAMS:
            raise ConfigError(f"streams must be 1 .. {MAX_STREAMS}, got {self.streams}")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if isinstance(m, ParallelConfig):
                lt, rt = m.left, m.right
                if lt.heads <= 0 or lt.kv_heads <= 0 or lt.heads % lt.kv_heads or lt.dim <= 0 or lt.vdim <= 0:
                    raise ConfigError(f"layers[{i}].mixer.left: heads must be a positive multiple of kv_heads, "
                                      "dim and vdim positive")
                if lt.rot_dims < 0 or lt.rot_dims % 2 or lt.rot_dims > lt.dim:
                    raise ConfigError(f"layers[{i}].mixer.left.rot.dims must be even and at most dim")
                if rt.heads <= 0 or rt.dim <= 0 or rt.vdim <= 0 or not rt.tau > 0:
                    raise ConfigError(f"layers[{i}].mixer.right: heads, dim, vdim and tau must be positive")
            else:
                if m.heads <= 0 or m.kv_heads <= 0 or m.heads % m.kv_heads or m.dim <= 0 or m.vdim <= 0:
                    raise ConfigError(f"layers[{i}].mixer: heads must be a positive multiple of kv_heads, "
                                      "dim and vdim positive")
                if not 1 <= m.conv <= 16:
                    raise ConfigError(f"layers[{i}].mixer.conv must be 1 .. 16 taps")
            mlp = layer.mlp
            if mlp is not None:
                if not (0 < mlp.top <= mlp.experts and mlp.expert_ff > 0):
                    raise ConfigError(f"layers[{i}].mlp: 0 < router.top <= router.experts and expert.ff > 0 are needed")
                if mlp.groups <= 0 or mlp.experts % mlp.groups or not 0 < mlp.keep <= mlp.groups:
                    raise ConfigError(f"layers[{i}].mlp.router.groups: experts must split into count equal groups, "
                                      "0 < keep <= count")
                if mlp.top > mlp.keep * (mlp.experts // mlp.groups):
                    raise ConfigError(f"layers[{i}].mlp.router: the kept groups hold fewer experts than top")


def _common_head_size(dim: int, vdim: int) -> int:
    fit = [s for s in ATTENTION_HEAD_SIZES if s >= max(dim, vdim)]
    return fit[0] if fit else 0


def _parallel_spec(cfg: MufevikConfig, m: ParallelConfig, prefix: str):
    from .spec import PartSpec
    lt, rt = m.left, m.right
    position = None
    if lt.rot_dims:
        position = PartSpec("position", "yarn_rope", {"dims": lt.rot_dims, "base": lt.rot_base, "scaling": None,
                                                      "max_positions": MAX_POSITIONS})
    left = PartSpec("mixer", "talking_attention", {
        "hidden_size": cfg.width, "heads": lt.heads, "kv_heads": lt.kv_heads, "dim": lt.dim, "vdim": lt.vdim,
        "scale": lt.scale, "rotary_dim": lt.rot_dims, "position": position,
        # the head size that keys and values are stored at on the bfloat16 path (0: as wide as they are)
        "head_dim": _common_head_size(lt.dim, lt.vdim)}, prefix=prefix + "left.")
    right = PartSpec("mixer", "gated_linear_attention", {
        "hidden_size": cfg.width, "heads": rt.heads, "dim": rt.dim, "vdim": rt.vdim, "tau": rt.tau,
        "norm_eps": cfg.eps, "decay_rank": rt.decay_rank}, prefix=prefix + "right.")
    return PartSpec("mixer", "parallel_pair", {
        "hidden_size": cfg.width, "eps": cfg.eps, "left": left, "right": right,
        "left_norm": "left.out", "right_norm": "right.out", "head_dim": left.params["head_dim"]}, prefix=prefix)


def _delta_spec(cfg: MufevikConfig, m: DeltaConfig, prefix: str):
    from .spec import PartSpec
    return PartSpec("mixer", "gated_delta", {
        "hidden_size": cfg.width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
        "conv": m.conv, "norm_eps": cfg.eps, "key_eps": UNIT_KEY_EPS}, prefix=prefix)


def _ffn_spec(cfg: MufevikConfig, mlp: MoeConfig, prefix: str):
    from .spec import PartSpec
    return PartSpec("ffn", "grouped_experts", {
        "hidden_size": cfg.width, "experts": mlp.experts, "top": mlp.top, "groups": mlp.groups, "keep": mlp.keep,
        "expert_size": mlp.expert_ff, "shared_size": mlp.shared_ff, "correction": "correction",
        "shared_gate": "shared.sg" if mlp.shared_ff else None}, prefix=prefix)


def build_spec(cfg: MufevikConfig):
    """Mufevik as data: per layer a block that reads and writes the residual streams around mixer and
    feed-forward; the final norm reads the sum of the streams, its gain carries the logit scale."""
    from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep

    streams = cfg.streams or 1
    layers, ignored = [], {}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norm = lambda name: PartSpec("norm", "scalar_rms_norm", {"size": cfg.width, "eps": cfg.eps, "weight": name,
                                                                 "streams": streams}, prefix=p)
        connect = lambda name: PartSpec("connect", "stream_connection", {
            "streams": streams, "stored": cfg.streams is not None}, prefix=p + name + ".")
        mixer = (_parallel_spec if layer.type == "parallel" else _delta_spec)(cfg, layer.mixer, p + "mix.")
        parts = {"norm1": norm("norm1"), "mixer": mixer, "connect1": connect("hc1")}
        if layer.mlp is not None:
            parts.update(norm2=norm("norm2"), ffn=_ffn_spec(cfg, layer.mlp, p + "mlp."), connect2=connect("hc2"))
        else:
            ignored[p + "norm2"] = "layer has no feed-forward"
            for name in ("in", "out", "mix"):
                ignored[p + "hc2." + name] = "layer has no feed-forward"
        layers.append(LayerSpec("hyper_connections", parts))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embed=PartSpec("embed", "token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "table": "embed"}),
        layers=layers, schedule=[ScheduleStep(i) for i in range(len(cfg.layers))],
        final_norm=PartSpec("norm", "scalar_rms_norm", {"size": cfg.width, "eps": cfg.eps, "weight": "final.norm",
                                                        "streams": streams, "gain": cfg.logit_scale}),
        head=PartSpec("head", "lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None,
                                          "tensor": "head"}),
        eos_token_ids=list(cfg.eos_token_id or ()), ignored_tensors=ignored)
