"""Typed configuration of Zudarax, read from the keys of its config.json.

A Zudarax layer has ONE norm, an RMS norm taken in groups (the row in ``norm.groups`` equal consecutive
parts, each over the root of its own mean square), which both its sublayers read:
``h = norm1(x); x <- x + (mixer(h) + ff(h))``.  Three mixers, all grouped-query attention over the paged
cache whose scores are worked on before they become weights:

* ``attention``: biases on q, k, v; a causal convolution of ``conv`` taps over time on every channel of
  q, k and v; RMS norm of q and of k over their whole rows; rotation of the leading ``rot.dims`` elements
  of each head; scores squashed to ``softcap * tanh(s / softcap)``; keys seen within the query's own block
  of ``mask.size`` positions; softmax.
* ``attention_2``: differential attention.  Each head has two maps of queries and keys, two softmax
  attentions over the same values, ``o = a1 - lambda a2`` with ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) +
  diff``, o over the root of its mean square per head times ``1 - diff``, times ``sigmoid(W_g h)`` per head.
* ``attention_3``: convolutions; rotation with YaRN-scaled frequencies (``rot.scaling``); the weight of a
  visible key is ``sigmoid(s + pb[h])``, not normalised over the keys.

The feed-forward is ``down(PolyNorm(up h))``.  config.json: ``architecture``, ``vocab``, ``width``,
``norm.{eps, groups}``, ``layers``: a list of ``{"type", "mixer": {...}, "mlp": {"kind": "dense", "ff"} |
null}``.  A layer's type says which tensors it has; every size and constant is read from its ``mixer``
entry, and an option that the entry does not name (``conv``, ``rot``, ``rot.scaling``, ``softcap``,
``mask``) is absent.  The design has no position limit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .hunyuan_dense import ConfigError

ARCHITECTURE = "Zudarax"
ALIASES = ("zudarax",)
# the design has no limit on positions; the engine's own (``EngineConfig.max_seq_len``) is capped here
MAX_POSITIONS = 1 << 17
MIXERS = ("attention", "attention_2", "attention_3")
# head sizes that the warp-level attention kernels are compiled for
ATTENTION_HEAD_SIZES = (16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 256)


@dataclass(frozen=True)
class ZudaraxMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int = 0                       # taps of the convolutions on q, k, v (0: none)
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_scaling: Optional[Tuple[Tuple[str, float], ...]] = None      # YaRN: factor, original, fast, slow
    softcap: float = 0.0
    chunk: int = 0                      # mask.size (0: every earlier position)
    diff: float = 0.0                   # attention_2: the constant of lambda and of the head norm's factor


@dataclass(frozen=True)
class ZudaraxLayer:
    type: str
    mixer: ZudaraxMixer
    ff: int                             # 0: no feed-forward


@dataclass(frozen=True)
class ZudaraxConfig:
    vocab: int
    width: int
    eps: float
    groups: int
    layers: Tuple[ZudaraxLayer, ...]
    eos_token_id: Optional[Tuple[int, ...]] = None

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "ZudaraxConfig":
        def need(obj, key, where):
            if not isinstance(obj, dict) or obj.get(key) is None:
                raise ConfigError(f"config.json lacks '{key}' in {where}")
            return obj[key]

        layers: List[ZudaraxLayer] = []
        for i, ld in enumerate(need(d, "layers", "the top level")):
            where = f"layers[{i}]"
            kind = str(need(ld, "type", where))
            if kind not in MIXERS:
                raise ConfigError(f"{where}: no mixer '{kind}'; this design has: {', '.join(MIXERS)}")
            m = need(ld, "mixer", where)
            heads, dim = int(need(m, "heads", where + ".mixer")), int(need(m, "dim", where + ".mixer"))
            rot = m.get("rot") or {}
            sc = rot.get("scaling")
            if sc is not None:
                for key in ("factor", "original", "fast", "slow"):
                    need(sc, key, where + ".mixer.rot.scaling")
            mixer = ZudaraxMixer(
                heads=heads, kv_heads=int(m.get("kv_heads") or heads), dim=dim, vdim=int(m.get("vdim") or dim),
                scale=float(m["scale"]) if m.get("scale") is not None else dim ** -0.5,
                conv=int(m.get("conv") or 0), rot_dims=int(rot.get("dims") or 0),
                rot_base=float(rot.get("base") or 10000.0),
                rot_scaling=tuple(sorted((k, float(v)) for k, v in sc.items())) if sc else None,
                softcap=float(m.get("softcap") or 0.0), chunk=int((m.get("mask") or {}).get("size") or 0),
                diff=float(need(m, "diff", where + ".mixer")) if kind == "attention_2" else 0.0)
            md = ld.get("mlp")
            ff = 0
            if md is not None:
                mk = str(md.get("kind") or "dense")
                if mk != "dense":
                    raise ConfigError(f"{where}.mlp: no feed-forward kind '{mk}'; this design has: dense")
                ff = int(need(md, "ff", where + ".mlp"))
            layers.append(ZudaraxLayer(kind, mixer, ff))
        eos = d.get("eos_token_id")
        eos = (int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos) if eos else None
        norm = need(d, "norm", "the top level")
        cfg = ZudaraxConfig(vocab=int(need(d, "vocab", "the top level")), width=int(need(d, "width", "the top level")),
                            eps=float(need(norm, "eps", "norm")), groups=int(norm.get("groups") or 1),
                            layers=tuple(layers), eos_token_id=eos)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be > 0, got {self.eps}")
        if self.groups <= 0 or self.width % self.groups:
            raise ConfigError(f"norm.groups {self.groups} must divide the width {self.width}")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.heads <= 0 or m.kv_heads <= 0 or m.heads % m.kv_heads or m.dim <= 0 or m.vdim <= 0:
                raise ConfigError(f"layers[{i}].mixer: heads must be a positive multiple of kv_heads, "
                                  "dim and vdim positive")
            if m.rot_dims < 0 or m.rot_dims % 2 or m.rot_dims > m.dim:
                raise ConfigError(f"layers[{i}].mixer.rot.dims must be even and at most dim")
            if not 0 <= m.conv <= 64:
                raise ConfigError(f"layers[{i}].mixer.conv must be at most 64 taps")
            if m.softcap < 0 or m.chunk < 0:
                raise ConfigError(f"layers[{i}].mixer: softcap and mask.size must not be negative")
            if layer.ff < 0:
                raise ConfigError(f"layers[{i}].mlp.ff must be positive")


def _stored_head(maps: int, dim: int, vdim: int) -> Tuple[int, int]:
    """(the head size that keys and values are stored at on the bfloat16 path, where a head's second
    map starts); (0, 0): none of the compiled sizes holds them.  Two maps share a key row in halves, each
    half a multiple of 16 elements."""
    for s in ATTENTION_HEAD_SIZES:
        if maps == 1 and s >= max(dim, vdim):
            return s, s
        if maps == 2 and s % 32 == 0 and s // 2 >= dim and s >= vdim:
            return s, s // 2
    return 0, 0


def _mixer_spec(cfg: ZudaraxConfig, kind: str, m: ZudaraxMixer, prefix: str):
    from .spec import PartSpec
    position = None
    if m.rot_dims:
        position = PartSpec("position", "yarn_rope", {
            "dims": m.rot_dims, "base": m.rot_base, "scaling": dict(m.rot_scaling) if m.rot_scaling else None,
            "max_positions": MAX_POSITIONS})
    maps = 2 if kind == "attention_2" else 1
    store, dpad = _stored_head(maps, m.dim, m.vdim)
    return PartSpec("mixer", "scored_attention", {
        "hidden_size": cfg.width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
        "scale": m.scale, "bias": kind == "attention", "conv": m.conv, "qk_norm": kind == "attention",
        "norm_eps": cfg.eps, "rotary_dim": m.rot_dims, "position": position, "softcap": m.softcap, "chunk": m.chunk,
        "weighting": "sigmoid" if kind == "attention_3" else "softmax", "head_bias": kind == "attention_3",
        "maps": maps, "diff": m.diff, "head_norm": kind == "attention_2", "gate": kind == "attention_2",
        "head_dim": store, "map_stride": dpad}, prefix=prefix)


def build_spec(cfg: ZudaraxConfig):
    """Zudarax as data: per layer one norm in groups, a mixer and a feed-forward that both read it."""
    from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep

    def norm(prefix, name):
        return PartSpec("norm", "group_rms_norm", {"size": cfg.width, "eps": cfg.eps, "groups": cfg.groups,
                                                   "weight": name}, prefix=prefix)
    layers, ignored = [], {}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"norm1": norm(p, "norm1"), "mixer": _mixer_spec(cfg, layer.type, layer.mixer, p + "mix.")}
        if layer.ff:
            parts["ffn"] = PartSpec("ffn", "poly_norm_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.ff,
                                                             "eps": cfg.eps}, prefix=p + "mlp.")
        layers.append(LayerSpec("parallel_shared_norm", parts))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embed=PartSpec("embed", "token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "table": "embed"}),
        layers=layers, schedule=[ScheduleStep(i) for i in range(len(cfg.layers))],
        final_norm=norm("", "final.norm"),
        head=PartSpec("head", "lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None,
                                          "tensor": "head"}),
        eos_token_ids=list(cfg.eos_token_id or ()), ignored_tensors=ignored)
