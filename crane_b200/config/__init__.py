"""Typed configurations and the architecture registry."""
from .hunyuan_dense import (ALIASES, ARCHITECTURE, ConfigError, HunyuanDenseConfig, RopeScaling,
                            build_spec, read_config_json)
from . import mufevik, radorax, vodelix, zudarax
from .radorax import RadoraxConfig
from .vodelix import VodelixConfig
from .mufevik import MufevikConfig
from .zudarax import ZudaraxConfig
from .registry import (Architecture, UnknownArchitecture, register_architecture, registered,
                       resolve)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep
from .engine_config import EngineConfig, parse_memory_limit

register_architecture(ARCHITECTURE, HunyuanDenseConfig.from_dict, build_spec, ALIASES)
register_architecture(radorax.ARCHITECTURE, RadoraxConfig.from_dict, radorax.build_spec, radorax.ALIASES)
register_architecture(vodelix.ARCHITECTURE, VodelixConfig.from_dict, vodelix.build_spec, vodelix.ALIASES)
register_architecture(mufevik.ARCHITECTURE, MufevikConfig.from_dict, mufevik.build_spec, mufevik.ALIASES)
register_architecture(zudarax.ARCHITECTURE, ZudaraxConfig.from_dict, zudarax.build_spec, zudarax.ALIASES)

__all__ = ["ConfigError", "HunyuanDenseConfig", "RadoraxConfig", "VodelixConfig", "MufevikConfig", "ZudaraxConfig", "RopeScaling", "read_config_json", "Architecture",
           "UnknownArchitecture", "register_architecture", "registered", "resolve", "LayerSpec",
           "ModelSpec", "PartSpec", "ScheduleStep", "EngineConfig", "parse_memory_limit"]
