"""Parts of a decoder and their registries."""
from .base import (CacheNeed, LayerCache, Part, Workspace, block_class, build_part, part_class,
                   register_block, register_part)
from .runtime import DeviceFault, Runtime
from . import (attention, block, delta_rule, embedding, feed_forward, latent_attention, norm, pair, position,   # register the parts
               recurrent, scored_attention)
from .model import DecoderModel, model_manifest

__all__ = ["CacheNeed", "LayerCache", "Part", "Workspace", "block_class", "build_part",
           "part_class", "register_block", "register_part", "Runtime", "DeviceFault",
           "DecoderModel", "model_manifest"]
