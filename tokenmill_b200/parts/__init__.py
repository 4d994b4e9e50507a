"""Parts a layer is made of. Importing this package registers the built-in kinds."""

from . import (attention, block, decay_memory, gated_memory, latent_attention, matrix_memory, norm, pair_mixer, rope, routed, sink_attention,  # noqa: F401
               state_space, swiglu)
from .base import LayerCache, StepInputs
from .model import CacheGroup, CacheLayout, DecoderModel
from .spec import LayerSpec, ModelSpec, PagedKVNeed, PartSpec, RunEntry, StateNeed, WeightSpec

__all__ = ["LayerCache", "StepInputs", "CacheGroup", "CacheLayout", "DecoderModel", "LayerSpec", "ModelSpec",
           "PagedKVNeed", "PartSpec", "RunEntry", "StateNeed", "WeightSpec"]
