from .base import (CacheSpec, CacheView, Part, Runtime, StateSpec, StateView, TensorDecl, WeightSource,
                   build_part, register_part, registered_parts)
from . import (attention, block, decay_attention, embedding, exp_gated_memory, gated_recurrence, latent_attention, mlp,  # noqa: F401
               multimap_attention, norm, parallel, rope, side_input, stream)  # noqa: F401  (register the built-in parts)
from .block import build_block
from .linear import Linear

__all__ = ["CacheSpec", "CacheView", "Part", "Runtime", "StateSpec", "StateView", "TensorDecl", "WeightSource",
           "build_part", "build_block", "register_part", "registered_parts", "Linear"]
