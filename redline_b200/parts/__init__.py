"""Parts a layer is put together from.  Importing the package registers the
built-in parts."""

from . import (attention, attention_maps, block, embedding, layernorm, linear_attention, mlp, moe, rmsnorm,  # noqa: F401
               rope)
from .base import (Block, Embedding, FeedForward, Head, LayerCache, Mixer, Norm, Part, PositionEncoding,
                   Runtime, Workspace, build_part, lookup, register)
from .spec import CacheSpec, CacheTensor, LayerCall, LayerSpec, ModelSpec, PartSpec, StateSpec, TensorSpec
