"""Parts a layer is put together from.  Importing the package registers the
built-in parts."""

from . import attention, block, embedding, mlp, rmsnorm, rope  # noqa: F401
from .base import (Block, Embedding, FeedForward, Head, LayerCache, Mixer, Norm, Part, PositionEncoding,
                   Runtime, Workspace, build_part, lookup, register)
from .spec import CacheSpec, CacheTensor, LayerCall, LayerSpec, ModelSpec, PartSpec, StateSpec, TensorSpec
