"""Descriptions of a model as data: which parts make a layer, and in which order
layers run.  An architecture's factory turns its configuration into a
``ModelSpec``; the model builder turns the spec into parts by looking every
``PartSpec.kind`` up in the part registries.  Nothing here knows a model's name.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer.

    kind    name under which the part's class is registered
    params  the part's own parameter object (its sizes and constants)
    names   the part's tensor names -> tensor names in the checkpoint
    """

    kind: str
    params: Any = None
    names: Dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A block: how a mixer and a feed-forward are arranged around the residual
    stream.  ``arrangement`` names a registered block class.  A layer that has a mixer
    only leaves ``ffn_norm`` and ``ffn`` out."""

    arrangement: str
    mixer_norm: PartSpec
    mixer: PartSpec
    ffn_norm: Optional[PartSpec] = None
    ffn: Optional[PartSpec] = None


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    layer        index into ``ModelSpec.layers``; an index may appear more than once
    cache_of     None: this call owns a cache of its own and writes it;
                 an int: index of an earlier call whose cache this call reads
                 (it then writes none)
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects from the checkpoint."""

    shape: Tuple[int, ...]
    optional: bool = False
    integer: bool = False  # integer tables are kept as int32


@dataclass(frozen=True)
class CacheTensor:
    """One tensor that a mixer caches for each token it has seen.

    name   how the mixer finds it in its ``LayerCache``
    shape  of one token, for instance (heads, head_dim).  The last axis is kept contiguous; the pool
           lays a tensor out as [pages, *shape[:-1], page_size, shape[-1]], so that the tokens of a page
           under one index of the leading axes (a head's keys) are one contiguous box.
    """

    name: str
    shape: Tuple[int, ...]

    def elements(self) -> int:
        n = 1
        for x in self.shape:
            n *= int(x)
        return n


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer needs cached for each token it has seen.

    kind     "full": every token stays; "window": only the last ``window`` tokens
    tensors  the tensors kept per token, each with a shape of its own (keys and values of the same
             shape for ordinary attention; one latent vector, or keys and values of different widths,
             for other mixers)
    Layers whose mixers ask for the same spec share one group of pages and one block table per request.
    """

    kind: str
    tensors: Tuple[CacheTensor, ...]
    window: int = 0

    @staticmethod
    def keys_values(kind: str, heads: int, head_dim: int, window: int = 0) -> "CacheSpec":
        """Keys "k" and values "v" of [heads, head_dim] per token: what grouped-query attention caches."""
        return CacheSpec(kind, (CacheTensor("k", (heads, head_dim)), CacheTensor("v", (heads, head_dim))), window)

    def elements_per_token(self) -> int:
        return sum(t.elements() for t in self.tensors)

    def group_key(self) -> Tuple:
        return (self.kind, self.tensors, self.window)


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size that a mixer keeps (none for attention)."""

    shape: Tuple[int, ...]
    dtype: str = "float32"
