"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from its ``PartSpec`` and the ``Runtime`` (device, activation type,
workspace); it declares the tensors it wants from the checkpoint under its own
names, receives them, and then runs on a ``StepContext``.  No part knows which
model it is in.  A new kind of part is added by subclassing one of the classes
below and registering it under a name:

    @register("mixer", "my_mixer")
    class MyMixer(Mixer): ...

after which a ``PartSpec(kind="my_mixer", ...)`` in a ``ModelSpec`` builds it.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from .spec import CacheSpec, PartSpec, StateSpec, TensorSpec

_REGISTRIES: Dict[str, Dict[str, type]] = {
    "norm": {}, "mixer": {}, "ffn": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


def register(family: str, kind: str) -> Callable[[type], type]:
    if family not in _REGISTRIES:
        raise KeyError(f"unknown part family '{family}' (known: {sorted(_REGISTRIES)})")

    def deco(cls: type) -> type:
        _REGISTRIES[family][kind] = cls
        return cls

    return deco


def lookup(family: str, kind: str) -> type:
    reg = _REGISTRIES[family]
    if kind not in reg:
        raise KeyError(f"no {family} part is registered as '{kind}' (known: {sorted(reg)})")
    return reg[kind]


def build_part(family: str, spec: PartSpec, rt: "Runtime"):
    return lookup(family, spec.kind)(spec, rt)


class Workspace:
    """Activation buffers shared by all layers (they run one after another).  A
    buffer is asked for by name with its widest shape and lives as long as the
    engine, so addresses are stable for CUDA graphs and no step allocates."""

    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self._retired: List[torch.Tensor] = []

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = f"{name}:{dtype}"
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            if buf is not None:
                self._retired.append(buf)   # a captured graph may still point at it
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:n].view(shape)

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


@dataclass
class Runtime:
    """What a part may know of the engine it runs in."""

    device: torch.device
    dtype: torch.dtype            # activation / cache type: float32 or bfloat16
    max_tokens: int               # most tokens in one step
    max_seqs: int                 # most sequences in one step
    max_seq_len: int              # longest sequence
    page_size: int
    workspace: Workspace = None   # type: ignore[assignment]

    def __post_init__(self):
        if self.workspace is None:
            self.workspace = Workspace(self.device)


@dataclass
class LayerCache:
    """The cache one call of a layer works on: the tensors its mixer's ``CacheSpec`` names, each
    [pages, *leading axes, page_size, last axis] in the pages of its cache group (for attention
    ``k`` and ``v`` [pages, heads, page_size, D]), and whether this call writes its tokens there."""

    group: int
    tensors: Dict[str, torch.Tensor]
    write: bool = True

    @property
    def k(self) -> torch.Tensor:
        return self.tensors["k"]

    @property
    def v(self) -> torch.Tensor:
        return self.tensors["v"]


class Part:
    def __init__(self, spec: PartSpec, rt: Runtime):
        self.spec = spec
        self.params = spec.params
        self.rt = rt

    def tensors(self) -> Dict[str, TensorSpec]:
        """Own tensor name -> what is expected of it."""
        return {}

    def fused(self) -> Dict[str, List[str]]:
        """Own name of a fused tensor -> the names (of ``tensors()``) whose tensors the part uses as one,
        laid one after another along their first axis.  The loader then puts them so on the device and
        ``load`` receives the fused name in place of the members (if the checkpoint has all of them)."""
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the tensors of ``tensors()`` that the checkpoint had, on the device (and those of
        ``fused()`` in place of their members)."""

    def nbytes(self) -> int:
        return 0


class Norm(Part):
    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
                 rows_idx: Optional[torch.Tensor] = None, rows: Optional[int] = None) -> None:
        """residual (float32) += delta; out = norm(residual).  With ``rows_idx`` only
        those rows are produced and residual is not changed."""
        raise NotImplementedError

    def rms_params(self) -> Optional[Tuple[torch.Tensor, float]]:
        """(weight, eps) if this norm is y = x * rsqrt(mean(x^2) + eps) * weight, which a
        consumer may then compute itself from the residual stream; None otherwise."""
        return None


@dataclass
class NormHandover:
    """An RMSNorm that the part before has half done in its last kernel, for the part after it.

    A part whose fused form ends in ``residual += ...`` and that finds ``ctx.next_norm`` set (the norm
    that will be applied to the stream next, an RMSNorm) may leave, instead of nothing,
    ``ctx.hand_out = NormHandover(norm, xw, sums)``: xw = bfloat16(residual * norm.weight) and per-row
    partial sums of residual^2.  The block passes it to the next part's fused form as ``ctx.hand_in``
    (only if it was made for that part's norm); a part that takes it skips its norm kernel, multiplies
    xw and scales the rows of the product by rsqrt(sum / width + eps).  A part that knows nothing of
    this ignores both fields and norms the stream itself."""

    norm: "Norm"
    xw: torch.Tensor        # [T, H] bfloat16
    sums: torch.Tensor      # [T, n] float32; a row's sum of squares is sums[row].sum()


def norm_handover(part: "Part", name: str, ctx, width: int, rows: int, tile: int = 16) -> Optional[NormHandover]:
    """The hand-over that ``part``'s last product is to fill for ``ctx.next_norm`` (buffers named after
    ``name`` in the workspace, for up to ``rows`` rows, a sum of squares for every ``tile`` features), or
    None if there is no such norm or it is not an RMSNorm of this width.  ``REDLINE_NORM_HANDOVER=0`` turns
    hand-overs off (every norm its own kernel)."""
    norm = ctx.next_norm
    if norm is None or os.environ.get("REDLINE_NORM_HANDOVER", "1") == "0":
        return None
    rms = norm.rms_params()
    if rms is None or rms[0].numel() != width:
        return None
    ws = part.rt.workspace
    return NormHandover(norm, ws.get(name + ".hand_xw", (rows, width), torch.bfloat16),
                        ws.get(name + ".hand_sums", (rows, (width + tile - 1) // tile), torch.float32))


def op_mark(ctx, op: str, weight: Optional[torch.Tensor] = None, rows: int = 0, nbytes: float = 0.0,
            flops: float = 0.0) -> None:
    """Tells the step's per-op profiler (``ctx.profiler``, None unless per-op profiling is on) that ``op``
    has been enqueued.  For a product with ``weight`` [N, K] over ``rows`` rows the bytes and operations are
    worked out here; other ops pass their own."""
    prof = getattr(ctx, "profiler", None)
    if prof is None:
        return
    if weight is not None:
        n, k = weight.shape
        elem = weight.element_size()
        nbytes += float(weight.numel() * elem + rows * (n + k) * elem)
        flops += 2.0 * rows * n * k
    prof.mark(op, nbytes, flops)


class PositionEncoding(Part):
    """How positions enter a mixer.  A rotary encoding exposes ``rotary_tables()``
    (cos, sin [max_pos, D/2] float32) and the attention mixer rotates q and k in the
    kernel that writes the cache; any other encoding implements ``apply`` on the
    projected q and k."""

    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        return None

    def apply(self, qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, ctx) -> None:
        """In place on qkv [T, (Hq + 2 Hkv) D]; the default does nothing."""


class Mixer(Part):
    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def tiling(self) -> Optional[Tuple[int, int]]:
        """(query rows of a tile, keys of a partition) in which this mixer's kernels want the step's
        work lists cut (``ctx.tile_*`` for sequences that bring several tokens, ``ctx.decode_info`` /
        ``ctx.decode_parts`` for single tokens), or None if it reads neither list.  All mixers of a
        model that name a tiling must name the same one."""
        return None

    def decode_variant(self, ctx) -> int:
        """Which of its kernels this mixer will run for the step's single-token sequences, as a number of its
        own (0 if it has one way only).  It must depend on nothing but ``ctx.num_decode``,
        ``ctx.decode_max_ctx`` and ``ctx.decode_sum_ctx``: a CUDA graph of a step is replayed only for steps
        whose mixers answer alike."""
        return 0

    def forward(self, x: torch.Tensor, ctx, cache: Optional[LayerCache],
                state: Optional[torch.Tensor]) -> torch.Tensor:
        """x [T, H] -> [T, H] (what is added to the residual stream).  ``state`` is this
        call's slot pool [slots, *state shape]; ``ctx.state_slot`` maps sequences to slots."""
        raise NotImplementedError

    def forward_into(self, residual: torch.Tensor, norm: Norm, ctx, cache: Optional[LayerCache],
                     state: Optional[torch.Tensor]) -> bool:
        """Optional fused form for small batches: residual += mixer(norm(residual)), the norm
        computed by the mixer's first kernel and the add by its last.  Returns False (and
        does nothing) when the part does not take this batch that way.  ``ctx.hand_in`` /
        ``ctx.next_norm`` / ``ctx.hand_out``: see ``NormHandover`` (optional)."""
        return False


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError

    def forward_into(self, residual: torch.Tensor, norm: Norm, ctx) -> bool:
        """Optional fused form: residual += ffn(norm(residual)); see ``Mixer.forward_into``."""
        return False


class Embedding(Part):
    def forward(self, ctx, out: torch.Tensor) -> None:
        """out [T, H] float32 <- embeddings of ctx.token_ids."""
        raise NotImplementedError

    def table(self) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    def forward(self, x: torch.Tensor, rows: int, out: torch.Tensor) -> None:
        """x [R, H] -> out [R, V] float32."""
        raise NotImplementedError

    def wants_table(self) -> bool:
        """True after ``load`` if the head has no weight of its own and is to share the embedding's
        table; the model then calls ``tie`` with it."""
        return False

    def tie(self, table: torch.Tensor) -> None:
        raise NotImplementedError

    def forward_from(self, residual: torch.Tensor, norm: Norm, rows_idx: torch.Tensor, rows: int,
                     out: torch.Tensor) -> bool:
        """Optional fused form: out[:rows] = head(norm(residual[rows_idx])).  False if not taken."""
        return False


class Block:
    """Arrangement of a mixer and a feed-forward around the float32 residual stream.
    ``forward`` gets the stream and a delta that has not been added yet (the previous
    block's last output, so that the add is fused with this block's first norm) and
    returns its own last output the same way."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm], ffn: Optional[FeedForward],
                 rt: Runtime):
        """``ffn_norm`` and ``ffn`` are None for a layer that has a mixer only."""
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.rt = mixer_norm, mixer, ffn_norm, ffn, rt

    def parts(self) -> List[Part]:
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def first_norm(self) -> Optional[Norm]:
        """The norm this block applies to the incoming stream first, if the block before may hand it
        over (``NormHandover``); None if the block does not begin with a norm of the stream."""
        return None

    def forward(self, residual: torch.Tensor, pending: Optional[torch.Tensor], ctx,
                cache: Optional[LayerCache], state: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        raise NotImplementedError
