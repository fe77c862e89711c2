"""A decoder put together from a ``ModelSpec``: embedding, blocks run in the order
the spec lists (an entry may name a layer twice, or read an earlier entry's cache),
final norm on the rows whose logits are wanted, head.  The forward pass is the
reference's (src/cuda/model/llama.cpp:56-151) with the residual stream in float32
and the final norm applied to the wanted rows only.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.manager import GroupInfo
from ..parts import base as parts_base
from ..parts.base import Block, Runtime, build_part, lookup, op_mark
from ..parts.spec import CacheSpec, ModelSpec, StateSpec, TensorSpec
from ..weights import loader
from ..weights.safetensors_io import CheckpointReader


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec, self.rt = spec, rt
        self.embedding = build_part("embedding", spec.embedding, rt)
        self.blocks: List[Block] = []
        for ls in spec.layers:
            block_cls = lookup("block", ls.arrangement)
            if (ls.ffn is None) != (ls.ffn_norm is None):
                raise ValueError("a layer has a feed-forward and its norm, or neither")
            self.blocks.append(block_cls(build_part("norm", ls.mixer_norm, rt), build_part("mixer", ls.mixer, rt),
                                         build_part("norm", ls.ffn_norm, rt) if ls.ffn_norm is not None else None,
                                         build_part("ffn", ls.ffn, rt) if ls.ffn is not None else None, rt))
        self.final_norm = build_part("norm", spec.final_norm, rt)
        self.head = build_part("head", spec.head, rt)
        self.nvtx_layers = False           # one NVTX range per layer call (set by the runner from the engine's options)
        self._check_order()

    # -------------------------------------------------------------- layout
    def _check_order(self) -> None:
        for i, call in enumerate(self.spec.order):
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"run order entry {i} names layer {call.layer} of {len(self.blocks)}")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < i:
                    raise ValueError(f"run order entry {i} reads the cache of entry {call.cache_of}, "
                                     "which does not come before it")
                if self.spec.order[call.cache_of].cache_of is not None:
                    raise ValueError(f"run order entry {i} reads the cache of entry {call.cache_of}, "
                                     "which owns none")
                a = self.blocks[call.layer].mixer.cache_spec()
                b = self.blocks[self.spec.order[call.cache_of].layer].mixer.cache_spec()
                if a is None or b is None or a.group_key() != b.group_key():
                    raise ValueError(f"run order entry {i} cannot read the cache of entry {call.cache_of}: "
                                     "the two mixers need different caches")

    def cache_groups(self) -> List[GroupInfo]:
        """Groups of cache-owning run-order entries whose mixers need the same cache."""
        groups: Dict[Tuple, GroupInfo] = {}
        for i, call in enumerate(self.spec.order):
            if call.cache_of is not None:
                continue
            cs = self.blocks[call.layer].mixer.cache_spec()
            if cs is None:
                continue
            groups.setdefault(cs.group_key(), GroupInfo(cs)).owners.append(i)
        return list(groups.values())

    def tiling(self) -> Optional[Tuple[int, int]]:
        """The one tiling of the step's work lists that this model's mixers ask for (None: no mixer reads them)."""
        named = {b.mixer.tiling() for b in self.blocks} - {None}
        if len(named) > 1:
            raise ValueError(f"the model's mixers want the step's work lists cut in different ways: {sorted(named)}")
        return next(iter(named)) if named else None

    def decode_variants(self, ctx) -> Tuple[int, ...]:
        """What every layer's mixer will run for the step's single-token sequences (``Mixer.decode_variant``):
        steps with the same answer can share a CUDA graph."""
        return tuple(b.mixer.decode_variant(ctx) for b in self.blocks)

    def state_specs(self) -> Dict[int, StateSpec]:
        out = {}
        for i, call in enumerate(self.spec.order):
            ss = self.blocks[call.layer].mixer.state_spec()
            if ss is not None:
                out[i] = ss
        return out

    # ------------------------------------------------------------- weights
    def _named_parts(self):
        yield self.embedding
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm
        yield self.head

    def expected_tensors(self) -> Dict[str, TensorSpec]:
        exp: Dict[str, TensorSpec] = {}
        for part in self._named_parts():
            for local, ts in part.tensors().items():
                name = part.spec.names.get(local)
                if name is None:
                    if ts.optional:
                        continue
                    raise ValueError(f"part '{part.spec.kind}' has no checkpoint name for its tensor '{local}'")
                exp[name] = ts
        return exp

    def load_weights(self, reader: CheckpointReader) -> None:
        rt = self.rt
        parts = list(self._named_parts())
        fused = {}                       # "<part number>:<fused name>" -> checkpoint names of its members
        for pi, part in enumerate(parts):
            for fname, members in part.fused().items():
                names = [part.spec.names.get(m) for m in members]
                if all(n is not None for n in names):
                    fused[f"{pi}:{fname}"] = names
        tensors = loader.load(reader, self.expected_tensors(), rt.dtype, rt.device, fused=fused)
        for pi, part in enumerate(parts):
            mine = {}
            for local in part.tensors():
                name = part.spec.names.get(local)
                if name is not None and name in tensors:
                    mine[local] = tensors[name]
            for fname in part.fused():
                if f"{pi}:{fname}" in tensors:
                    mine[fname] = tensors[f"{pi}:{fname}"]
            part.load(mine)
        if self.head.wants_table():
            # no head tensor in use: the head shares the embedding table
            self.head.tie(self.embedding.table())

    def weight_bytes(self) -> int:
        return sum(p.nbytes() for p in self._named_parts())

    # ------------------------------------------------------------- forward
    def forward(self, ctx, caches, states, logits: torch.Tensor) -> torch.Tensor:
        """Runs the step's tokens; returns logits[:R] (float32) at the wanted rows.
        ``caches[i]`` / ``states[i]`` belong to run-order entry i (None where unused)."""
        rt = self.rt
        T, R = ctx.T, ctx.R
        ws = rt.workspace
        residual = ws.get("residual", (rt.max_tokens, self.spec.hidden_size), torch.float32)[:T]
        self.embedding.forward(ctx, residual)
        op_mark(ctx, "embed", nbytes=T * self.spec.hidden_size * (4.0 + (2 if rt.dtype == torch.bfloat16 else 4)))
        pending = None
        order = self.spec.order
        ctx.block_hand = None
        for i, call in enumerate(order):
            # (the block after this one may take over its first norm from this block's last kernel)
            ctx.block_next_norm = self.blocks[order[i + 1].layer].first_norm() if i + 1 < len(order) else None
            if self.nvtx_layers:
                torch.cuda.nvtx.range_push(f"layer call {i} (layer {call.layer})")
            pending = self.blocks[call.layer].forward(residual, pending, ctx, caches[i], states[i])
            if self.nvtx_layers:
                torch.cuda.nvtx.range_pop()
        ctx.block_hand = ctx.block_next_norm = None
        head_w = getattr(self.head, "weight", None)
        if R > 0 and pending is None and self.head.forward_from(residual, self.final_norm, ctx.logit_rows, R, logits):
            op_mark(ctx, "final_norm+lm_head", head_w, R, nbytes=R * logits.shape[1] * 2.0)
        elif R > 0:
            xr = ws.get("head.in", (logits.shape[0], self.spec.hidden_size), rt.dtype)[:R]
            self.final_norm.add_norm(residual, pending, xr, rows_idx=ctx.logit_rows, rows=R)
            op_mark(ctx, "final_norm", nbytes=R * self.spec.hidden_size * 6.0)
            self.head.forward(xr, R, logits)
            op_mark(ctx, "lm_head", head_w, R, nbytes=R * logits.shape[1] * 2.0)     # (the logits are float32: 2 more bytes each)
        return logits[:R]
