"""Token embedding (a row gather, no scaling: src/cuda/kernels/elementwise.cu:19-24)
and the output head (logits in float32: src/cuda/model/llama.cpp:143-150)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import Embedding, Head, register
from .spec import TensorSpec


@dataclass(frozen=True)
class EmbeddingParams:
    vocab_size: int
    hidden_size: int


@register("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.params.vocab_size, self.params.hidden_size))}

    def load(self, tensors) -> None:
        self.weight = tensors["weight"]

    def table(self) -> torch.Tensor:
        return self.weight

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx, out: torch.Tensor) -> None:
        kernels.embedding(ctx.token_ids[:ctx.T], self.weight, out, ctx.status)


@dataclass(frozen=True)
class HeadParams:
    vocab_size: int
    hidden_size: int
    tied: bool  # the configuration ties the head to the embedding table


@register("head", "lm_head")
class LMHead(Head):
    """``weight`` is optional: a checkpoint without it shares the embedding table
    (src/cuda/model/weights.cpp:237-246); the model builder then calls ``tie``."""

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.params.vocab_size, self.params.hidden_size), optional=True)}

    def load(self, tensors) -> None:
        self.weight = None if self.params.tied else tensors.get("weight")
        self.shared = False

    def wants_table(self) -> bool:
        return self.weight is None

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table
        self.shared = True

    def nbytes(self) -> int:
        return 0 if self.shared or self.weight is None else self.weight.numel() * self.weight.element_size()

    def forward(self, x: torch.Tensor, rows: int, out: torch.Tensor) -> None:
        linear(x[:rows], self.weight, out[:rows])

    def forward_from(self, residual, norm, rows_idx, rows: int, out: torch.Tensor) -> bool:
        rms = norm.rms_params()
        # (for a very tall matrix the library product already runs at the bandwidth limit;
        #  the fused form pays off where the product is short and launches dominate)
        if (rms is None or self.rt.dtype != torch.bfloat16 or self.weight.shape[0] > 32768
                or not kernels.skinny_ok(rows, self.weight, self.rt.dtype)):
            return False
        kernels.gemm_skinny(self.weight, out, kernels.EPI_F32, rows, residual=residual, norm_w=rms[0], eps=rms[1],
                            rows_idx=rows_idx)
        return True
