"""Draws one token per logits row on the GPU (greedy, temperature, top-k, top-p) and
gives its log-probability under the raw logits; see csrc/sampling.cu."""

from __future__ import annotations

import torch

from ..ops import kernels


class Sampler:
    def __init__(self, max_rows: int, device: torch.device):
        self.tokens = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.logprobs = torch.zeros(max_rows, dtype=torch.float32, device=device)
        self.scratch = torch.zeros(max_rows * kernels.SAMPLE_CHUNKS * 4, dtype=torch.float32, device=device)

    def sample(self, logits: torch.Tensor, ctx) -> None:
        """Fills tokens[:R] and logprobs[:R] from logits[:R] with the rows' parameters in ctx."""
        kernels.sample(logits, ctx.R, ctx.temperature, ctx.top_k, ctx.top_p, ctx.seed_lo, ctx.seed_hi,
                       ctx.sample_pos, self.tokens, self.logprobs, scratch=self.scratch)
