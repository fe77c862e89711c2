"""Per-request sampling options, with the reference's names, meanings and defaults
(src/core/sequence.h:10-20)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Tuple


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0      # <= 0 selects greedy decoding
    top_k: int = 0                # 0 disables top-k
    top_p: float = 1.0            # 1 disables top-p
    seed: int = 0
    max_new_tokens: int = 128
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    def validate(self) -> None:
        if self.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.seed < 0 or self.seed >= 2 ** 64:
            raise ValueError("seed must fit in 64 bits")
