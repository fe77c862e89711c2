"""Rotary position encoding: inverse frequencies with none / linear / llama3
scaling in double precision, angle = float32(pos) * float32(inv_freq) formed in
float32, pairs (i, i + D/2) rotated (reference: src/core/model_config.cpp:126-169,
src/cuda/kernels/rope_kv.cu:26-51).  ``NoPosition`` is the encoding that does
nothing."""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch

from ..config.model_config import RopeScaling
from .base import PositionEncoding, register


@dataclass(frozen=True)
class RotaryParams:
    head_dim: int
    theta: float
    scaling: RopeScaling
    max_positions: int


def rope_inv_freq(head_dim: int, theta: float, scaling: RopeScaling) -> List[float]:
    half = head_dim // 2
    inv = [theta ** (-(2.0 * i) / head_dim) for i in range(half)]
    if scaling.type == "linear":
        return [f / scaling.factor for f in inv]
    if scaling.type == "llama3":
        orig = float(scaling.original_max_position_embeddings)
        long_wave = orig / scaling.low_freq_factor    # longer than this: fully scaled
        short_wave = orig / scaling.high_freq_factor  # shorter than this: untouched
        span = scaling.high_freq_factor - scaling.low_freq_factor
        scaled = []
        for f in inv:
            wave = 2.0 * math.pi / f
            if wave < short_wave:
                scaled.append(f)
            elif wave > long_wave:
                scaled.append(f / scaling.factor)
            else:
                t = (orig / wave - scaling.low_freq_factor) / span
                scaled.append((1.0 - t) * f / scaling.factor + t * f)
        return scaled
    return inv


def rope_tables(params: RotaryParams, num_positions: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos, sin [num_positions, D/2] float32 on the CPU."""
    inv = np.asarray(rope_inv_freq(params.head_dim, params.theta, params.scaling), dtype=np.float64)
    angle = np.arange(num_positions, dtype=np.float32)[:, None] * inv.astype(np.float32)[None, :]
    angle = angle.astype(np.float32).astype(np.float64)
    return (torch.from_numpy(np.cos(angle).astype(np.float32)),
            torch.from_numpy(np.sin(angle).astype(np.float32)))


@register("position", "rope")
class RotaryPosition(PositionEncoding):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        n = min(self.params.max_positions, rt.max_seq_len) if rt.max_seq_len > 0 else self.params.max_positions
        cos, sin = rope_tables(self.params, max(n, 1))
        self.cos = cos.to(rt.device)
        self.sin = sin.to(rt.device)

    def rotary_tables(self):
        return self.cos, self.sin

    def nbytes(self) -> int:
        return 2 * self.cos.numel() * 4


@register("position", "none")
class NoPosition(PositionEncoding):
    pass
