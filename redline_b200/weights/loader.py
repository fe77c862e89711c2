"""Loads a checkpoint's tensors by name into the parts of a model.

The model says which tensors it expects (name -> shape, optional or not); the
loader compares that with what the checkpoint holds and raises ONE error that lists
every missing tensor, every unexpected tensor and every wrong shape.  Then each
tensor goes to the device in the engine's type: floating tensors stay bfloat16
(float16 is converted), except that a tensor stored in 32-bit stays 32-bit; in a
float32 engine everything floating becomes float32; integer tables become int32.
Error cases follow src/cuda/model/weights.cpp:180-246 and src/core/safetensors.cpp.
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Tuple

import torch

from ..parts.spec import TensorSpec
from .safetensors_io import CheckpointReader

# Buffers some exporters write that no part asks for; they are recomputed here.
IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


class WeightsError(ValueError):
    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"{where}: checkpoint does not match the model"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(exp)}" for n, got, exp in wrong))
        super().__init__("\n".join(lines))


def check(reader: CheckpointReader, expected: Dict[str, TensorSpec], ignorable: Iterable[str] = ()) -> None:
    have = set(reader.names())
    ignorable = set(ignorable)
    missing = sorted(n for n, s in expected.items() if n not in have and not s.optional)
    unexpected = sorted(n for n in have if n not in expected and n not in ignorable
                        and not n.endswith(IGNORED_SUFFIXES))
    wrong = []
    for n, s in sorted(expected.items()):
        if n in have:
            _, shape = reader.info(n)
            if tuple(shape) != tuple(s.shape):
                wrong.append((n, tuple(shape), tuple(s.shape)))
    if missing or unexpected or wrong:
        raise WeightsError(reader.model_dir, missing, unexpected, wrong)


def to_engine(t: torch.Tensor, spec: TensorSpec, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    if spec.integer or not t.dtype.is_floating_point:
        return t.to(device=device, dtype=torch.int32)
    if dtype == torch.float32 or t.dtype == torch.float32:
        return t.to(device=device, dtype=torch.float32)
    return t.to(device=device, dtype=torch.bfloat16)


def load(reader: CheckpointReader, expected: Dict[str, TensorSpec], dtype: torch.dtype,
         device: torch.device, ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Checkpoint name -> device tensor for every expected tensor the file has."""
    check(reader, expected, ignorable)
    out = {}
    for n, s in expected.items():
        if reader.has(n):
            out[n] = to_engine(reader.tensor(n), s, dtype, device).contiguous()
    return out
