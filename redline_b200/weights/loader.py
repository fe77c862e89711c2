"""Loads a checkpoint's tensors by name into the parts of a model.

The model says which tensors it expects (name -> shape, optional or not); the
loader compares that with what the checkpoint holds and raises ONE error that lists
every missing tensor, every unexpected tensor and every wrong shape.  Then the
tensors go to the device, into ONE allocation, through two pinned staging buffers
that take turns, each in the engine's type: floating tensors stay bfloat16
(float16 is converted), except that a tensor stored in 32-bit stays 32-bit; in a
float32 engine everything floating becomes float32; integer tables become int32.
Tensors that a part uses as one (q, k and v; gate and up) are laid one after
another there, so that fusing them costs no second copy.
Error cases follow src/cuda/model/weights.cpp:180-246 and src/core/safetensors.cpp.
"""

from __future__ import annotations

import sys
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


def engine_dtype(stored: torch.dtype, spec: TensorSpec, dtype: torch.dtype) -> torch.dtype:
    """The type a tensor has in the engine: integer tables int32; floating tensors the engine's type,
    except that a tensor stored in 32-bit stays 32-bit."""
    if spec.integer or not stored.is_floating_point:
        return torch.int32
    if dtype == torch.float32 or stored == torch.float32:
        return torch.float32
    return torch.bfloat16


def to_engine(t: torch.Tensor, spec: TensorSpec, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    return t.to(device=device, dtype=engine_dtype(t.dtype, spec, dtype))


ALIGN = 256                 # every tensor starts on a 256-byte boundary of the blob
STAGE_BYTES = 64 << 20      # size of each of the two pinned staging buffers


class BlobUploader:
    """One device allocation for all weights, filled through two pinned host buffers that take turns:
    while the copy engine moves one to the device, the host converts and copies the next piece of the
    file into the other (reference: src/cuda/model/weights.cpp:15-46,129-174)."""

    def __init__(self, total_bytes: int, device: torch.device, stage_bytes: int = STAGE_BYTES):
        self.device = device
        self.blob = torch.empty(max(total_bytes, 1), dtype=torch.uint8, device=device)
        self.on_gpu = device.type == "cuda"
        if self.on_gpu:
            n = max(ALIGN, min(stage_bytes, (total_bytes + ALIGN - 1) // ALIGN * ALIGN))
            self.stage = [torch.empty(n, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
            self.events = [torch.cuda.Event(), torch.cuda.Event()]
            self.busy = [False, False]
            self.stream = torch.cuda.Stream(device)
            self.turn = 0

    def view(self, offset: int, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for x in shape:
            n *= int(x)
        esize = torch.empty((), dtype=dtype).element_size()
        return self.blob[offset:offset + n * esize].view(dtype).view(tuple(shape))

    def put(self, offset: int, src: torch.Tensor, dtype: torch.dtype) -> None:
        """Copies the CPU tensor ``src`` (converted to ``dtype``) to the blob at ``offset``."""
        flat = src.reshape(-1)
        esize = torch.empty((), dtype=dtype).element_size()
        if not self.on_gpu:
            self.blob[offset:offset + flat.numel() * esize].view(dtype).copy_(flat)
            return
        per = self.stage[0].numel() // esize
        for i in range(0, flat.numel(), per):
            piece = flat[i:i + per]
            b = self.turn & 1
            self.turn += 1
            if self.busy[b]:
                self.events[b].synchronize()              # the copy that last used this buffer has left it
            host = self.stage[b][:piece.numel() * esize].view(dtype)
            host.copy_(piece)                             # (converts float16 / float32 on the way if need be)
            with torch.cuda.stream(self.stream):
                self.blob[offset + i * esize:offset + (i + piece.numel()) * esize].view(dtype).copy_(host, non_blocking=True)
                self.events[b].record(self.stream)
            self.busy[b] = True

    def finish(self) -> None:
        if self.on_gpu:
            self.stream.synchronize()
            torch.cuda.current_stream(self.device).wait_stream(self.stream)


def load(reader: CheckpointReader, expected: Dict[str, TensorSpec], dtype: torch.dtype,
         device: torch.device, ignorable: Iterable[str] = (),
         fused: Dict[str, List[str]] = None) -> Dict[str, torch.Tensor]:
    """Checkpoint name -> device tensor for every expected tensor the file has, all of them views of ONE
    device allocation.  ``fused`` maps a name of the caller's choice to checkpoint names whose tensors
    are to lie one after another (along their first axis) as one tensor: a group all of whose members
    the file has, with the same trailing shape, comes back under that name as one tensor (in 32-bit if a
    member is stored in 32-bit) and its members do not come back singly."""
    check(reader, expected, ignorable)
    plan = []                      # (result name, [(checkpoint name, rows)], shape, dtype)
    grouped = set()
    for key, members in (fused or {}).items():
        if not members or not all(reader.has(m) and m in expected for m in members):
            continue
        shapes = [tuple(reader.info(m)[1]) for m in members]
        if any(len(sh) == 0 or sh[1:] != shapes[0][1:] for sh in shapes):
            continue
        dts = {engine_dtype(reader.tensor(m).dtype, expected[m], dtype) for m in members}
        dt = torch.float32 if torch.float32 in dts else next(iter(dts))
        if len(dts) > 1 and dts != {torch.float32, torch.bfloat16}:
            continue
        plan.append((key, list(members), (sum(sh[0] for sh in shapes),) + shapes[0][1:], dt))
        grouped.update(members)
    for n, s in expected.items():
        if reader.has(n) and n not in grouped:
            plan.append((n, [n], tuple(reader.info(n)[1]), engine_dtype(reader.tensor(n).dtype, s, dtype)))
    offsets, total = [], 0
    for _, _, shape, dt in plan:
        n = 1
        for x in shape:
            n *= int(x)
        offsets.append(total)
        total += (n * torch.empty((), dtype=dt).element_size() + ALIGN - 1) // ALIGN * ALIGN
    narrowed = sorted(m for _, members, _, dt in plan for m in members
                      if dt == torch.bfloat16 and reader.tensor(m).dtype == torch.float16)
    if narrowed:
        # said once and aloud: float16 has three more mantissa bits than the bfloat16 the engine computes in
        print(f"[redline_b200] {reader.model_dir}: {len(narrowed)} float16 tensors are converted to bfloat16 "
              f"(first: {narrowed[0]}); --dtype float32 keeps every stored bit", file=sys.stderr, flush=True)
    up = BlobUploader(total, device)
    out: Dict[str, torch.Tensor] = {}
    for (key, members, shape, dt), off in zip(plan, offsets):
        esize = torch.empty((), dtype=dt).element_size()
        at = off
        for m in members:
            t = reader.tensor(m)
            up.put(at, t, dt)
            at += t.numel() * esize
        out[key] = up.view(off, shape, dt)
    up.finish()
    return out
