"""Options of the engine, with the reference's names and defaults
(src/cuda/engine/engine.h:37-66, apps/cli_common.cpp:68-118) minus quantisation and
speculation, plus the compute type."""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Dict

import torch

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


@dataclass
class EngineConfig:
    model: str = ""
    dtype: str = "bfloat16"
    max_num_seqs: int = 32
    max_num_batched_tokens: int = 2048
    max_seq_len: int = 4096
    max_logit_rows: int = 0            # 0: max(max_num_seqs, 64)
    block_size: int = 16               # tokens per cache page
    kv_cache_tokens: int = 0           # 0: from the memory budget
    gpu_memory_utilization: float = 0.90
    cuda_graphs: bool = True
    async_scheduling: bool = True
    mix_prefill_decode: bool = True
    admission_watermark: float = 0.01
    nvtx_layers: bool = False          # one NVTX range per step and per layer call (for nsys timelines)
    track_memory: bool = False         # sample the device's used memory every step (peak in memory_report)
    device: int = 0

    # names the reference's Python entry point and command line use for the same options
    ALIASES = {"max_seqs": "max_num_seqs", "max_batched_tokens": "max_num_batched_tokens"}

    @classmethod
    def from_options(cls, model: str, options: Dict[str, Any]) -> "EngineConfig":
        known = {f.name for f in fields(cls)}
        kw: Dict[str, Any] = {"model": model}
        for k, v in options.items():
            if v is None:
                continue
            k = cls.ALIASES.get(k, k)
            if k not in known:
                raise TypeError(f"unknown engine option '{k}' (known: {sorted(known | set(cls.ALIASES))})")
            kw[k] = v
        c = cls(**kw)
        c.validate()
        return c

    def validate(self) -> None:
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {self.dtype}")
        if self.block_size not in (16, 32, 64):
            raise ValueError(f"block_size must be 16, 32 or 64, got {self.block_size}")
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0 or self.max_seq_len <= 1:
            raise ValueError("max_num_seqs, max_num_batched_tokens and max_seq_len must be positive")
        if self.max_num_batched_tokens < self.max_num_seqs:
            raise ValueError("max_num_batched_tokens must be >= max_num_seqs")

    @property
    def torch_dtype(self) -> torch.dtype:
        return DTYPES[self.dtype]

    @property
    def logit_rows(self) -> int:
        return self.max_logit_rows if self.max_logit_rows > 0 else max(self.max_num_seqs, 64)
