"""Random-weights mode: writes a model folder (config.json, model.safetensors) from
a configuration and a seed, which then loads like any checkpoint.  Matrices are
N(0, 0.02^2), norm weights 1 + N(0, 0.1^2); tensors are drawn and written one at a
time (the reference's writer of random test models: src/cpu/random_model.cpp:19-171)."""

from __future__ import annotations

import os

import torch

from ..config.model_config import ModelConfig
from ..config.registry import get_architecture
from .safetensors_io import SafetensorsWriter


def write_random_model(model_dir: str, config: ModelConfig, seed: int = 0,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    arch = get_architecture(config.architecture)
    if arch.random_tensors is None:
        raise NotImplementedError(f"{config.architecture} has no random-weights generator")
    os.makedirs(model_dir, exist_ok=True)
    config.save(model_dir)
    plan = [(name, dtype, shape) for name, shape, _ in arch.random_tensors(config, seed, dtype)]
    w = SafetensorsWriter(os.path.join(model_dir, "model.safetensors"), plan, {"format": "pt"})
    for name, _, make in arch.random_tensors(config, seed, dtype):
        w.write(name, make())
    w.close()
    return model_dir
