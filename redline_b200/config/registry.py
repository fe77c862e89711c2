"""One registry from an architecture's name (``architectures[0]`` of config.json)
to its configuration class and its factory of a ``ModelSpec``.

Adding an architecture = one call of ``register_architecture`` with a function that
reads the architecture's config.json keys and a function that lays the model out
as parts; nothing in the engine, the cache or the scheduler changes.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional

from .model_config import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_hf: Callable[[Dict[str, Any], Optional[str]], ModelConfig]
    build_spec: Callable[[ModelConfig], Any]   # -> parts.spec.ModelSpec
    random_tensors: Optional[Callable] = None  # (config, seed, dtype) -> iterator of (name, tensor)


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def known_architectures():
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture '{name}' is not supported; known: {known_architectures()}")
    return _ARCHITECTURES[name]


def _ensure_builtin() -> None:
    from .. import models  # noqa: F401  (registers the built-in architectures)


def config_from_dict(cfg: Dict[str, Any], model_dir: Optional[str] = None) -> ModelConfig:
    archs = cfg.get("architectures")
    if not archs:
        raise ConfigError("config.json has no 'architectures'")
    return get_architecture(archs[0]).config_from_hf(cfg, model_dir)


def load_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path) as f:
            cfg = json.load(f)
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e.strerror}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    return config_from_dict(cfg, model_dir)


def model_spec(config: ModelConfig):
    return get_architecture(config.architecture).build_spec(config)
