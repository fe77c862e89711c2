"""Typed model configurations read from an architecture's own ``config.json`` keys.

``ModelConfig`` is what the rest of the framework may ask of any architecture;
``LlamaConfig`` holds what ``LlamaForCausalLM`` adds.  Keys, defaults and the
accepted rope-scaling types follow the reference's reading of HF configs
(python/redline/convert.py:86-150) and its validation
(src/core/model_config.cpp:97-116).  No size or constant that ``config.json``
gives is repeated anywhere else in the package.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A ``config.json`` that cannot be used, with the key that is at fault."""


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of rotary embeddings (src/core/model_config.h:26-32)."""

    type: str = "none"  # none | linear | llama3
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @staticmethod
    def from_hf(cfg: Dict[str, Any]) -> Tuple[float, "RopeScaling"]:
        """Returns (rope_theta, scaling) from ``rope_scaling`` / ``rope_parameters``
        and ``rope_theta`` (python/redline/convert.py:86-105)."""
        params = cfg.get("rope_parameters") or {}
        scaling = cfg.get("rope_scaling") or params or None
        theta = float(cfg.get("rope_theta", params.get("rope_theta", 10000.0)))
        if not scaling:
            return theta, RopeScaling()
        rtype = scaling.get("rope_type", scaling.get("type", "default"))
        if rtype in ("default", None, "none"):
            return theta, RopeScaling()
        if rtype == "linear":
            return theta, RopeScaling(type="linear", factor=float(_need(scaling, "factor", "rope_scaling")))
        if rtype == "llama3":
            return theta, RopeScaling(
                type="llama3",
                factor=float(_need(scaling, "factor", "rope_scaling")),
                low_freq_factor=float(scaling.get("low_freq_factor", 1.0)),
                high_freq_factor=float(scaling.get("high_freq_factor", 4.0)),
                original_max_position_embeddings=int(
                    scaling.get("original_max_position_embeddings", 8192)),
            )
        raise ConfigError(f"rope_scaling type '{rtype}' is not supported (none, default, linear, llama3)")

    def to_hf(self) -> Optional[Dict[str, Any]]:
        if self.type == "none":
            return None
        if self.type == "linear":
            return {"rope_type": "linear", "factor": self.factor}
        return {
            "rope_type": "llama3",
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


def _need(d: Dict[str, Any], key: str, where: str = "config.json") -> Any:
    if key not in d or d[key] is None:
        raise ConfigError(f"{where} has no '{key}'")
    return d[key]


@dataclass(frozen=True)
class ModelConfig:
    """What every architecture's configuration gives the engine."""

    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    bos_token_id: int
    eos_token_ids: Tuple[int, ...]

    def to_hf(self) -> Dict[str, Any]:  # pragma: no cover - overridden
        raise NotImplementedError

    def save(self, model_dir: str) -> None:
        os.makedirs(model_dir, exist_ok=True)
        with open(os.path.join(model_dir, "config.json"), "w") as f:
            json.dump(self.to_hf(), f, indent=1)


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    """``LlamaForCausalLM``: pre-norm decoder, RMSNorm, grouped-query attention with
    rotary embeddings, SiLU-gated feed-forward (src/cuda/model/llama.cpp:56-151)."""

    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    attention_bias: bool = False
    mlp_bias: bool = False
    tie_word_embeddings: bool = False

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def gqa_group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @classmethod
    def from_hf(cls, cfg: Dict[str, Any], model_dir: Optional[str] = None) -> "LlamaConfig":
        archs = cfg.get("architectures") or ["LlamaForCausalLM"]
        act = cfg.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act '{act}' is not supported: the feed-forward is SiLU-gated")
        theta, scaling = RopeScaling.from_hf(cfg)
        heads = int(_need(cfg, "num_attention_heads"))
        hidden = int(_need(cfg, "hidden_size"))
        eos = cfg.get("eos_token_id")
        if model_dir is not None:
            gen = os.path.join(model_dir, "generation_config.json")
            if os.path.exists(gen):
                with open(gen) as f:
                    eos = json.load(f).get("eos_token_id", eos)
        if eos is None:
            eos = []
        elif isinstance(eos, int):
            eos = [eos]
        bos = cfg.get("bos_token_id")
        c = cls(
            architecture=archs[0],
            vocab_size=int(_need(cfg, "vocab_size")),
            hidden_size=hidden,
            max_position_embeddings=int(cfg.get("max_position_embeddings", 4096)),
            bos_token_id=int(bos) if bos is not None else -1,
            eos_token_ids=tuple(int(e) for e in eos),
            intermediate_size=int(_need(cfg, "intermediate_size")),
            num_hidden_layers=int(_need(cfg, "num_hidden_layers")),
            num_attention_heads=heads,
            num_key_value_heads=int(cfg.get("num_key_value_heads") or heads),
            head_dim=int(cfg.get("head_dim") or hidden // heads),
            rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-5)),
            rope_theta=theta,
            rope_scaling=scaling,
            attention_bias=bool(cfg.get("attention_bias", False)),
            mlp_bias=bool(cfg.get("mlp_bias", False)),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        )
        c.validate()
        return c

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim must be even for rotary embeddings, got {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.rope_scaling.type != "none" and not self.rope_scaling.factor > 0:
            raise ConfigError("rope_scaling.factor must be positive")
        if self.rope_scaling.type == "llama3" and \
                self.rope_scaling.high_freq_factor == self.rope_scaling.low_freq_factor:
            raise ConfigError("rope_scaling: high_freq_factor must differ from low_freq_factor")

    def to_hf(self) -> Dict[str, Any]:
        eos: Any = list(self.eos_token_ids)
        if len(eos) == 1:
            eos = eos[0]
        elif not eos:
            eos = None
        return {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_hf(),
            "max_position_embeddings": self.max_position_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "tie_word_embeddings": self.tie_word_embeddings,
            "bos_token_id": self.bos_token_id if self.bos_token_id >= 0 else None,
            "eos_token_id": eos,
            "torch_dtype": "bfloat16",
        }
