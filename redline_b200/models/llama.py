"""``LlamaForCausalLM`` laid out as parts: token embedding, ``num_hidden_layers``
pre-norm blocks of (RMSNorm, grouped-query attention with rotary embeddings,
RMSNorm, SiLU-gated feed-forward), a final RMSNorm and the head, which shares the
embedding table when the configuration ties it or the checkpoint has no
``lm_head.weight``.  Tensor names are HF's (reference: python/redline/convert.py:
194-272 maps the same names onto its own fused ones).
"""

from __future__ import annotations

from typing import Iterator, Tuple

import torch

from ..config.model_config import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..parts.attention import AttentionParams
from ..parts.embedding import EmbeddingParams, HeadParams
from ..parts.mlp import GatedMLPParams
from ..parts.rmsnorm import RMSNormParams
from ..parts.rope import RotaryParams
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def llama_spec(c: LlamaConfig) -> ModelSpec:
    position = PartSpec("rope", RotaryParams(c.head_dim, c.rope_theta, c.rope_scaling, c.max_position_embeddings))
    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        attn_names = {n: f"{p}self_attn.{n}_proj.weight" for n in "qkvo"}
        attn_names.update({f"{n}_bias": f"{p}self_attn.{n}_proj.bias" for n in "qkvo"})
        mlp_names = {n: f"{p}mlp.{n}_proj.weight" for n in ("gate", "up", "down")}
        mlp_names.update({f"{n}_bias": f"{p}mlp.{n}_proj.bias" for n in ("gate", "up", "down")})
        layers.append(LayerSpec(
            arrangement="prenorm",
            mixer_norm=PartSpec("rmsnorm", RMSNormParams(c.hidden_size, c.rms_norm_eps),
                                {"weight": p + "input_layernorm.weight"}),
            mixer=PartSpec("gqa_attention",
                           AttentionParams(c.hidden_size, c.num_attention_heads, c.num_key_value_heads,
                                           c.head_dim, position, bias=c.attention_bias,
                                           out_bias=c.attention_bias),
                           attn_names),
            ffn_norm=PartSpec("rmsnorm", RMSNormParams(c.hidden_size, c.rms_norm_eps),
                              {"weight": p + "post_attention_layernorm.weight"}),
            ffn=PartSpec("swiglu_mlp", GatedMLPParams(c.hidden_size, c.intermediate_size, bias=c.mlp_bias),
                         mlp_names),
        ))
    return ModelSpec(
        hidden_size=c.hidden_size,
        vocab_size=c.vocab_size,
        max_positions=c.max_position_embeddings,
        embedding=PartSpec("token_embedding", EmbeddingParams(c.vocab_size, c.hidden_size),
                           {"weight": "model.embed_tokens.weight"}),
        layers=tuple(layers),
        order=tuple(LayerCall(i) for i in range(c.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", RMSNormParams(c.hidden_size, c.rms_norm_eps), {"weight": "model.norm.weight"}),
        head=PartSpec("lm_head", HeadParams(c.vocab_size, c.hidden_size, c.tie_word_embeddings),
                      {"weight": "lm_head.weight"}),
    )


def llama_random_tensors(c: LlamaConfig, seed: int, dtype: torch.dtype) -> Iterator[Tuple[str, tuple, object]]:
    """Yields (name, shape, make) in file order; ``make()`` draws the tensor: matrices
    N(0, 0.02^2), norm weights 1 + N(0, 0.1^2), one seeded generator run in order."""
    g = torch.Generator().manual_seed(seed)

    def mat(n, k):
        return lambda: (torch.randn(n, k, generator=g) * 0.02).to(dtype)

    def norm(n):
        return lambda: (1.0 + 0.1 * torch.randn(n, generator=g)).to(dtype)

    H, D, I = c.hidden_size, c.head_dim, c.intermediate_size
    yield "model.embed_tokens.weight", (c.vocab_size, H), mat(c.vocab_size, H)
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        yield p + "input_layernorm.weight", (H,), norm(H)
        yield p + "self_attn.q_proj.weight", (c.q_size, H), mat(c.q_size, H)
        yield p + "self_attn.k_proj.weight", (c.kv_size, H), mat(c.kv_size, H)
        yield p + "self_attn.v_proj.weight", (c.kv_size, H), mat(c.kv_size, H)
        yield p + "self_attn.o_proj.weight", (H, c.q_size), mat(H, c.q_size)
        yield p + "post_attention_layernorm.weight", (H,), norm(H)
        yield p + "mlp.gate_proj.weight", (I, H), mat(I, H)
        yield p + "mlp.up_proj.weight", (I, H), mat(I, H)
        yield p + "mlp.down_proj.weight", (H, I), mat(H, I)
    yield "model.norm.weight", (H,), norm(H)
    if not c.tie_word_embeddings:
        yield "lm_head.weight", (c.vocab_size, H), mat(c.vocab_size, H)


register_architecture(Architecture(
    name="LlamaForCausalLM",
    config_from_hf=LlamaConfig.from_hf,
    build_spec=llama_spec,
    random_tensors=llama_random_tensors,
))
