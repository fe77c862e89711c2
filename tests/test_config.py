"""Configuration: keys, defaults, errors, the architecture registry."""

import json
import math
import os

import pytest

import tiny_configs as C
from redline_b200.config import (ConfigError, EngineConfig, LlamaConfig, RopeScaling, config_from_dict,
                                 known_architectures, load_config, model_spec)
from redline_b200.parts.rope import RotaryParams, rope_inv_freq, rope_tables


def test_llama_keys_and_defaults():
    c = config_from_dict(C.TINY_B)
    assert isinstance(c, LlamaConfig)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 384, 3, 1)
    assert c.head_dim == 128 and c.gqa_group == 3 and c.q_size == 384 and c.kv_size == 128
    assert c.rope_scaling == RopeScaling("llama3", 8.0, 1.0, 4.0, 64)
    assert c.tie_word_embeddings and c.eos_token_ids == (7, 9) and c.bos_token_id == 0
    d = dict(C.TINY_A)
    for k in ("num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "rope_scaling",
              "tie_word_embeddings", "max_position_embeddings", "bos_token_id", "eos_token_id"):
        d.pop(k)
    c = config_from_dict(d)
    assert c.num_key_value_heads == 4 and c.head_dim == 64 and c.rms_norm_eps == 1e-5
    assert c.rope_theta == 10000.0 and c.rope_scaling.type == "none" and not c.tie_word_embeddings
    assert c.max_position_embeddings == 4096 and c.bos_token_id == -1 and c.eos_token_ids == ()


def test_rope_parameters_spelling_and_legacy_type_key():
    d = dict(C.TINY_A)
    d.pop("rope_theta"), d.pop("rope_scaling")
    d["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "linear", "factor": 4.0}
    c = config_from_dict(d)
    assert c.rope_theta == 12345.0 and c.rope_scaling == RopeScaling("linear", 4.0)
    d = dict(C.TINY_A, rope_scaling={"type": "llama3", "factor": 2.0})
    c = config_from_dict(d)
    assert c.rope_scaling == RopeScaling("llama3", 2.0, 1.0, 4.0, 8192)


@pytest.mark.parametrize("patch,word", [
    ({"architectures": ["MambaForCausalLM"]}, "not supported"),
    ({"architectures": None}, "architectures"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 63}, "even"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "linear"}}, "factor"),
    ({"vocab_size": None}, "vocab_size"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_config_errors_name_the_fault(patch, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict(dict(C.TINY_A, **patch))
    assert word in str(e.value)


def test_unknown_architecture_lists_known():
    with pytest.raises(ConfigError) as e:
        config_from_dict(dict(C.TINY_A, architectures=["Nope"]))
    assert "LlamaForCausalLM" in str(e.value) and "LlamaForCausalLM" in known_architectures()


def test_round_trip_through_a_folder(tmp_path):
    c = config_from_dict(C.TINY_B)
    c.save(str(tmp_path))
    assert load_config(str(tmp_path)) == c
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [1, 2, 3]}))
    assert load_config(str(tmp_path)).eos_token_ids == (1, 2, 3)
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "missing"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_spec_is_data_with_sizes_from_the_configuration():
    c = config_from_dict(C.TINY_B)
    s = model_spec(c)
    assert len(s.layers) == 3 and [k.layer for k in s.order] == [0, 1, 2]
    assert all(k.cache_of is None for k in s.order)
    m = s.layers[1].mixer
    assert m.kind == "gqa_attention" and m.params.num_kv_heads == 1 and m.params.head_dim == 128
    assert m.params.position.kind == "rope" and m.params.position.params.theta == 500000.0
    assert m.names["q"] == "model.layers.1.self_attn.q_proj.weight"
    assert s.layers[2].ffn.params.intermediate_size == 1024 and s.layers[0].mixer_norm.params.eps == 1e-5
    assert s.head.params.tied and s.head.names["weight"] == "lm_head.weight"


def test_rope_tables_follow_the_formula():
    p = RotaryParams(128, 500000.0, RopeScaling("llama3", 8.0, 1.0, 4.0, 64), 4096)
    inv = rope_inv_freq(p.head_dim, p.theta, p.scaling)
    base = rope_inv_freq(p.head_dim, p.theta, RopeScaling())
    assert inv[0] == base[0] and inv[-1] == pytest.approx(base[-1] / 8.0)
    cos, sin = rope_tables(p, 50)
    assert cos.shape == (50, 64) and float(cos[0].min()) == 1.0 and float(sin[0].abs().max()) == 0.0
    assert float(cos[7, 0]) == pytest.approx(math.cos(7.0), abs=1e-6)
    import plain_llama as P
    pc, ps = P.rope_tables(P.plain_config(C.TINY_B), 50)
    assert (pc.float() - cos).abs().max() < 1e-6 and (ps.float() - sin).abs().max() < 1e-6


def test_engine_options():
    c = EngineConfig.from_options("m", {"max_seqs": 4, "max_batched_tokens": 64, "dtype": "float32", "device": None})
    assert c.max_num_seqs == 4 and c.max_num_batched_tokens == 64 and c.logit_rows == 64
    with pytest.raises(TypeError):
        EngineConfig.from_options("m", {"max_sequences": 4})
    with pytest.raises(ValueError):
        EngineConfig.from_options("m", {"block_size": 8})
    with pytest.raises(ValueError):
        EngineConfig.from_options("m", {"dtype": "float16"})
