"""The tests' own small configurations, as HF ``config.json`` dictionaries.

TINY_A and TINY_B differ in every size and option the architecture has: layers,
width, heads, kv heads (group 2 and 3), head size, feed-forward width (704 is
5.5 x 128), vocabulary (1000 is no multiple of 16), rope base, rope scaling,
the norms' eps, tied or untied head.  TINY_C has a head size that is no power of
two and a width that is no multiple of 128.
"""

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 256,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "intermediate_size": 704,
    "vocab_size": 512,
    "rope_theta": 10000.0,
    "rope_scaling": None,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False,
    "max_position_embeddings": 2048,
    "hidden_act": "silu",
    "bos_token_id": 1,
    "eos_token_id": 2,
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 3,
    "hidden_size": 384,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "head_dim": 128,
    "intermediate_size": 1024,
    "vocab_size": 1000,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64,
    },
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "max_position_embeddings": 4096,
    "hidden_act": "silu",
    "bos_token_id": 0,
    "eos_token_id": [7, 9],
}

TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 200,
    "num_attention_heads": 5,
    "num_key_value_heads": 5,
    "head_dim": 48,
    "intermediate_size": 328,
    "vocab_size": 331,
    "rope_theta": 50000.0,
    "rope_scaling": {"rope_type": "linear", "factor": 2.0},
    "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False,
    "max_position_embeddings": 1024,
    "hidden_act": "silu",
    "bos_token_id": 1,
    "eos_token_id": 2,
}

ALL = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C}
