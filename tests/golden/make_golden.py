"""Makes tests/golden/*.npz: logits of the reference project's own CPU model.

Usage:  python tests/golden/make_golden.py /path/to/redline_ref

``redline_ref`` is the reference's CPU oracle, built from its unmodified source
with ``cmake -S <reference> -B build -DREDLINE_BUILD_CUDA=OFF && cmake --build
build --target redline_ref``.  For TINY_A and TINY_B this script draws the tests'
seeded weights (tests/plain_llama.py: random_weights), writes them in the
reference's model-file layout (fused ``wqkv`` and ``w_gate_up``, the configuration
as ``redline_config`` metadata; python/redline/format.py:1-25,
python/redline/convert.py:194-272), runs ``redline_ref --tokens ... --logits-out``
and stores its float32 logits with the token ids.  tests/test_plain.py compares
the plain implementation with these files; nothing else reads them.
"""

import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import plain_llama as P  # noqa: E402
import tiny_configs  # noqa: E402

CASES = {
    # name: (config, seed, sharpen, number of tokens)
    "tiny_a": (tiny_configs.TINY_A, 11, 8.0, 24),
    "tiny_b": (tiny_configs.TINY_B, 12, 8.0, 20),
}


def rlm_tensors(c: P.PlainConfig, w: dict) -> dict:
    out = {"tok_embeddings.weight": w["model.embed_tokens.weight"]}
    for i in range(c.num_layers):
        p, q = f"model.layers.{i}.", f"layers.{i}."
        out[q + "attn_norm.weight"] = w[p + "input_layernorm.weight"]
        out[q + "wqkv.weight"] = torch.cat(
            [w[p + f"self_attn.{n}_proj.weight"] for n in "qkv"], dim=0)
        out[q + "wo.weight"] = w[p + "self_attn.o_proj.weight"]
        out[q + "ffn_norm.weight"] = w[p + "post_attention_layernorm.weight"]
        out[q + "w_gate_up.weight"] = torch.cat(
            [w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]], dim=0)
        out[q + "w_down.weight"] = w[p + "mlp.down_proj.weight"]
    out["norm.weight"] = w["model.norm.weight"]
    if "lm_head.weight" in w:
        out["lm_head.weight"] = w["lm_head.weight"]
    return out


def redline_config(c: P.PlainConfig) -> dict:
    d = {
        "architecture": "llama", "vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
        "intermediate_size": c.intermediate_size, "num_layers": c.num_layers,
        "num_heads": c.num_heads, "num_kv_heads": c.num_kv_heads, "head_dim": c.head_dim,
        "rms_norm_eps": c.rms_norm_eps, "rope_theta": c.rope_theta,
        "max_position_embeddings": c.max_position_embeddings,
        "tie_word_embeddings": c.tie_word_embeddings,
    }
    if c.rope_scaling:
        d["rope_scaling"] = dict(c.rope_scaling)
    return d


def main():
    ref_bin = sys.argv[1]
    here = os.path.dirname(os.path.abspath(__file__))
    for name, (cfg_json, seed, sharpen, ntok) in CASES.items():
        c = P.plain_config(cfg_json)
        w = P.random_weights(cfg_json, seed, sharpen)
        tokens = np.random.RandomState(seed).randint(0, c.vocab_size, size=ntok).tolist()
        with tempfile.TemporaryDirectory() as tmp:
            model = os.path.join(tmp, "m.rlm")
            P.write_safetensors(model, rlm_tensors(c, w),
                                {"format": "redline", "redline_config": json.dumps(redline_config(c))})
            out = os.path.join(tmp, "logits.f32")
            subprocess.run([ref_bin, "--model", model, "--tokens", ",".join(map(str, tokens)),
                            "--logits-out", out], check=True)
            logits = np.fromfile(out, dtype=np.float32).reshape(ntok, c.vocab_size)
        np.savez_compressed(os.path.join(here, name + ".npz"), tokens=np.asarray(tokens, dtype=np.int32),
                            logits=logits, seed=seed, sharpen=sharpen)
        print(name, logits.shape, float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
