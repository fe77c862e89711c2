"""Safetensors reading and writing, the loader's one error, the random-weights mode."""

import json
import os
import struct

import pytest
import torch

import plain_llama as P
import tiny_configs as C
from redline_b200.config import config_from_dict, model_spec
from redline_b200.engine.model import DecoderModel
from redline_b200.parts.base import Runtime
from redline_b200.weights import (CheckpointReader, SafetensorsError, SafetensorsFile, WeightsError, save_file,
                                  write_random_model)


def cpu_model(cfg_json, dtype=torch.bfloat16):
    rt = Runtime(torch.device("cpu"), dtype, 64, 4, 256, 16)
    return DecoderModel(model_spec(config_from_dict(cfg_json)), rt)


def test_round_trip_and_foreign_reader(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "d": torch.randn(2, 2).to(torch.float16), "e": torch.zeros(0, 4)}
    path = str(tmp_path / "x.safetensors")
    save_file(path, t, {"k": "v"})
    f = SafetensorsFile(path)
    assert f.metadata == {"k": "v"} and sorted(f.names()) == sorted(t)
    for n, x in t.items():
        assert f.info(n)[1] == tuple(x.shape) and torch.equal(f.tensor(n), x)
    st = pytest.importorskip("safetensors.torch")     # an independent reader agrees
    other = st.load_file(path)
    assert all(torch.equal(other[n], x) for n, x in t.items())
    # and the tests' own writer is read by the product reader
    P.write_safetensors(path, t)
    assert all(torch.equal(SafetensorsFile(path).tensor(n), x) for n, x in t.items())


def test_reader_errors(tmp_path):
    p = str(tmp_path / "x.safetensors")
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFile(p)
    open(p, "wb").write(b"abc")
    with pytest.raises(SafetensorsError, match="too small"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="corrupt header"):
        SafetensorsFile(p)
    h = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(h)) + h + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(p)
    h = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(h)) + h + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 16"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        CheckpointReader(str(tmp_path / "nowhere"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    w = P.random_weights(C.TINY_A, 0, dtype=torch.bfloat16)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 256, dtype=torch.bfloat16)
    w["model.layers.5.extra.weight"] = torch.zeros(3)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(32)   # tolerated
    P.write_model_dir(str(tmp_path), C.TINY_A, w)
    m = cpu_model(C.TINY_A)
    with pytest.raises(WeightsError) as e:
        m.load_weights(CheckpointReader(str(tmp_path)))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.5.extra.weight"]
    assert err.wrong == [("model.layers.0.self_attn.k_proj.weight", (64, 256), (128, 256))]
    msg = str(err)
    for word in ("missing", "unexpected", "wrong shapes", "up_proj", "extra", "[64, 256]", "[128, 256]"):
        assert word in msg


def test_dtypes_kept_and_head_tied(tmp_path, capsys):
    w = P.random_weights(C.TINY_B, 1, dtype=torch.bfloat16)
    w["model.norm.weight"] = w["model.norm.weight"].float()               # stored in 32-bit: stays
    w["model.layers.0.mlp.down_proj.weight"] = w["model.layers.0.mlp.down_proj.weight"].to(torch.float16)
    P.write_model_dir(str(tmp_path), C.TINY_B, w)
    m = cpu_model(C.TINY_B)
    capsys.readouterr()
    m.load_weights(CheckpointReader(str(tmp_path)))
    said = capsys.readouterr().err                                          # float16 is narrowed, and said so
    assert "1 float16 tensors are converted to bfloat16" in said and "down_proj" in said
    assert m.final_norm.weight.dtype == torch.float32
    assert m.blocks[0].ffn.w_down.dtype == torch.bfloat16
    assert m.embedding.weight.dtype == torch.bfloat16
    assert m.head.weight.data_ptr() == m.embedding.weight.data_ptr() and m.head.nbytes() == 0
    q = w["model.layers.2.self_attn.q_proj.weight"]
    assert torch.equal(m.blocks[2].mixer.w_qkv[:q.shape[0]], q)
    m32 = cpu_model(C.TINY_B, torch.float32)
    m32.load_weights(CheckpointReader(str(tmp_path)))
    assert "float16" not in capsys.readouterr().err                         # (a float32 engine keeps every bit)
    assert m32.embedding.weight.dtype == torch.float32 and m32.blocks[1].mixer.w_qkv.dtype == torch.float32
    # untied configuration whose file has no lm_head: the table is shared all the same
    wa = P.random_weights(C.TINY_A, 1, dtype=torch.bfloat16)
    del wa["lm_head.weight"]
    P.write_model_dir(str(tmp_path / "a"), C.TINY_A, wa)
    ma = cpu_model(C.TINY_A)
    ma.load_weights(CheckpointReader(str(tmp_path / "a")))
    assert ma.head.weight.data_ptr() == ma.embedding.weight.data_ptr()


def test_weights_lie_in_one_allocation_with_fused_tensors_side_by_side(tmp_path):
    """Every weight is a view of one allocation; q, k and v (and gate and up) are laid one after another
    there, so the fused tensors a layer multiplies by cost no second copy; a member stored in 32-bit
    makes its fused tensor 32-bit."""
    w = P.random_weights(C.TINY_B, 2, dtype=torch.bfloat16)
    w["model.layers.1.self_attn.k_proj.weight"] = w["model.layers.1.self_attn.k_proj.weight"].float()
    P.write_model_dir(str(tmp_path), C.TINY_B, w)
    m = cpu_model(C.TINY_B)
    m.load_weights(CheckpointReader(str(tmp_path)))
    tensors = [m.embedding.weight, m.final_norm.weight]
    for i, b in enumerate(m.blocks):
        p = f"model.layers.{i}."
        qkv = torch.cat([w[p + f"self_attn.{n}_proj.weight"].float() for n in "qkv"])
        assert torch.equal(b.mixer.w_qkv.float(), qkv)
        gu = torch.cat([w[p + f"mlp.{n}_proj.weight"] for n in ("gate", "up")])
        assert torch.equal(b.ffn.w_gate_up, gu)
        assert b.mixer.w_qkv.dtype == (torch.float32 if i == 1 else torch.bfloat16)
        tensors += [b.mixer.w_qkv, b.mixer.w_o, b.ffn.w_gate_up, b.ffn.w_down, b.mixer_norm.weight, b.ffn_norm.weight]
    base = tensors[0].untyped_storage().data_ptr()
    assert all(t.untyped_storage().data_ptr() == base for t in tensors)
    assert all((t.data_ptr() - base) % 256 == 0 and t.is_contiguous() for t in tensors)
    spans = sorted((t.data_ptr(), t.data_ptr() + t.numel() * t.element_size()) for t in tensors)
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))          # no two tensors overlap


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    c = config_from_dict(C.TINY_A)
    d = write_random_model(str(tmp_path / "m"), c, seed=3)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    r = CheckpointReader(d)
    m = cpu_model(C.TINY_A)
    m.load_weights(r)
    e = r.tensor("model.embed_tokens.weight").float()
    n = r.tensor("model.layers.0.input_layernorm.weight").float()
    assert r.info("model.embed_tokens.weight")[0] == "BF16"
    assert abs(float(e.std()) - 0.02) < 0.002 and abs(float(n.mean()) - 1.0) < 0.03 and 0.05 < float(n.std()) < 0.15
    write_random_model(str(tmp_path / "m2"), c, seed=3)
    write_random_model(str(tmp_path / "m3"), c, seed=4)
    a, b, c3 = (CheckpointReader(str(tmp_path / x)).tensor("model.layers.1.mlp.down_proj.weight") for x in ("m", "m2", "m3"))
    assert torch.equal(a, b) and not torch.equal(a, c3)
