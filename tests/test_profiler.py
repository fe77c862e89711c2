"""The work figures that the per-op profiler attaches to an op (bytes to move, floating-point
operations) and the table it prints: plain arithmetic, checked on the CPU."""

from types import SimpleNamespace

import torch

from redline_b200.engine.profiler import attention_work, format_op_profile, linear_work


def test_linear_work_counts_the_weight_once_and_two_flops_per_multiply_add():
    w = torch.empty(3072, 2048, dtype=torch.bfloat16)
    nbytes, flops = linear_work(8, w, 2, 2)
    assert nbytes == 3072 * 2048 * 2 + 8 * 2048 * 2 + 8 * 3072 * 2
    assert flops == 2 * 8 * 3072 * 2048


def test_attention_work_of_single_tokens_and_portions():
    host = SimpleNamespace(q_len=[1, 1, 5], start_pos=[99, 3, 10])
    w = attention_work(host, num_heads=4, num_kv_heads=2, head_dim=64, window=0, elem=2)
    kv_row, q_row = 2 * 2 * 64 * 2, 2 * 4 * 64 * 2
    assert w["decode"] == ((100 + 4) * kv_row + 2 * q_row, 4.0 * 4 * 64 * (100 + 4))
    pairs = 5 * 10 + 5 * 6 / 2            # rows see 11, 12, 13, 14, 15 keys
    assert pairs == 11 + 12 + 13 + 14 + 15
    assert w["prefill"] == (15 * kv_row + 5 * q_row, 4.0 * 4 * 64 * pairs)
    win = attention_work(host, 4, 2, 64, window=8, elem=2)
    assert win["decode"][1] == 4.0 * 4 * 64 * (8 + 4) and win["prefill"][1] == 4.0 * 4 * 64 * 5 * 8


def test_table_text_groups_ops_by_scope():
    rows = [{"op": "decode/embed", "ms_per_pass": 0.002, "calls_per_pass": 1, "pct": 10.0, "gb_s": 100.0, "tflop_s": 0.0},
            {"op": "decode/qkv_proj", "ms_per_pass": 0.018, "calls_per_pass": 16, "pct": 90.0, "gb_s": 3000.0,
             "tflop_s": 1.5, "roofline_frac": 0.46},
            {"op": "prefill/embed", "ms_per_pass": 0.01, "calls_per_pass": 1, "pct": 100.0}]
    text = format_op_profile(rows)
    assert text.count("per-op device time") == 2 and "qkv_proj" in text and "0.46" in text
