"""bench.py's host-side parts: the byte and FLOP counts of its roofline, the summary of the clock
samples, and the refusal of more than one GPU (no kernels run)."""

import os
import subprocess
import sys

import bench

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bytes_and_flops_of_the_bench_configuration():
    cfg = dict(bench.BENCH_CONFIG)
    n = bench.model_numbers(cfg)
    L, H, I, V = 16, 2048, 8192, 128256
    assert (cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]) == (L, H, I, V)
    per_layer = 3072 * H + H * 2048 + 3 * I * H                       # qkv, o, gate + up + down
    assert n["layer_mat"] == per_layer
    assert n["weight_bytes"] == 2.0 * (L * (per_layer + 2 * H) + V * H + H)
    assert n["kv_bytes_per_token"] == 2 * 2 * L * 8 * 64              # k and v, bfloat16, 8 kv heads of 64
    T = 2048
    flops = bench.prefill_flops(cfg, T)
    gemm = 2.0 * T * per_layer * L + 2.0 * V * H
    attn = L * 32 * 4.0 * 64 * (T * (T + 1) / 2)
    assert abs(flops - (gemm + attn)) < 1e-6 * flops
    assert 0.06 < attn / flops < 0.08                                 # the attention's share at 2,048 tokens


def test_clock_summary_takes_the_timed_samples_and_widens_a_short_region():
    s = bench.ClockSampler(0)
    line = "{}, 1965, 700.0, Not Active, Not Active, Not Active, {}"
    s.lines = [line.format(1500, "Not Active")] * 6 + [line.format(1900 + i, "Active") for i in range(5)]
    full = s.summary(6, 11)
    assert full["samples"] == 5 and full["sm_mhz"] == 1902.0 and full["sm_max_mhz"] == 1965.0
    assert full["reasons"] == ["sw_power_cap"] and full["widened"] is False
    short = s.summary(10, 11)                                         # one sample only: the warm-up before it counts too
    assert short["widened"] is True and short["samples"] == 8 and short["sm_mhz"] >= 1500.0
    s.lines = ["garbage", "N/A, N/A, 1, a, b, c, d"]
    assert s.summary(0, 2)["samples"] == 0 and s.summary(0, 2)["sm_mhz"] is None


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True,
                       timeout=120)
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "single-GPU" in p.stdout
