#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Llama 3.2 1B sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the running batch (default: 8 requests at a context
of 4,096).  One JSON line is printed:

  value     decoded tokens per second, device time: CUDA events around each of K
            steps driven through ``Engine.step`` (summed, so host gaps do not count)
  e2e       the same K-step measure by the wall clock through the Python entry point:
            every step uploads its metadata from pinned host memory and the host reads
            the sampled tokens back
  prefill   one 2,048-token prompt alone on an idle GPU, host preparation included:
            tokens/s and the fraction of the measured bf16 tensor-core peak that its
            FLOPs reach ("back_to_back_ms": per prompt when prompts follow one another)
  roofline  bytes a decode step has to read (every weight once, the cache of the
            live requests) / its time, against the measured copy bandwidth
  points    decode tokens/s at batch 1, 8 and 64 with 512-token prompts (the metric's
            decode workload), each with its step time and its fraction of the copy
            bandwidth (the same byte count at its batch and context)

Weights are random (N(0, 0.02^2)), token ids uniform random: the sizes are what is
measured.  ``--impl reference`` runs the unmodified reference (built by
baseline/build_reference.sh into baseline/_ref) on the same workload through its own
``redline_bench``.  More than one GPU is not supported: the engine is single-GPU.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Any, Dict, List, Optional

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Llama 3.2 1B (the benchmark configuration): every size comes from here.
BENCH_CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 16, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
    "hidden_act": "silu", "bos_token_id": 128000, "eos_token_id": 128001,
}
CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048
POINT_PROMPT = 512
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> Dict[str, Any]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int = 0):
        self.device = device
        self.proc: Optional[subprocess.Popen] = None
        self.lines: List[str] = []

    def start(self) -> None:
        exe = shutil.which("nvidia-smi")
        if not exe:
            return
        self.proc = subprocess.Popen([exe, f"--id={self.device}", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits", "-lms", "25"],
                                     stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self) -> None:
        assert self.proc and self.proc.stdout
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self) -> int:
        return len(self.lines)

    def stop(self) -> None:
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, lo: int = 0, hi: Optional[int] = None) -> Dict[str, Any]:
        """Samples lo..hi (marks around the timed region).  A region too short for three samples is
        widened backwards into the warm-up steps before it, which run the same load; "widened" says so."""
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        hi = len(self.lines) if hi is None else hi
        widened = hi - lo < 3
        if widened:
            lo = max(0, hi - 8)
        for line in self.lines[lo:hi]:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm), "widened": widened}


def bench_config(cfg: Dict[str, Any], steps: int, warmup: int, peaks_source: str) -> Dict[str, Any]:
    """The ``config`` of the JSON line: every size, flat.  Both arms print the same dictionary."""
    return {
        "model": "llama-3.2-1b-sizes", "layers": cfg["num_hidden_layers"], "layers_full": 16,
        "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
        "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
        "global_batch": BATCH, "seq_len": CONTEXT, "context_at_timing": timed_prompt(steps, warmup) + warmup + steps // 2,
        "page_size": 16, "parallelism": "single-gpu", "l2": "step reads weights + cache >> L2, no flush",
        "points_prompt": POINT_PROMPT, "prefill_tokens": PREFILL_TOKENS, "peaks": peaks_source,
    }


def timed_prompt(steps: int, warmup: int) -> int:
    """Prompt length of the headline run: the requests reach the context limit just after the timed steps."""
    return CONTEXT - (warmup + 2 * steps + 34)


def model_numbers(cfg: Dict[str, Any]) -> Dict[str, float]:
    """Parameter counts, bytes and FLOPs of the configuration (bf16 weights and cache)."""
    L, H, I, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Hq, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    layer_mat = (Hq + 2 * Hkv) * D * H + H * Hq * D + 3 * I * H
    layer = layer_mat + 2 * H
    head = V * H
    weight_bytes = 2.0 * (L * layer + head + H)          # every weight a decode step reads, once
    kv_bytes_per_token = 2.0 * 2 * L * Hkv * D
    return {"layer_mat": layer_mat, "weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token,
            "head": head, "L": L, "Hq": Hq, "D": D}


def prefill_flops(cfg: Dict[str, Any], T: int, rows: int = 1) -> float:
    n = model_numbers(cfg)
    gemm = 2.0 * T * n["layer_mat"] * n["L"] + 2.0 * rows * n["head"]
    attn = n["L"] * n["Hq"] * 4.0 * n["D"] * (T * (T + 1) / 2.0)   # QK^T and PV over the causal half
    return gemm + attn


def write_model(tmp: str, layers: Optional[int]) -> str:
    from redline_b200.config import config_from_dict
    from redline_b200.weights import write_random_model
    cfg = dict(BENCH_CONFIG)
    if layers:
        cfg["num_hidden_layers"] = layers
    d = os.path.join(tmp, "llama_1b_random")
    t0 = time.time()
    write_random_model(d, config_from_dict(cfg), seed=0)
    print(f"[bench] wrote random weights to {d} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return d


def decode_run(model: str, batch: int, prompt_len: int, steps: int, warmup: int, sampler: ClockSampler,
               max_seq_len: int) -> Dict[str, Any]:
    """Prefills ``batch`` random prompts, then W warm-up decode steps, K device-timed steps
    and K wall-clock steps, all through Engine.step (host tokens in and out every step)."""
    import numpy as np
    import torch
    from redline_b200.engine.engine import Engine
    from redline_b200.sampling import SamplingParams

    new_tokens = warmup + 2 * steps + 32
    eng = Engine(model, dtype="bfloat16", max_num_seqs=batch, max_num_batched_tokens=2048, max_seq_len=max_seq_len,
                 kv_cache_tokens=batch * ((prompt_len + new_tokens + 15) // 16 * 16 + 16))
    rng = np.random.RandomState(0)
    V = eng.vocab_size
    for i in range(batch):
        eng.add_request(rng.randint(0, V, size=prompt_len).tolist(),
                        SamplingParams(max_new_tokens=new_tokens, ignore_eos=True, seed=i))
    eng.record_steps = True
    t0 = time.time()
    while True:                                   # prefill until every sequence is decoding
        eng.step()
        if eng.records and eng.records[-1].kind == "decode" and eng.records[-1].num_seqs == batch:
            break
        if not eng.has_unfinished():
            raise RuntimeError("requests finished before the decode phase")
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    prefill_s = time.time() - t0

    # ---- K steps, device time: the per-step CUDA event pairs of the engine's step records
    eng.records.clear()
    launches0 = eng.runner.num_kernel_launches
    mark0 = sampler.mark()
    torch.cuda.synchronize()
    for _ in range(steps):
        eng.step()
    while len(eng.records) < steps:               # the last launched step is read one call later
        eng.step()
    torch.cuda.synchronize()
    recs = eng.records[:steps]
    assert all(r.kind == "decode" and r.num_seqs == batch for r in recs), "timed steps must be pure decode"
    gpu_ms = sum(r.gpu_ms for r in recs)
    launches = (eng.runner.num_kernel_launches - launches0) * steps // max(len(eng.records), 1)
    graph = all(r.cuda_graph for r in recs)
    host_ms = sorted(r.host_ms for r in recs)[len(recs) // 2]

    # ---- K steps, wall clock, host tokens in and out
    eng.record_steps = False
    done_before = sum(len(s.tokens) for s in eng._seqs.values())
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t1
    mark1 = sampler.mark()                        # the clocks cover both timed regions
    assert len(eng._seqs) == batch, "a request finished inside the timed region"
    produced = sum(len(s.tokens) for s in eng._seqs.values()) - done_before
    ctx_mid = prompt_len + warmup + steps // 2
    words = eng.runner.builder.capacity_words
    from redline_b200.engine.batch import Layout
    lay = Layout(batch, batch, batch, 0, len(eng.runner.groups), eng.runner.builder.B)
    out = {
        "tok_s": batch * steps / (gpu_ms / 1e3), "ms_per_step": gpu_ms / steps,
        "e2e_tok_s": produced / wall, "e2e_ms_per_step": wall * 1e3 / steps,
        "launches": launches, "cuda_graph": graph, "host_ms_p50": host_ms, "ctx_mid": ctx_mid,
        "h2d_bytes": lay.words * 4, "d2h_bytes": batch * 8, "prefill_s": prefill_s,
        "clocks": sampler.summary(mark0, mark1),
    }
    del eng
    torch.cuda.empty_cache()
    return out


def profile_step(args) -> int:
    """For profilers: sets the decode batch up as the default run does, then brackets ONE decode
    step with cudaProfilerStart/Stop (use ``ncu --profile-from-start off``) and prints its time."""
    import numpy as np
    import torch
    from redline_b200.engine.engine import Engine
    from redline_b200.sampling import SamplingParams
    tmp = tempfile.mkdtemp(prefix="redline_bench_")
    try:
        model = write_model(tmp, args.layers)
        batch, prompt = args.profile_batch, args.profile_prompt or (CONTEXT - 96)
        # every request must still be running when the last one has been admitted: one decoded token per
        # request and step while the others' prompts are being prefilled
        if prompt + 2 * batch * ((prompt + 2047) // 2048) + 16 > CONTEXT:
            raise SystemExit("--profile-batch / --profile-prompt: the first requests would reach the context "
                             "limit before the last one is admitted; use a shorter --profile-prompt")
        eng = Engine(model, dtype="bfloat16", max_num_seqs=batch, max_num_batched_tokens=2048, max_seq_len=CONTEXT,
                     kv_cache_tokens=max(batch * (prompt + 128), CONTEXT + 64), cuda_graphs=not args.profile_eager, async_scheduling=False)
        rng = np.random.RandomState(0)
        for i in range(batch):
            eng.add_request(rng.randint(0, eng.vocab_size, size=prompt).tolist(),
                            SamplingParams(max_new_tokens=CONTEXT - prompt - 8, ignore_eos=True))
        eng.record_steps = True
        while not (eng.records and eng.records[-1].kind == "decode" and eng.records[-1].num_seqs == batch):
            eng.step()
        for _ in range(3):
            eng.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        eng.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        for _ in range(3):
            eng.step()
        print(json.dumps({"profiled": "one decode step", "batch": batch, "context": prompt + 4,
                          "gpu_ms_per_step": [round(r.gpu_ms, 4) for r in eng.records[-4:]]}))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return 0


def profile_prefill(args) -> int:
    """One prompt of PREFILL_TOKENS tokens between cudaProfilerStart and cudaProfilerStop (after three
    untimed ones), for `ncu --profile-from-start off`."""
    import numpy as np
    import torch
    from redline_b200.engine.engine import Engine
    tmp = tempfile.mkdtemp(prefix="redline_bench_")
    try:
        model = write_model(tmp, args.layers)
        T = PREFILL_TOKENS
        eng = Engine(model, dtype="bfloat16", max_num_seqs=2, max_num_batched_tokens=T, max_seq_len=T + 16,
                     kv_cache_tokens=2 * T + 64, cuda_graphs=True, async_scheduling=False)
        toks = np.random.RandomState(1).randint(0, eng.vocab_size, size=T).tolist()
        for i in range(4):
            torch.cuda.synchronize()
            if i == 3:
                torch.cuda.profiler.start()
            eng.step_tokens([("p", toks, [T - 1])], graphs=True)       # (as prefill_run: the step is a CUDA graph)
            torch.cuda.synchronize()
            if i == 3:
                torch.cuda.profiler.stop()
            eng.close_request("p")
        print(json.dumps({"profiled": "one prompt step", "tokens": T}))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return 0


def prefill_run(model: str, tokens: int, reps: int = 6, warmup: int = 3) -> Dict[str, Any]:
    """Prompts of ``tokens`` tokens through Engine.step_tokens (host token ids in, logits of the last
    position on the device).  "ms": per prompt when ``reps`` prompts are submitted one after another
    between one pair of CUDA events (the host's preparation of a prompt then runs while the GPU works on
    the one before, as in serving); "latency_ms": one prompt alone on an idle GPU, host preparation
    included (median of ``reps``).  A step that is one full portion of a prompt is replayed as a CUDA graph,
    sampler included, as in generation."""
    import numpy as np
    import torch
    from redline_b200.engine.engine import Engine
    eng = Engine(model, dtype="bfloat16", max_num_seqs=2, max_num_batched_tokens=tokens, max_seq_len=tokens + 16,
                 kv_cache_tokens=2 * tokens + 64, cuda_graphs=True, async_scheduling=False)
    rng = np.random.RandomState(1)
    toks = rng.randint(0, eng.vocab_size, size=tokens).tolist()
    times = []
    for i in range(warmup + reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step_tokens([("p", toks, [tokens - 1])], graphs=True)
        b.record()
        torch.cuda.synchronize()
        eng.close_request("p")
        if i >= warmup:
            times.append(a.elapsed_time(b))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for i in range(reps):
        eng.step_tokens([(f"q{i}", toks, [tokens - 1])], graphs=True)
        eng.close_request(f"q{i}")
    b.record()
    torch.cuda.synchronize()
    del eng
    torch.cuda.empty_cache()
    times.sort()
    return {"ms": a.elapsed_time(b) / reps, "latency_ms": times[len(times) // 2]}


def run_ours(args) -> Dict[str, Any]:
    import torch
    pk = peaks()
    tmp = tempfile.mkdtemp(prefix="redline_bench_")
    sampler = ClockSampler(0)
    try:
        model = write_model(tmp, args.layers)
        cfg = dict(BENCH_CONFIG)
        if args.layers:
            cfg["num_hidden_layers"] = args.layers
        nums = model_numbers(cfg)
        sampler.start()
        K, W = args.steps, args.warmup
        main = decode_run(model, BATCH, timed_prompt(K, W), K, W, sampler, CONTEXT)
        pre = prefill_run(model, PREFILL_TOKENS)
        pts = {}
        hbm = pk.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"])
        for b in (1, 8, 64):
            r = decode_run(model, b, POINT_PROMPT, min(K, 64), W, sampler, 1024)
            bytes_b = nums["weight_bytes"] + b * r["ctx_mid"] * nums["kv_bytes_per_token"]
            pts[f"decode_b{b}"] = round(r["tok_s"], 1)
            pts[f"decode_b{b}_e2e"] = round(r["e2e_tok_s"], 1)
            pts[f"decode_b{b}_ms"] = round(r["ms_per_step"], 4)
            pts[f"decode_b{b}_frac"] = round(bytes_b / (r["ms_per_step"] / 1e3) / 1e9 / hbm, 4)
    finally:
        sampler.stop()
        shutil.rmtree(tmp, ignore_errors=True)
    step_bytes = nums["weight_bytes"] + BATCH * main["ctx_mid"] * nums["kv_bytes_per_token"]
    achieved = step_bytes / (main["ms_per_step"] / 1e3) / 1e9
    pf = prefill_flops(cfg, PREFILL_TOKENS)
    peak_tflops = pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])
    return {
        "metric": "decode tok/s at batch 8, context 4096 (Llama 3.2 1B sizes)",
        "value": round(main["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "ours",
        "config": bench_config(cfg, K, W, pk["source"]), "cuda_graph": main["cuda_graph"],
        "e2e": {"value": round(main["e2e_tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": main["h2d_bytes"],
                "d2h_bytes_per_step": main["d2h_bytes"], "ms_per_step": round(main["e2e_ms_per_step"], 4),
                "host_ms_p50": round(main["host_ms_p50"], 4)},
        "gpu_launches": int(main["launches"]),
        "clocks": main["clocks"],
        "prefill": {"value": round(PREFILL_TOKENS / (pre["latency_ms"] / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pre["latency_ms"], 3),
                    "frac": round(pf / (pre["latency_ms"] / 1e3) / (peak_tflops * 1e12), 4),
                    "back_to_back_ms": round(pre["ms"], 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk.get("hbm_gbs"), "unit": "GB/s",
                     "frac": round(achieved / pk.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]), 4)},
        "points": pts,
    }


def full_width_steps(trace: Dict[str, Any], batch: int) -> List[Dict[str, float]]:
    """The pure-decode steps of a reference trace (its ``redline-trace-v1`` format: ``step_fields`` names
    the columns of ``steps``) that hold all ``batch`` sequences, in order, as dicts with gpu_ms and the
    time since the step before finished."""
    col = {name: i for i, name in enumerate(trace["step_fields"])}
    out, prev_done = [], None
    for row in trace["steps"]:
        done = row[col["t_done_ms"]]
        if row[col["kind"]] == "decode" and row[col["seqs"]] == batch:
            out.append({"gpu_ms": row[col["gpu_ms"]],
                        "wall_ms": done - prev_done if prev_done is not None else row[col["gpu_ms"]]})
        prev_done = done
    return out


def run_reference(args) -> Dict[str, Any]:
    """The unmodified reference on the same workload through its own redline_bench.  Its report sums
    over every decode step, also those while requests are still being admitted or have already
    finished; to time what the other arm times, the per-step trace it writes is read and only steps
    that hold all BATCH sequences count: W of them are skipped, the next K are the timed ones."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    binary = os.path.join(ref, "build", "redline_bench")
    if not os.path.exists(binary):
        return {"impl": "reference", "unavailable": "baseline/_ref/build/redline_bench is not built "
                                                    "(run baseline/build_reference.sh on the build machine)"}
    tmp = tempfile.mkdtemp(prefix="redline_ref_")
    K, W = args.steps, args.warmup
    try:
        model = write_model(tmp, None)
        rlm = os.path.join(tmp, "model.rlm")
        env = dict(os.environ, PYTHONPATH=ref + os.pathsep + os.environ.get("PYTHONPATH", ""))
        r = subprocess.run([sys.executable, "-m", "redline.convert", "--model", model, "--out", rlm, "--device", "cpu"], env=env, capture_output=True, text=True)
        if r.returncode != 0:
            return {"impl": "reference", "unavailable": "the reference's converter failed: " + r.stderr.strip()[-300:]}
        prompt = timed_prompt(K, W)
        # long enough that W + K steps hold every sequence: the first sequences decode while the
        # prompts of the later ones are still being prefilled, and finish that much earlier
        new_tokens = min(W + K + 4 * BATCH + 8, CONTEXT - prompt - 1)
        out, trace_path = os.path.join(tmp, "report.json"), os.path.join(tmp, "trace.json")
        cmd = [binary, "--model", rlm, "--synthetic", f"{BATCH},{prompt},{new_tokens}", "--max-seqs", str(BATCH),
               "--max-seq-len", str(CONTEXT), "--out", out, "--trace-out", trace_path]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            return {"impl": "reference", "unavailable": "redline_bench failed: " + r.stderr.strip()[-300:]}
        with open(out) as f:
            rep = json.load(f)
        with open(trace_path) as f:
            full = full_width_steps(json.load(f), BATCH)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    timed = full[W:W + K] if len(full) > W else full
    if not timed:
        return {"impl": "reference", "unavailable": f"its trace has no decode step with all {BATCH} sequences"}
    gpu_ms = sum(t["gpu_ms"] for t in timed) / len(timed)
    wall_ms = sum(t["wall_ms"] for t in timed) / len(timed)
    return {
        "metric": "decode tok/s at batch 8, context 4096 (Llama 3.2 1B sizes)", "impl": "reference",
        "value": round(BATCH / (gpu_ms / 1e3), 1), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(gpu_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic (random weights, uniform random token ids)",
        "config": bench_config(BENCH_CONFIG, K, W, peaks()["source"]),
        "timed_steps": len(timed), "seqs_per_timed_step": BATCH, "full_width_decode_steps": len(full),
        "e2e": {"value": round(BATCH / (wall_ms / 1e3), 1), "unit": "tok/s", "ms_per_step": round(wall_ms, 4),
                "note": "host tokens in and out every step through the reference's own engine loop; it does "
                        "not report the bytes it copies"},
        "whole_run": {"decode_tok_s_gpu": round(rep["decode_throughput_gpu_tok_s"], 1),
                      "decode_tok_s": round(rep["decode_throughput_tok_s"], 1),
                      "decode_step_gpu_ms_mean": round(rep["decode_step_gpu_ms"]["mean"], 4)},
        "prefill": {"value": round(rep["prefill_throughput_gpu_tok_s"], 1)},
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--profile-step", action="store_true", help="bracket one decode step with cudaProfilerStart/Stop and exit")
    ap.add_argument("--profile-prefill", action="store_true", help="bracket one prompt step of 2,048 tokens with cudaProfilerStart/Stop and exit")
    ap.add_argument("--profile-batch", type=int, default=BATCH)
    ap.add_argument("--profile-prompt", type=int, default=0, help="with --profile-step: prompt length (default: context - 96)")
    ap.add_argument("--profile-eager", action="store_true", help="with --profile-step: no CUDA graph")
    args = ap.parse_args()
    if args.gpus != 1:
        print("redline_b200 is a single-GPU engine: bench.py runs at --gpus 1 only")
        return 2
    if args.profile_step:
        return profile_step(args)
    if args.profile_prefill:
        return profile_prefill(args)
    args.warmup = max(args.warmup, 3)
    args.steps = max(1, min(args.steps, 1000))
    res = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
