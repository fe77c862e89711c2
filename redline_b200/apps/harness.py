"""Benchmark harness: runs a workload through the engine and reports latency and
throughput the way the reference's harness does (src/cuda/bench/harness.cpp:16-244,
src/core/stats.cpp:8-36, src/core/workload.cpp:32-102): time to first token, inter-token
latency, time per output token, end-to-end latency (percentiles by linear
interpolation), output / decode / prefill throughput by the wall clock and by CUDA
events, host overhead per step, share of steps replayed as CUDA graphs, preemptions,
memory, plus the achieved fraction of the HBM roofline of decode steps.
"""

from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from ..sampling.params import SamplingParams


# ------------------------------------------------------------------- statistics

def percentile(values: Sequence[float], q: float) -> float:
    if not values:
        return 0.0
    v = sorted(values)
    pos = q / 100.0 * (len(v) - 1)
    lo = int(math.floor(pos))
    hi = min(lo + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (pos - lo)


def summarize(values: Sequence[float]) -> Dict[str, float]:
    if not values:
        return {"count": 0, "mean": 0.0, "p50": 0.0, "p90": 0.0, "p95": 0.0, "p99": 0.0, "min": 0.0, "max": 0.0, "std": 0.0}
    mean = sum(values) / len(values)
    var = sum((x - mean) ** 2 for x in values) / len(values)
    return {"count": len(values), "mean": mean, "p50": percentile(values, 50), "p90": percentile(values, 90),
            "p95": percentile(values, 95), "p99": percentile(values, 99), "min": min(values), "max": max(values),
            "std": math.sqrt(var)}


# -------------------------------------------------------------------- workloads

@dataclass
class WorkloadRequest:
    id: int
    prompt: List[int]
    params: SamplingParams
    arrival_time: float = 0.0


@dataclass
class Workload:
    name: str
    requests: List[WorkloadRequest]
    settings: Dict[str, Any] = field(default_factory=dict)
    description: str = ""


def _random_prompt(n: int, low: int, high: int, rng: np.random.RandomState) -> List[int]:
    return rng.randint(low, high, size=n).tolist()


def parse_workload(doc: Dict[str, Any], vocab_size: int) -> Workload:
    """A workload document: name, settings, seed, vocab_low / vocab_high, and requests with
    either ``prompt_ids`` or ``prompt_len`` (seeded uniform ids that avoid the low, usually
    special, ids), ``max_new_tokens``, sampling options, ``arrival_time``."""
    rng = np.random.RandomState(int(doc.get("seed", 0)) % (2 ** 32))
    low = int(doc.get("vocab_low", min(1000, vocab_size // 4)))
    high = int(doc.get("vocab_high", vocab_size))
    if not (low < high <= vocab_size):
        raise ValueError("bad synthetic vocab range")
    reqs: List[WorkloadRequest] = []
    next_id = 0
    for r in doc["requests"]:
        rid = int(r.get("id", next_id))
        next_id = rid + 1
        if "prompt_ids" in r:
            prompt = [int(t) for t in r["prompt_ids"]]
            for t in prompt:
                if not 0 <= t < vocab_size:
                    raise ValueError(f"prompt token id {t} out of range")
        else:
            prompt = _random_prompt(int(r["prompt_len"]), low, high, rng)
        if not prompt:
            raise ValueError(f"request {rid} has an empty prompt")
        sp = SamplingParams(temperature=float(r.get("temperature", 0.0)), top_k=int(r.get("top_k", 0)),
                            top_p=float(r.get("top_p", 1.0)), seed=int(r.get("seed", rid)),
                            max_new_tokens=int(r.get("max_new_tokens", 128)),
                            stop_token_ids=tuple(int(t) for t in r.get("stop_token_ids", ())),
                            ignore_eos=bool(r.get("ignore_eos", True)))
        reqs.append(WorkloadRequest(rid, prompt, sp, float(r.get("arrival_time", 0.0))))
    return Workload(doc.get("name", "workload"), reqs, doc.get("settings") or {}, doc.get("description", ""))


def load_workload(path: str, vocab_size: int) -> Workload:
    with open(path) as f:
        return parse_workload(json.load(f), vocab_size)


def synthetic_workload(num_requests: int, prompt_len: int, output_len: int, vocab_size: int, seed: int = 0) -> Workload:
    rng = np.random.RandomState(seed)
    low = min(1000, vocab_size // 4)
    reqs = [WorkloadRequest(i, _random_prompt(prompt_len, low, vocab_size, rng),
                            SamplingParams(max_new_tokens=output_len, ignore_eos=True, seed=i))
            for i in range(num_requests)]
    return Workload(f"synthetic_n{num_requests}_in{prompt_len}_out{output_len}", reqs,
                    {"num_requests": num_requests, "prompt_len": prompt_len, "output_len": output_len})


# ---------------------------------------------------------------------- the run

@dataclass
class BenchOptions:
    online: bool = False          # honour arrival times
    warmup_requests: int = 2
    warmup_tokens: int = 8
    keep_per_request: bool = False
    trace_path: str = ""
    hbm_gbs: float = 0.0          # > 0: report decode steps against this bandwidth
    bf16_tflops: float = 0.0      # > 0: with profile_ops, report compute-bound ops against this peak
    profile_ops: bool = False     # per-op device time breakdown (steps run eagerly; skews throughput)


def _warmup(engine, w: Workload, opts: BenchOptions) -> None:
    import dataclasses
    reqs = []
    for r in w.requests[:opts.warmup_requests]:
        sp = dataclasses.replace(r.params, max_new_tokens=min(r.params.max_new_tokens, opts.warmup_tokens))
        reqs.append((r.prompt, sp))
    if reqs:
        engine.generate_requests(reqs)
    import torch
    torch.cuda.synchronize()


def run_benchmark(engine, workload: Workload, opts: Optional[BenchOptions] = None) -> Dict[str, Any]:
    import torch
    opts = opts or BenchOptions()
    _warmup(engine, workload, opts)
    engine.records.clear()
    engine.record_steps = True
    engine.reset_peak_memory()
    if opts.profile_ops:
        engine.set_op_profiling(True)
        engine.reset_op_profile()
    order = sorted(workload.requests, key=lambda r: r.arrival_time if opts.online else 0.0)
    wave = int(workload.settings.get("batch_size", 0)) if not opts.online else 0
    outputs: List[Dict[str, Any]] = []
    nxt = 0
    base_id = engine._next_id
    t0 = time.perf_counter()
    step_done: List[float] = []
    while nxt < len(order) or engine.has_unfinished():
        now = time.perf_counter()
        if opts.online:
            while nxt < len(order) and t0 + order[nxt].arrival_time <= now:
                r = order[nxt]
                nxt += 1
                engine.add_request(r.prompt, r.params, base_id + r.id, t0 + r.arrival_time)
        elif wave == 0 or not engine.has_unfinished():
            end = len(order) if wave == 0 else min(len(order), nxt + wave)
            while nxt < end:
                r = order[nxt]
                nxt += 1
                engine.add_request(r.prompt, r.params, base_id + r.id, now)
        if not engine.has_unfinished():
            if nxt >= len(order):
                break
            wait = t0 + order[nxt].arrival_time - time.perf_counter()
            if wait > 0:
                time.sleep(wait)
            continue
        n_before = len(engine.records)
        outputs.extend(engine.step())
        step_done.extend([time.perf_counter()] * (len(engine.records) - n_before))
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    engine.record_steps = False
    duration = t_end - t0

    ttft, e2e, tpot, itl = [], [], [], []
    out_tokens = prompt_tokens = preemptions = 0
    per_request = []
    for o in outputs:
        n = len(o["output_ids"])
        out_tokens += n
        prompt_tokens += len(o["prompt_ids"])
        preemptions += o["num_preemptions"]
        ttft.append(o["ttft_s"] * 1e3)
        e2e.append(o["e2e_s"] * 1e3)
        tt = o["token_times"]
        if n > 1:
            tpot.append((tt[-1] - tt[0]) * 1e3 / (n - 1))
        itl.extend((tt[i] - tt[i - 1]) * 1e3 for i in range(1, len(tt)))
        if opts.keep_per_request:
            per_request.append({"id": o["id"] - base_id, "prompt_tokens": len(o["prompt_ids"]), "output_tokens": n,
                                "ttft_ms": o["ttft_s"] * 1e3, "e2e_ms": o["e2e_s"] * 1e3,
                                "finish_reason": o["finish_reason"]})

    steps = engine.records
    decode_gpu_ms = prefill_gpu_ms = decode_wall = 0.0
    decode_tokens = prefill_tokens = graph_steps = 0
    decode_step_gpu, host_overhead = [], []
    prev_done = t0
    for s, done in zip(steps, step_done):
        host_overhead.append(s.host_ms)
        graph_steps += 1 if s.cuda_graph else 0
        if s.kind == "decode":
            decode_gpu_ms += s.gpu_ms
            decode_tokens += s.tokens_out
            decode_wall += done - prev_done
            decode_step_gpu.append(s.gpu_ms)
        else:
            prefill_gpu_ms += s.gpu_ms
            prefill_tokens += s.num_prefill_tokens
        prev_done = done
    report: Dict[str, Any] = {
        "workload": workload.name, "workload_settings": workload.settings,
        "mode": "online" if opts.online else "offline", "engine": engine.describe(),
        "num_requests": len(outputs), "duration_s": duration, "prompt_tokens": prompt_tokens,
        "output_tokens": out_tokens, "request_throughput_rps": len(outputs) / duration,
        "output_throughput_tok_s": out_tokens / duration,
        "decode_throughput_tok_s": decode_tokens / decode_wall if decode_wall > 0 else 0.0,
        "decode_throughput_gpu_tok_s": decode_tokens / (decode_gpu_ms / 1e3) if decode_gpu_ms > 0 else 0.0,
        "prefill_throughput_gpu_tok_s": prefill_tokens / (prefill_gpu_ms / 1e3) if prefill_gpu_ms > 0 else 0.0,
        "ttft_ms": summarize(ttft), "itl_ms": summarize(itl), "tpot_ms": summarize(tpot),
        "e2e_latency_ms": summarize(e2e), "decode_step_gpu_ms": summarize(decode_step_gpu),
        "host_overhead_ms": summarize(host_overhead), "num_steps": len(steps),
        "cuda_graph_step_fraction": graph_steps / len(steps) if steps else 0.0,
        "preemptions": preemptions, "memory": engine.memory_report(),
    }
    if opts.hbm_gbs > 0 and decode_step_gpu:
        wb = engine.runner.model.weight_bytes()
        report["decode_roofline"] = {"weight_bytes": wb, "hbm_gbs": opts.hbm_gbs,
                                     "weights_only_frac_p50": wb / (percentile(decode_step_gpu, 50) / 1e3) / 1e9 / opts.hbm_gbs}
    if opts.keep_per_request:
        report["requests"] = per_request
    if opts.profile_ops:
        report["op_profile"] = engine.op_profile(opts.hbm_gbs, opts.bf16_tflops)
        engine.set_op_profiling(False)
    if opts.trace_path:
        with open(opts.trace_path, "w") as f:
            json.dump({"report": {k: v for k, v in report.items() if k != "requests"},
                       "steps": [s.__dict__ for s in steps]}, f)
    return report


def format_report_summary(r: Dict[str, Any]) -> str:
    return (f"{r['workload']}: {r['num_requests']} req, out {r['output_throughput_tok_s']:.1f} tok/s, "
            f"decode {r['decode_throughput_tok_s']:.1f} tok/s (gpu {r['decode_throughput_gpu_tok_s']:.1f}), "
            f"prefill gpu {r['prefill_throughput_gpu_tok_s']:.1f} tok/s, TTFT p50 {r['ttft_ms']['p50']:.2f} ms, "
            f"ITL p50 {r['itl_ms']['p50']:.2f} ms (p99 {r['itl_ms']['p99']:.2f}), "
            f"graphs {100 * r['cuda_graph_step_fraction']:.0f}% of steps, preemptions {r['preemptions']}")
