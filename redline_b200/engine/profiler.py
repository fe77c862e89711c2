"""Per-op device time of eager steps, with the bytes and floating-point operations of each op and
the fraction of the roofline it reaches.

CUDA events are recorded on the step's stream between consecutive ops; the host enqueues a whole
step ahead of the GPU, so the time between two events is the device time of the op in between
(plus its launch gap).  A CUDA graph cannot be cut this way, so the runner steps eagerly while
profiling is on; throughput measured meanwhile is skewed.  The parts of a layer call
``ctx.profiler.mark`` after their kernels when a profiler is attached to the step, with what the
op had to read and compute (reference: src/cuda/op_profiler.h:21-103; the op names are those of
src/cuda/model/llama.cpp:76-150, the byte / FLOP columns and the roofline fraction are additions).
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch


class OpProfiler:
    def __init__(self) -> None:
        self._pool: List[torch.cuda.Event] = []
        self._used = 0
        self._names: List[str] = []
        self._work: List[tuple] = []
        self._scope = ""
        self._stats: Dict[str, List[float]] = {}     # name -> [ms, calls, bytes, flops]
        self._order: List[str] = []
        self._passes: Dict[str, int] = {}

    # ------------------------------------------------------------------ one pass
    def begin(self, scope: str) -> None:
        """Starts a forward pass; ops are attributed to "<scope>/<op>"."""
        self._scope = scope
        self._used = 0
        self._names = []
        self._work = []
        self._record("", 0.0, 0.0)

    def mark(self, op: str, nbytes: float = 0.0, flops: float = 0.0) -> None:
        """Marks the end of ``op``: everything enqueued since the mark before.  ``nbytes`` is what the
        op has to move through device memory at least (operands read once, results written once),
        ``flops`` its floating-point operations."""
        self._record(f"{self._scope}/{op}", nbytes, flops)

    def end(self) -> None:
        """Waits for the pass and adds the times of its ops to the totals."""
        if self._used < 2:
            return
        self._pool[self._used - 1].synchronize()
        for i in range(1, self._used):
            name = self._names[i]
            st = self._stats.get(name)
            if st is None:
                st = self._stats[name] = [0.0, 0, 0.0, 0.0]
                self._order.append(name)
            st[0] += self._pool[i - 1].elapsed_time(self._pool[i])
            st[1] += 1
            st[2] += self._work[i][0]
            st[3] += self._work[i][1]
        self._passes[self._scope] = self._passes.get(self._scope, 0) + 1
        self._used = 0

    def reset(self) -> None:
        self._stats.clear()
        self._order.clear()
        self._passes.clear()

    def _record(self, name: str, nbytes: float, flops: float) -> None:
        if self._used == len(self._pool):
            self._pool.append(torch.cuda.Event(enable_timing=True))
        self._pool[self._used].record()
        self._names.append(name)
        self._work.append((nbytes, flops))
        self._used += 1

    # -------------------------------------------------------------------- report
    def report(self, hbm_gbs: float = 0.0, tflops: float = 0.0) -> List[Dict[str, Any]]:
        """Rows {op, ms_per_pass, calls_per_pass, pct, gbytes_per_pass, gflop_per_pass, gb_s, tflop_s,
        roofline_frac} in first-seen order; pct is within the op's scope.  ``roofline_frac`` is the time
        the op would take at the given peaks (the slower of its bytes at ``hbm_gbs`` and its operations
        at ``tflops``) over the time it took; absent without peaks or without work figures."""
        scope_ms: Dict[str, float] = {}
        for name, st in self._stats.items():
            scope = name.split("/", 1)[0]
            scope_ms[scope] = scope_ms.get(scope, 0.0) + st[0]
        rows = []
        for name in self._order:
            ms, calls, nbytes, flops = self._stats[name]
            scope = name.split("/", 1)[0]
            passes = max(1, self._passes.get(scope, 1))
            row: Dict[str, Any] = {
                "op": name, "ms_per_pass": ms / passes, "calls_per_pass": calls / passes,
                "pct": 100.0 * ms / scope_ms[scope] if scope_ms[scope] > 0 else 0.0,
                "gbytes_per_pass": nbytes / passes / 1e9, "gflop_per_pass": flops / passes / 1e9,
            }
            if ms > 0:
                row["gb_s"] = nbytes / (ms / 1e3) / 1e9
                row["tflop_s"] = flops / (ms / 1e3) / 1e12
                floor_s = 0.0
                if hbm_gbs > 0:
                    floor_s = max(floor_s, nbytes / (hbm_gbs * 1e9))
                if tflops > 0:
                    floor_s = max(floor_s, flops / (tflops * 1e12))
                if floor_s > 0:
                    row["roofline_frac"] = floor_s / (ms / 1e3)
            rows.append(row)
        return rows


def format_op_profile(rows: List[Dict[str, Any]]) -> str:
    """The per-op table as text, one scope after another."""
    out = []
    scope = None
    for r in rows:
        s, op = r["op"].split("/", 1)
        if s != scope:
            scope = s
            out.append(f"-- {s}: per-op device time of one step (eager)")
            out.append(f"{'op':<22}{'ms':>9}{'calls':>7}{'%':>7}{'GB/s':>9}{'TFLOP/s':>9}{'of roofline':>13}")
        frac = f"{r['roofline_frac']:.2f}" if "roofline_frac" in r else "-"
        out.append(f"{op:<22}{r['ms_per_pass']:>9.4f}{r['calls_per_pass']:>7.0f}{r['pct']:>7.1f}"
                   f"{r.get('gb_s', 0.0):>9.0f}{r.get('tflop_s', 0.0):>9.1f}{frac:>13}")
    return "\n".join(out) + ("\n" if out else "")


def tensor_bytes(*tensors: Optional[torch.Tensor]) -> float:
    return float(sum(t.numel() * t.element_size() for t in tensors if t is not None))


def linear_work(rows: int, w: torch.Tensor, act_elem: int, out_elem: int) -> tuple:
    """(bytes, flops) of out[rows, N] = x[rows, K] . w[N, K]^T: the weight once, x and out once."""
    n, k = w.shape
    return (float(w.numel() * w.element_size() + rows * k * act_elem + rows * n * out_elem), 2.0 * rows * n * k)


def attention_work(host, num_heads: int, num_kv_heads: int, head_dim: int, window: int, elem: int) -> dict:
    """What the attention of a step has to read and compute, from the step's host-side description
    (``host.q_len`` / ``host.start_pos`` per sequence): {"decode": (bytes, flops), "prefill": (bytes, flops)}.
    A single token reads the keys and values of its context once per kv head; a portion of n tokens
    after p earlier ones reads its p + n keys and values once and computes over the causal part."""
    dec_b = dec_f = pre_b = pre_f = 0.0
    kv_row = 2.0 * num_kv_heads * head_dim * elem            # K and V of one token
    q_row = 2.0 * num_heads * head_dim * elem                # q read, output written
    for n, p in zip(host.q_len, host.start_pos):
        if n == 1:
            keys = p + 1 if window <= 0 else min(p + 1, window)
            dec_b += keys * kv_row + q_row
            dec_f += 4.0 * num_heads * head_dim * keys
        elif n > 1:
            pairs = n * p + n * (n + 1) / 2.0                # (query, key) pairs of the causal part
            if window > 0:
                pairs = sum(min(p + i + 1, window) for i in range(n))
            pre_b += (p + n) * kv_row + n * q_row
            pre_f += 4.0 * num_heads * head_dim * pairs
    return {"decode": (dec_b, dec_f), "prefill": (pre_b, pre_f)}
