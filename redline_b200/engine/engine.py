"""The engine: requests in, tokens out.

``Engine`` puts the scheduler above the step function.  ``step()`` plans one batch,
launches it, and (with asynchronous scheduling) reads the tokens of the batch
before it, so the GPU never waits for the host: a sequence whose newest token is
still on the device is planned anyway and the next step takes the token from the
sampler's output there.  Pure decode batches are replayed as CUDA graphs of a
padded fixed shape.  Options, request fields and outputs have the reference's
names (src/cuda/engine/engine.h:37-129, src/cuda/engine/engine.cpp:360-553,681-733;
python/redline/runtime.py:43-92).

The same object also serves the trace replay: ``open_request`` / ``step_tokens`` /
``close_request`` run given tokens through the same step function without
scheduler or sampler.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence as Seq, Tuple

import torch

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from .batch import RowSampling, Segment
from .runner import EngineError, ModelRunner
from .scheduler import FINISHED, Scheduler, SchedulerConfig, Sequence, StepPlan


@dataclass
class StepRecord:
    """One step as the engine saw it (reference: src/cuda/engine/engine.h:68-87)."""

    step: int
    kind: str               # prefill | decode | mixed
    num_seqs: int
    num_tokens: int
    num_prefill_tokens: int
    num_decode_tokens: int
    cuda_graph: bool
    host_ms: float
    gpu_ms: float = 0.0
    tokens_out: int = 0
    num_preempted: int = 0
    kv_pages_used: int = 0
    kv_pages_total: int = 0
    num_running: int = 0
    num_waiting: int = 0


@dataclass
class _InFlight:
    step: int
    plan: StepPlan
    sample_rows: List[int]
    slot: int
    record: StepRecord


def make_output(seq: Sequence) -> Dict[str, Any]:
    return {
        "id": seq.id,
        "prompt_ids": list(seq.tokens[:seq.prompt_len]),
        "output_ids": list(seq.tokens[seq.prompt_len:]),
        "logprobs": list(seq.logprobs),
        "finish_reason": seq.finish_reason,
        "ttft_s": seq.first_token_time - seq.arrival_time,
        "e2e_s": seq.finish_time - seq.arrival_time,
        "token_times": list(seq.token_times),
        "num_preemptions": seq.num_preemptions,
    }


class Engine:
    def __init__(self, model: str, **options: Any):
        self.cfg = EngineConfig.from_options(model, options)
        self.runner = ModelRunner(self.cfg)
        self._init_rest()

    @classmethod
    def from_runner(cls, runner: ModelRunner) -> "Engine":
        """An engine around an existing runner (a model built from a spec in code)."""
        e = cls.__new__(cls)
        e.cfg = runner.cfg
        e.runner = runner
        e._init_rest()
        return e

    def _init_rest(self) -> None:
        cfg = self.cfg
        self.scheduler = Scheduler(
            SchedulerConfig(cfg.max_num_seqs, cfg.max_num_batched_tokens, cfg.max_seq_len,
                            cfg.mix_prefill_decode, cfg.admission_watermark), self.runner.cache)
        self._seqs: Dict[int, Sequence] = {}
        self._next_id = 0
        self._next_step = 0
        self._inflight: Deque[_InFlight] = deque()
        dev = self.runner.device
        rows = self.runner.max_rows
        self._tok_host = [torch.zeros(rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._lp_host = [torch.zeros(rows, dtype=torch.float32, pin_memory=True) for _ in range(2)]
        self._ev_done = [torch.cuda.Event() for _ in range(2)]
        self._ev_start = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        self._ev_stop = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        self.record_steps = False
        self.records: List[StepRecord] = []
        self.num_preemptions = 0
        self.peak_device_used = 0                  # with track_memory: the most device memory seen in use after a step
        self._op_profile_rows: List[Dict[str, Any]] = []
        self._replay_pos: Dict[object, int] = {}
        # Called after every launched step with ([(request id, position)] of the rows whose logits
        # the step computed, in row order, and the float32 logits [rows, vocab] on the device, valid
        # until the next launch).  For tests and tools that want the logits of scheduled generation.
        self.on_logits: Optional[Callable[[List[Tuple[int, int]], torch.Tensor], None]] = None

    # ------------------------------------------------------------ properties
    @property
    def vocab_size(self) -> int:
        return self.runner.vocab_size

    @property
    def model_config(self):
        return self.runner.model_config

    # --------------------------------------------------------------- requests
    def add_request(self, prompt: Seq[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[int] = None, arrival_time: float = 0.0) -> int:
        params = params or SamplingParams()
        params.validate()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("empty prompt")
        for t in prompt:
            if not 0 <= t < self.vocab_size:
                raise ValueError(f"token id {t} out of range [0, {self.vocab_size})")
        rid = self._next_id if request_id is None else int(request_id)
        if rid in self._seqs:
            raise ValueError(f"duplicate request id {rid}")
        self._next_id = max(self._next_id, rid + 1)
        stop = set(params.stop_token_ids)
        if not params.ignore_eos:
            stop |= set(self.model_config.eos_token_ids)
        seq = Sequence(id=rid, tokens=prompt, prompt_len=len(prompt), params=params,
                       stop_ids=frozenset(stop),
                       arrival_time=arrival_time if arrival_time > 0 else time.perf_counter())
        self.scheduler.add(seq)
        self._seqs[rid] = seq
        return rid

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or bool(self._inflight)

    # ------------------------------------------------------------------ step
    def step(self) -> List[Dict[str, Any]]:
        outputs: List[Dict[str, Any]] = []
        t0 = time.perf_counter()
        prev = self._inflight[-1].step if self._inflight else -1
        plan = self.scheduler.schedule(self._next_step, prev)
        launched = not plan.empty
        if launched:
            self._inflight.append(self._launch(plan, t0))
        keep = 1 if (self.cfg.async_scheduling and launched) else 0
        while len(self._inflight) > keep:
            self._process(self._inflight.popleft(), outputs)
        if not (launched or self._inflight or outputs or not self.scheduler.has_unfinished()):
            raise EngineError("scheduler made no progress")
        return outputs

    def _launch(self, plan: StepPlan, t0: float) -> _InFlight:
        step = self._next_step
        self._next_step += 1
        self.num_preemptions += plan.num_preempted
        segments: List[Segment] = []
        sample_rows: List[int] = []
        row = 0
        for e in plan.seqs:
            seq = e.seq
            if e.input_from_device:
                toks: Seq[int] = (0,)
            else:
                toks = seq.tokens[e.start_pos:e.start_pos + e.num_tokens]
            sp = seq.params
            segments.append(Segment(seq.cache, toks, e.start_pos, (e.num_tokens - 1,) if e.sample else (),
                                    e.src_row if e.input_from_device else -1,
                                    RowSampling(sp.temperature, sp.top_k, sp.top_p, sp.seed)))
            if e.sample:
                sample_rows.append(row)
                seq.num_pending += 1
                seq.pending_step = step
                seq.pending_row = row
                row += 1
            else:
                sample_rows.append(-1)
        slot = step % 2
        graphs_before = self.runner.num_graph_steps
        if self.cfg.nvtx_layers:
            torch.cuda.nvtx.range_push(f"step {step}: {plan.num_prefill_tokens} prompt + {plan.num_decode_tokens} decode tokens")
        if self.record_steps:
            self._ev_start[slot].record()
        logits, _ = self.runner.run(segments, sample=True)
        if self.record_steps:
            self._ev_stop[slot].record()
        if self.cfg.nvtx_layers:
            torch.cuda.nvtx.range_pop()
        if self.cfg.track_memory:
            free, total = torch.cuda.mem_get_info(self.runner.device)
            self.peak_device_used = max(self.peak_device_used, total - free)
        if self.on_logits is not None and row > 0:
            self.on_logits([(e.seq.id, e.start_pos + e.num_tokens - 1) for e in plan.seqs if e.sample], logits[:row])
        if row > 0:
            self._tok_host[slot][:row].copy_(self.runner.sampler.tokens[:row], non_blocking=True)
            self._lp_host[slot][:row].copy_(self.runner.sampler.logprobs[:row], non_blocking=True)
        self._ev_done[slot].record()
        self.scheduler.after_step(plan)
        kind = "decode" if plan.num_prefill_tokens == 0 else ("prefill" if plan.num_decode_tokens == 0 else "mixed")
        rec = StepRecord(step, kind, len(plan.seqs), plan.num_tokens, plan.num_prefill_tokens,
                         plan.num_decode_tokens, self.runner.num_graph_steps > graphs_before,
                         (time.perf_counter() - t0) * 1e3, num_preempted=plan.num_preempted)
        if self.record_steps:
            c = self.runner.cache
            rec.kv_pages_total = c.num_total_pages(0) if c.groups else 0
            rec.kv_pages_used = rec.kv_pages_total - (c.num_free_pages(0) if c.groups else 0)
            rec.num_running = len(self.scheduler.running)
            rec.num_waiting = len(self.scheduler.waiting) + len(self.scheduler.parked)
        return _InFlight(step, plan, sample_rows, slot, rec)

    def _process(self, f: _InFlight, outputs: List[Dict[str, Any]]) -> None:
        self._ev_done[f.slot].synchronize()
        now = time.perf_counter()
        n = sum(1 for r in f.sample_rows if r >= 0)
        tokens = self._tok_host[f.slot][:n].tolist() if n else []
        lps = self._lp_host[f.slot][:n].tolist() if n else []
        appended = 0
        for e, row in zip(f.plan.seqs, f.sample_rows):
            if row < 0:
                continue
            seq = e.seq
            seq.num_pending -= 1
            if seq.status == FINISHED:      # stopped earlier; the extra token is dropped
                self._maybe_release(seq)
                continue
            appended += 1
            if self._append(seq, tokens[row], lps[row], now):
                seq.finish_time = now
                self.scheduler.finish(seq, seq.finish_reason)
                outputs.append(make_output(seq))
                self._maybe_release(seq)
            else:
                self.scheduler.on_tokens_received(seq)
        if self.record_steps:
            f.record.gpu_ms = self._ev_start[f.slot].elapsed_time(self._ev_stop[f.slot])
            f.record.tokens_out = appended
            self.records.append(f.record)

    def _append(self, seq: Sequence, token: int, logprob: float, now: float) -> bool:
        seq.tokens.append(int(token))
        seq.logprobs.append(float(logprob))
        seq.token_times.append(now)
        if seq.first_token_time < 0:
            seq.first_token_time = now
        if token in seq.stop_ids:
            seq.finish_reason = "stop"
            return True
        if len(seq.tokens) - seq.prompt_len >= seq.params.max_new_tokens or \
                len(seq.tokens) >= self.cfg.max_seq_len:
            seq.finish_reason = "length"
            return True
        return False

    def _maybe_release(self, seq: Sequence) -> None:
        if seq.status == FINISHED and seq.num_pending == 0:
            self._seqs.pop(seq.id, None)

    # -------------------------------------------------------------- generate
    def generate_requests(self, requests: Seq[Tuple[Seq[int], SamplingParams]]) -> List[Dict[str, Any]]:
        """Runs (prompt, params) pairs to completion; outputs ordered by request."""
        if self._replay_pos:
            raise EngineError("requests opened with open_request / step_tokens are still open; close them first "
                              "(they hold cache pages the scheduler does not count)")
        ids = [self.add_request(p, sp) for p, sp in requests]
        outs: Dict[int, Dict[str, Any]] = {}
        while self.has_unfinished():
            for o in self.step():
                outs[o["id"]] = o
        self.runner.check_status()
        return [outs[i] for i in ids]

    def generate(self, prompts: Seq[Seq[int]], max_new_tokens: int = 128, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int = 0, ignore_eos: bool = False,
                 stop_token_ids: Seq[int] = ()) -> List[Dict[str, Any]]:
        """Request i samples with seed + i (reference: python/bindings/redline_ext.cpp:70-83)."""
        reqs = [(p, SamplingParams(temperature, top_k, top_p, seed + i, max_new_tokens,
                                   tuple(stop_token_ids), ignore_eos)) for i, p in enumerate(prompts)]
        return self.generate_requests(reqs)

    # ----------------------------------------------------------------- score
    def score(self, tokens: Seq[int]) -> List[float]:
        """log p(tokens[i] | tokens[:i]) for i = 1 .. len - 1, teacher forced, in portions
        (reference: src/cuda/engine/engine.cpp:693-733).  The engine must be idle."""
        if self.has_unfinished():
            raise EngineError("score needs an idle engine")
        tokens = [int(t) for t in tokens]
        if len(tokens) < 2:
            return []
        if len(tokens) > self.cfg.max_seq_len:
            raise ValueError("sequence longer than max_seq_len")
        key = ("score", id(tokens))
        rc = self.runner.open(key)
        out: List[float] = []
        try:
            if not self.runner.cache.reserve(rc, len(tokens) - 1):
                raise EngineError("not enough cache pages to score this sequence")
            chunk = min(self.cfg.max_num_batched_tokens, self.runner.max_rows)
            n = len(tokens) - 1
            target = torch.empty(chunk, dtype=torch.int32, device=self.runner.device)
            lp = torch.empty(chunk, dtype=torch.float32, device=self.runner.device)
            from ..ops import kernels
            for s in range(0, n, chunk):
                m = min(chunk, n - s)
                logits, _ = self.runner.run([Segment(rc, tokens[s:s + m], s, tuple(range(m)))])
                target[:m].copy_(torch.tensor(tokens[s + 1:s + 1 + m], dtype=torch.int32))
                kernels.gather_logprob(logits, m, target, lp)
                out.extend(lp[:m].tolist())
        finally:
            self.runner.close(key)
        self.runner.check_status()
        return out

    # ---------------------------------------------------------------- replay
    def open_request(self, key: object) -> None:
        if self.has_unfinished():
            raise EngineError("open_request needs an engine without unfinished scheduled requests")
        self.runner.open(key)
        self._replay_pos[key] = 0

    def close_request(self, key: object) -> None:
        self.runner.close(key)
        self._replay_pos.pop(key, None)

    def step_tokens(self, entries: Seq[Tuple[object, Seq[int], Seq[int]]], graphs: bool = False) -> torch.Tensor:
        """One step of given tokens: entries are (request key, its next tokens, wanted
        indices among them).  Returns float32 logits [wanted, vocab] on the device, in the
        order of the entries and of their wanted indices.  Requests are opened on first
        use; a step larger than the engine's token or row limits is run as several
        batches, which changes nothing about what a position attends to.  With ``graphs`` a
        batch of single tokens that all want their logits runs the way generation runs it:
        padded to a fixed shape, sampler included, replayed as a CUDA graph (if the engine
        has ``cuda_graphs`` on).  Requests given tokens here hold pages that the scheduler
        does not know of, so this is refused while scheduled requests are unfinished."""
        if self.has_unfinished():
            raise EngineError("step_tokens needs an engine without unfinished scheduled requests")
        cache = self.runner.cache
        pieces: List[List[Segment]] = [[]]
        used_t = used_r = 0
        max_t, max_r, max_s = self.cfg.max_num_batched_tokens, self.runner.max_rows, self.cfg.max_num_seqs
        total_rows = 0
        order: List[int] = []      # row of the computed (sorted, unique) logits for every wanted place
        for key, toks, want in entries:
            if key not in self._replay_pos:
                self.open_request(key)
            rc = cache.get(key)
            toks = [int(t) for t in toks]
            if not toks:
                if len(want):
                    raise ValueError(f"request {key!r}: logits wanted of a step that brings no tokens")
                continue
            want = [int(w) for w in want]
            for w in want:
                if not 0 <= w < len(toks):
                    raise ValueError(f"request {key!r}: wanted place {w} outside its {len(toks)} tokens")
            uniq = sorted(set(want))
            order.extend(total_rows + uniq.index(w) for w in want)
            pos = self._replay_pos[key]
            if pos + len(toks) > self.cfg.max_seq_len:
                raise EngineError(f"request {key!r} would grow to {pos + len(toks)} tokens, beyond "
                                  f"max_seq_len {self.cfg.max_seq_len}")
            if not cache.reserve(rc, pos + len(toks)):
                raise EngineError(f"out of cache pages for request {key!r} at {pos + len(toks)} tokens")
            i = 0
            while i < len(toks):
                if max_t - used_t <= 0 or len(pieces[-1]) >= max_s or used_r >= max_r:
                    pieces.append([])
                    used_t = used_r = 0
                n = min(max_t - used_t, len(toks) - i)
                w = [x - i for x in uniq if i <= x < i + n]
                if len(w) > max_r - used_r:          # cut the portion where the rows run out
                    w = w[:max_r - used_r]
                    n = w[-1] + 1
                pieces[-1].append(Segment(rc, toks[i:i + n], pos + i, tuple(w)))
                used_t += n
                used_r += len(w)
                total_rows += len(w)
                i += n
            self._replay_pos[key] = pos + len(toks)
        out = torch.empty((total_rows, self.vocab_size), dtype=torch.float32, device=self.runner.device)
        r = 0
        for segs in pieces:
            if not segs:
                continue
            logits, _ = self.runner.run(segs, sample=graphs)
            n = sum(len(sg.want) for sg in segs)       # (a graph step is padded: its context counts more rows)
            out[r:r + n].copy_(logits[:n])
            r += n
        for key, toks, _ in entries:
            if len(toks):
                cache.release_passed(cache.get(key), self._replay_pos[key])
        if order != list(range(total_rows)):
            out = out[torch.tensor(order, dtype=torch.long, device=out.device)]
        return out

    # --------------------------------------------------------------- reports
    def set_op_profiling(self, on: bool) -> None:
        """Per-op device time of every step from now on (reference: Engine::set_op_profiling,
        src/cuda/engine/engine.h:120-124).  Steps run eagerly meanwhile, which skews throughput."""
        self.runner.set_op_profiling(on)

    def reset_op_profile(self) -> None:
        if self.runner.profiler is not None:
            self.runner.profiler.reset()

    def op_profile(self, hbm_gbs: float = 0.0, tflops: float = 0.0) -> List[Dict[str, Any]]:
        """Rows of the per-op table (engine.profiler.OpProfiler.report), with roofline fractions against
        the given peaks."""
        return self.runner.profiler.report(hbm_gbs, tflops) if self.runner.profiler is not None else []

    def reset_peak_memory(self) -> None:
        free, total = torch.cuda.mem_get_info(self.runner.device)
        self.peak_device_used = total - free
        torch.cuda.reset_peak_memory_stats(self.runner.device)

    def memory_report(self) -> Dict[str, Any]:
        rep: Dict[str, Any] = dict(self.runner.memory_report())
        free, total = torch.cuda.mem_get_info(self.runner.device)
        rep["device_total"] = total
        rep["device_used"] = total - free
        self.peak_device_used = max(self.peak_device_used, total - free)
        rep["peak_device_used_bytes"] = self.peak_device_used
        rep["torch_peak"] = torch.cuda.max_memory_allocated(self.runner.device)
        return rep

    def describe(self) -> Dict[str, Any]:
        c = self.runner.cache
        return {
            "engine": "redline_b200",
            "model": self.cfg.model,
            "architecture": self.model_config.architecture,
            "dtype": self.cfg.dtype,
            "config": {k: getattr(self.cfg, k) for k in (
                "max_num_seqs", "max_num_batched_tokens", "max_seq_len", "block_size", "kv_cache_tokens",
                "gpu_memory_utilization", "cuda_graphs", "async_scheduling", "mix_prefill_decode", "nvtx_layers",
                "track_memory")},
            "cache_groups": [{"kind": g.spec.kind, "window": g.spec.window, "layers": len(g.owners),
                              "tensors": {t.name: list(t.shape) for t in g.spec.tensors},
                              "pages": c.num_total_pages(i)} for i, g in enumerate(c.groups)],
            "weight_bytes": self.runner.model.weight_bytes(),
        }
