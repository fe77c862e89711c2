"""Continuous batching on the host: which sequences run in the next step and how
many tokens each of them brings.

Every ``schedule()`` plans one step under a token budget: first one token for every
running sequence that is decoding, then portions of prompts (running sequences that
are mid-prompt first, then new admissions in arrival order).  A new sequence is
admitted only while a watermark of pages stays free, unless nothing is running.
When a decoding sequence cannot get its next page, the newest running sequence that
is not yet in the plan is preempted (all its pages go back, it is queued again at
the front and later recomputed from its prompt plus what it has generated); if there
is none, the sequence itself is.  A sequence whose newest token is still on the GPU
("pending") may be planned anyway: its next step reads the token on the device.
Policy of the reference's scheduler (src/core/scheduler.cpp:24-218).

This module is host code only; it talks to the ``CacheManager`` and to nothing on
the GPU.  The plan loop is native code (``rl_sched_plan`` in csrc/host_core.cpp, beside the
cache manager's state it works on); the request objects, the queues and the life cycle
(add, finish, preempt on request, tokens received) are kept here.
"""

from __future__ import annotations

import ctypes
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional

from ..cache import native
from ..cache.manager import CacheManager, RequestCache
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass(eq=False)
class Sequence:
    """Host state of one request (reference: src/core/sequence.h:31-67)."""

    id: int
    tokens: List[int]                  # tokens the host knows: prompt + received samples
    prompt_len: int
    params: SamplingParams
    stop_ids: frozenset = frozenset()
    status: str = WAITING
    finish_reason: str = ""
    num_computed: int = 0              # positions whose cache writes have been enqueued
    num_pending: int = 0               # tokens sampled on the GPU that the host has not read yet
    pending_step: int = -1
    pending_row: int = -1
    requeue_when_received: bool = False
    cache: Optional[RequestCache] = None
    num_preemptions: int = 0
    arrival_time: float = 0.0
    first_token_time: float = -1.0
    finish_time: float = -1.0
    token_times: List[float] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)

    @property
    def total_len(self) -> int:
        return len(self.tokens) + self.num_pending

    @property
    def num_generated(self) -> int:
        return self.total_len - self.prompt_len

    @property
    def num_uncomputed(self) -> int:
        return self.total_len - self.num_computed


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 32
    max_num_batched_tokens: int = 2048
    max_seq_len: int = 4096
    mix_prefill_decode: bool = True
    admission_watermark: float = 0.01


@dataclass
class ScheduledSeq:
    seq: Sequence
    start_pos: int
    num_tokens: int
    sample: bool                      # a new token is drawn after the last position
    input_from_device: bool = False
    src_row: int = -1


@dataclass
class StepPlan:
    step_id: int = 0
    seqs: List[ScheduledSeq] = field(default_factory=list)
    num_tokens: int = 0
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    num_preempted: int = 0

    @property
    def empty(self) -> bool:
        return not self.seqs

    @property
    def pure_decode(self) -> bool:
        return bool(self.seqs) and all(s.num_tokens == 1 and s.sample for s in self.seqs)


class SchedulerError(ValueError):
    pass


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, cache: CacheManager):
        if cfg.max_num_seqs <= 0 or cfg.max_num_batched_tokens < cfg.max_num_seqs:
            raise SchedulerError("max_num_batched_tokens must be >= max_num_seqs > 0")
        self.cfg = cfg
        self.cache = cache
        self.running: List[Sequence] = []      # admission order, oldest first
        self.waiting: Deque[Sequence] = deque()
        self.parked: List[Sequence] = []       # preempted with a token still in flight

    # ------------------------------------------------------------- requests
    def add(self, seq: Sequence) -> None:
        if seq.prompt_len <= 0:
            raise SchedulerError("empty prompt")
        if seq.total_len >= self.cfg.max_seq_len:
            raise SchedulerError(f"prompt of length {seq.total_len} does not fit max_seq_len="
                                 f"{self.cfg.max_seq_len}")
        worst = min(self.cfg.max_seq_len, seq.total_len + seq.params.max_new_tokens)
        for g in range(len(self.cache.groups)):
            if self.cache.blocks_for(worst) > self.cache.num_total_pages(g):
                raise SchedulerError(f"request {seq.id} needs more cache pages than the whole cache holds")
        seq.status = WAITING
        self.waiting.append(seq)

    def needs_compute(self, seq: Sequence) -> bool:
        if seq.status == FINISHED:
            return False
        if seq.num_uncomputed > 1:
            return True
        if seq.num_uncomputed == 0:
            return False
        if seq.num_generated >= seq.params.max_new_tokens:
            return False
        if seq.total_len >= self.cfg.max_seq_len:
            return False
        return True

    def has_unfinished(self) -> bool:
        return bool(self.running or self.waiting or self.parked)

    # ---------------------------------------------------------------- pages
    def _drop_cache(self, seq: Sequence) -> None:
        if seq.cache is not None:
            self.cache.close(seq.id)
            seq.cache = None

    def preempt(self, seq: Sequence) -> None:
        self._drop_cache(seq)
        seq.num_computed = 0
        seq.status = WAITING
        seq.num_preemptions += 1
        if seq in self.running:
            self.running.remove(seq)
        if seq.num_pending > 0:
            seq.requeue_when_received = True
            self.parked.append(seq)
        else:
            self.waiting.appendleft(seq)

    def on_tokens_received(self, seq: Sequence) -> None:
        if not seq.requeue_when_received or seq.num_pending > 0:
            return
        seq.requeue_when_received = False
        if seq in self.parked:
            self.parked.remove(seq)
        if seq.status != FINISHED:
            self.waiting.appendleft(seq)

    def finish(self, seq: Sequence, reason: str) -> None:
        if seq.status == FINISHED:
            return
        seq.status = FINISHED
        seq.finish_reason = reason
        self._drop_cache(seq)
        if seq in self.running:
            self.running.remove(seq)
        if seq in self.waiting:
            self.waiting.remove(seq)
        if seq in self.parked:
            self.parked.remove(seq)

    def after_step(self, plan: StepPlan) -> None:
        """Window groups give back the pages that every later token is past."""
        for e in plan.seqs:
            if e.seq.cache is not None and e.seq.status == RUNNING:
                self.cache.release_passed(e.seq.cache, e.seq.num_computed)

    # ------------------------------------------------------------- planning
    def schedule(self, step_id: int, prev_step_id: int = -1) -> StepPlan:
        """Plans one step.  The plan loop itself is native (``rl_sched_plan`` in csrc/host_core.cpp): it
        works on the cache manager's state directly; here the sequences' numbers are handed to it and
        what it decided is written back to the sequences and the queues."""
        import numpy as np
        cfg = self.cfg
        # every running sequence, and as much of the waiting queue's front as could be admitted
        nw = min(len(self.waiting), cfg.max_num_seqs)
        seqs: List[Sequence] = list(self.running) + [self.waiting[i] for i in range(nw)]
        nr = len(self.running)
        n = len(seqs)
        flat: List[int] = []
        for q in seqs:
            flat += (q.cache.rid if q.cache is not None else -1, len(q.tokens), q.num_pending, q.num_computed,
                     q.prompt_len, min(q.params.max_new_tokens, 2**31 - 1),
                     1 if (q.num_pending > 0 and q.pending_step == prev_step_id) else 0, q.pending_row, 0, 0, 0)
        nf = len(native.SCHED_SEQ_FIELDS)
        rec = np.array(flat, dtype=np.int32).reshape(n, nf) if n else np.zeros((1, nf), dtype=np.int32)
        entries = np.empty((max(n, 1), len(native.SCHED_ENTRY_FIELDS)), dtype=np.int32)
        order = np.empty((3, max(n, 1)), dtype=np.int32)
        counts = np.zeros(6, dtype=np.int32)
        ncfg = native.RlSchedCfg(cfg.max_num_seqs, cfg.max_num_batched_tokens, cfg.max_seq_len,
                                 1 if cfg.mix_prefill_decode else 0, cfg.admission_watermark)
        code = self.cache._lib.rl_sched_plan(self.cache._h, ctypes.byref(ncfg), rec.ctypes.data, nr, nw,
                                             entries.ctypes.data, order[0].ctypes.data, order[1].ctypes.data,
                                             order[2].ctypes.data, counts.ctypes.data)
        ne, n_run, n_wait, n_park, n_pre, bad = counts.tolist()
        # ---- what the planner did to the sequences
        for q, r in zip(seqs, rec.tolist()):
            rid, computed, where, preempted, changed = r[0], r[3], r[8], r[9], r[10]
            q.num_computed = computed
            if preempted:
                q.num_preemptions += preempted
            if changed:
                if q.cache is not None:
                    self.cache.forget(q.id)
                q.cache = self.cache.adopt(q.id, rid) if rid >= 0 else None
            if where == 0:
                q.status = RUNNING
            else:
                q.status = WAITING
                if where == 2:
                    q.requeue_when_received = True
        order_l = order.tolist()
        self.running = [seqs[i] for i in order_l[0][:n_run]]
        for _ in range(nw):
            self.waiting.popleft()
        self.waiting.extendleft(seqs[i] for i in reversed(order_l[1][:n_wait]))
        self.parked.extend(seqs[i] for i in order_l[2][:n_park])
        if code == -10:
            raise SchedulerError(f"sequence {seqs[bad].id} needs a device token that is not available")
        if code != 0:
            raise SchedulerError(f"the planner refused its arguments (code {code})")
        plan = StepPlan(step_id=step_id, num_preempted=n_pre)
        for i, start, num, sample, from_device, src_row in entries[:ne].tolist():
            plan.seqs.append(ScheduledSeq(seqs[i], start, num, bool(sample), bool(from_device), src_row))
            plan.num_tokens += num
            if num == 1 and sample:
                plan.num_decode_tokens += 1
            else:
                plan.num_prefill_tokens += num
        return plan
