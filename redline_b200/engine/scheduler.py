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
the GPU.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional

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
    def _watermark(self, group: int) -> int:
        return int(self.cfg.admission_watermark * self.cache.num_total_pages(group))

    def _ensure(self, seq: Sequence, num_positions: int) -> bool:
        if seq.cache is None:
            seq.cache = self.cache.open(seq.id)
        return self.cache.reserve(seq.cache, num_positions)

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
        plan = StepPlan(step_id=step_id)
        budget = self.cfg.max_num_batched_tokens

        def add_entry(seq: Sequence, n: int) -> None:
            nonlocal budget
            e = ScheduledSeq(seq, seq.num_computed, n, seq.num_computed + n == seq.total_len)
            if e.start_pos >= len(seq.tokens):
                if not (n == 1 and seq.num_pending > 0 and seq.pending_step == prev_step_id):
                    raise SchedulerError(f"sequence {seq.id} needs a device token that is not available")
                e.input_from_device = True
                e.src_row = seq.pending_row
            seq.num_computed += n
            budget -= n
            plan.num_tokens += n
            if n == 1 and e.sample:
                plan.num_decode_tokens += 1
            else:
                plan.num_prefill_tokens += n
            plan.seqs.append(e)

        def schedule_prefill() -> None:
            for seq in list(self.running):
                if budget <= 0:
                    return
                if seq.num_uncomputed <= 1:
                    continue
                # a pending token cannot be part of a multi-token portion
                known = len(seq.tokens) - seq.num_computed
                chunk = min(known if seq.num_pending else seq.num_uncomputed, budget)
                if chunk <= 0:
                    continue
                if not self._ensure(seq, seq.num_computed + chunk):
                    return
                add_entry(seq, chunk)
            while self.waiting and budget > 0 and len(self.running) < self.cfg.max_num_seqs:
                seq = self.waiting[0]
                chunk = min(seq.num_uncomputed, budget)
                if self.running:
                    need = self.cache.blocks_for(seq.num_computed + chunk)
                    short = any(self.cache.num_free_pages(g) - need < self._watermark(g)
                                for g in range(len(self.cache.groups)))
                    if short:
                        return
                if self.cache.num_open() >= self.cache.num_state_slots and seq.cache is None:
                    return
                if not self._ensure(seq, seq.num_computed + chunk):
                    self._drop_cache(seq)
                    return
                self.waiting.popleft()
                seq.status = RUNNING
                self.running.append(seq)
                add_entry(seq, chunk)

        def schedule_decode() -> None:
            i = 0
            while i < len(self.running):
                seq = self.running[i]
                if budget <= 0:
                    break
                if seq.num_uncomputed != 1 or not self.needs_compute(seq):
                    i += 1
                    continue
                self_preempted = False
                while not self._ensure(seq, seq.num_computed + 1):
                    victim = self.running[-1]
                    in_plan = any(e.seq is victim for e in plan.seqs)
                    if victim is seq or in_plan:
                        self.preempt(seq)
                        self_preempted = True
                        break
                    self.preempt(victim)
                    plan.num_preempted += 1
                if self_preempted:
                    plan.num_preempted += 1
                    continue            # running shrank at position i
                add_entry(seq, 1)
                i += 1

        if self.cfg.mix_prefill_decode:
            schedule_decode()
            schedule_prefill()
        else:
            schedule_prefill()
            if plan.empty:
                schedule_decode()

        # Sequences stuck mid-prompt can hold every page with none able to go on:
        # free the newest until the oldest can continue.
        while plan.empty and len(self.running) > 1:
            if not any(self.needs_compute(s) for s in self.running):
                break
            self.preempt(self.running[-1])
            plan.num_preempted += 1
            schedule_prefill()
            if plan.empty:
                schedule_decode()
        return plan
