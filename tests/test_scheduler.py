"""The scheduler's decisions, with token delivery simulated on the host (no GPU):
portions under a budget, decode beside prefill, pending device tokens, finishing,
what happens when pages run out (scenarios of the reference's tests/cpp/test_core.cpp:188-301)."""

import pytest

from redline_b200.cache import CacheManager, GroupInfo
from redline_b200.engine.scheduler import FINISHED, RUNNING, Scheduler, SchedulerConfig, SchedulerError, Sequence
from redline_b200.parts.spec import CacheSpec
from redline_b200.sampling import SamplingParams


def make(pages=64, max_seqs=4, budget=32, max_len=256, mix=True, watermark=0.01):
    cache = CacheManager([GroupInfo(CacheSpec.keys_values("full", 2, 64), [0, 1])], [pages + 1], 16, max_seqs)
    return Scheduler(SchedulerConfig(max_seqs, budget, max_len, mix, watermark), cache), cache


def seq(i, n, new=8):
    return Sequence(id=i, tokens=list(range(n)), prompt_len=n, params=SamplingParams(max_new_tokens=new))


def deliver(sched, plan, step, token=5, sync=True):
    """What the engine does around a step: mark samples pending, then (sync) receive them."""
    row = 0
    got = []
    for e in plan.seqs:
        if e.sample:
            e.seq.num_pending += 1
            e.seq.pending_step, e.seq.pending_row = step, row
            row += 1
            got.append(e.seq)
    if sync:
        receive(sched, got, token)
    return got


def receive(sched, seqs, token=5):
    for s in seqs:
        s.num_pending -= 1
        if s.status == FINISHED:
            continue
        s.tokens.append(token)
        if len(s.tokens) - s.prompt_len >= s.params.max_new_tokens:
            sched.finish(s, "length")
        else:
            sched.on_tokens_received(s)


def test_chunked_prefill_then_decode_beside_a_new_prompt():
    sched, cache = make(budget=32)
    a, b = seq(0, 52), seq(1, 8)
    sched.add(a), sched.add(b)
    p = sched.schedule(0)
    assert [(e.seq.id, e.start_pos, e.num_tokens, e.sample) for e in p.seqs] == [(0, 0, 32, False)]
    deliver(sched, p, 0)
    p = sched.schedule(1)          # the rest of a, then b fills what is left of the budget
    assert [(e.seq.id, e.start_pos, e.num_tokens, e.sample) for e in p.seqs] == [(0, 32, 20, True), (1, 0, 8, True)]
    assert p.num_prefill_tokens == 28 and not p.pure_decode
    deliver(sched, p, 1)
    p = sched.schedule(2)
    assert [(e.seq.id, e.start_pos, e.num_tokens, e.sample) for e in p.seqs] == [(0, 52, 1, True), (1, 8, 1, True)]
    assert p.pure_decode and p.num_decode_tokens == 2
    assert a.cache.tables[0] == [1, 2, 3, 4] and b.cache.tables[0] == [5]
    cache.check_invariants()


def test_pending_token_is_read_on_the_device_and_everything_is_returned_at_the_end():
    sched, cache = make()
    a = seq(0, 5, new=3)
    sched.add(a)
    p0 = sched.schedule(0)
    inflight = deliver(sched, p0, 0, sync=False)          # token of step 0 not read yet
    p1 = sched.schedule(1, prev_step_id=0)
    assert [(e.start_pos, e.num_tokens, e.input_from_device, e.src_row) for e in p1.seqs] == [(5, 1, True, 0)]
    with pytest.raises(SchedulerError):                    # two steps behind is not available
        a.num_computed -= 1
        a.pending_step = -7
        sched.schedule(2, prev_step_id=0)
    a.pending_step = 0
    a.num_computed += 1
    receive(sched, inflight)
    inflight = deliver(sched, p1, 1, sync=False)
    p2 = sched.schedule(2, prev_step_id=1)
    assert len(p2.seqs) == 1 and p2.seqs[0].input_from_device
    receive(sched, inflight)
    inflight = deliver(sched, p2, 2, sync=False)
    assert sched.schedule(3, prev_step_id=2).empty         # 3 tokens are wanted, all are in flight or here
    receive(sched, inflight)
    assert a.status == FINISHED and a.finish_reason == "length" and len(a.tokens) == 8
    assert not sched.has_unfinished() and cache.num_open() == 0 and cache.num_free_pages(0) == 64


def test_pages_run_out_newest_is_preempted_and_recomputed():
    sched, cache = make(pages=6, budget=64, watermark=0.0)
    a, b = seq(0, 40, new=30), seq(1, 40, new=30)
    sched.add(a), sched.add(b)
    preempted = 0
    finished = []
    for step in range(200):
        p = sched.schedule(step)
        preempted += p.num_preempted
        if p.empty:
            break
        for e in p.seqs:
            assert e.seq.status == RUNNING and len(e.seq.cache.tables[0]) * 16 >= e.start_pos + e.num_tokens
        deliver(sched, p, step)
        cache.check_invariants()
    assert preempted > 0 and b.num_preemptions > 0 and a.num_preemptions == 0
    assert a.status == FINISHED and b.status == FINISHED and len(a.tokens) == 70 and len(b.tokens) == 70
    assert cache.num_free_pages(0) == 6 and cache.num_open() == 0


def test_recompute_covers_generated_tokens_and_samples_only_at_the_end():
    sched, cache = make(pages=8, budget=16, watermark=0.0)
    a = seq(0, 20, new=50)
    sched.add(a)
    for step in range(6):
        deliver(sched, sched.schedule(step), step)
    n = len(a.tokens)
    sched.preempt(a)
    assert a.cache is None and a.num_computed == 0 and cache.num_free_pages(0) == 8
    plans = []
    for step in range(6, 9):
        p = sched.schedule(step)
        plans.append([(e.start_pos, e.num_tokens, e.sample) for e in p.seqs])
        deliver(sched, p, step)
    assert plans[0] == [(0, 16, False)] and plans[1] == [(16, n - 16, True)] and plans[2] == [(n, 1, True)]


def test_watermark_and_request_too_large_and_no_mix():
    sched, cache = make(pages=10, budget=128, watermark=0.5)
    a, b = seq(0, 60), seq(1, 40)
    sched.add(a), sched.add(b)
    p = sched.schedule(0)      # a takes 4 pages; admitting b (3 pages) would leave 3 < 5 free
    assert [e.seq.id for e in p.seqs] == [0]
    with pytest.raises(SchedulerError, match="whole cache"):
        sched.add(seq(2, 150, new=100))
    with pytest.raises(SchedulerError, match="max_seq_len"):
        sched.add(seq(3, 256))
    with pytest.raises(SchedulerError, match="empty"):
        sched.add(Sequence(id=4, tokens=[], prompt_len=0, params=SamplingParams()))

    sched, cache = make(budget=32, mix=False)
    a, b = seq(0, 8), seq(1, 8)
    sched.add(a)
    deliver(sched, sched.schedule(0), 0)
    sched.add(b)
    p = sched.schedule(1)      # prefill-only steps come first when mixing is off
    assert [(e.seq.id, e.num_tokens) for e in p.seqs] == [(1, 8)]
    deliver(sched, p, 1)
    p = sched.schedule(2)
    assert p.pure_decode and len(p.seqs) == 2


def test_starved_prompts_free_the_newest_until_the_oldest_goes_on():
    sched, cache = make(pages=5, budget=48, watermark=0.0, max_len=512)
    a, b = seq(0, 70, new=4), seq(1, 60, new=4)
    sched.add(a), sched.add(b)
    p = sched.schedule(0)      # a: 48 tokens (3 pages)
    deliver(sched, p, 0)
    a_first = [(e.seq.id, e.num_tokens) for e in p.seqs]
    assert a_first == [(0, 48)]
    p = sched.schedule(1)      # a: 22 more (2 pages); nothing left for b
    deliver(sched, p, 1)
    done = False
    for step in range(2, 60):
        p = sched.schedule(step)
        if p.empty:
            done = True
            break
        deliver(sched, p, step)
        cache.check_invariants()
    assert done and a.status == FINISHED and b.status == FINISHED


@pytest.mark.parametrize("asynchronous", [False, True])
def test_random_workloads_keep_the_invariants_and_everything_finishes(asynchronous):
    """Random arrivals, lengths, pools and limits: every plan stays within the budget and the sequence
    limit, a sequence's portions follow one another without gaps, no page is lost or held twice, and every
    request that was accepted finishes (with its tokens received one step late if asynchronous)."""
    import random
    for seed in range(60):
        rng = random.Random(seed)
        pages, max_seqs = rng.choice([6, 10, 20, 40, 200]), rng.choice([1, 2, 3, 4, 8])
        budget = max(rng.choice([4, 16, 32, 100]), max_seqs)
        max_len, mix = rng.choice([64, 128, 400]), rng.random() < 0.7
        sched, cache = make(pages, max_seqs, budget, max_len, mix, rng.choice([0.0, 0.01, 0.1, 0.3]))
        accepted, inflight, nid, step = [], [], 0, 0
        computed = {}
        while step < 60 or sched.has_unfinished() or inflight:
            assert step < 5000, f"seed {seed}: the workload does not come to an end"
            if step < 60:
                for _ in range(rng.choice([0, 0, 1, 1, 2])):
                    s = seq(nid, rng.randint(1, max_len - 2), rng.randint(1, 40))
                    nid += 1
                    try:
                        sched.add(s)
                        accepted.append(s)
                    except SchedulerError:
                        pass
            plan = sched.schedule(step, step - 1)
            assert plan.num_tokens <= budget and len(sched.running) <= max_seqs
            assert plan.num_tokens == sum(e.num_tokens for e in plan.seqs) == plan.num_prefill_tokens + plan.num_decode_tokens
            assert len({e.seq.id for e in plan.seqs}) == len(plan.seqs)
            for e in plan.seqs:
                assert e.seq.status == RUNNING and e.seq in sched.running and e.seq.cache is not None
                # a portion begins where the last one ended, or at 0 after a preemption
                assert e.start_pos == computed.get(e.seq.id, 0) or e.start_pos == 0
                computed[e.seq.id] = e.start_pos + e.num_tokens
                assert e.seq.num_computed == computed[e.seq.id] <= len(e.seq.tokens) + e.seq.num_pending
                assert e.seq.cache.num_tokens >= computed[e.seq.id]
                assert e.sample == (computed[e.seq.id] == len(e.seq.tokens) + e.seq.num_pending)
                assert e.input_from_device == (e.start_pos >= len(e.seq.tokens))
            for s in list(sched.waiting) + sched.parked:
                assert s.cache is None and s.num_computed == 0
            got = deliver(sched, plan, step, sync=False)
            sched.after_step(plan)
            todo, inflight = (inflight, got) if asynchronous else (got, [])
            for s in todo:                                  # as the engine does: length limits end a request
                s.num_pending -= 1
                if s.status == FINISHED:
                    continue
                s.tokens.append(5)
                if len(s.tokens) - s.prompt_len >= s.params.max_new_tokens or len(s.tokens) >= max_len:
                    sched.finish(s, "length")
                else:
                    sched.on_tokens_received(s)
            cache.check_invariants()
            step += 1
        assert all(s.status == FINISHED for s in accepted), f"seed {seed}"
        assert cache.num_open() == 0 and cache.num_free_pages(0) == cache.num_total_pages(0)
