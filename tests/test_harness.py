"""Statistics and workloads of the benchmark harness (host side)."""

import pytest

from redline_b200.apps.harness import parse_workload, percentile, summarize, synthetic_workload


def test_percentiles_interpolate_linearly():
    v = [1.0, 2.0, 3.0, 4.0]
    assert percentile(v, 50) == 2.5 and percentile(v, 0) == 1.0 and percentile(v, 100) == 4.0
    assert percentile(v, 90) == pytest.approx(3.7) and percentile([], 50) == 0.0
    s = summarize(v)
    assert s["count"] == 4 and s["mean"] == 2.5 and s["std"] == pytest.approx(1.1180339887) and s["p99"] == pytest.approx(3.97)


def test_workloads():
    w = synthetic_workload(3, 17, 5, vocab_size=5000, seed=1)
    assert w.name == "synthetic_n3_in17_out5" and len(w.requests) == 3
    assert all(len(r.prompt) == 17 and min(r.prompt) >= 1000 and max(r.prompt) < 5000 for r in w.requests)
    assert w.requests[2].params.max_new_tokens == 5 and w.requests[2].params.ignore_eos and w.requests[2].params.seed == 2
    assert synthetic_workload(3, 17, 5, 5000, seed=1).requests[1].prompt == w.requests[1].prompt
    doc = {"name": "x", "seed": 3, "settings": {"batch_size": 2}, "requests": [
        {"prompt_ids": [5, 6, 7], "max_new_tokens": 4, "temperature": 0.5, "top_k": 3},
        {"prompt_len": 9, "arrival_time": 0.25, "stop_token_ids": [11]}]}
    w = parse_workload(doc, 400)
    assert w.requests[0].prompt == [5, 6, 7] and w.requests[0].params.top_k == 3 and w.settings == {"batch_size": 2}
    assert len(w.requests[1].prompt) == 9 and min(w.requests[1].prompt) >= 100 and w.requests[1].arrival_time == 0.25
    assert w.requests[1].id == 1 and w.requests[1].params.stop_token_ids == (11,)
    with pytest.raises(ValueError):
        parse_workload({"requests": [{"prompt_ids": [400]}]}, 400)
    with pytest.raises(ValueError):
        parse_workload({"requests": [{"prompt_ids": []}]}, 400)
