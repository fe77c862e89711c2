"""Generation through the entry point: greedy against the plain implementation; the
engine's modes (graphs, asynchronous scheduling, mixed batches) give the same tokens;
prompts cut into portions under a small budget; a pool so small that sequences are
preempted and recomputed; stop tokens; seeded sampling; scoring; the command line."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as P
import tiny_configs as C
from gpu_utils import make_model, oracle_logits, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gen_models")
    return {n: make_model(tmp, C.ALL[n], seed=40 + i, sharpen=5.0) for i, n in enumerate(["tiny_a", "tiny_b"])}


def check_greedy(cfg_json, w, prompt, output, margin):
    """Every generated token's oracle logit is within ``margin`` of the oracle's maximum
    given the same prefix (0: it is the arg max); the reference's check for its
    half-precision engine uses 0.1 (tests/cuda/test_engine.cpp:77-95)."""
    seq = list(prompt) + list(output)
    logits = oracle_logits(cfg_json, w, seq[:-1])
    for i, tok in enumerate(output):
        row = logits[len(prompt) - 1 + i]
        assert row[tok] >= row.max() - margin, (i, tok, int(row.argmax()), float(row.max() - row[tok]))


@pytest.mark.parametrize("name,dtype,margin", [("tiny_a", "float32", 1e-4), ("tiny_b", "float32", 1e-4),
                                                ("tiny_a", "bfloat16", 0.1), ("tiny_b", "bfloat16", 0.1)])
def test_greedy_through_the_entry_point(name, dtype, margin, models):
    from redline_b200.runtime import Engine
    d, w = models[name]
    V = C.ALL[name]["vocab_size"]
    lens = [5, 17, 33] if name == "tiny_a" else [1, 40, 70, 129]
    prompts = [random_tokens(V, n, 60 + n) for n in lens]
    eng = Engine(d, dtype=dtype, max_seqs=4, max_batched_tokens=32, max_seq_len=256, kv_cache_tokens=1024)
    outs = eng.generate(prompts, max_new_tokens=12, ignore_eos=True)
    assert [o["id"] for o in outs] == list(range(len(prompts)))
    for p, o in zip(prompts, outs):
        assert o["prompt_ids"] == p and len(o["output_ids"]) == 12 and o["finish_reason"] == "length"
        assert len(o["logprobs"]) == 12 and all(lp <= 0 for lp in o["logprobs"]) and o["ttft_s"] > 0
        check_greedy(C.ALL[name], w, p, o["output_ids"], margin)
    if dtype == "float32":
        pc = P.plain_config(C.ALL[name])
        assert outs[1]["output_ids"] == P.greedy_generate(pc, w, prompts[1], 12)
        lp = torch.log_softmax(torch.from_numpy(oracle_logits(C.ALL[name], w, prompts[0] + outs[0]["output_ids"])), -1)
        want = [float(lp[len(prompts[0]) - 1 + i, t]) for i, t in enumerate(outs[0]["output_ids"])]
        assert np.abs(np.array(outs[0]["logprobs"]) - np.array(want)).max() < 1e-3
    assert eng.vocab_size == V and eng.describe()["architecture"] == "LlamaForCausalLM"
    assert eng.memory_report()["weights"] > 0


def test_modes_give_the_same_tokens(models):
    """Graphs on or off, asynchronous or not, mixed batches or not: in float32 the same tokens."""
    from redline_b200.engine.engine import Engine
    d, w = models["tiny_a"]
    prompts = [random_tokens(512, n, 70 + n) for n in (40, 46, 41, 44, 45, 43)]
    results = []
    for graphs, asyn, mix in [(False, False, True), (True, True, True), (True, False, False), (False, True, True)]:
        # (6 sequences at most: no power of two, so the widest decode steps need the limit itself as a graph size)
        eng = Engine(d, dtype="float32", max_num_seqs=6, max_num_batched_tokens=64, max_seq_len=256,
                     kv_cache_tokens=2048, cuda_graphs=graphs, async_scheduling=asyn, mix_prefill_decode=mix)
        eng.record_steps = True
        outs = eng.generate(prompts, max_new_tokens=24, ignore_eos=True)
        results.append([o["output_ids"] for o in outs])
        kinds = {r.kind for r in eng.records}
        assert "decode" in kinds
        if mix:
            assert "mixed" in kinds, kinds       # portions of later prompts ran beside decoded tokens
        else:
            assert "mixed" not in kinds, kinds
        if graphs:
            assert eng.runner.num_graph_steps > 0 and any(r.num_seqs == 6 for r in eng.records)
            assert all(r.cuda_graph for r in eng.records if r.kind == "decode")
        else:
            assert eng.runner.num_graph_steps == 0
        assert eng.runner.cache.num_open() == 0
        eng.runner.cache.check_invariants()
    assert all(r == results[0] for r in results[1:])
    for p, o in zip(prompts, results[0]):
        check_greedy(C.TINY_A, w, p, o, 1e-4)


def test_preemption_in_a_small_pool_changes_nothing(models):
    from redline_b200.engine.engine import Engine
    d, w = models["tiny_a"]
    prompts = [random_tokens(512, n, 90 + n) for n in (40, 35, 44, 38)]
    big = Engine(d, dtype="float32", max_num_seqs=4, max_num_batched_tokens=64, max_seq_len=128, kv_cache_tokens=1024)
    want = [o["output_ids"] for o in big.generate(prompts, max_new_tokens=30, ignore_eos=True)]
    small = Engine(d, dtype="float32", max_num_seqs=4, max_num_batched_tokens=64, max_seq_len=128,
                   kv_cache_tokens=160, admission_watermark=0.0)
    outs = small.generate(prompts, max_new_tokens=30, ignore_eos=True)
    assert small.num_preemptions > 0 and sum(o["num_preemptions"] for o in outs) > 0
    assert [o["output_ids"] for o in outs] == want
    assert small.runner.cache.num_open() == 0 and small.runner.cache.num_free_pages(0) == 10


def test_stop_tokens_and_seeded_sampling(models):
    from redline_b200.engine.engine import Engine
    d, w = models["tiny_b"]
    eng = Engine(d, dtype="float32", max_num_seqs=4, max_num_batched_tokens=64, max_seq_len=256, kv_cache_tokens=1024)
    p = random_tokens(1000, 20, 5)
    base = eng.generate([p], max_new_tokens=16, ignore_eos=True)[0]["output_ids"]
    stop = base[5]
    first = base.index(stop)
    o = eng.generate([p], max_new_tokens=16, ignore_eos=True, stop_token_ids=[stop])[0]
    assert o["finish_reason"] == "stop" and o["output_ids"] == base[:first + 1]
    # eos from config.json stops unless ignored (TINY_B's eos ids are 7 and 9)
    a = eng.generate([p, p[:7]], max_new_tokens=12, temperature=0.8, seed=11, ignore_eos=True)
    b = eng.generate([p, p[:7]], max_new_tokens=12, temperature=0.8, seed=11, ignore_eos=True)
    c = eng.generate([p, p[:7]], max_new_tokens=12, temperature=0.8, seed=12, ignore_eos=True)
    assert [x["output_ids"] for x in a] == [x["output_ids"] for x in b]
    assert [x["output_ids"] for x in a] != [x["output_ids"] for x in c]
    # request i uses seed + i: the second request of seed 11 is the first of seed 12
    d2 = eng.generate([p[:7]], max_new_tokens=12, temperature=0.8, seed=12, ignore_eos=True)
    assert d2[0]["output_ids"] == a[1]["output_ids"]
    # the first drawn token is the plain restatement's draw from the oracle's logits
    logits = oracle_logits(C.TINY_B, w, p).astype(np.float32)[-1]
    assert a[0]["output_ids"][0] == P.gumbel_draw(logits, 0.8, 0, 1.0, 11, len(p))
    with pytest.raises(ValueError):
        eng.generate([[1000]], max_new_tokens=2)
    with pytest.raises(ValueError):
        eng.generate([[]], max_new_tokens=2)


def test_score_in_portions(models):
    from redline_b200.engine.engine import Engine
    d, w = models["tiny_a"]
    eng = Engine(d, dtype="float32", max_num_seqs=2, max_num_batched_tokens=64, max_logit_rows=40, max_seq_len=256,
                 kv_cache_tokens=512)
    toks = random_tokens(512, 150, 8)
    got = np.array(eng.score(toks))
    lp = torch.log_softmax(torch.from_numpy(oracle_logits(C.TINY_A, w, toks)), -1)
    want = np.array([float(lp[i, toks[i + 1]]) for i in range(len(toks) - 1)])
    assert got.shape == want.shape and np.abs(got - want).max() < 1e-3
    assert eng.runner.cache.num_open() == 0


def test_command_line(models, tmp_path):
    d, w = models["tiny_a"]
    p = random_tokens(512, 9, 3)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "redline_generate"), "--model", d, "--dtype", "float32",
           "--prompt-ids", ",".join(map(str, p)), "--prompt-ids", "5,6,7", "--max-new-tokens", "6", "--ignore-eos",
           "--max-seqs", "4", "--max-seq-len", "128", "--kv-cache-tokens", "512"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(x) for x in r.stdout.splitlines() if x.startswith("{")]
    assert [x["id"] for x in lines] == [0, 1] and all(len(x["output_ids"]) == 6 for x in lines)
    assert lines[0]["output_ids"] == P.greedy_generate(P.plain_config(C.TINY_A), w, p, 6)
    assert set(lines[0]) == {"id", "output_ids", "logprobs", "finish_reason", "ttft_ms", "e2e_ms"}
    r = subprocess.run(cmd[:5] + ["--bogus"], capture_output=True, text=True, timeout=600)
    assert r.returncode != 0
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(C.TINY_C))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "redline_generate"), "--random-weights", str(cfg),
                        "--weights-seed", "3", "--model", str(tmp_path / "rand"), "--prompt-ids", "1,2,3",
                        "--max-new-tokens", "4", "--ignore-eos", "--max-seq-len", "64", "--kv-cache-tokens", "256",
                        "--max-seqs", "2"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert os.path.exists(tmp_path / "rand" / "model.safetensors")
    assert len(json.loads([x for x in r.stdout.splitlines() if x.startswith("{")][0])["output_ids"]) == 4


def test_benchmark_harness_report(models, tmp_path):
    """The fields of the report (reference: tests/cuda/test_engine.cpp:233-248) and the
    redline_bench program."""
    from redline_b200.runtime import Engine
    d, _ = models["tiny_a"]
    eng = Engine(d, dtype="bfloat16", max_seqs=4, max_batched_tokens=64, max_seq_len=256, kv_cache_tokens=1024)
    doc = {"name": "t", "requests": [{"prompt_len": 20 + 7 * i, "max_new_tokens": 10} for i in range(5)]}
    rep = eng.benchmark(doc, warmup=1)
    assert rep["num_requests"] == 5 and rep["output_tokens"] == 50 and rep["prompt_tokens"] == sum(20 + 7 * i for i in range(5))
    for k in ("ttft_ms", "itl_ms", "tpot_ms", "e2e_latency_ms", "decode_step_gpu_ms", "host_overhead_ms"):
        assert rep[k]["count"] > 0 and rep[k]["p50"] > 0, k
    assert rep["decode_throughput_gpu_tok_s"] > 0 and rep["prefill_throughput_gpu_tok_s"] > 0
    assert rep["output_throughput_tok_s"] > 0 and 0 < rep["cuda_graph_step_fraction"] <= 1
    assert rep["memory"]["weights"] > 0 and rep["engine"]["engine"] == "redline_b200"
    out = tmp_path / "rep.json"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "redline_bench"), "--model", d, "--synthetic", "3,16,6",
                        "--max-seqs", "4", "--max-seq-len", "128", "--kv-cache-tokens", "512", "--out", str(out),
                        "--per-request"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    rep = json.loads(out.read_text())
    assert rep["workload"] == "synthetic_n3_in16_out6" and rep["output_tokens"] == 18 and len(rep["requests"]) == 3


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_per_op_profile_of_engine_steps(dtype, models, tmp_path):
    """--profile-ops: CUDA events between the ops of eager steps give a table per kind of step with
    every op of a layer, their calls per step, shares that add up, and roofline fractions; the tokens
    are those of an unprofiled run; NVTX ranges and memory tracking can be on meanwhile (reference:
    src/cuda/op_profiler.h:21-103, apps/redline_bench.cpp:39-49, apps/cli_common.cpp:89-90)."""
    from redline_b200.apps.harness import BenchOptions, parse_workload, run_benchmark
    from redline_b200.engine.engine import Engine
    from redline_b200.engine.profiler import format_op_profile
    d, _ = models["tiny_a"]
    layers = C.TINY_A["num_hidden_layers"]
    doc = {"name": "t", "requests": [{"prompt_len": 20 + 7 * i, "max_new_tokens": 10} for i in range(5)]}
    outs = {}
    for profile in (False, True):
        eng = Engine(d, dtype=dtype, max_num_seqs=4, max_num_batched_tokens=64, max_seq_len=256, kv_cache_tokens=1024,
                     nvtx_layers=profile, track_memory=profile)
        w = parse_workload(doc, eng.vocab_size)
        rep = run_benchmark(eng, w, BenchOptions(warmup_requests=1, profile_ops=profile, hbm_gbs=6500.0, bf16_tflops=1600.0))
        outs[profile] = rep
        if not profile:
            assert "op_profile" not in rep and rep["cuda_graph_step_fraction"] > 0
            continue
        assert rep["cuda_graph_step_fraction"] == 0                    # profiled steps are eager
        assert rep["memory"]["peak_device_used_bytes"] >= rep["memory"]["weights"]
        rows = rep["op_profile"]
        by_scope = {}
        for r in rows:
            scope, op = r["op"].split("/", 1)
            by_scope.setdefault(scope, {})[op] = r
            assert r["ms_per_pass"] > 0 and r["calls_per_pass"] > 0
        assert "decode" in by_scope and ("prefill" in by_scope or "mixed" in by_scope)
        for scope, ops in by_scope.items():
            assert abs(sum(r["pct"] for r in ops.values()) - 100.0) < 1e-6
            assert ops["embed"]["calls_per_pass"] == 1 and ops["sample"]["calls_per_pass"] == 1
            per_layer = [o for o in ops if "qkv_proj" in o or "o_proj" in o or "gate_up" in o or "down_proj" in o]
            assert len(per_layer) == 4 and all(ops[o]["calls_per_pass"] == layers for o in per_layer), (scope, list(ops))
            assert any("attention" in o for o in ops) and any("lm_head" in o for o in ops)
            products = [ops[o] for o in per_layer]
            assert all(r["gflop_per_pass"] > 0 and r["gbytes_per_pass"] > 0 and 0 < r["roofline_frac"] < 1.5 for r in products)
        text = format_op_profile(rows)
        assert "decode: per-op device time" in text and "of roofline" in text
    assert outs[True]["output_tokens"] == outs[False]["output_tokens"] == 50
    # the program's flag
    out = tmp_path / "rep.json"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "redline_bench"), "--model", d, "--synthetic", "3,16,6",
                        "--max-seqs", "4", "--max-seq-len", "128", "--kv-cache-tokens", "512", "--out", str(out),
                        "--profile-ops", "--nvtx-layers", "--track-memory", "--dtype", dtype],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "per-op device time" in r.stderr
    rep = json.loads(out.read_text())
    assert rep["op_profile"] and rep["engine"]["config"]["nvtx_layers"] and rep["engine"]["config"]["track_memory"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_logits_of_generation_with_graphs_and_tokens_fed_on_the_device(name, dtype, tmp_path):
    """Scheduled generation on its product path (CUDA graphs of padded decode batches, the next step
    launched before this step's tokens are read, so it takes them from the sampler's output on the
    device; a pool so small that sequences are preempted and recomputed): the logits of every position
    that was sampled from, against the plain implementation run on the finished sequences, with the
    tolerances of the replay tests; and the tokens are the arg max of those logits."""
    from gpu_utils import check_logits, engine_for, make_model
    cfg = C.ALL[name]
    d, w = make_model(tmp_path, cfg, seed=61, sharpen=6.0 if dtype == "float32" else 3.0)
    eng = engine_for(d, dtype, cuda_graphs=True, async_scheduling=True, max_num_seqs=8, max_num_batched_tokens=48,
                     kv_cache_tokens=320, max_seq_len=160)
    V = cfg["vocab_size"]
    prompts = [random_tokens(V, n, 90 + n) for n in (40, 5, 61, 33, 17, 50)]
    seen = {}

    def keep(where, logits):
        host = logits.cpu().numpy()
        for (rid, pos), row in zip(where, host):
            seen[rid, pos] = row.copy()

    eng.on_logits = keep
    eng.record_steps = True
    outs = eng.generate(prompts, max_new_tokens=40, ignore_eos=True)
    assert eng.runner.num_graph_steps > 0 and eng.num_preemptions > 0
    assert any(r.kind == "mixed" for r in eng.records)
    for o, p in zip(outs, prompts):
        seq = p + o["output_ids"]
        rows = list(range(len(p) - 1, len(seq) - 1))
        got = np.stack([seen[o["id"], r] for r in rows])
        check_logits(got, cfg, w, seq[:-1], dtype, rows=rows)
        assert [int(g.argmax()) for g in got] == o["output_ids"]
    assert eng.runner.cache.num_open() == 0
    eng.runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_prompt_portions_replay_one_graph(dtype, tmp_path):
    """Steps that are one full portion of a prompt (as many tokens as the engine takes a step) are one CUDA
    graph per number of wanted rows: captured for the first portion, replayed for the next two, which start
    later, lie in other pages and attend to a cached past.  Logits against the plain implementation, and
    the same as without graphs."""
    from gpu_utils import check_logits, engine_for, make_model
    cfg = C.TINY_A
    d, w = make_model(tmp_path, cfg, seed=71, sharpen=6.0 if dtype == "float32" else 3.0)
    V = cfg["vocab_size"]
    long = random_tokens(V, 3 * 128 + 20, 7)
    short = random_tokens(V, 128, 8)
    got = {}
    for graphs in (True, False):
        eng = engine_for(d, dtype, cuda_graphs=graphs, async_scheduling=False, max_num_seqs=2,
                         max_num_batched_tokens=128, kv_cache_tokens=1024, max_seq_len=512)
        rows = []
        for i in range(3):                               # full portions; the third wants its last row
            out = eng.step_tokens([("a", long[128 * i:128 * (i + 1)], [127] if i == 2 else [])], graphs=True)
            rows.append(out.cpu().numpy())
        rows.append(eng.step_tokens([("a", long[384:], [0, 19])], graphs=True).cpu().numpy())     # the rest: eager
        rows.append(eng.step_tokens([("b", short, [127])], graphs=True).cpu().numpy())
        got[graphs] = rows
        if graphs:
            keys = sorted(k for k in eng.runner._graphs if k[0] == "portion")
            assert keys == [("portion", 128, 0), ("portion", 128, 1)], keys
            assert eng.runner.num_graph_steps == 4
        else:
            assert eng.runner.num_graph_steps == 0
        eng.runner.check_status()
        eng.close_request("a")
        eng.close_request("b")
        eng.runner.cache.check_invariants()
    a_rows = np.concatenate([got[True][2], got[True][3]])
    check_logits(a_rows, cfg, w, long, dtype, rows=[383, 384, 403])
    check_logits(got[True][4], cfg, w, short, dtype, rows=[127])
    if dtype == "float32":
        for x, y in zip(got[True], got[False]):
            assert np.array_equal(x, y)


def test_generation_of_a_long_prompt_replays_the_portion_graph(models):
    """Through the scheduler (asynchronous, graphs on): a 400-token prompt in an engine of 128 tokens a step
    runs three full portions as one CUDA graph before its short rest; the tokens are the plain greedy ones."""
    from redline_b200.engine.engine import Engine
    d, w = models["tiny_a"]
    prompt = random_tokens(512, 400, 5)
    eng = Engine(d, dtype="float32", max_num_seqs=2, max_num_batched_tokens=128, max_seq_len=512, kv_cache_tokens=1024,
                 cuda_graphs=True, async_scheduling=True)
    out = eng.generate([prompt], max_new_tokens=10, ignore_eos=True)[0]
    assert ("portion", 128, 0) in eng.runner._graphs
    assert out["output_ids"] == P.greedy_generate(P.plain_config(C.TINY_A), w, prompt, 10)
    eng.runner.check_status()
