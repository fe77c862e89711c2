"""Logits at the real layer sizes: a random-weight model with the layer sizes of Llama 3.2 1B
(width 2048, 32 query and 8 kv heads of 64, feed-forward 8192, vocabulary 128,256, llama3
scaling with factor 32, tied head) and TWO layers instead of sixteen, so that the plain
float64 implementation can follow.  The engine's logits are compared with it, in float32 and
in bfloat16, on the paths that only these sizes reach:

* a 300-token prompt whole and cut at 130 / 170: the tcgen05 gate/up product, the library
  products at hundreds of rows, the tcgen05 prompt attention without and with a cached past,
  the head over 128,256 columns;
* 40 single-token steps of 8 sequences at contexts beyond 2,048 keys: the decode attention of
  one cluster per (sequence, kv head), and with that one switched off the streaming kernel (more
  than 1,024 (item, head, partition) units), both with the rotation and the cache write inside,
  after the skinny products with the norms handed over; eagerly and, in bfloat16, as CUDA graphs
  of the padded batch with the sampler inside;
* 8 sequences of very different lengths and then 8 of similar ones in one engine: the engine
  chooses the streaming kernel for the first and the clusters for the second, a CUDA graph each;
* a pure-decode batch of 24 sequences: library products at 24 rows and a launch of many
  short attention rows;
* generation through the scheduler with CUDA graphs and asynchronous scheduling, tokens fed
  from the sampler's output on the device: the logits of every generated position.

The plain implementation runs its float64 torch operations on the GPU here (the same code,
weights handed to it there): on the CPU the thousands of tokens would take minutes.
"""

import numpy as np
import pytest
import torch

import plain_llama as P
from gpu_utils import BF16_REL_ROUNDED, F32_REL, engine_for, make_model, random_tokens, rel_max

pytestmark = pytest.mark.gpu

LAYERS = 2          # of the 16 that Llama 3.2 1B has; every layer SIZE below is the real one
REAL = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": LAYERS, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
    "hidden_act": "silu", "bos_token_id": 128000, "eos_token_id": 128001,
}
V = REAL["vocab_size"]
DTYPES = ["float32", "bfloat16"]


class Models(dict):
    """(folder, weights on the GPU) by dtype.  At this width a query and a key of random weights already
    have scores of about +-1 to +-3, so attention is far from uniform without help; the float32 model,
    whose tolerance of 1e-4 finds any fault of logic, is sharpened twice over on top."""

    def __missing__(self, dtype):
        d, w = make_model(self.tmp, REAL, seed=40 if dtype == "float32" else 41,
                          sharpen=2.0 if dtype == "float32" else 1.0)
        self[dtype] = (d, {k: v.cuda() for k, v in w.items()})
        return self[dtype]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    m = Models()
    m.tmp = tmp_path_factory.mktemp("real_size")
    yield m
    m.clear()
    torch.cuda.empty_cache()


def oracle_rows(w, tokens, rows, dtype):
    """The plain implementation's logits at ``rows`` of ``tokens`` (bfloat16: the oracle that rounds
    what a 16-bit engine stores)."""
    P.STORE_DTYPE = torch.bfloat16 if dtype == "bfloat16" else None
    try:
        out = P.forward(P.plain_config(REAL), w, list(tokens))[list(rows)].cpu().numpy()
    finally:
        P.STORE_DTYPE = None
    torch.cuda.empty_cache()
    return out


def check(got, want, dtype, what):
    err = rel_max(got, want)
    tol = F32_REL if dtype == "float32" else BF16_REL_ROUNDED
    worst = int(np.abs(got - want).max(axis=1).argmax())
    assert err < tol, f"{what}: {dtype} logits differ, rel-max {err:.3e} (worst row {worst})"
    return err


def real_engine(models, dtype, **kw):
    opts = dict(kv_cache_tokens=8 * 2304, max_seq_len=2304, max_num_seqs=8, max_num_batched_tokens=2048,
                max_logit_rows=320)
    opts.update(kw)
    return engine_for(models[dtype][0], dtype, **opts)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_whole_and_cut_with_a_cached_past(dtype, models):
    w = models[dtype][1]
    eng = real_engine(models, dtype, kv_cache_tokens=1024, max_seq_len=512, max_num_seqs=2)
    toks = random_tokens(V, 300, 1)
    want = oracle_rows(w, toks, range(300), dtype)
    whole = eng.step_tokens([("w", toks, list(range(300)))]).cpu().numpy()
    eng.close_request("w")
    check(whole, want, dtype, "whole prompt")
    first = eng.step_tokens([("c", toks[:130], list(range(130)))]).cpu().numpy()
    second = eng.step_tokens([("c", toks[130:], list(range(170)))]).cpu().numpy()
    eng.close_request("c")
    check(np.concatenate([first, second]), want, dtype, "prompt cut at 130")
    eng.runner.check_status()
    eng.runner.cache.check_invariants()


@pytest.mark.parametrize("dtype,graphs,clusters", [("float32", False, True), ("bfloat16", False, True),
                                                   ("bfloat16", True, True), ("bfloat16", True, False)])
def test_eight_sequences_decoding_beyond_2048_keys(dtype, graphs, clusters, models, monkeypatch):
    """8 sequences of similar length: the decode attention of these steps gives every (sequence, kv head) a
    cluster of two CTAs.  With that kernel switched off, 8 sequences x 8 kv heads x 17 or 18 partitions of
    128 keys are more than 1,024 units: the streaming kernel.  Both also rotate q and k and write the cache."""
    from redline_b200.ops import kernels
    monkeypatch.setenv("REDLINE_DECODE_ROWS", "1" if clusters else "0")
    w = models[dtype][1]
    eng = real_engine(models, dtype, cuda_graphs=graphs)
    steps = 40
    lens = [2050 + 7 * i for i in range(8)]             # the prompts; every sequence then decodes 40 tokens
    seqs = [random_tokens(V, n + steps, 10 + i) for i, n in enumerate(lens)]
    got = [[] for _ in seqs]
    for i, (s, n) in enumerate(zip(seqs, lens)):         # prompts longer than a step are cut by the engine
        got[i].append(eng.step_tokens([(i, s[:n], [n - 1])]).cpu().numpy())
    assert 8 * 8 * ((min(lens) + 127) // 128) >= 1024
    graph_steps = eng.runner.num_graph_steps
    for t in range(steps - 1):
        out = eng.step_tokens([(i, s[n + t:n + t + 1], [0]) for i, (s, n) in enumerate(zip(seqs, lens))],
                              graphs=graphs).cpu().numpy()
        for i in range(8):
            got[i].append(out[i:i + 1])
    assert (eng.runner.num_graph_steps - graph_steps == steps - 1) if graphs else eng.runner.num_graph_steps == 0
    if graphs:                                            # which kernel the mixers named for these steps
        assert {v for _, variants in eng.runner._graphs for v in variants} == ({4} if clusters else {0})
    eng.runner.check_status()
    assert int(kernels.tc_status(eng.runner.device).item()) == 0
    for i, (s, n) in enumerate(zip(seqs, lens)):
        want = oracle_rows(w, s[:n + steps - 1], range(n - 1, n + steps - 1), dtype)
        check(np.concatenate(got[i]), want, dtype, f"sequence {i}")
        eng.close_request(i)
    eng.runner.cache.check_invariants()


def test_lengths_decide_the_decode_attention_kernel(models):
    """One engine, CUDA graphs on: 8 sequences of which one is fifty times as long as the others decode
    together (the keys are shared among all warps: the streaming kernel), then 8 of similar length (a cluster
    per row).  The logits of both against the plain implementation, and one graph for each choice."""
    from redline_b200.ops import kernels
    dtype = "bfloat16"
    w = models[dtype][1]
    dev = torch.device("cuda")
    assert kernels.attn_decode_rows_pays(8, 8, 64, 4096, 8 * 4096, 0, dev)
    assert not kernels.attn_decode_rows_pays(8, 8, 64, 4096, 4096 + 7 * 128, 0, dev)
    assert kernels.attn_decode_rows_pays(64, 8, 64, 516, 64 * 516, 0, dev)                 # (three warps to a row)
    assert not kernels.attn_decode_rows_pays(64, 8, 64, 4096, 4096 + 63 * 64, 0, dev)
    eng = real_engine(models, dtype, cuda_graphs=True)
    steps = 6
    for phase, lens in enumerate([[2100, 40, 41, 42, 43, 44, 45, 46], [300 + 3 * i for i in range(8)]]):
        seqs = [random_tokens(V, n + steps, 80 + 10 * phase + i) for i, n in enumerate(lens)]
        got = [[] for _ in seqs]
        for i, (s, n) in enumerate(zip(seqs, lens)):
            got[i].append(eng.step_tokens([(i, s[:n], [n - 1])]).cpu().numpy())
        for t in range(steps - 1):
            out = eng.step_tokens([(i, s[n + t:n + t + 1], [0]) for i, (s, n) in enumerate(zip(seqs, lens))],
                                  graphs=True).cpu().numpy()
            for i in range(8):
                got[i].append(out[i:i + 1])
        chosen = {v for _, variants in eng.runner._graphs for v in variants}
        assert chosen == ({0} if phase == 0 else {0, 4}), chosen
        for i, (s, n) in enumerate(zip(seqs, lens)):
            want = oracle_rows(w, s[:n + steps - 1], range(n - 1, n + steps - 1), dtype)
            check(np.concatenate(got[i]), want, dtype, f"phase {phase}, sequence {i}")
            eng.close_request(i)
    eng.runner.check_status()
    eng.runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
def test_twenty_four_sequences_decoding_together(dtype, models):
    """17 to 64 rows: the products of these steps are the tcgen05 products with the weights as the wide
    operand (K split over a cluster), the attention a launch of 192 rows of five or six partitions each:
    more rows than clusters are resident, so a cluster takes two, one after the other."""
    w = models[dtype][1]
    eng = real_engine(models, dtype, kv_cache_tokens=24 * 768, max_seq_len=768, max_num_seqs=24, max_logit_rows=64)
    steps = 8
    lens = [640 + 5 * i for i in range(24)]
    seqs = [random_tokens(V, n + steps, 50 + i) for i, n in enumerate(lens)]
    got = [[] for _ in seqs]
    for lo in range(0, 24, 3):                            # the prompts, three to a step
        out = eng.step_tokens([(i, seqs[i][:lens[i]], [lens[i] - 1]) for i in range(lo, lo + 3)]).cpu().numpy()
        for j, i in enumerate(range(lo, lo + 3)):
            got[i].append(out[j:j + 1])
    for t in range(steps - 1):
        out = eng.step_tokens([(i, s[n + t:n + t + 1], [0]) for i, (s, n) in enumerate(zip(seqs, lens))]).cpu().numpy()
        for i in range(24):
            got[i].append(out[i:i + 1])
    eng.runner.check_status()
    for i, (s, n) in enumerate(zip(seqs, lens)):
        want = oracle_rows(w, s[:n + steps - 1], range(n - 1, n + steps - 1), dtype)
        check(np.concatenate(got[i]), want, dtype, f"sequence {i}")
        eng.close_request(i)


@pytest.mark.parametrize("dtype", DTYPES)
def test_generation_with_graphs_and_tokens_fed_on_the_device(dtype, models):
    """The product path of serving: scheduler, chunked prompts beside decoded tokens, padded decode
    batches replayed as CUDA graphs, the next step launched before this step's tokens are read (it
    takes them from the sampler's output on the device).  The logits of every position that was
    sampled from are collected and compared with the plain implementation run on the finished
    sequences; so are the tokens (greedy: the arg max of those logits)."""
    w = models[dtype][1]
    eng = real_engine(models, dtype, cuda_graphs=True, async_scheduling=True, max_num_batched_tokens=512,
                      kv_cache_tokens=8 * 1024, max_seq_len=1024)
    prompts = [random_tokens(V, n, 80 + i) for i, n in enumerate((300, 17, 620, 129, 450, 64, 200, 513))]
    new = 24
    seen = {}

    def keep(where, logits):
        host = logits.cpu().numpy()
        for (rid, pos), row in zip(where, host):
            seen[rid, pos] = row.copy()

    eng.on_logits = keep
    eng.record_steps = True
    outs = eng.generate(prompts, max_new_tokens=new, ignore_eos=True)
    assert eng.runner.num_graph_steps > 0 and any(r.kind == "mixed" for r in eng.records)
    for o, p in zip(outs, prompts):
        seq = p + o["output_ids"]
        rows = range(len(p) - 1, len(seq) - 1)
        want = oracle_rows(w, seq[:-1], rows, dtype)
        got = np.stack([seen[o["id"], r] for r in rows])
        check(got, want, dtype, f"request {o['id']}")
        assert [int(g.argmax()) for g in got] == o["output_ids"]
    eng.runner.check_status()
