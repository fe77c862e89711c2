"""Replay of the same requests under every way of cutting the work, in 32-bit and in
bfloat16, each compared with the plain implementation: whole; most in one step and
the last 32 tokens one by one; portions of changing size down to two tokens; mixed,
up to four live requests with so few pages that they are used again; long decoding;
the first tokens of a sequence; and through bin/trace_run itself."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as P
import tiny_configs as C
from gpu_utils import check_logits, engine_for, make_model, oracle_logits, random_tokens, rel_max

pytestmark = pytest.mark.gpu

CONFIGS = ["tiny_a", "tiny_b", "tiny_c"]
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"tiny_a": 150, "tiny_b": 129, "tiny_c": 97}


class Models(dict):
    """(folder, weights) by (configuration, dtype).  The 32-bit runs, whose tolerance of 1e-4 finds
    any fault of logic, use sharply peaked attention (q and k weights times 6).  The bfloat16 runs
    use a milder 3: at 6 the flipped roundings of a 16-bit engine alone reach 3.5e-2 of max |logit|
    in single rows (measured), which is the size of the tolerance."""

    def __missing__(self, key):
        name, dtype = key
        i = CONFIGS.index(name)
        self[key] = make_model(self.tmp, C.ALL[name], seed=20 + i + (0 if dtype == "float32" else 10),
                               sharpen=6.0 if dtype == "float32" else 3.0)
        return self[key]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    m = Models()
    m.tmp = tmp_path_factory.mktemp("models")
    return m


@pytest.fixture(scope="module")
def engines(models):
    cache = {}

    def get(name, dtype, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in cache:
            cache[key] = engine_for(models[name, dtype][0], dtype, **kw)
        return cache[key]

    yield get
    cache.clear()


def vocab(name):
    return C.ALL[name]["vocab_size"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_whole(name, dtype, models, engines):
    eng, (_, w) = engines(name, dtype), models[name, dtype]
    toks = random_tokens(vocab(name), LENGTHS[name], 1)
    out = eng.step_tokens([("w", toks, list(range(len(toks))))]).cpu().numpy()
    eng.close_request("w")
    check_logits(out, C.ALL[name], w, toks, dtype)
    eng.runner.cache.check_invariants()


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_last_32_tokens_one_by_one(name, dtype, graphs, models, engines):
    """With ``graphs`` the single-token steps run as generation runs them: padded to a fixed shape, the
    sampler behind the head, captured once and replayed as a CUDA graph whose launches are sized for the
    longest sequence the engine allows."""
    eng, (_, w) = engines(name, dtype, cuda_graphs=graphs), models[name, dtype]
    toks = random_tokens(vocab(name), LENGTHS[name], 2)
    n0 = len(toks) - 32
    before = eng.runner.num_graph_steps
    outs = [eng.step_tokens([("d", toks[:n0], [n0 - 1])], graphs=graphs).cpu().numpy()]
    for i in range(n0, len(toks)):
        outs.append(eng.step_tokens([("d", toks[i:i + 1], [0])], graphs=graphs).cpu().numpy())
    eng.close_request("d")
    assert eng.runner.num_graph_steps - before == (32 if graphs else 0)
    check_logits(np.concatenate(outs), C.ALL[name], w, toks, dtype, rows=range(n0 - 1, len(toks)))


@pytest.mark.parametrize("name", CONFIGS)
def test_norms_handed_over_between_the_products_of_small_steps(name, models, monkeypatch):
    """In steps of up to 8 tokens the bfloat16 engine hands every norm but a step's first and last from
    the product before it to the product after it: fewer launches, the same logits within the tolerance
    against the oracle as with every norm a kernel of its own."""
    from redline_b200.ops import kernels
    d, w = models[name, "bfloat16"]
    toks = random_tokens(vocab(name), 40, 9)
    layers = C.ALL[name]["num_hidden_layers"]
    launches, outs = {}, {}
    for mode in ("1", "0"):
        monkeypatch.setenv("REDLINE_NORM_HANDOVER", mode)
        eng = engine_for(d, "bfloat16")
        got = [eng.step_tokens([("h", toks[:20], [19])]).cpu().numpy()]
        i = 20
        for n in (1, 3, 8, 2, 5, 1):                      # small steps of several sizes
            before = kernels.LAUNCHES
            got.append(eng.step_tokens([("h", toks[i:i + n], list(range(n)))]).cpu().numpy())
            launches.setdefault(mode, []).append(kernels.LAUNCHES - before)
            i += n
        eng.close_request("h")
        outs[mode] = np.concatenate(got)
        check_logits(outs[mode], C.ALL[name], w, toks[:i], "bfloat16", rows=range(19, i))
    assert all(a == b - (2 * layers - 1) for a, b in zip(launches["1"], launches["0"])), launches
    assert rel_max(outs["1"], outs["0"]) < 2e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_portions_of_changing_size(name, dtype, models, engines):
    eng, (_, w) = engines(name, dtype), models[name, dtype]
    toks = random_tokens(vocab(name), LENGTHS[name], 3)
    sizes = [17, 5, 2, 31, 2, 1, 33, 2, 16, 3, 64]
    outs, i = [], 0
    for s in sizes:
        s = min(s, len(toks) - i)
        if s <= 0:
            break
        outs.append(eng.step_tokens([("p", toks[i:i + s], list(range(s)))]).cpu().numpy())
        i += s
    eng.close_request("p")
    assert i == len(toks)
    check_logits(np.concatenate(outs), C.ALL[name], w, toks, dtype)


def mixed_schedule(lengths, pool_tokens, seed):
    """Steps of [(id, start, n)] and ends: up to four live requests, portions of some
    beside single tokens of others; a request is admitted when the pool (each request
    rounded up to 64 tokens) has room, so later requests reuse the pages of ended ones."""
    rng = np.random.RandomState(seed)
    pending = list(enumerate(lengths))
    live = {}
    steps = []
    while pending or live:
        used = sum((lengths[i] + 63) // 64 * 64 for i in live)
        while pending and len(live) < 4 and used + (pending[0][1] + 63) // 64 * 64 <= pool_tokens:
            i, n = pending.pop(0)
            live[i] = 0
            used += (n + 63) // 64 * 64
        entries, ends = [], []
        for i in list(live):
            if rng.rand() < 0.15 and len(live) > 1:
                continue                     # left out of this step, goes on later
            done = live[i]
            mode = rng.rand()
            n = 1 if mode < 0.45 else int(rng.choice([2, 2, 3, 5, 16, 17, 31, 40]))
            n = min(n, lengths[i] - done)
            entries.append((i, done, n))
            live[i] = done + n
            if live[i] == lengths[i]:
                ends.append(i)
                del live[i]
        if entries:
            steps.append((entries, ends))
    return steps


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_mixed_with_pages_used_again(name, dtype, graphs, models, engines):
    """With ``graphs`` the steps that hold single tokens only are padded with dummy rows on the reserved
    page and replayed as CUDA graphs, between eager steps that hold portions."""
    lengths = [129, 70, 40, 97, 33, 150, 64, 5]
    pool = 384
    eng, (_, w) = engines(name, dtype, kv_cache_tokens=pool, cuda_graphs=graphs), models[name, dtype]
    graph_steps = eng.runner.num_graph_steps
    toks = {i: random_tokens(vocab(name), n, 100 + i) for i, n in enumerate(lengths)}
    got = {i: [] for i in toks}
    pages_seen = {}
    reused = False
    for entries, ends in mixed_schedule(lengths, pool, seed=7):
        batch = [(f"r{i}", toks[i][s:s + n], list(range(n))) for i, s, n in entries]
        out = eng.step_tokens(batch, graphs=graphs).cpu().numpy()
        r = 0
        for i, s, n in entries:
            got[i].append(out[r:r + n])
            r += n
            for p in eng.runner.cache.get(f"r{i}").tables[0]:
                if pages_seen.setdefault(p, i) != i:
                    reused = True
        for i in ends:
            eng.close_request(f"r{i}")
        eng.runner.cache.check_invariants()
    assert reused, "the pool was large enough that no page was handed out twice"
    assert eng.runner.cache.num_open() == 0
    assert (eng.runner.num_graph_steps > graph_steps) == graphs
    for i in toks:
        check_logits(np.concatenate(got[i]), C.ALL[name], w, toks[i], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype, models, engines):
    name = "tiny_b"
    eng, (_, w) = engines(name, dtype, kv_cache_tokens=1024, max_seq_len=1024), models[name, dtype]
    toks = random_tokens(vocab(name), 700, 9)       # crosses two 256-key partitions while decoding
    eng.step_tokens([("l", toks[:200], [])])
    outs, rows = [], []
    for i in range(200, 700):
        want = [0] if (i % 50 == 0 or i in (255, 256, 257, 511, 512, 513, 699)) else []
        o = eng.step_tokens([("l", toks[i:i + 1], want)])
        if want:
            outs.append(o.cpu().numpy())
            rows.append(i)
    eng.close_request("l")
    check_logits(np.concatenate(outs), C.ALL[name], w, toks, dtype, rows=rows)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_first_tokens_of_a_sequence(name, dtype, models, engines):
    eng, (_, w) = engines(name, dtype), models[name, dtype]
    toks = random_tokens(vocab(name), 6, 4)
    outs = [eng.step_tokens([("f", toks[i:i + 1], [0])]).cpu().numpy() for i in range(3)]
    outs.append(eng.step_tokens([("f", toks[3:6], [0, 1, 2])]).cpu().numpy())
    eng.close_request("f")
    check_logits(np.concatenate(outs), C.ALL[name], w, toks, dtype)
    one = eng.step_tokens([("g", toks[:1], [0, 0])]).cpu().numpy()      # a place may be asked for twice
    eng.close_request("g")
    assert np.array_equal(one[0], one[1])
    check_logits(one[:1], C.ALL[name], w, toks[:1], dtype)


def test_wanted_rows_come_in_the_order_asked(models, engines):
    eng, (_, w) = engines("tiny_a", "float32"), models["tiny_a", "float32"]
    toks = random_tokens(512, 40, 5)
    a = eng.step_tokens([("o", toks, [39, 0, 17, 0])]).cpu().numpy()
    eng.close_request("o")
    ref = oracle_logits(C.TINY_A, w, toks)[[39, 0, 17, 0]]
    assert rel_max(a, ref) < 1e-4


def test_bfloat16_against_the_unrounded_oracle(models, engines):
    """The reference's own bounds for its half-precision engine: log-probabilities of the
    given next tokens within mean 0.03 and max 0.3 of the 32-bit model's."""
    for name in CONFIGS:
        eng, (_, w) = engines(name, "bfloat16"), models[name, "bfloat16"]
        toks = random_tokens(vocab(name), LENGTHS[name], 6)
        out = eng.step_tokens([("u", toks, list(range(len(toks))))]).cpu().double()
        eng.close_request("u")
        ref = torch.from_numpy(oracle_logits(C.ALL[name], w, toks))
        nxt = torch.tensor(toks[1:])
        lp = torch.log_softmax(out, -1)[:-1].gather(1, nxt[:, None])
        lr = torch.log_softmax(ref, -1)[:-1].gather(1, nxt[:, None])
        d = (lp - lr).abs()
        assert float(d.mean()) < 0.03 and float(d.max()) < 0.3, (name, float(d.mean()), float(d.max()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(dtype, models, tmp_path):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 out, 'done <step>' after each."""
    name = "tiny_b"
    model_dir, w = models[name, dtype]
    a, b = random_tokens(1000, 70, 11), random_tokens(1000, 45, 12)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[40:42], "want": [1]},
                                {"id": "b", "tokens": b[:45], "want": [44]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[42:43], "want": []}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": a[43:70], "want": [26]},
                                {"id": "c", "tokens": b[:2], "want": [1, 0]}], "end": ["a", "c"]},
    ]
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_dir,
                           "--dtype", dtype, "--out", str(out), "--max-tokens", "256"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    assert not (out / "2.f32").exists()
    V = 1000
    f = {i: np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V) for i in (0, 1, 3)}
    assert f[0].shape[0] == 2 and f[1].shape[0] == 2 and f[3].shape[0] == 3
    check_logits(np.concatenate([f[0], f[1][:1], f[3][:1]]), C.ALL[name], w, a, dtype, rows=[0, 39, 41, 69])
    check_logits(f[1][1:], C.ALL[name], w, b, dtype, rows=[44])
    check_logits(f[3][1:], C.ALL[name], w, b[:2], dtype, rows=[1, 0])
