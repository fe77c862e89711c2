"""The sampling kernel: greedy with ties, log-probabilities, the seeded draw against the
plain restatement, empirical frequencies against the exact warped distribution
(cases of the reference's tests/cuda/test_sampling.cu:84-161)."""

import numpy as np
import pytest
import torch

import plain_llama as P
from redline_b200.ops import kernels

pytestmark = pytest.mark.gpu
DEV = "cuda"


def run(logits, temperature, top_k, top_p, seeds, positions, two_stage=None):
    """two_stage None: both ways must agree (greedy rows take the two-stage arg max when scratch is given)."""
    if two_stage is None:
        a = run(logits, temperature, top_k, top_p, seeds, positions, two_stage=False)
        b = run(logits, temperature, top_k, top_p, seeds, positions, two_stage=True)
        assert np.array_equal(a[0], b[0]) and np.abs(a[1] - b[1]).max() < 1e-4
        return b
    R = logits.shape[0]
    f = lambda v, dt: torch.tensor(np.broadcast_to(np.asarray(v), (R,)).copy(), dtype=dt, device=DEV)  # noqa: E731
    seeds = np.broadcast_to(np.asarray(seeds, dtype=np.uint64), (R,))
    lo = torch.tensor((seeds & 0xFFFFFFFF).astype(np.int64), device=DEV).to(torch.int32)
    hi = torch.tensor((seeds >> 32).astype(np.int64), device=DEV).to(torch.int32)
    tok = torch.empty(R, dtype=torch.int32, device=DEV)
    lp = torch.empty(R, dtype=torch.float32, device=DEV)
    scratch = torch.full((R * kernels.SAMPLE_CHUNKS * 4,), float("nan"), device=DEV) if two_stage else None
    kernels.sample(logits, R, f(temperature, torch.float32), f(top_k, torch.int32), f(top_p, torch.float32),
                   lo, hi, f(positions, torch.int32), tok, lp, scratch=scratch)
    return tok.cpu().numpy(), lp.cpu().numpy()


def test_greedy_ties_and_logprobs():
    V = 1000
    l = torch.randn(12, V, device=DEV)
    l[3, 17] = l[3, 900] = l[3].max() + 1.0          # a tie: the smaller index wins
    l[5, 0] = 50.0
    tok, lp = run(l, 0.0, 0, 1.0, 0, 0)
    ref = l.double().cpu()
    assert tok.tolist() == [int(ref[i].argmax()) if i != 3 else 17 for i in range(12)]
    want = torch.log_softmax(ref, -1)[torch.arange(12), torch.tensor(tok.astype(np.int64))]
    assert np.abs(lp - want.numpy()).max() < 1e-4
    # 16 rows and more: the first stage cuts a row into fewer, longer pieces (and marks the unused slots
    # empty); a vocabulary that is no multiple of anything, a tie across two pieces, a maximum in the last one
    for V, R in [(128256, 16), (331, 20), (50001, 33)]:
        l = torch.randn(R, V, device=DEV)
        l[1, 5] = l[1, V - 2] = l[1].max() + 2.0
        l[2, V - 1] = 40.0
        tok, lp = run(l, 0.0, 0, 1.0, 0, 0)
        ref = l.double().cpu()
        assert tok.tolist() == [int(ref[i].argmax()) if i != 1 else 5 for i in range(R)]
        want = torch.log_softmax(ref, -1)[torch.arange(R), torch.tensor(tok.astype(np.int64))]
        assert np.abs(lp - want.numpy()).max() < 1e-4


@pytest.mark.parametrize("T,k,p", [(1.0, 0, 1.0), (0.7, 5, 1.0), (1.3, 0, 0.8), (0.9, 20, 0.6)])
def test_seeded_draw_equals_the_plain_restatement(T, k, p):
    V = 331
    l = (torch.randn(40, V) * 2).float()
    pos = np.arange(40) + 3
    tok, _ = run(l.to(DEV), T, k, p, 1234567890123, pos)
    for r in range(40):
        assert tok[r] == P.gumbel_draw(l[r].numpy(), T, k, p, 1234567890123, int(pos[r])), r
    tok2, _ = run(l.to(DEV), T, k, p, 1234567890123, pos)
    assert np.array_equal(tok, tok2)
    # a row's draw depends on (seed, position), not on where the row sits in the batch
    perm = np.random.RandomState(0).permutation(40)
    tok3, _ = run(l[perm].to(DEV), T, k, p, 1234567890123, pos[perm])
    assert np.array_equal(tok3, tok[perm])


@pytest.mark.parametrize("T,k,p", [(1.0, 0, 1.0), (0.7, 4, 1.0), (1.5, 0, 0.7), (0.8, 6, 0.9)])
def test_frequencies_follow_the_warped_distribution(T, k, p):
    V, R = 16, 6000
    row = np.array([2.0, 1.5, 1.5, 1.0, 0.7, 0.3, 0.0, -0.2, -0.5, -1.0, -1.0, -2.0, -3.0, -3.5, -5.0, -8.0],
                   dtype=np.float32)
    l = torch.tensor(np.tile(row, (R, 1)), device=DEV)
    tok, _ = run(l, T, k, p, 99, np.arange(R))
    want = P.warped_distribution(row, T, k, p)
    freq = np.bincount(tok, minlength=V) / R
    assert np.all(freq[want == 0] == 0), "a token outside the kept set was drawn"
    assert np.abs(freq - want).max() < 0.025


def test_large_vocabulary_top_k_membership():
    V = 128256
    l = torch.randn(4, V, device=DEV)
    tok, lp = run(l, 1.0, 50, 1.0, [1, 2, 3, 4], [10, 10, 10, 10])
    top = torch.topk(l, 50, dim=-1).indices.cpu().numpy()
    assert all(tok[r] in top[r] for r in range(4)) and np.all(np.isfinite(lp))
    tok_g, lp_g = run(l, 0.0, 0, 1.0, 0, 0)
    assert tok_g.tolist() == l.argmax(-1).tolist()
    want = torch.log_softmax(l.double(), -1).max(-1).values.cpu().numpy()
    assert np.abs(lp_g - want).max() < 1e-4
    # greedy and sampled rows in one launch
    temp = np.array([0.0, 1.0, 0.0, 0.7], dtype=np.float32)
    tok_m, _ = run(l, temp, 50, 1.0, [1, 2, 3, 4], [10, 10, 10, 10])
    assert tok_m[0] == tok_g[0] and tok_m[2] == tok_g[2] and tok_m[1] in top[1] and tok_m[3] in top[3]


def test_gather_logprob():
    l = torch.randn(9, 777, device=DEV) * 3
    tgt = torch.randint(0, 777, (9,), device=DEV, dtype=torch.int32)
    out = torch.empty(9, device=DEV)
    kernels.gather_logprob(l, 9, tgt, out)
    want = torch.log_softmax(l.double(), -1)[torch.arange(9), tgt.long()]
    assert (out.double() - want).abs().max().item() < 1e-4
