"""The plain implementation against the reference's own CPU model (tests/golden) and
against itself."""

import math
import os

import numpy as np
import pytest
import torch

import plain_llama as P
import tiny_configs as C

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_matches_reference_cpu_model(name):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg = C.ALL[name]
    w = P.random_weights(cfg, int(g["seed"]), float(g["sharpen"]))
    logits = P.forward(P.plain_config(cfg), w, g["tokens"].tolist()).numpy()
    ref = g["logits"]
    assert logits.shape == ref.shape
    # the reference stores float32 with double accumulators; rel-max as its own export test (1e-4)
    assert np.abs(logits - ref).max() / np.abs(ref).max() < 1e-4


def test_prefix_logits_do_not_depend_on_what_follows():
    cfg = C.TINY_A
    pc = P.plain_config(cfg)
    w = P.random_weights(cfg, 3, 6.0)
    toks = np.random.RandomState(0).randint(0, pc.vocab_size, size=20).tolist()
    full = P.forward(pc, w, toks)
    part = P.forward(pc, w, toks[:11])
    assert torch.allclose(full[:11], part, atol=1e-10)


def test_llama3_scaling_endpoints():
    sc = {"type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    base = P.rope_inv_freq(128, 500000.0, None)
    scaled = P.rope_inv_freq(128, 500000.0, sc)
    assert scaled[0] == base[0]                       # wavelength 2 pi < 64 / 4: untouched
    assert scaled[-1] == pytest.approx(base[-1] / 8)  # very long wavelength: divided by the factor
    mids = [i for i, f in enumerate(base) if 16 <= 2 * math.pi / f <= 64]
    assert mids and all(base[i] / 8 <= scaled[i] <= base[i] for i in mids)
    lin = P.rope_inv_freq(64, 1e4, {"type": "linear", "factor": 2.0})
    assert lin == [f / 2 for f in P.rope_inv_freq(64, 1e4, None)]


def test_window_attention_is_full_attention_when_the_window_covers_all():
    q = torch.randn(9, 4, 16, dtype=torch.float64)
    k = torch.randn(9, 2, 16, dtype=torch.float64)
    v = torch.randn(9, 2, 16, dtype=torch.float64)
    a = P.causal_attention(q, k, v, 0.25)
    assert torch.allclose(a, P.causal_attention(q, k, v, 0.25, window=9))
    b = P.causal_attention(q, k, v, 0.25, window=3)
    assert torch.allclose(a[:3], b[:3]) and not torch.allclose(a[5:], b[5:])
    # row 8 with window 3 sees keys 6, 7, 8 only
    c = P.causal_attention(q[6:], k[6:], v[6:], 0.25)
    assert torch.allclose(b[8], c[2])


def test_warped_distribution_and_draws():
    l = np.array([2.0, 1.0, 0.5, 0.5, -1.0, -3.0], dtype=np.float32)
    p = P.warped_distribution(l, 1.0, 0, 1.0)
    assert p.sum() == pytest.approx(1.0) and np.all(np.diff(p[[0, 1, 2]]) < 0)
    p = P.warped_distribution(l, 0.7, 3, 1.0)      # ties at the 3rd value are kept
    assert (p > 0).tolist() == [True, True, True, True, False, False]
    p = P.warped_distribution(l, 1.0, 0, 0.5)      # the top token alone has mass > 0.5
    assert (p > 0).tolist() == [True, False, False, False, False, False]
    draws = [P.gumbel_draw(l, 1.0, 0, 1.0, seed=7, position=i) for i in range(400)]
    freq = np.bincount(draws, minlength=6) / 400.0
    assert np.abs(freq - P.warped_distribution(l, 1.0, 0, 1.0)).max() < 0.08
    assert P.gumbel_draw(l, 1.0, 0, 1.0, 7, 3) == P.gumbel_draw(l, 1.0, 0, 1.0, 7, 3)


def test_philox_known_answer():
    # Random123 known-answer test for philox4x32-10 with zero counter and key.
    assert P.philox4x32_10((0, 0, 0, 0), (0, 0)) == (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)
