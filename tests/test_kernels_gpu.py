"""Each CUDA kernel alone against a plain float64 torch restatement of the same op,
at sizes other than the engine's: head sizes in steps of 16, odd group counts, widths
and vocabularies that are no power of two, shuffled page ids, lengths that cross page,
tile and partition edges, a far key that must be found among hundreds."""

import math

import numpy as np
import pytest
import torch

import plain_llama as P
from redline_b200.ops import kernels
from redline_b200.ops.linear import linear

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 1.2e-2}     # of max |ref|: float32 sums, one bfloat16 rounding


def close(got, ref, tol):
    err = (got.double().cpu() - ref.double().cpu()).abs().max().item() / (ref.abs().max().item() + 1e-30)
    assert err < tol, f"rel-max error {err:.3e} >= {tol}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,vocab", [(200, 331), (2048, 1000), (72, 17)])
def test_embedding(dtype, hidden, vocab):
    table = torch.randn(vocab, hidden, device=DEV).to(DT[dtype])
    ids = torch.randint(0, vocab, (37,), device=DEV, dtype=torch.int32)
    out = torch.full((37, hidden), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.embedding(ids, table, out, status)
    assert torch.equal(out, table[ids.long()].float()) and status.item() == 0
    ids[3] = vocab
    kernels.embedding(ids, table, out, status)
    assert status.item() == 1 and out[3].abs().max().item() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,eps", [(200, 3e-6), (2048, 1e-5), (72, 1e-2), (4100, 1e-6)])
def test_add_rmsnorm(dtype, hidden, eps):
    T = 19
    res = torch.randn(T, hidden, device=DEV) * 3
    delta = torch.randn(T, hidden, device=DEV).to(DT[dtype])
    w = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(DT[dtype])
    want_res = res.double() + delta.double()
    ref = P.rmsnorm(want_res.cpu(), w.cpu(), eps)
    out = torch.empty(T, hidden, device=DEV, dtype=DT[dtype])
    r = res.clone()
    kernels.add_rmsnorm(r, delta, w, out, eps)
    close(out, ref, TOL[dtype])
    assert torch.allclose(r.double(), want_res, atol=1e-6)          # the stream holds the float32 sum
    r2 = res.clone()                                                 # no delta: a plain norm, stream untouched
    kernels.add_rmsnorm(r2, None, w, out, eps)
    close(out, P.rmsnorm(res.double().cpu(), w.cpu(), eps), TOL[dtype])
    assert torch.equal(r2, res)
    idx = torch.tensor([4, 4, 0, 18], dtype=torch.int32, device=DEV)  # rows picked, stream left alone
    out4 = torch.empty(4, hidden, device=DEV, dtype=DT[dtype])
    r3 = res.clone()
    kernels.add_rmsnorm(r3, delta, w, out4, eps, rows_idx=idx)
    close(out4, ref[idx.long().cpu()], TOL[dtype])
    assert torch.equal(r3, res)
    wf = w.float()                                                   # a weight stored in 32-bit
    kernels.add_rmsnorm(res.clone(), delta, wf, out, eps)
    close(out, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inter", [704, 328, 1000])
def test_swiglu(dtype, inter):
    gu = (torch.randn(11, 2 * inter, device=DEV) * 4).to(DT[dtype])
    out = torch.empty(11, inter, device=DEV, dtype=DT[dtype])
    kernels.swiglu(gu, out)
    g, u = gu[:, :inter].double().cpu(), gu[:, inter:].double().cpu()
    close(out, P.swiglu(g, u), TOL[dtype])


@pytest.mark.parametrize("tx,tw,ty", [("float32", "float32", "float32"), ("bfloat16", "bfloat16", "float32"),
                                       ("bfloat16", "float32", "bfloat16"), ("float32", "bfloat16", "bfloat16")])
@pytest.mark.parametrize("M,N,K", [(1, 331, 200), (37, 1000, 384), (130, 70, 1024), (5, 64, 18)])
def test_gemm_simt(tx, tw, ty, M, N, K):
    x = torch.randn(M, K, device=DEV).to(DT[tx])
    w = torch.randn(N, K, device=DEV).to(DT[tw])
    y = torch.empty(M, N, device=DEV, dtype=DT[ty])
    kernels.gemm_tn_simt(x, w, y)
    close(y, x.double() @ w.double().T, TOL[ty] if ty == "bfloat16" else 2e-6)
    if M > 1:       # a row does not depend on its neighbours: bit for bit
        y1 = torch.empty(1, N, device=DEV, dtype=DT[ty])
        kernels.gemm_tn_simt(x[M // 2:M // 2 + 1], w, y1)
        assert torch.equal(y1[0], y[M // 2])


@pytest.mark.parametrize("M,N,K", [(1, 3072, 2048), (8, 1000, 384), (200, 704, 256), (64, 331, 200)])
def test_linear_bfloat16(M, N, K):
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    y = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    close(linear(x, w, y), ref, 1.2e-2)
    yf = torch.empty(M, N, device=DEV, dtype=torch.float32)
    close(linear(x, w, yf), ref, 1e-4)


@pytest.mark.parametrize("M,N,K", [(64, 2048, 8192), (2048, 2048, 2048), (24, 3072, 2048), (300, 8192, 2048)])
def test_library_products_accumulate_in_float32(M, N, K):
    """Products of more than 16 rows are library calls.  The engine pins them to float32 accumulation all
    the way (no bfloat16 reduction of the parts of a split k dimension, no TF32): the float32 result is the
    float64 product to within float32 sums, and the bfloat16 result is the ROUNDED float64 product in all
    but the elements whose value lies within the float32 sum's error of a rounding boundary (at K = 8192
    the sum is off by about 2e-5 where a bfloat16 step is 8e-3: one element in two hundred; a reduction in
    bfloat16, off by half a step, would move every third)."""
    from redline_b200.engine.runner import pin_library_products
    pin_library_products()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    yf = torch.empty(M, N, device=DEV, dtype=torch.float32)
    # a float32 sum of K terms, each rounded to 2^-24 of the running sum (a bfloat16 partial sum: 2^-9)
    close(linear(x, w, yf), ref, 2.0 ** -23 * math.sqrt(K))
    y = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    linear(x, w, y)
    moved = (y != ref.to(torch.bfloat16)).float().mean().item()
    assert moved < 2e-2, f"{moved:.2%} of the bfloat16 results are not the rounded exact product"
    assert not torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction and not torch.backends.cuda.matmul.allow_tf32


def plain_rope_tables(D, theta, num_pos, scaling=None):
    """cos / sin [num_pos, D / 2] in float32 from the oracle's own table builder (not the product's)."""
    pc = P.PlainConfig(vocab_size=0, hidden_size=0, intermediate_size=0, num_layers=0, num_heads=0, num_kv_heads=0,
                       head_dim=D, rms_norm_eps=0.0, rope_theta=theta, rope_scaling=scaling, tie_word_embeddings=False,
                       max_position_embeddings=num_pos)
    cos, sin = P.rope_tables(pc, num_pos)
    return cos.float().contiguous(), sin.float().contiguous()


def paged_setup(dtype, Hq, Hkv, D, lens_past, lens_new, page_size, seed, sharp=None, cos=None, sin=None):
    """Random q/k/v for several sequences; pages with shuffled ids; returns everything a
    kernel launch needs plus the dense per-sequence tensors for the reference."""
    g = torch.Generator().manual_seed(seed)
    S = len(lens_past)
    total = [p + n for p, n in zip(lens_past, lens_new)]
    max_blocks = max((t + page_size - 1) // page_size for t in total) + 1
    npages = sum((t + page_size - 1) // page_size for t in total) + 3
    perm = (torch.randperm(npages - 1, generator=g) + 1).tolist()
    bt = torch.zeros(S, max_blocks, dtype=torch.int32)
    it = iter(perm)
    for s in range(S):
        for b in range((total[s] + page_size - 1) // page_size):
            bt[s, b] = next(it)
    qkv_w = (Hq + 2 * Hkv) * D
    seqs = []
    for s in range(S):
        x = torch.randn(total[s], qkv_w, generator=g)
        seqs.append(x)
    if sharp is not None:
        sharp(seqs, cos, sin)
    seqs = [x.to(DT[dtype]) for x in seqs]
    return dict(S=S, total=total, bt=bt, npages=npages, seqs=seqs, max_blocks=max_blocks)


def reference_attention(seqs, Hq, Hkv, D, cos, sin, scale, window, dtype):
    """Per sequence: rotate q, k (rounded to the cache type), causal attention in float64."""
    outs = []
    P.STORE_DTYPE = DT[dtype] if dtype == "bfloat16" else None
    try:
        for x in seqs:
            T = x.shape[0]
            x = x.double().cpu()
            q = x[:, :Hq * D].reshape(T, Hq, D)
            k = x[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D)
            v = x[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
            q = P.rope_rotate(q, cos[:T].double(), sin[:T].double())
            k = P.rope_rotate(k, cos[:T].double(), sin[:T].double())
            P.STORE_DTYPE = None
            outs.append(P.causal_attention(q, k, v, scale, window).reshape(T, Hq * D))
            P.STORE_DTYPE = DT[dtype] if dtype == "bfloat16" else None
    finally:
        P.STORE_DTYPE = None
    return outs


def run_attention(dtype, Hq, Hkv, D, lens_past, lens_new, page_size=16, window=0, seed=0, sharp=None,
                  poison=True, decode_impl=0, prefill_impl=0):
    """Writes the past through rope_kv_write, then runs the new tokens (decode kernel for
    single tokens, prefill kernel for portions) and compares with the reference."""
    cos, sin = plain_rope_tables(D, 10000.0, max(p + n for p, n in zip(lens_past, lens_new)) + 1)
    st = paged_setup(dtype, Hq, Hkv, D, lens_past, lens_new, page_size, seed, sharp, cos, sin)
    S, total, seqs = st["S"], st["total"], st["seqs"]
    scale = 1.0 / math.sqrt(D)
    ref = reference_attention(seqs, Hq, Hkv, D, cos, sin, scale, window, dtype)
    fill = float("nan") if poison else 0.0
    kc = torch.full((st["npages"], Hkv, page_size, D), fill, device=DEV, dtype=DT[dtype])
    vc = torch.full((st["npages"], Hkv, page_size, D), fill, device=DEV, dtype=DT[dtype])
    kc[0], vc[0] = 0, 0
    bt = st["bt"].to(DEV)
    cosd, sind = cos.to(DEV), sin.to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def launch(ranges):
        """ranges: per sequence (start, n) of tokens to run now."""
        toks, pos, seq_of, slots = [], [], [], []
        dec, tiles = [], []
        t = 0
        for s, (a, n) in enumerate(ranges):
            if n == 0:
                continue
            toks.append(seqs[s][a:a + n])
            for i in range(a, a + n):
                pos.append(i)
                seq_of.append(s)
                slots.append(int(st["bt"][s, i // page_size]) * page_size + i % page_size)
            if n == 1:
                dec.append(t)
            else:
                for r0 in range(0, n, kernels.PREFILL_TILE_ROWS):
                    tiles.append((s, t + r0, min(kernels.PREFILL_TILE_ROWS, n - r0)))
            t += n
        qkv = torch.cat(toks).to(DEV).contiguous()
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
        pos_d, seq_d, slot_d = i32(pos), i32(seq_of), i32(slots)
        kernels.rope_kv_write(qkv, pos_d, slot_d, cosd, sind, kc, vc, Hq, Hkv, D, page_size, status)
        out = torch.full((t, Hq * D), float("nan"), device=DEV, dtype=DT[dtype])
        if dec:
            parts = (max(total) + kernels.DECODE_PARTITION - 1) // kernels.DECODE_PARTITION
            po = torch.full((len(dec) * Hq * parts * D,), float("nan"), device=DEV)
            pm = torch.full((len(dec) * Hq * parts * 2,), float("nan"), device=DEV)
            items = i32([[tk, seq_of[tk], pos[tk] + 1, 0] for tk in dec])
            counters = torch.zeros(len(dec) * Hkv, dtype=torch.int32, device=DEV)
            kernels.attn_decode(qkv, qkv.shape[1], kc, vc, bt, items, po, pm, parts, counters, out,
                                len(dec), Hq, Hkv, D, page_size, window, scale, decode_impl)
            assert int(counters.abs().max()) == 0, "the merge counters must be left at zero"
        if tiles:
            kernels.attn_prefill(qkv, qkv.shape[1], kc, vc, bt, i32([x[0] for x in tiles]),
                                 i32([x[1] for x in tiles]), i32([x[2] for x in tiles]), pos_d, out, len(tiles),
                                 Hq, Hkv, D, page_size, window, scale, prefill_impl)
        return out

    if any(lens_past):
        launch([(0, p) for p in lens_past])
    out = launch([(p, n) for p, n in zip(lens_past, lens_new)])
    assert status.item() == 0
    want = torch.cat([ref[s][p:p + n] for s, (p, n) in enumerate(zip(lens_past, lens_new)) if n])
    assert not torch.isnan(out.float()).any(), "attention read a cache slot that was never written"
    close(out, want, 2e-5 if dtype == "float32" else 1.6e-2)


ATTN_SHAPES = [  # Hq, Hkv, D
    (4, 2, 64), (3, 1, 128), (5, 5, 48), (8, 1, 16), (6, 2, 80), (2, 1, 256), (14, 2, 32),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,D", ATTN_SHAPES)
def test_attention_prefill_whole_and_with_a_cached_past(dtype, Hq, Hkv, D):
    # impl 1: the CUDA-core kernel; 0: the tensor-core kernel where it applies (bfloat16, D 64 / 128)
    for impl in (0, 1):
        run_attention(dtype, Hq, Hkv, D, [0, 0, 0], [1 + 4, 33, 129], seed=1, prefill_impl=impl)
        run_attention(dtype, Hq, Hkv, D, [17, 64, 5], [40, 2, 70], seed=2, prefill_impl=impl)


@pytest.mark.parametrize("Hq,Hkv,D", [(4, 2, 64), (32, 8, 64), (3, 1, 128), (5, 5, 64), (24, 8, 128)])
@pytest.mark.parametrize("page_size", [16, 32, 64])
def test_attention_prefill_tensor_core_kernel(Hq, Hkv, D, page_size):
    """impl 2 insists on the tensor-core kernel: portions that start and end anywhere relative to its
    64-row and 64-key tiles, pasts of every alignment, every page size, and windows."""
    run_attention("bfloat16", Hq, Hkv, D, [0, 0, 0, 0], [2, 63, 64, 65], page_size=page_size, seed=21, prefill_impl=2)
    run_attention("bfloat16", Hq, Hkv, D, [0, 1, 63, 64, 200], [300, 129, 2, 70, 131], page_size=page_size, seed=22,
                  prefill_impl=2)
    for window in (1, 20, 64, 100, 300):
        run_attention("bfloat16", Hq, Hkv, D, [0, 90, 290], [150, 35, 66], page_size=page_size, window=window, seed=23,
                      prefill_impl=2)


@pytest.mark.parametrize("Hq,Hkv,D", [(4, 2, 64), (32, 8, 64), (5, 5, 64), (3, 1, 64), (24, 8, 128), (3, 1, 128),
                                      (4, 4, 128), (16, 1, 64)])
@pytest.mark.parametrize("page_size", [16, 32, 64])
def test_attention_prefill_tcgen05_kernel(Hq, Hkv, D, page_size):
    """impl 3 insists on the tcgen05 kernel (head sizes 64 and 128): portions that start and end anywhere
    relative to its 128-row and 128-key tiles, pasts of every alignment, many key tiles per query tile
    (every stage and the S, P and O columns of tensor memory in use again and again, a row's reference
    maximum moved and O rescaled on the way), groups of one, two, three and more heads (pairs of heads
    share a CTA; the last head of an odd group has one alone), every page size, and windows."""
    run_attention("bfloat16", Hq, Hkv, D, [0, 0, 0, 0], [2, 127, 128, 129], page_size=page_size, seed=41, prefill_impl=3)
    run_attention("bfloat16", Hq, Hkv, D, [0, 1, 127, 128, 500], [600, 257, 2, 130, 131], page_size=page_size, seed=42,
                  prefill_impl=3)
    for window in (1, 20, 128, 200, 600):
        run_attention("bfloat16", Hq, Hkv, D, [0, 90, 590], [300, 35, 130], page_size=page_size, window=window, seed=43,
                      prefill_impl=3)
    assert int(kernels.tc_status(torch.device(DEV)).item()) == 0


def test_attention_prefill_tcgen05_kernel_long_rows_with_a_growing_maximum():
    """2,100 keys per row, with queries and keys made so that a row's largest score keeps growing with
    the key's position (every later tile raises the maximum by far more than 2^8): the reference maximum
    moves and O is rescaled in tensor memory at nearly every tile; then the opposite, the largest score
    at the row's first key.  More items than SMs at Hq = 32, so CTAs take several items each."""
    def growing(sign):
        def sharp(seqs, cos, sin):
            for x in seqs:
                T = x.shape[0]
                ramp = torch.arange(T, dtype=torch.float32)[:, None] * (sign * 0.02)
                x[:, 32 * 64:(32 + 8) * 64] += ramp          # the keys drift along one direction ...
                x[:, :32 * 64] += 1.0                        # ... that every query has a share of
        return sharp
    for sign in (1.0, -1.0):
        run_attention("bfloat16", 32, 8, 64, [0, 1000], [2100, 700], seed=45, sharp=growing(sign), prefill_impl=3)
    assert int(kernels.tc_status(torch.device(DEV)).item()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,D", ATTN_SHAPES)
def test_attention_decode_lengths_across_pages_and_partitions(dtype, Hq, Hkv, D):
    # impl 1: the CUDA-core kernel; 0: the tensor-core kernel where it applies (bfloat16, D 64 / 128)
    for impl in (0, 1):
        run_attention(dtype, Hq, Hkv, D, [0, 4, 15, 16, 128], [1, 1, 1, 1, 1], seed=3, decode_impl=impl)
        run_attention(dtype, Hq, Hkv, D, [255, 256, 257, 699], [1, 1, 1, 1], seed=4, decode_impl=impl)


@pytest.mark.parametrize("Hq,Hkv,D", [(4, 2, 64), (32, 8, 64), (3, 1, 128), (16, 1, 64), (24, 8, 128), (7, 7, 64)])
@pytest.mark.parametrize("page_size", [16, 32, 64])
def test_attention_decode_tensor_core_kernel(Hq, Hkv, D, page_size):
    """impl 2 insists on the tensor-core kernel: group sizes 1 to 16, both head sizes, every page size,
    lengths around the 32-key rounds, the 64-key warps and the 256-key partitions, and windows."""
    run_attention("bfloat16", Hq, Hkv, D, [0, 31, 32, 33, 63, 64, 65], [1] * 7, page_size=page_size, seed=11, decode_impl=2)
    run_attention("bfloat16", Hq, Hkv, D, [255, 256, 300, 511, 512, 1030], [1] * 6, page_size=page_size, seed=12, decode_impl=2)
    for window in (1, 20, 100, 300):
        run_attention("bfloat16", Hq, Hkv, D, [5, 99, 290, 700], [1] * 4, page_size=page_size, window=window, seed=13,
                      decode_impl=2)


@pytest.mark.parametrize("Hq,Hkv,D", [(4, 2, 64), (32, 8, 64), (3, 1, 128), (16, 1, 64), (24, 8, 128), (7, 7, 64)])
@pytest.mark.parametrize("page_size", [16, 32, 64, 128])
def test_attention_decode_streaming_kernel(Hq, Hkv, D, page_size):
    """impl 3 insists on the streaming kernel (persistent CTAs, every warp with its own two-stage ring
    of 32-key sub-blocks): the same cases as the one-partition kernel and a page size of a whole
    partition."""
    run_attention("bfloat16", Hq, Hkv, D, [0, 31, 32, 33, 63, 64, 65], [1] * 7, page_size=page_size, seed=11, decode_impl=3)
    run_attention("bfloat16", Hq, Hkv, D, [255, 256, 300, 511, 512, 1030], [1] * 6, page_size=page_size, seed=12, decode_impl=3)
    for window in (1, 20, 100, 300):
        run_attention("bfloat16", Hq, Hkv, D, [5, 99, 290, 700], [1] * 4, page_size=page_size, window=window, seed=13,
                      decode_impl=3)
    assert int(kernels.tc_status(torch.device(DEV)).item()) == 0


@pytest.mark.parametrize("Hq,Hkv,D", [(4, 2, 64), (32, 8, 64), (3, 1, 128), (16, 1, 64), (24, 8, 128), (7, 7, 64)])
@pytest.mark.parametrize("page_size", [16, 32, 64, 128])
def test_attention_decode_rows_kernel(Hq, Hkv, D, page_size):
    """impl 4 insists on the kernel that gives every (item, kv head) a cluster of its own and merges the
    partial results through distributed shared memory: the same cases as the other tensor-core kernels
    (rows shorter than a sub-block, rows that end on a sub-block's or a page's edge, windows)."""
    run_attention("bfloat16", Hq, Hkv, D, [0, 31, 32, 33, 63, 64, 65], [1] * 7, page_size=page_size, seed=11, decode_impl=4)
    run_attention("bfloat16", Hq, Hkv, D, [255, 256, 300, 511, 512, 1030], [1] * 6, page_size=page_size, seed=12, decode_impl=4)
    for window in (1, 20, 100, 300):
        run_attention("bfloat16", Hq, Hkv, D, [5, 99, 290, 700], [1] * 4, page_size=page_size, window=window, seed=13,
                      decode_impl=4)
    assert int(kernels.tc_status(torch.device(DEV)).item()) == 0


def test_attention_decode_rows_kernel_long_rows_and_many_rows():
    """Clusters of 2 (64 rows of 4,000 keys: every warp a run of several sub-blocks), of 8 (8 rows), of one
    CTA (128 rows of many lengths), and more rows than clusters are resident (320 and 1,000 rows: a CTA takes
    several, one after another, and its rings and sums are used again)."""
    decode_only_case(32, 8, 64, [4000 + 13 * i for i in range(8)], 16, 0, 4, seed=61)
    decode_only_case(32, 8, 64, [4096], 16, 0, 4, seed=62)
    decode_only_case(16, 8, 128, [1500, 3000, 77, 2047, 2048, 4096, 4097], 32, 0, 4, seed=63)
    decode_only_case(32, 8, 64, [2000 + 97 * i for i in range(12)] + [1, 130, 5, 640], 64, 1000, 4, seed=64)
    decode_only_case(32, 8, 64, [1 + (37 * i) % 700 for i in range(40)], 16, 0, 4, seed=65)
    decode_only_case(8, 8, 128, [1 + (53 * i) % 300 for i in range(125)], 32, 100, 4, seed=66)
    assert int(kernels.tc_status(torch.device(DEV)).item()) == 0


def decode_only_case(Hq, Hkv, D, lens, page_size, window, impl, seed):
    """Decode attention straight on a random cache (no rotation, no cache write): the reference
    gathers each item's keys and does the softmax in float64."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    blocks = [(n + page_size - 1) // page_size for n in lens]
    npages = sum(blocks) + 1
    perm = (torch.randperm(npages - 1, generator=g) + 1).tolist()
    bt = torch.zeros(B, max(blocks) + 1, dtype=torch.int32)
    it = iter(perm)
    for b in range(B):
        for i in range(blocks[b]):
            bt[b, i] = next(it)
    kc = torch.randn(npages, Hkv, page_size, D, generator=g).to(torch.bfloat16).to(DEV)
    vc = torch.randn(npages, Hkv, page_size, D, generator=g).to(torch.bfloat16).to(DEV)
    q = torch.randn(B, Hq * D, generator=g).to(torch.bfloat16).to(DEV)
    scale = 1.0 / math.sqrt(D)
    parts = (max(lens) + kernels.DECODE_PARTITION - 1) // kernels.DECODE_PARTITION
    po = torch.full((B * Hq * parts * D,), float("nan"), device=DEV)
    pm = torch.full((B * Hq * parts * 2,), float("nan"), device=DEV)
    items = torch.tensor([[b, b, lens[b], 0] for b in range(B)], dtype=torch.int32, device=DEV)
    counters = torch.zeros(B * Hkv, dtype=torch.int32, device=DEV)
    out = torch.full((B, Hq * D), float("nan"), device=DEV, dtype=torch.bfloat16)
    btd = bt.to(DEV)
    for _ in range(2):       # twice: the counters and the ring are left ready for the next launch
        kernels.attn_decode(q, q.shape[1], kc, vc, btd, items, po, pm, parts, counters, out, B, Hq, Hkv, D,
                            page_size, window, scale, impl)
    assert int(counters.abs().max()) == 0
    G = Hq // Hkv
    for b in range(B):
        n = lens[b]
        lo = max(0, n - window) if window > 0 else 0
        pages = btd[b, :blocks[b]].long()
        k = kc[pages].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, lo:n].double()     # [Hkv, keys, D]
        v = vc[pages].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, lo:n].double()
        qb = q[b].double().reshape(Hkv, G, D)
        p = torch.softmax(torch.einsum("hgd,hkd->hgk", qb, k) * scale, dim=-1)
        want = torch.einsum("hgk,hkd->hgd", p, v).reshape(Hq * D)
        close(out[b], want, 1.6e-2)


def test_attention_decode_streaming_kernel_many_units_per_cta():
    """Several thousand (item, head, partition) units over at most one CTA per SM: every warp has a run
    of several partitions, rows of partitions are cut by the ends of runs and merged from their pieces,
    with contexts of many lengths in one launch."""
    lens = [2000 + 97 * i for i in range(12)] + [1, 130, 5, 640]
    decode_only_case(32, 8, 64, lens, 16, 0, 3, seed=31)
    decode_only_case(32, 8, 64, lens, 64, 1000, 3, seed=32)
    decode_only_case(16, 8, 128, [1500, 3000, 77, 2047, 2048, 4096, 4097], 32, 0, 3, seed=33)
    decode_only_case(32, 8, 64, lens, 16, 0, 2, seed=31)
    assert int(kernels.tc_status(torch.device(DEV)).item()) == 0


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 64), (16, 2, 128), (4, 4, 64)])
@pytest.mark.parametrize("page_size,window", [(16, 0), (64, 0), (16, 300)])
@pytest.mark.parametrize("mode", ["stream", "one", "rows"])
def test_attention_decode_with_rotation_and_cache_write_in_the_kernel(Hq, Hkv, D, page_size, window, mode):
    """attn_decode_rope against rope_kv_write followed by attn_decode: the same outputs, and the same k and
    v rows written into the cache at the tokens' own positions (and nowhere else); with many partitions
    (the streaming kernel), with few (the one-partition kernel), and by the kernel of one cluster per row."""
    g = torch.Generator().manual_seed(51)
    streams = mode == "stream"
    lens = [700, 1, 129, 2048, 33, 1500, 260, 2047]          # context lengths including the new token
    lens = lens * 4 if streams else (lens[:5] if mode == "one" else lens)
    B = len(lens)
    cos, sin = plain_rope_tables(D, 10000.0, 2200)
    cos, sin = cos.to(DEV).contiguous(), sin.to(DEV).contiguous()
    blocks = [(n + page_size - 1) // page_size for n in lens]
    npages = sum(blocks) + 1
    perm = (torch.randperm(npages - 1, generator=g) + 1).tolist()
    bt = torch.zeros(B, max(blocks) + 1, dtype=torch.int32)
    it = iter(perm)
    for b in range(B):
        for i in range(blocks[b]):
            bt[b, i] = next(it)
    btd = bt.to(DEV)
    kc0 = torch.randn(npages, Hkv, page_size, D, generator=g).to(torch.bfloat16).to(DEV)
    vc0 = torch.randn(npages, Hkv, page_size, D, generator=g).to(torch.bfloat16).to(DEV)
    qkv0 = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(torch.bfloat16).to(DEV)
    scale = 1.0 / math.sqrt(D)
    parts = (max(lens) + kernels.DECODE_PARTITION - 1) // kernels.DECODE_PARTITION
    items = torch.tensor([[b, b, lens[b], 0] for b in range(B)], dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    slots = torch.tensor([int(bt[b, (lens[b] - 1) // page_size]) * page_size + (lens[b] - 1) % page_size
                          for b in range(B)], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def buffers():
        po = torch.full((B * Hq * parts * D,), float("nan"), device=DEV)
        pm = torch.full((B * Hq * parts * 2,), float("nan"), device=DEV)
        return po, pm, torch.zeros(B * Hkv, dtype=torch.int32, device=DEV), \
            torch.full((B, Hq * D), float("nan"), device=DEV, dtype=torch.bfloat16)

    # the two kernels
    kc1, vc1, qkv1 = kc0.clone(), vc0.clone(), qkv0.clone()
    kernels.rope_kv_write(qkv1, pos, slots, cos, sin, kc1, vc1, Hq, Hkv, D, page_size, status)
    po, pm, cnt, want = buffers()
    kernels.attn_decode(qkv1, qkv1.shape[1], kc1, vc1, btd, items, po, pm, parts, cnt, want, B, Hq, Hkv, D,
                        page_size, window, scale, 2 if mode == "one" else 3)
    # the one kernel
    kc2, vc2, qkv2 = kc0.clone(), vc0.clone(), qkv0.clone()
    po, pm, cnt, got = buffers()
    if mode != "rows":
        assert kernels.attn_decode_streams(qkv2, qkv2.shape[1], kc2, vc2, po, cnt, got, parts, B, Hq, Hkv, D,
                                           page_size) == streams
    assert kernels.attn_decode_rope_ok(qkv2, qkv2.shape[1], kc2, vc2, po, cnt, got, parts, B, Hq, Hkv, D, page_size,
                                       Hq * D, (Hq + Hkv) * D)
    kernels.attn_decode_rope(qkv2, qkv2.shape[1], kc2, vc2, btd, items, po, pm, parts, cnt, got, B, Hq, Hkv, D,
                             page_size, window, scale, cos, sin, Hq * D, (Hq + Hkv) * D, status,
                             impl=4 if mode == "rows" else 0)
    assert status.item() == 0 and int(cnt.abs().max()) == 0
    assert torch.equal(qkv2, qkv0), "the token rows stay unrotated"
    close(got, want, 4e-3)
    close(kc2, kc1, 1e-2)
    assert torch.equal(vc2, vc1)
    changed = (kc2 != kc0).any(dim=-1)                 # [pages, heads, slots]: only the tokens' own slots may differ
    allowed = torch.zeros_like(changed)
    for b in range(B):
        sl = int(slots[b])
        allowed[sl // page_size, :, sl % page_size] = True
    assert not (changed & ~allowed).any()


@pytest.mark.parametrize("window", [0, 200])
def test_attention_decode_streaming_kernel_many_short_rows(window):
    """Several rows per SM, short and long ones side by side, rows that end exactly at a partition's end,
    one-key rows."""
    lens = [516] * 24 + [1500, 33, 1, 129, 2048, 700, 1025, 260, 128, 1024] * 4
    decode_only_case(32, 8, 64, lens, 16, window, 3, seed=37)
    decode_only_case(32, 8, 64, lens[::-1], 16, window, 0, seed=38)
    decode_only_case(16, 8, 128, [516, 77, 1300, 640] * 16, 32, window, 3, seed=39)


def test_attention_decode_beyond_256_partitions():
    """A context of 40,000 keys has 313 partitions, more than the one-partition kernel can merge: the
    default choice must take the streaming kernel there (and the CUDA-core kernel must agree)."""
    decode_only_case(8, 2, 64, [40000, 33000, 7], 16, 0, 0, seed=35)
    decode_only_case(8, 2, 64, [40000], 16, 0, 1, seed=36)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_mixed_launch_and_other_page_sizes(dtype):
    run_attention(dtype, 4, 2, 64, [300, 31, 0, 90], [1, 33, 2, 1], page_size=32, seed=5)
    run_attention(dtype, 3, 1, 128, [63, 64, 200], [1, 65, 1], page_size=64, seed=6)
    # pages of 48 and 80 keys are no power of two: the tensor-core kernels, which find a key's page with a
    # shift and a mask, must leave such launches to the CUDA-core kernels
    run_attention(dtype, 4, 2, 64, [300, 31, 0, 90], [1, 33, 2, 1], page_size=48, seed=7)
    run_attention(dtype, 8, 2, 128, [100, 700, 5], [1, 1, 140], page_size=80, seed=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 7, 16, 40, 300])
def test_attention_window(dtype, window):
    run_attention(dtype, 4, 2, 64, [0, 50, 290], [45, 35, 1], window=window, seed=7)
    run_attention(dtype, 3, 3, 32, [99, 300], [1, 1], window=window, seed=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_is_found_among_hundreds(dtype):
    """One key far back is made to match the last query after rotation (both are the
    inverse rotation of the same vector u, |u|^2 = 4 D), so its score is 32 while all
    others are about N(0, 4): the output is that key's value, and a kernel that loses a
    partition, a page or a tile gives something else entirely."""
    Hq, Hkv, D = 4, 2, 64
    half = D // 2

    def unrotate(u, c, s):
        return torch.cat([u[:half] * c + u[half:] * s, u[half:] * c - u[:half] * s])

    for far, total in [(3, 700), (255, 700), (256, 530), (511, 530), (17, 300)]:
        def sharp(seqs, cos, sin, far=far, total=total):
            x = seqs[0]
            u = torch.full((D,), 2.0)
            for h in range(Hq):
                x[total - 1, h * D:(h + 1) * D] = unrotate(u, cos[total - 1], sin[total - 1])
            for h in range(Hkv):
                x[far, (Hq + h) * D:(Hq + h + 1) * D] = unrotate(u, cos[far], sin[far])
        run_attention(dtype, Hq, Hkv, D, [total - 1], [1], seed=9, sharp=sharp)     # decode kernel
        run_attention(dtype, Hq, Hkv, D, [total - 1], [1], seed=9, sharp=sharp, decode_impl=1)
        if dtype == "bfloat16":
            run_attention(dtype, Hq, Hkv, D, [total - 1], [1], seed=9, sharp=sharp, decode_impl=2)
            run_attention(dtype, Hq, Hkv, D, [total - 1], [1], seed=9, sharp=sharp, decode_impl=3)
            run_attention(dtype, Hq, Hkv, D, [total - 1], [1], seed=9, sharp=sharp, decode_impl=4)
        run_attention(dtype, Hq, Hkv, D, [total - 40], [40], seed=9, sharp=sharp)   # prefill kernel
        run_attention(dtype, Hq, Hkv, D, [total - 40], [40], seed=9, sharp=sharp, prefill_impl=1)
        if dtype == "bfloat16":
            run_attention(dtype, Hq, Hkv, D, [total - 40], [40], seed=9, sharp=sharp, prefill_impl=2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rope_kv_write_values_and_skipped_writes(dtype):
    Hq, Hkv, D, ps = 3, 2, 48, 16
    cos, sin = plain_rope_tables(D, 5e4, 512, {"type": "linear", "factor": 2.0})
    T = 9
    x = torch.randn(T, (Hq + 2 * Hkv) * D).to(DT[dtype])
    pos = torch.tensor([0, 1, 15, 16, 17, 100, 255, 300, 511], dtype=torch.int32)
    slots = torch.tensor([32, 33, 47, 80, 81, -1, 16, 17, 95], dtype=torch.int32)
    kc = torch.zeros(6, Hkv, ps, D, device=DEV, dtype=DT[dtype])
    vc = torch.zeros_like(kc)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    qkv = x.to(DEV).clone()
    kernels.rope_kv_write(qkv, pos.to(DEV), slots.to(DEV), cos.to(DEV), sin.to(DEV), kc, vc, Hq, Hkv, D, ps, status)
    xd = x.double()
    c, s = cos[pos.long()].double(), sin[pos.long()].double()
    q = P.rope_rotate(xd[:, :Hq * D].reshape(T, Hq, D), c, s)
    k = P.rope_rotate(xd[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D), c, s)
    v = xd[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    tol = 1e-6 if dtype == "float32" else 8e-3
    close(qkv[:, :Hq * D], q.reshape(T, -1), tol)
    close(qkv[:, Hq * D:(Hq + Hkv) * D], k.reshape(T, -1), tol)
    assert torch.equal(qkv[:, (Hq + Hkv) * D:].cpu(), x[:, (Hq + Hkv) * D:])
    written = torch.zeros(6 * ps, dtype=torch.bool)
    for t in range(T):
        sl = int(slots[t])
        if sl < 0:
            continue
        written[sl] = True
        close(kc[sl // ps, :, sl % ps, :], k[t], tol)
        assert torch.equal(vc[sl // ps, :, sl % ps, :].cpu().double(), v[t])
    flat_k = kc.permute(0, 2, 1, 3).reshape(6 * ps, -1)
    assert flat_k[~written.to(DEV)].abs().max().item() == 0      # nothing else was touched
    assert status.item() == 0
    kernels.rope_kv_write(qkv, torch.full((T,), 512, dtype=torch.int32, device=DEV), None, cos.to(DEV),
                          sin.to(DEV), kc, vc, Hq, Hkv, D, ps, status)
    assert status.item() == 2                                     # a position beyond the table is flagged
    status.zero_()
    before = kc.clone()
    far = torch.tensor([6 * ps, 6 * ps + 5, 2 ** 30] + [-1] * (T - 3), dtype=torch.int32, device=DEV)
    kernels.rope_kv_write(x.to(DEV).clone(), pos.to(DEV), far, cos.to(DEV), sin.to(DEV), kc, vc, Hq, Hkv, D, ps, status)
    assert status.item() == 4 and torch.equal(kc, before)         # a slot beyond the pool: flagged, not written


def test_resolve_ids_and_bias_and_residual():
    ids = torch.tensor([5, 6, 7, 8], dtype=torch.int32, device=DEV)
    src = torch.tensor([-1, 2, -1, 0], dtype=torch.int32, device=DEV)
    sampled = torch.tensor([100, 200, 300], dtype=torch.int32, device=DEV)
    kernels.resolve_ids(ids, src, sampled, 4)
    assert ids.tolist() == [5, 300, 7, 100]
    x = torch.randn(5, 33, device=DEV).to(torch.bfloat16)
    b = torch.randn(33, device=DEV)
    want = (x.float() + b).to(torch.bfloat16)
    kernels.add_bias(x, b)
    assert torch.equal(x, want)
    r = torch.randn(7, 50, device=DEV)
    d = torch.randn(7, 50, device=DEV).to(torch.bfloat16)
    want = r + d.float()
    kernels.add_residual(r, d)
    assert torch.equal(r, want)


SKINNY_SHAPES = [(1, 3072, 2048), (8, 2048, 8192), (3, 331, 200), (9, 1000, 384), (16, 64, 328), (13, 704, 256),
                 (16, 2048, 2048), (5, 16, 8), (8, 5000, 264), (16, 300, 8192)]


@pytest.mark.parametrize("M,N,K", SKINNY_SHAPES)
def test_gemm_skinny_plain_epilogues(M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M * N + K)
    x = torch.randn(M + 3, K, device=DEV, generator=g).to(torch.bfloat16)[:M]
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    y = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    kernels.gemm_skinny(w, y, kernels.EPI_BF16, M, x=x)
    close(y, ref, 1.2e-2)
    yf = torch.full((M, N), float("nan"), device=DEV)
    kernels.gemm_skinny(w, yf, kernels.EPI_F32, M, x=x)
    close(yf, ref, 2e-5)
    res = torch.randn(M, N, device=DEV, generator=g)
    want = res.double() + ref.to(torch.bfloat16).double()
    kernels.gemm_skinny(w, res, kernels.EPI_ADD_RESIDUAL, M, x=x)
    close(res, want, 1e-2)
    if M > 1:       # a row does not depend on its neighbours, bit for bit, nor on the padding it gets
        y1 = torch.empty(1, N, device=DEV)
        kernels.gemm_skinny(w, y1, kernels.EPI_F32, 1, x=x[M // 2:M // 2 + 1])
        assert torch.equal(y1[0], yf[M // 2])
    y2 = torch.empty(M, N, device=DEV)
    kernels.gemm_skinny(w, y2, kernels.EPI_F32, M, x=x)
    assert torch.equal(y2, yf)      # and not on the run


@pytest.mark.parametrize("M,N,K", [(1, 8192, 2048), (8, 704, 256), (7, 328, 200), (12, 1024, 384), (16, 96, 4096)])
@pytest.mark.parametrize("w32", [False, True])
def test_gemm_skinny_norm_prologue_and_gated_epilogue(M, N, K, w32):
    g = torch.Generator(device="cuda").manual_seed(N + K)
    T = M + 5
    res = torch.randn(T, K, device=DEV, generator=g) * 2
    nw = (1 + 0.1 * torch.randn(K, device=DEV, generator=g)).to(torch.float32 if w32 else torch.bfloat16)
    idx = torch.randperm(T, device=DEV, generator=g)[:M].to(torch.int32)
    w = (torch.randn(2 * N, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    eps = 1e-5
    P.STORE_DTYPE = torch.bfloat16
    try:
        xn = P.rmsnorm(res.double().cpu(), nw.cpu(), eps)                 # rounded to bfloat16, as the kernel does
        xg = P.rmsnorm(res[idx.long()].double().cpu(), nw.cpu(), eps)
        gate, up = P.linear(xn[:M], w[:N].cpu()), P.linear(xn[:M], w[N:].cpu())
        want_act = P.swiglu(gate, up)
    finally:
        P.STORE_DTYPE = None
    act = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    kernels.gemm_skinny(w, act, kernels.EPI_SWIGLU, M, residual=res, norm_w=nw, eps=eps)
    close(act, want_act, 2e-2)
    logits = torch.full((M, 2 * N), float("nan"), device=DEV)
    kernels.gemm_skinny(w, logits, kernels.EPI_F32, M, residual=res, norm_w=nw, eps=eps, rows_idx=idx)
    close(logits, xg @ w.double().cpu().T, 1e-2)
    y = torch.empty(M, 2 * N, device=DEV, dtype=torch.bfloat16)
    kernels.gemm_skinny(w, y, kernels.EPI_BF16, M, residual=res, norm_w=nw, eps=eps)
    close(y, xn[:M] @ w.double().cpu().T, 1.5e-2)
    # the gated product without the fused norm
    xb = xn[:M].to(torch.bfloat16).to(DEV)
    act2 = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    kernels.gemm_skinny(w, act2, kernels.EPI_SWIGLU, M, x=xb)
    close(act2, want_act, 2e-2)


@pytest.mark.parametrize("M,H,N2,K1", [(8, 2048, 3072, 2048), (5, 328, 200, 72), (1, 1000, 96, 8192), (8, 4400, 64, 256)])
@pytest.mark.parametrize("w32", [False, True])
def test_gemm_skinny_norm_handed_over_between_two_products(M, H, N2, K1, w32):
    """residual += x W1^T leaves bfloat16(residual * norm_weight) and per-tile sums of squares; the next
    product takes them and scales its rows: together the RMSNorm between the two, against float64."""
    g = torch.Generator(device="cuda").manual_seed(M + H + N2)
    x = torch.randn(M, K1, device=DEV, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(H, K1, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    res = torch.randn(M + 2, H, device=DEV, generator=g)[:M] * 3
    nw = (1 + 0.1 * torch.randn(H, device=DEV, generator=g)).to(torch.float32 if w32 else torch.bfloat16)
    w2 = (torch.randn(2 * N2, H, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    eps = 1e-5
    want_res = res.double() + (x.double() @ w1.double().T).to(torch.bfloat16).double()
    xw, sums = kernels.norm_handover_buffers(8, H, DEV)
    xw.fill_(float("nan"))
    sums.fill_(float("nan"))
    kernels.gemm_skinny(w1, res, kernels.EPI_ADD_RESIDUAL, M, x=x, hand_out=(nw, xw, sums))
    close(res, want_res, 1e-2)
    got = res.double()                                     # what the kernel itself stored
    close(xw[:M], got * nw.double(), 5e-3)
    assert torch.isnan(xw[M:]).all()
    ss = (got * got).sum(1)
    assert ((sums[:M].double().sum(1) - ss).abs() <= 1e-5 * ss).all()
    inv = torch.rsqrt(ss / H + eps)[:, None]
    ref = (xw[:M].double() @ w2.double().T) * inv          # from the xw the kernel stored ...
    exact = ((got * inv) * nw.double()) @ w2.double().T    # ... and the norm as it is defined
    y = torch.full((M, 2 * N2), float("nan"), device=DEV, dtype=torch.bfloat16)
    kernels.gemm_skinny(w2, y, kernels.EPI_BF16, M, x=xw[:M], hand_in=sums, eps=eps)
    close(y, ref, 1.2e-2)
    close(y, exact, 1.5e-2)
    yf = torch.full((M, 2 * N2), float("nan"), device=DEV)
    kernels.gemm_skinny(w2, yf, kernels.EPI_F32, M, x=xw[:M], hand_in=sums, eps=eps)
    close(yf, ref, 2e-5)
    act = torch.full((M, N2), float("nan"), device=DEV, dtype=torch.bfloat16)
    kernels.gemm_skinny(w2, act, kernels.EPI_SWIGLU, M, x=xw[:M], hand_in=sums, eps=eps)
    P.STORE_DTYPE = torch.bfloat16
    try:
        want_act = P.swiglu(P.stored(ref[:, :N2].cpu()), P.stored(ref[:, N2:].cpu()))
    finally:
        P.STORE_DTYPE = None
    close(act, want_act, 2e-2)
    # without the hand-over the same call is the plain product
    kernels.gemm_skinny(w2, yf, kernels.EPI_F32, M, x=xw[:M])
    close(yf, xw[:M].double() @ w2.double().T, 2e-5)
    with pytest.raises(kernels.KernelError):               # a hand-over only from `residual +=`
        kernels.gemm_skinny(w1, torch.zeros(M, H, device=DEV), kernels.EPI_F32, M, x=x, hand_out=(nw, xw, sums))


def test_gemm_skinny_refuses_what_it_cannot_do():
    w = torch.zeros(32, 20, device=DEV, dtype=torch.bfloat16)      # K no multiple of 8
    x = torch.zeros(4, 20, device=DEV, dtype=torch.bfloat16)
    assert not kernels.skinny_ok(4, w, torch.bfloat16)
    with pytest.raises(kernels.KernelError):
        kernels.gemm_skinny(w, torch.zeros(4, 32, device=DEV, dtype=torch.bfloat16), kernels.EPI_BF16, 4, x=x)
    w = torch.zeros(32, 64, device=DEV, dtype=torch.bfloat16)
    assert not kernels.skinny_ok(17, w, torch.bfloat16) and kernels.skinny_ok(16, w, torch.bfloat16)
    with pytest.raises(kernels.KernelError):
        kernels.gemm_skinny(w, torch.zeros(4, 32, device=DEV), kernels.EPI_BF16, 4,
                            x=torch.zeros(4, 64, device=DEV, dtype=torch.bfloat16))


MID_SHAPES = [(64, 3072, 2048), (17, 2048, 8192), (128, 331, 200), (33, 1000, 72), (100, 704, 256), (1, 128, 8),
              (96, 8192, 2048), (32, 64, 4096)]


@pytest.mark.parametrize("M,N,K", MID_SHAPES)
def test_gemm_mid_epilogues(M, N, K):
    """The tcgen05 product for up to 128 rows (weights as the wide operand, K split over the CTAs of a
    cluster) against float64: both storing epilogues, edge tiles in N and K, every width of the token
    operand, every cluster size from 1 to 8; a second run gives the same bits (the partial tiles are added
    in a fixed order)."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M + 2, K, device=DEV, generator=g).to(torch.bfloat16)[:M]
    w = (torch.randn(2 * N, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    status = kernels.tc_status(x.device)
    y = torch.full((M, 2 * N), float("nan"), device=DEV, dtype=torch.bfloat16)
    kernels.gemm_mid(x, w, y, kernels.EPI_BF16)
    close(y, ref, 1.2e-2)
    y2 = torch.full((M + 1, 2 * N + 8), float("nan"), device=DEV, dtype=torch.bfloat16)[:M, :2 * N]    # a strided output
    kernels.gemm_mid(x, w, y2, kernels.EPI_BF16)
    assert torch.equal(y2, y)
    act = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    kernels.gemm_mid(x, w, act, kernels.EPI_SWIGLU)
    P.STORE_DTYPE = torch.bfloat16
    try:
        want_act = P.swiglu(P.stored(ref[:, :N].cpu()), P.stored(ref[:, N:].cpu()))
    finally:
        P.STORE_DTYPE = None
    close(act, want_act, 2e-2)
    act2 = torch.empty_like(act)
    kernels.gemm_mid(x, w, act2, kernels.EPI_SWIGLU)
    assert torch.equal(act2, act)
    assert int(status.item()) == 0
    with pytest.raises(kernels.KernelError):
        kernels.gemm_mid(torch.zeros(129, K, device=DEV, dtype=torch.bfloat16), w,
                         torch.zeros(129, 2 * N, device=DEV, dtype=torch.bfloat16))


@pytest.mark.parametrize("M,H,N2,K1", [(64, 2048, 3072, 2048), (17, 328, 200, 72), (128, 1000, 96, 8192),
                                       (33, 4400, 64, 256), (100, 2048, 8192, 8192), (1, 136, 40, 640)])
@pytest.mark.parametrize("w32", [False, True])
def test_gemm_mid_residual_epilogue_and_norm_handed_over(M, H, N2, K1, w32):
    """residual += x W1^T in the product's epilogue, which also leaves bfloat16(residual * norm_weight) and
    the sums of squares per feature tile; the next product takes them and scales its rows: together the
    RMSNorm between the two, against float64.  Rows and features beyond the product are not touched."""
    g = torch.Generator(device="cuda").manual_seed(M + H + N2)
    x = torch.randn(M, K1, device=DEV, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(H, K1, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    res_all = torch.randn(M + 2, H + 4, device=DEV, generator=g) * 3
    before = res_all.clone()
    res = res_all[:M, :H]
    nw = (1 + 0.1 * torch.randn(H, device=DEV, generator=g)).to(torch.float32 if w32 else torch.bfloat16)
    w2 = (torch.randn(2 * N2, H, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    eps = 1e-5
    status = kernels.tc_status(x.device)
    want_res = res.double() + x.double() @ w1.double().T
    plain = res.clone()
    kernels.gemm_mid(x, w1, None, kernels.EPI_ADD_RESIDUAL, residual=plain)         # without a hand-over
    close(plain, want_res, 5e-5)                           # the product is added in float32, not rounded first
    xw, sums = kernels.mid_handover_buffers(H, DEV)
    xw.fill_(float("nan"))
    sums.fill_(float("nan"))
    kernels.gemm_mid(x, w1, None, kernels.EPI_ADD_RESIDUAL, residual=res, hand_out=(nw, xw, sums))
    assert torch.equal(res, plain)
    assert torch.equal(res_all[M:], before[M:]) and torch.equal(res_all[:, H:], before[:, H:])
    got = res.double()                                     # what the kernel itself stored
    close(xw[:M], got * nw.double(), 5e-3)
    assert torch.isnan(xw[M:]).all()
    ss = (got * got).sum(1)
    assert ((sums[:M].double().sum(1) - ss).abs() <= 1e-5 * ss).all()
    inv = torch.rsqrt(ss / H + eps)[:, None]
    ref = (xw[:M].double() @ w2.double().T) * inv          # from the xw the kernel stored ...
    exact = ((got * inv) * nw.double()) @ w2.double().T    # ... and the norm as it is defined
    y = torch.full((M, 2 * N2), float("nan"), device=DEV, dtype=torch.bfloat16)
    kernels.gemm_mid(xw[:M], w2, y, kernels.EPI_BF16, hand_in=sums, eps=eps)
    close(y, ref, 1.2e-2)
    close(y, exact, 1.5e-2)
    act = torch.full((M, N2), float("nan"), device=DEV, dtype=torch.bfloat16)
    kernels.gemm_mid(xw[:M], w2, act, kernels.EPI_SWIGLU, hand_in=sums, eps=eps)
    P.STORE_DTYPE = torch.bfloat16
    try:
        want_act = P.swiglu(P.stored(ref[:, :N2].cpu()), P.stored(ref[:, N2:].cpu()))
    finally:
        P.STORE_DTYPE = None
    close(act, want_act, 2e-2)
    assert int(status.item()) == 0
    with pytest.raises(kernels.KernelError):               # a hand-over only from `residual +=`
        kernels.gemm_mid(x, w1, torch.zeros(M, H, device=DEV, dtype=torch.bfloat16), kernels.EPI_BF16,
                         hand_out=(nw, xw, sums))
    with pytest.raises(kernels.KernelError):               # the stream is float32
        kernels.gemm_mid(x, w1, None, kernels.EPI_ADD_RESIDUAL, residual=res.to(torch.bfloat16))


TC_SHAPES = [(128, 128, 64), (17, 331, 200), (256, 384, 512), (130, 200, 72), (2048, 3072, 2048), (300, 1000, 384),
             (1, 128, 8), (640, 2048, 8192)]


@pytest.mark.parametrize("tile_n", [128, 256, 512])
@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemm_tc_epilogues(M, N, K, tile_n):
    """The tcgen05 / TMEM / TMA product against float64, every epilogue, edge tiles in M, N and K; one CTA per
    tile of 128 or 256 features, and CTA pairs on 256 x 256 tiles (tile_n 512)."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M + 2, K, device=DEV, generator=g).to(torch.bfloat16)[:M]
    w = (torch.randn(2 * N, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    status = kernels.tc_status(x.device)
    y = torch.full((M, 2 * N), float("nan"), device=DEV, dtype=torch.bfloat16)
    kernels.gemm_tc(x, w, y, kernels.EPI_BF16, tile_n)
    close(y, ref, 1.2e-2)
    yf = torch.full((M, 2 * N), float("nan"), device=DEV)
    kernels.gemm_tc(x, w, yf, kernels.EPI_F32, tile_n)
    close(yf, ref, 2e-5)
    res = torch.randn(M, 2 * N, device=DEV, generator=g)
    want = res.double() + ref.to(torch.bfloat16).double()
    kernels.gemm_tc(x, w, res, kernels.EPI_ADD_RESIDUAL, tile_n)
    close(res, want, 1e-2)
    act = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    kernels.gemm_tc(x, w, act, kernels.EPI_SWIGLU, tile_n)
    P.STORE_DTYPE = torch.bfloat16
    try:
        want_act = P.swiglu(P.stored(ref[:, :N].cpu()), P.stored(ref[:, N:].cpu()))
    finally:
        P.STORE_DTYPE = None
    close(act, want_act, 2e-2)
    y2 = torch.empty(M, 2 * N, device=DEV)
    kernels.gemm_tc(x, w, y2, kernels.EPI_F32, tile_n)
    assert torch.equal(y2, yf)                       # the same bits on every run
    if M > 1:                                        # and a row does not depend on the rows beside it
        y1 = torch.empty(1, 2 * N, device=DEV)
        kernels.gemm_tc(x[M // 2:M // 2 + 1], w, y1, kernels.EPI_F32, tile_n)
        assert torch.equal(y1[0], yf[M // 2])
    assert int(status.item()) == 0                   # no wait inside the kernel ran out


def test_gemm_tc_refuses_what_it_cannot_do():
    x = torch.zeros(4, 20, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(32, 20, device=DEV, dtype=torch.bfloat16)
    assert not kernels.gemm_tc_ok(x, w)
    with pytest.raises(kernels.KernelError):
        kernels.gemm_tc(x, w, torch.zeros(4, 32, device=DEV, dtype=torch.bfloat16))
