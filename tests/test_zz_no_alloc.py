"""rl_attn_decode_noalloc: the decode-attention entry point for callers that cannot
allocate device memory (a plug-in under a fixed memory budget, a real-time loop that
must stay out of the allocator).  It keeps its scratch in a fixed array inside the
library.  The tests call it through its exported C symbol, twice in a row with different
shapes (the second call finds the first one's leftovers in the array), and check each
result against a float64 restatement of the attention and against the ordinary entry
point (which gets scratch buffers from the caller), within the tolerance the other
kernel tests use: on launches that the one-partition kernels take and on one large
enough for the streaming kernel, whose pieces, merges and counters then live in the
array.  A request beyond the array's size must be refused with a message and without
launching anything.

This file sorts last so that a run that stops at the first failure has already run
every other test."""

import ctypes
import math
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 8 << 20
ARGTYPES = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
            c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_char_p, c_int]


def setup_case(dtype, ctx, Hq, Hkv, D, ps, seed):
    g = torch.Generator().manual_seed(seed)
    B = len(ctx)
    pages_per_seq = (max(ctx) + ps - 1) // ps
    npages = B * pages_per_seq + 1
    k = torch.randn(npages, Hkv, ps, D, generator=g).to(dtype).cuda()
    v = torch.randn(npages, Hkv, ps, D, generator=g).to(dtype).cuda()
    bt = (torch.randperm(npages - 1, generator=g) + 1)[:B * pages_per_seq].view(B, pages_per_seq).to(torch.int32).cuda()
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(dtype).cuda()
    items = torch.tensor([[i, i, ctx[i], 0] for i in range(B)], dtype=torch.int32).cuda()
    return k, v, bt, qkv, items


def attention_in_float64(qkv, k, v, bt, ctx, Hq, Hkv, D, ps, scale):
    """softmax(q k^T * scale) v per item over the keys its block table names, in float64."""
    G = Hq // Hkv
    out = []
    for b, n in enumerate(ctx):
        pages = bt[b, :(n + ps - 1) // ps].long()
        kb = k[pages].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n].double()
        vb = v[pages].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n].double()
        q = qkv[b, :Hq * D].double().reshape(Hkv, G, D)
        p = torch.softmax(torch.einsum("hgd,hkd->hgk", q, kb) * scale, dim=-1)
        out.append(torch.einsum("hgk,hkd->hgd", p, vb).reshape(Hq * D))
    return torch.stack(out)


def call_both(fn, dtype, ctx, Hq, Hkv, D, ps, seed):
    """One call of each entry point on the same inputs; returns (no-alloc result, ordinary result,
    float64 result, whether the launch is one the streaming kernel takes)."""
    from redline_b200.ops import kernels
    k, v, bt, qkv, items = setup_case(dtype, ctx, Hq, Hkv, D, ps, seed)
    B, scale = len(ctx), 1.0 / math.sqrt(D)
    parts = (max(ctx) + kernels.DECODE_PARTITION - 1) // kernels.DECODE_PARTITION
    plain = torch.full((B, Hq * D), float("nan"), dtype=dtype, device="cuda")
    po = torch.empty(B * Hq * parts * D, device="cuda")
    pm = torch.empty(B * Hq * parts * 2, device="cuda")
    cnt = torch.zeros(B * Hkv, dtype=torch.int32, device="cuda")
    kernels.attn_decode(qkv, qkv.shape[1], k, v, bt, items, po, pm, parts, cnt, plain, B, Hq, Hkv, D, ps, 0, scale)
    streams = dtype == torch.bfloat16 and bool(kernels.attn_decode_streams(
        qkv, qkv.shape[1], k, v, po, cnt, plain, parts, B, Hq, Hkv, D, ps))
    got = torch.full((B, Hq * D), float("nan"), dtype=dtype, device="cuda")
    err = ctypes.create_string_buffer(512)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = fn(kernels.DTYPE_CODE[dtype], qkv.data_ptr(), qkv.shape[1], k.data_ptr(), v.data_ptr(), bt.data_ptr(),
            bt.shape[1], items.data_ptr(), parts, got.data_ptr(), got.stride(0), B, Hq, Hkv, ps, 0, scale, stream,
            err, len(err))
    assert rc == 0, (rc, err.value)
    torch.cuda.synchronize()
    want = attention_in_float64(qkv, k, v, bt, ctx, Hq, Hkv, D, ps, scale)
    return got, plain, want, streams


def entry_point(D):
    from redline_b200.ops import kernels
    fn = kernels._attn(D).rl_attn_decode_noalloc
    fn.argtypes = ARGTYPES
    fn.restype = c_int
    return fn


def rel(a, ref):
    return (a.double() - ref.double()).abs().max().item() / ref.double().abs().max().item()


@pytest.mark.parametrize("dtype,D,Hq,Hkv", [(torch.bfloat16, 64, 8, 2), (torch.float32, 64, 4, 2), (torch.bfloat16, 48, 6, 3)])
def test_no_alloc_entry_point_matches_the_ordinary_one(dtype, D, Hq, Hkv):
    from redline_b200.ops import kernels
    fn = entry_point(D)
    ps, scale = 16, 1.0 / math.sqrt(D)
    tol = 2e-5 if dtype == torch.float32 else 1.6e-2
    # two calls in a row with different shapes: the second finds the first one's leftovers in the scratch
    for call, ctx in enumerate([[700, 129, 5], [33, 1000, 256, 257, 128]]):
        got, plain, want, _ = call_both(fn, dtype, ctx, Hq, Hkv, D, ps, seed=call)
        assert not torch.isnan(got.float()).any()
        assert rel(got, want) < tol, (call, rel(got, want))        # against the float64 restatement
        assert rel(got, plain) < tol, (call, rel(got, plain))      # and against the ordinary entry point
    # a request that needs more scratch than the array holds is refused, with both numbers in the message
    B = 64
    k, v, bt, qkv, items = setup_case(dtype, [5] * B, Hq, Hkv, D, ps, seed=9)
    parts = SCRATCH_BYTES // (B * Hq * (D + 2) * 4) + 1
    need = B * Hq * parts * (D + 2) * 4
    assert need > SCRATCH_BYTES
    got = torch.full((B, Hq * D), 7.0, dtype=dtype, device="cuda")
    err = ctypes.create_string_buffer(512)
    rc = fn(kernels.DTYPE_CODE[dtype], qkv.data_ptr(), qkv.shape[1], k.data_ptr(), v.data_ptr(), bt.data_ptr(),
            bt.shape[1], items.data_ptr(), parts, got.data_ptr(), got.stride(0), B, Hq, Hkv, ps, 0, scale,
            c_void_p(torch.cuda.current_stream().cuda_stream), err, len(err))
    torch.cuda.synchronize()
    assert rc == -1 and str(SCRATCH_BYTES).encode() in err.value and b"scratch" in err.value
    assert float(got.float().min()) == 7.0          # nothing was launched


def test_no_alloc_entry_point_with_the_streaming_kernel_in_the_array():
    """16 sequences of about 1,100 keys with 8 kv heads are 1,152 (item, head, partition) units: the
    launch goes to the streaming kernel, whose pieces, statistics and arrival counters then lie in the
    built-in array (about 1.2 MB of it).  Two calls in a row with other lengths; after them a small
    launch of the one-partition kernel finds the array as the streaming kernel left it."""
    fn = entry_point(64)
    for call, ctx in enumerate([[1100 + 3 * i for i in range(16)], [1152 - 7 * i for i in range(16)]]):
        got, plain, want, streams = call_both(fn, torch.bfloat16, ctx, 32, 8, 64, 16, seed=20 + call)
        assert streams, "this launch was meant for the streaming kernel"
        assert not torch.isnan(got.float()).any()
        assert rel(got, want) < 1.6e-2, (call, rel(got, want))
        assert rel(got, plain) < 1.6e-2, (call, rel(got, plain))
    got, plain, want, streams = call_both(fn, torch.bfloat16, [300, 17, 129], 32, 8, 64, 16, seed=23)
    assert not streams
    assert rel(got, want) < 1.6e-2 and rel(got, plain) < 1.6e-2
