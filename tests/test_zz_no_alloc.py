"""rl_attn_decode_noalloc: the decode-attention entry point for callers that cannot
allocate device memory (a plug-in under a fixed memory budget, a real-time loop that
must stay out of the allocator).  It keeps its scratch in a fixed array inside the
library.  The test calls it through its exported C symbol, twice in a row, and checks
each result against the ordinary entry point (which gets scratch buffers from the
caller), within the tolerance the other kernel tests use; then that a request beyond the
array's size is refused with a message and without launching anything.

This file sorts last so that a run that stops at the first failure has already run
every other test."""

import ctypes
import math
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 8 << 20


def setup_case(dtype, B, ctx, Hq, Hkv, D, ps, seed):
    g = torch.Generator().manual_seed(seed)
    pages_per_seq = (max(ctx) + ps - 1) // ps
    npages = B * pages_per_seq + 1
    k = torch.randn(npages, Hkv, ps, D, generator=g).to(dtype).cuda()
    v = torch.randn(npages, Hkv, ps, D, generator=g).to(dtype).cuda()
    bt = (torch.randperm(npages - 1, generator=g) + 1)[:B * pages_per_seq].view(B, pages_per_seq).to(torch.int32).cuda()
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(dtype).cuda()
    items = torch.tensor([[i, i, ctx[i], 0] for i in range(B)], dtype=torch.int32).cuda()
    return k, v, bt, qkv, items


@pytest.mark.parametrize("dtype,D,Hq,Hkv", [(torch.bfloat16, 64, 8, 2), (torch.float32, 64, 4, 2), (torch.bfloat16, 48, 6, 3)])
def test_no_alloc_entry_point_matches_the_ordinary_one(dtype, D, Hq, Hkv):
    from redline_b200.ops import kernels
    lib = kernels._attn(D)
    fn = lib.rl_attn_decode_noalloc
    fn.argtypes = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                   c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_char_p, c_int]
    fn.restype = c_int
    ps, scale = 16, 1.0 / math.sqrt(D)
    tol = 2e-5 if dtype == torch.float32 else 1.6e-2
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    err = ctypes.create_string_buffer(512)
    # two calls in a row with different shapes: the second finds the first one's leftovers in the scratch
    for call, (B, ctx) in enumerate([(3, [700, 129, 5]), (5, [33, 1000, 256, 257, 128])]):
        k, v, bt, qkv, items = setup_case(dtype, B, ctx, Hq, Hkv, D, ps, seed=call)
        parts = (max(ctx) + kernels.DECODE_PARTITION - 1) // kernels.DECODE_PARTITION
        want = torch.full((B, Hq * D), float("nan"), dtype=dtype, device="cuda")
        po = torch.empty(B * Hq * parts * D, device="cuda")
        pm = torch.empty(B * Hq * parts * 2, device="cuda")
        cnt = torch.zeros(B * Hkv, dtype=torch.int32, device="cuda")
        kernels.attn_decode(qkv, qkv.shape[1], k, v, bt, items, po, pm, parts, cnt, want, B, Hq, Hkv, D, ps, 0, scale)
        got = torch.full((B, Hq * D), float("nan"), dtype=dtype, device="cuda")
        rc = fn(kernels.DTYPE_CODE[dtype], qkv.data_ptr(), qkv.shape[1], k.data_ptr(), v.data_ptr(), bt.data_ptr(),
                bt.shape[1], items.data_ptr(), parts, got.data_ptr(), got.stride(0), B, Hq, Hkv, ps, 0, scale, stream,
                err, len(err))
        assert rc == 0, (rc, err.value)
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        diff = (got.double() - want.double()).abs().max().item() / want.double().abs().max().item()
        assert diff < tol, (call, diff)
    # a request that needs more scratch than the array holds is refused, with both numbers in the message
    B = 64
    parts = SCRATCH_BYTES // (B * Hq * (D + 2) * 4) + 1
    need = B * Hq * parts * (D + 2) * 4
    assert need > SCRATCH_BYTES
    got.fill_(7.0)
    rc = fn(kernels.DTYPE_CODE[dtype], qkv.data_ptr(), qkv.shape[1], k.data_ptr(), v.data_ptr(), bt.data_ptr(),
            bt.shape[1], items.data_ptr(), parts, got.data_ptr(), got.stride(0), B, Hq, Hkv, ps, 0, scale, stream, err,
            len(err))
    torch.cuda.synchronize()
    assert rc == -1 and str(SCRATCH_BYTES).encode() in err.value and b"scratch" in err.value
    assert float(got.float().min()) == 7.0          # nothing was launched
