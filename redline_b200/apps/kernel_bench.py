"""Times single kernels of the package at given sizes and reports their achieved
bandwidth or FLOP rate against the measured peaks (MEASURED_PEAKS.json beside the
package, if present).

    python -m redline_b200.apps.kernel_bench attn_decode --batch 8 --ctx 4096
    python -m redline_b200.apps.kernel_bench skinny --rows 8 --n 3072 --k 2048 [--norm] [--epilogue swiglu]
    python -m redline_b200.apps.kernel_bench attn_prefill --tokens 2048
    python -m redline_b200.apps.kernel_bench gemm_tc --rows 2048 --n 8192 --k 2048 --epilogue swiglu [--library]

Each kernel runs over several distinct copies of its large operands (more than the
L2 holds), captured in a CUDA graph so that launch overhead of the host is not
measured; times are CUDA events around graph replays.  The same commands are what
the profiles under ``profiles/`` were captured with (under ncu).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

from ..ops import kernels

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f)
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def graph_time_us(fn, calls: int, replays: int = 20, use_graph: bool = True) -> float:
    """Mean time of one call of fn in microseconds."""
    fn(0)
    torch.cuda.synchronize()
    if use_graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(calls):
                fn(i)
        run = g.replay
    else:
        def run():
            for i in range(calls):
                fn(i)
    run()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(replays):
        run()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / replays / calls * 1e3


def bench_attn_decode(args) -> None:
    dev = "cuda"
    B, ctx, Hq, Hkv, D, ps = args.batch, args.ctx, args.heads, args.kv_heads, args.head_dim, args.page_size
    pages_per_seq = (ctx + ps - 1) // ps
    npages = B * pages_per_seq + 1
    layers = max(1, min(args.copies, int(3e9 // (npages * Hkv * ps * D * 2 * 2))))
    kv = [(torch.randn(npages, Hkv, ps, D, device=dev).to(torch.bfloat16),
           torch.randn(npages, Hkv, ps, D, device=dev).to(torch.bfloat16)) for _ in range(layers)]
    perm = torch.randperm(npages - 1) + 1
    bt = perm[:B * pages_per_seq].view(B, pages_per_seq).to(torch.int32).to(dev)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=dev).to(torch.bfloat16)
    items = torch.tensor([[i, i, ctx, 0] for i in range(B)], dtype=torch.int32, device=dev)
    parts = (ctx + kernels.DECODE_PARTITION - 1) // kernels.DECODE_PARTITION
    po = torch.empty(B * Hq * parts * D, device=dev)
    pm = torch.empty(B * Hq * parts * 2, device=dev)
    cnt = torch.zeros(B * Hkv, dtype=torch.int32, device=dev)
    out = torch.empty(B, Hq * D, device=dev, dtype=torch.bfloat16)

    def fn(i):
        k, v = kv[i % layers]
        kernels.attn_decode(qkv, qkv.shape[1], k, v, bt, items, po, pm, parts, cnt, out, B, Hq, Hkv, D, ps, 0,
                            1.0 / math.sqrt(D), args.impl)

    us = graph_time_us(fn, layers, use_graph=not args.no_graph)
    nbytes = B * ctx * Hkv * D * 2 * 2
    pk = peaks()
    print(json.dumps({"kernel": "attn_decode", "impl": args.impl, "batch": B, "ctx": ctx, "heads": Hq, "kv_heads": Hkv,
                      "head_dim": D, "us": round(us, 2), "GB/s": round(nbytes / us / 1e3, 1),
                      "frac_of_measured_hbm": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3), "copies": layers}))


def bench_skinny(args) -> None:
    dev = "cuda"
    M, N, K = args.rows, args.n, args.k
    epi = {"bf16": kernels.EPI_BF16, "f32": kernels.EPI_F32, "residual": kernels.EPI_ADD_RESIDUAL,
           "swiglu": kernels.EPI_SWIGLU}[args.epilogue]
    wn = 2 * N if epi == kernels.EPI_SWIGLU else N
    copies = max(2, min(args.copies, int(1e9 // (wn * K * 2))))
    ws = [(torch.randn(wn, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    res = torch.randn(M, K, device=dev)
    nw = torch.ones(K, device=dev, dtype=torch.bfloat16)
    ydt = {kernels.EPI_BF16: torch.bfloat16, kernels.EPI_F32: torch.float32, kernels.EPI_ADD_RESIDUAL: torch.float32,
           kernels.EPI_SWIGLU: torch.bfloat16}[epi]
    y = torch.zeros(M, N, device=dev, dtype=ydt)

    def fn(i):
        w = ws[i % copies]
        if args.library:
            torch.mm(x, w.t(), out=yl)
        elif args.norm:
            kernels.gemm_skinny(w, y, epi, M, residual=res, norm_w=nw, eps=1e-5)
        elif args.hand_out:
            kernels.gemm_skinny(w, y, epi, M, x=x, hand_out=(nwn, xw, sums))
        elif args.hand_in:
            kernels.gemm_skinny(w, y, epi, M, x=x, hand_in=sums_in, eps=1e-5)
        else:
            kernels.gemm_skinny(w, y, epi, M, x=x)

    yl = torch.empty(M, wn, device=dev, dtype=torch.bfloat16)
    nwn = torch.ones(N, device=dev, dtype=torch.bfloat16)          # a norm handed over: to the next product ...
    xw, sums = kernels.norm_handover_buffers(8, N, dev)
    sums_in = torch.ones(8, (K + 15) // 16, device=dev)            # ... and from the one before
    us = graph_time_us(fn, copies, use_graph=not args.no_graph)
    nbytes = wn * K * 2
    pk = peaks()
    print(json.dumps({"kernel": "library_mm" if args.library else "gemm_skinny", "rows": M, "n": N, "k": K,
                      "epilogue": args.epilogue, "norm": bool(args.norm), "us": round(us, 2),
                      "GB/s": round(nbytes / us / 1e3, 1),
                      "frac_of_measured_hbm": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3), "copies": copies}))


def bench_gemm_tc(args) -> None:
    dev = "cuda"
    M, N, K = args.rows, args.n, args.k
    epi = {"bf16": kernels.EPI_BF16, "f32": kernels.EPI_F32, "residual": kernels.EPI_ADD_RESIDUAL,
           "swiglu": kernels.EPI_SWIGLU}[args.epilogue]
    wn = 2 * N if epi == kernels.EPI_SWIGLU else N
    copies = max(2, min(args.copies, int(1e9 // (wn * K * 2))))
    ws = [(torch.randn(wn, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    ydt = {kernels.EPI_BF16: torch.bfloat16, kernels.EPI_F32: torch.float32, kernels.EPI_ADD_RESIDUAL: torch.float32,
           kernels.EPI_SWIGLU: torch.bfloat16}[epi]
    y = torch.zeros(M, N, device=dev, dtype=ydt)
    yl = torch.empty(M, wn, device=dev, dtype=torch.bfloat16)

    def fn(i):
        w = ws[i % copies]
        if args.library:
            torch.mm(x, w.t(), out=yl)
        else:
            kernels.gemm_tc(x, w, y, epi, args.tile_n)

    us = graph_time_us(fn, copies, use_graph=not args.no_graph)
    flops = 2.0 * M * wn * K
    pk = peaks()
    print(json.dumps({"kernel": "library_mm" if args.library else "gemm_tc", "rows": M, "n": N, "k": K,
                      "epilogue": args.epilogue, "tile_n": args.tile_n, "us": round(us, 2),
                      "TFLOP/s": round(flops / us / 1e6, 1),
                      "frac_of_measured_bf16": round(flops / us / 1e6 / pk["bf16_tflops"], 3), "copies": copies}))


def bench_gemm_mid(args) -> None:
    dev = "cuda"
    M, N, K = args.rows, args.n, args.k
    epi = {"bf16": kernels.EPI_BF16, "swiglu": kernels.EPI_SWIGLU, "residual": kernels.EPI_ADD_RESIDUAL}[args.epilogue]
    wn = 2 * N if epi == kernels.EPI_SWIGLU else N
    copies = max(2, min(args.copies, int(1e9 // (wn * K * 2))))
    ws = [(torch.randn(wn, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    y = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
    yl = torch.empty(M, wn, device=dev, dtype=torch.bfloat16)
    res = torch.zeros(M, N, device=dev)
    nw = torch.ones(N, device=dev, dtype=torch.bfloat16)
    out = (nw,) + kernels.mid_handover_buffers(N, dev) if args.hand_out else None
    sums_in = torch.ones(M, kernels.mid_sum_columns(K), device=dev) if args.hand_in else None

    def fn(i):
        if args.library:
            torch.mm(x, ws[i % copies].t(), out=yl)
        elif epi == kernels.EPI_ADD_RESIDUAL:
            kernels.gemm_mid(x, ws[i % copies], None, epi, residual=res, hand_out=out)
        else:
            kernels.gemm_mid(x, ws[i % copies], y, epi, hand_in=sums_in, eps=1e-5)

    us = graph_time_us(fn, copies, use_graph=not args.no_graph)
    nbytes = wn * K * 2
    pk = peaks()
    print(json.dumps({"kernel": "library_mm" if args.library else "gemm_mid", "rows": M, "n": N, "k": K,
                      "epilogue": args.epilogue, "us": round(us, 2), "GB/s": round(nbytes / us / 1e3, 1),
                      "frac_of_measured_hbm": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3), "copies": copies}))


def bench_attn_prefill(args) -> None:
    dev = "cuda"
    T, Hq, Hkv, D, ps = args.tokens, args.heads, args.kv_heads, args.head_dim, args.page_size
    npages = (T + ps - 1) // ps + 1
    k = torch.randn(npages, Hkv, ps, D, device=dev).to(torch.bfloat16)
    v = torch.randn(npages, Hkv, ps, D, device=dev).to(torch.bfloat16)
    bt = (torch.arange(npages - 1, dtype=torch.int32) + 1).view(1, -1).to(dev)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev).to(torch.bfloat16)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    rows = kernels.PREFILL_TILE_ROWS
    nt = (T + rows - 1) // rows
    tile_seq = torch.zeros(nt, dtype=torch.int32, device=dev)
    tile_tok = (torch.arange(nt, dtype=torch.int32) * rows).to(dev)
    tile_rows = torch.tensor([min(rows, T - i * rows) for i in range(nt)], dtype=torch.int32, device=dev)
    out = torch.empty(T, Hq * D, device=dev, dtype=torch.bfloat16)

    def fn(i):
        kernels.attn_prefill(qkv, qkv.shape[1], k, v, bt, tile_seq, tile_tok, tile_rows, pos, out, nt, Hq, Hkv, D, ps,
                             0, 1.0 / math.sqrt(D), args.impl)

    # (16 launches to a graph: the launch of the graph itself then hardly counts)
    us = graph_time_us(fn, 16 if T <= 4096 else 2, replays=5, use_graph=not args.no_graph)
    flops = Hq * 4.0 * D * (T * (T + 1) / 2.0)
    pk = peaks()
    print(json.dumps({"kernel": "attn_prefill", "impl": args.impl, "tokens": T, "heads": Hq, "kv_heads": Hkv, "head_dim": D,
                      "us": round(us, 1), "TFLOP/s": round(flops / us / 1e6, 1),
                      "frac_of_measured_bf16": round(flops / us / 1e6 / pk["bf16_tflops"], 4)}))


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="kernel", required=True)
    for name in ("attn_decode", "attn_prefill", "skinny", "gemm_tc", "gemm_mid"):
        p = sub.add_parser(name)
        p.add_argument("--heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=64)
        p.add_argument("--page-size", type=int, default=16)
        p.add_argument("--copies", type=int, default=16, help="distinct copies of the large operand")
        p.add_argument("--no-graph", action="store_true", help="launch eagerly (for profilers)")
        if name == "attn_decode":
            p.add_argument("--batch", type=int, default=8)
            p.add_argument("--ctx", type=int, default=4096)
            p.add_argument("--impl", type=int, default=0,
                           help="0 auto, 1 CUDA cores, 2 one-partition mma.sync kernel, 3 streaming kernel")
        if name == "attn_prefill":
            p.add_argument("--tokens", type=int, default=2048)
            p.add_argument("--impl", type=int, default=0, help="0 auto, 1 CUDA cores, 2 mma.sync kernel, 3 tcgen05 kernel")
        if name == "gemm_tc":
            p.add_argument("--rows", type=int, default=2048)
            p.add_argument("--n", type=int, default=3072)
            p.add_argument("--k", type=int, default=2048)
            p.add_argument("--epilogue", default="bf16", choices=["bf16", "f32", "residual", "swiglu"])
            p.add_argument("--tile-n", type=int, default=0, choices=[0, 128, 256, 512],
                           help="0: the kernel chooses; 128 / 256: one CTA per tile of that width; 512: CTA pairs")
            p.add_argument("--library", action="store_true", help="time the library product instead")
        if name == "skinny":
            p.add_argument("--rows", type=int, default=8)
            p.add_argument("--n", type=int, default=3072)
            p.add_argument("--k", type=int, default=2048)
            p.add_argument("--norm", action="store_true", help="fuse the RMSNorm of a float32 residual")
            p.add_argument("--hand-out", action="store_true", help="with --epilogue residual: hand the next norm over")
            p.add_argument("--hand-in", action="store_true", help="take a norm that was handed over (at most 8 rows)")
            p.add_argument("--epilogue", default="bf16", choices=["bf16", "f32", "residual", "swiglu"])
            p.add_argument("--library", action="store_true", help="time the library product instead")
        if name == "gemm_mid":
            p.add_argument("--rows", type=int, default=64)
            p.add_argument("--n", type=int, default=3072)
            p.add_argument("--k", type=int, default=2048)
            p.add_argument("--epilogue", default="bf16", choices=["bf16", "swiglu", "residual"])
            p.add_argument("--hand-out", action="store_true", help="with --epilogue residual: hand the next norm over")
            p.add_argument("--hand-in", action="store_true", help="take a norm that was handed over")
            p.add_argument("--library", action="store_true", help="time the library product instead")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        print("kernel_bench needs a CUDA device", file=sys.stderr)
        return 1
    {"attn_decode": bench_attn_decode, "attn_prefill": bench_attn_prefill, "skinny": bench_skinny,
     "gemm_tc": bench_gemm_tc, "gemm_mid": bench_gemm_mid}[args.kernel](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
