"""ctypes bindings of the package's CUDA kernels, taking torch tensors.

Every function launches on torch's current stream and raises ``KernelError`` when
the launch fails.  There is no CPU fallback: without a CUDA device or without the
compiled extension these functions raise.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p
from typing import Dict, Optional, Tuple

import torch

from . import build

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


_libs: Dict[Tuple, ctypes.CDLL] = {}


def _lib(name: str, source: str, defines: Optional[Dict[str, object]] = None) -> ctypes.CDLL:
    key = (name, source, tuple(sorted((defines or {}).items())))
    lib = _libs.get(key)
    if lib is None:
        path = build.compile_module(name, source, defines)
        lib = ctypes.CDLL(path)
        _libs[key] = lib
    return lib


def _fn(lib: ctypes.CDLL, name: str, argtypes):
    f = getattr(lib, name)
    if f.argtypes is None:
        f.argtypes = argtypes
        f.restype = c_int
    return f


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


LAUNCHES = 0   # kernels of this package launched (or captured into a graph) so far


def _check(code: int, what: str, n: int = 1) -> None:
    global LAUNCHES
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
    LAUNCHES += n


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported (float32, bfloat16)") from None


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("redline_b200 kernels run on CUDA tensors only; there is no CPU fallback")


# ------------------------------------------------------------------ elementwise

def _ew() -> ctypes.CDLL:
    return _lib("elementwise", "elementwise.cu")


def resolve_ids(ids: torch.Tensor, src: torch.Tensor, sampled: torch.Tensor, n: int) -> None:
    """ids[i] = sampled[src[i]] where src[i] >= 0."""
    _need_cuda(ids, src, sampled)
    f = _fn(_ew(), "rl_resolve_ids", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(src), _ptr(sampled), n, _stream()), "resolve_ids")


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[t] = float(table[ids[t]]); out is the float32 residual stream [T, H]."""
    _need_cuda(ids, table, out)
    f = _fn(_ew(), "rl_embedding", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(ids), _ptr(table), _code(table.dtype), _ptr(out), ids.numel(), table.shape[1],
             table.shape[0], _ptr(status), _stream()), "embedding")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                out: torch.Tensor, eps: float, rows_idx: Optional[torch.Tensor] = None,
                rows: Optional[int] = None) -> None:
    """residual += delta (if given); out = rmsnorm(residual) * weight.  With
    ``rows_idx`` only those rows are normalised (out row i <- row rows_idx[i]) and
    residual is left as it is."""
    _need_cuda(residual, weight, out)
    n = rows if rows is not None else (rows_idx.numel() if rows_idx is not None else residual.shape[0])
    f = _fn(_ew(), "rl_add_rmsnorm", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                       c_int, c_int, c_float, c_void_p])
    if delta is not None and delta.dtype != out.dtype:
        raise KernelError("add_rmsnorm: delta and out must have the same dtype")
    _check(f(_ptr(residual), _ptr(delta), _ptr(weight), _code(weight.dtype), _ptr(out), _code(out.dtype),
             _ptr(rows_idx), n, residual.shape[-1], float(eps), _stream()), "add_rmsnorm")


def add_residual(residual: torch.Tensor, delta: torch.Tensor) -> None:
    _need_cuda(residual, delta)
    f = _fn(_ew(), "rl_add_residual", [c_void_p, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_ptr(residual), _ptr(delta), _code(delta.dtype), delta.numel(), _stream()), "add_residual")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need_cuda(gate_up, out)
    f = _fn(_ew(), "rl_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), _code(out.dtype), gate_up.shape[0], out.shape[1], _stream()), "swiglu")


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    _need_cuda(x, bias)
    f = _fn(_ew(), "rl_add_bias", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _code(x.dtype), _ptr(bias), _code(bias.dtype), x.shape[0], x.shape[1], _stream()), "add_bias")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slots: Optional[torch.Tensor],
                  cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], kcache: Optional[torch.Tensor],
                  vcache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                  page_size: int, status: torch.Tensor, tokens: Optional[int] = None) -> None:
    """Rotates q and k heads of qkv [T, (Hq + 2 Hkv) D] in place and writes k, v to
    the cache slot of each token (``slots`` None or negative: no write; a slot beyond the pool is
    not written and sets bit 4 of ``status``)."""
    _need_cuda(qkv, positions)
    f = _fn(_ew(), "rl_rope_kv_write", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_void_p,
                                         c_void_p])
    max_pos = cos.shape[0] if cos is not None else 2 ** 31 - 1
    num_slots = kcache.shape[0] * page_size if kcache is not None else 0
    _check(f(_ptr(qkv), _code(qkv.dtype), _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin), _ptr(kcache),
             _ptr(vcache), tokens if tokens is not None else qkv.shape[0], num_heads, num_kv_heads, head_dim,
             page_size, max_pos, num_slots, _ptr(status), _stream()), "rope_kv_write")


# ------------------------------------------------------------------------ gemm

def gemm_tn_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: Optional[int] = None) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T, float accumulation on the CUDA cores."""
    _need_cuda(x, w, out)
    f = _fn(_lib("gemm_simt", "gemm_simt.cu"), "rl_gemm_tn_simt",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    M = rows if rows is not None else x.shape[0]
    N, K = w.shape
    if x.shape[1] != K or out.shape[1] != N or x.stride(1) != 1 or out.stride(1) != 1 or not w.is_contiguous():
        raise KernelError(f"gemm_tn_simt: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(f(_ptr(x), _code(x.dtype), _ptr(w), _code(w.dtype), _ptr(out), _code(out.dtype), M, N, K,
             x.stride(0), out.stride(0), _stream()), "gemm_tn_simt")



# ---------------------------------------------------------------- skinny gemm

SKINNY_MAX_ROWS = 16
SKINNY_UNSTAGED_ROWS = 8    # up to here bfloat16 activations are read from global memory, not staged
EPI_BF16, EPI_F32, EPI_ADD_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
_sm_count: Dict[int, int] = {}


def sm_count(device: torch.device) -> int:
    i = device.index if device.index is not None else torch.cuda.current_device()
    if i not in _sm_count:
        _sm_count[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _sm_count[i]


def skinny_ok(rows: int, w: torch.Tensor, x_dtype: torch.dtype) -> bool:
    """Whether gemm_skinny takes this product: few rows, bfloat16 operands, K a multiple of 8."""
    return (rows <= SKINNY_MAX_ROWS and w.dtype == torch.bfloat16 and x_dtype == torch.bfloat16
            and w.shape[1] % 8 == 0 and w.is_contiguous())


def norm_handover_buffers(rows: int, width: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Buffers for a norm handed over between two skinny products: xw [rows, width] bfloat16 and the
    per-tile sums of squares [rows, ceil(width / 16)] float32."""
    return (torch.zeros((rows, width), dtype=torch.bfloat16, device=device),
            torch.zeros((rows, (width + 15) // 16), dtype=torch.float32, device=device))


def gemm_skinny(w: torch.Tensor, y: torch.Tensor, epilogue: int, rows: int, x: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                eps: float = 0.0, rows_idx: Optional[torch.Tensor] = None,
                hand_out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
                hand_in: Optional[torch.Tensor] = None) -> None:
    """y = epilogue(x @ w^T) for at most 16 rows on the tensor cores (csrc/gemm_skinny.cu).

    x given: bfloat16 activations [rows, K].  residual + norm_w given instead: x is
    bfloat16(rmsnorm(residual[rows_idx]) * norm_w) formed inside the kernel.
    epilogue EPI_BF16 / EPI_F32: store into y; EPI_ADD_RESIDUAL: y (float32 stream) += product;
    EPI_SWIGLU: w is [2 N, K] (gate rows, then up rows), y = silu(gate) * up, [rows, N].

    The RMSNorm between a product that ends in ``residual +=`` and the product after it can be handed
    over instead of run as a kernel: with ``hand_out = (next_norm_weight, xw, sums)`` (EPI_ADD_RESIDUAL)
    the product also leaves xw = bfloat16(residual * next_norm_weight) and per-tile sums of residual^2
    (buffers of ``norm_handover_buffers``); the next product is then called with ``x = xw``,
    ``hand_in = sums`` and the norm's ``eps`` (at most 8 rows) and scales its rows by
    rsqrt(sum / K + eps): the same norm, with the rounding to bfloat16 before the scaling."""
    _need_cuda(w, y)
    f = _fn(_lib("gemm_skinny", "gemm_skinny.cu"), "rl_gemm_skinny_handover",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_float, c_int, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
             c_void_p])
    K = w.shape[1]
    N = w.shape[0] // 2 if epilogue == EPI_SWIGLU else w.shape[0]
    norm = residual is not None
    if norm:
        if norm_w is None or residual.dtype != torch.float32 or residual.shape[1] != K or residual.stride(0) != K:
            raise KernelError("gemm_skinny: the fused norm needs a contiguous float32 residual [*, K] and a weight")
        ldx = 0
    else:
        if x is None or x.dtype != torch.bfloat16 or x.shape[1] != K or x.stride(1) != 1:
            raise KernelError("gemm_skinny: x must be bfloat16 [rows, K]")
        ldx = x.stride(0)
    want = {EPI_BF16: torch.bfloat16, EPI_F32: torch.float32, EPI_ADD_RESIDUAL: torch.float32,
            EPI_SWIGLU: torch.bfloat16}[epilogue]
    if y.dtype != want or y.shape[1] != N or y.stride(1) != 1:
        raise KernelError(f"gemm_skinny: output must be {want} [rows, {N}]")
    next_w = xw = ss_out = None
    ldxw = ss_n = 0
    if hand_out is not None:
        next_w, xw, ss_out = hand_out
        tiles = (N + 15) // 16
        if (epilogue != EPI_ADD_RESIDUAL or xw.dtype != torch.bfloat16 or xw.shape[1] != N or xw.stride(1) != 1
                or xw.shape[0] < rows or ss_out.dtype != torch.float32 or not ss_out.is_contiguous()
                or ss_out.shape[1] != tiles or ss_out.shape[0] < rows or next_w.numel() != N
                or next_w.dtype not in (torch.float32, torch.bfloat16)):
            raise KernelError("gemm_skinny: hand_out needs EPI_ADD_RESIDUAL, a norm weight [N], xw bfloat16 "
                              "[rows, N] and sums float32 [rows, ceil(N / 16)]")
        ldxw = xw.stride(0)
    if hand_in is not None:
        if (norm or rows > SKINNY_UNSTAGED_ROWS or epilogue == EPI_ADD_RESIDUAL or hand_in.dtype != torch.float32
                or not hand_in.is_contiguous() or hand_in.shape[0] < rows):
            raise KernelError("gemm_skinny: hand_in needs bfloat16 x of at most 8 rows and sums float32 [rows, n]")
        ss_n = hand_in.shape[1]
    _check(f(_ptr(w), _ptr(x), ldx, _ptr(residual), _ptr(norm_w),
             1 if (norm_w is not None and norm_w.dtype == torch.float32) else 0, _ptr(rows_idx), float(eps),
             1 if norm else 0, _ptr(y), y.stride(0), epilogue, rows, N, K, _ptr(next_w),
             1 if (next_w is not None and next_w.dtype == torch.float32) else 0, _ptr(xw), ldxw, _ptr(ss_out),
             _ptr(hand_in), ss_n, sm_count(w.device), _stream()),
           "gemm_skinny")


# ------------------------------------------------------------ tcgen05 gemm

_tc_status: Dict[int, torch.Tensor] = {}


def tc_status(device: torch.device) -> torch.Tensor:
    """The device word in which the tcgen05 kernels report a wait that ran out (bit 0: gemm_tc,
    bit 2: prompt-portion attention, bit 3: gemm_mid)."""
    i = device.index if device.index is not None else torch.cuda.current_device()
    if i not in _tc_status:
        _tc_status[i] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_status[i]


def gemm_tc_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether gemm_tc takes this product: bfloat16 operands, K a multiple of 8, 16-byte aligned rows."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.is_contiguous()
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, epilogue: int = EPI_BF16, tile_n: int = 0) -> None:
    """y = epilogue(x @ w^T) with tcgen05 tensor cores, TMEM accumulators and TMA loads
    (csrc/gemm_tc.cu): bfloat16 x [M, K], w [N, K] (EPI_SWIGLU: [2 N, K], gate rows then up rows).
    Epilogues as gemm_skinny's.  tile_n: 0 lets the kernel choose its tiling; 128 or 256 force one CTA per
    128-row tile of that width, 512 forces CTA pairs (tcgen05.mma.cta_group::2) on 256 x 256 tiles."""
    _need_cuda(x, w, y)
    f = _fn(_lib("gemm_tc", "gemm_tc.cu"), "rl_gemm_tc",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p])
    M, K = x.shape
    N = w.shape[0] // 2 if epilogue == EPI_SWIGLU else w.shape[0]
    want = {EPI_BF16: torch.bfloat16, EPI_F32: torch.float32, EPI_ADD_RESIDUAL: torch.float32,
            EPI_SWIGLU: torch.bfloat16}[epilogue]
    if w.shape[1] != K or y.dtype != want or y.shape[1] != N or y.stride(1) != 1 or not gemm_tc_ok(x, w):
        raise KernelError(f"gemm_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} y{tuple(y.shape)} {y.dtype}")
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(y), y.stride(0), epilogue, M, N, K, _ptr(tc_status(x.device)),
             sm_count(x.device), tile_n, _stream()), "gemm_tc")


# ------------------------------------------------- tcgen05 gemm for 17 to 128 rows

MID_MAX_ROWS = 128


def gemm_mid_ok(rows: int, x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether gemm_mid takes this product: at most 128 rows, bfloat16 operands, K a multiple of 8,
    16-byte aligned rows."""
    return 0 < rows <= MID_MAX_ROWS and gemm_tc_ok(x, w)


MID_ROUTED_ROWS = 64


def mid_rows(rows: int, *weights: torch.Tensor) -> bool:
    """Whether a part should take ``rows`` rows with gemm_mid products over these weights: at most 64 rows
    (measured on a B200 with 1B-model weights, decode steps of 32 / 48 / 64 sequences: 1.21 / 1.33 / 1.253 ms
    against 1.23 / 1.36 / 1.267 with the library's products and separate norm and SwiGLU kernels; at 96 and
    128 rows 1.72 / 1.91 against 1.67 / 1.90, so those stay with the library), bfloat16 weights with 16-byte
    aligned rows.  ``REDLINE_MID_PRODUCTS=0`` says no (for comparisons)."""
    if rows <= 0 or rows > MID_ROUTED_ROWS or os.environ.get("REDLINE_MID_PRODUCTS", "1") == "0":
        return False
    return all(w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0
               for w in weights)


def mid_handover_buffers(width: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Buffers for a norm handed over between two gemm_mid products: xw [128, width] bfloat16 and the
    per-feature-tile sums of squares [128, ceil(width / 128)] float32."""
    return (torch.zeros((MID_MAX_ROWS, width), dtype=torch.bfloat16, device=device),
            torch.zeros((MID_MAX_ROWS, mid_sum_columns(width)), dtype=torch.float32, device=device))


def mid_sum_columns(width: int) -> int:
    return (width + 127) // 128


def gemm_mid(x: torch.Tensor, w: torch.Tensor, y: Optional[torch.Tensor], epilogue: int = EPI_BF16,
             residual: Optional[torch.Tensor] = None,
             hand_out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
             hand_in: Optional[torch.Tensor] = None, eps: float = 0.0) -> None:
    """epilogue(x @ w^T) for up to 128 rows with tcgen05 tensor cores (csrc/gemm_mid.cu): the weight rows
    are the 128-row operand, the tokens the narrow one, K is split over the CTAs of a thread-block cluster
    and the partial tiles are added through distributed shared memory in a fixed order.  bfloat16 x [M, K],
    w [N, K] (EPI_SWIGLU: [2 N, K], gate rows then up rows).

    EPI_BF16 / EPI_SWIGLU: y bfloat16 [M, N].  EPI_ADD_RESIDUAL: ``residual`` float32 [M, N] += the product
    (y is not used); with ``hand_out = (next_norm_weight, xw, sums)`` (buffers of ``mid_handover_buffers``)
    it also leaves xw = bfloat16(residual * weight) and the sums of residual^2 per feature tile.  A product
    called with ``x = xw``, ``hand_in = sums`` and the norm's ``eps`` scales row m of its result by
    rsqrt(sums[m].sum() / K + eps): the product of the normed stream."""
    lib = _lib("gemm_mid", "gemm_mid.cu")
    f = _fn(lib, "rl_gemm_mid",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
             c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p])
    M, K = x.shape
    gated = epilogue == EPI_SWIGLU
    N = w.shape[0] // 2 if gated else w.shape[0]
    if epilogue not in (EPI_BF16, EPI_SWIGLU, EPI_ADD_RESIDUAL) or w.shape[1] != K or not gemm_mid_ok(M, x, w):
        raise KernelError(f"gemm_mid: shapes x{tuple(x.shape)} w{tuple(w.shape)} epilogue {epilogue}")
    if epilogue == EPI_ADD_RESIDUAL:
        _need_cuda(x, w, residual)
        if (residual is None or residual.dtype != torch.float32 or residual.shape[0] < M or residual.shape[1] != N
                or residual.stride(1) != 1 or residual.stride(0) % 4 != 0):
            raise KernelError("gemm_mid: EPI_ADD_RESIDUAL needs residual float32 [M, N] with 16-byte aligned rows")
    else:
        _need_cuda(x, w, y)
        if (y is None or y.dtype != torch.bfloat16 or y.shape[0] < M or y.shape[1] != N or y.stride(1) != 1
                or hand_out is not None):
            raise KernelError(f"gemm_mid: y must be bfloat16 [M, {N}] (and only EPI_ADD_RESIDUAL hands a norm out)")
    norm_w = xw = sums_out = None
    if hand_out is not None:
        norm_w, xw, sums_out = hand_out
        if (norm_w.numel() != N or norm_w.dtype not in (torch.bfloat16, torch.float32) or not norm_w.is_contiguous()
                or xw.dtype != torch.bfloat16 or xw.shape[0] < M or xw.shape[1] != N or xw.stride(1) != 1
                or sums_out.dtype != torch.float32 or sums_out.shape[0] < M or sums_out.stride(1) != 1
                or sums_out.shape[1] < mid_sum_columns(N)):
            raise KernelError("gemm_mid: hand_out needs a norm weight [N], xw bfloat16 [M, N] and sums float32 "
                              "[M, ceil(N / 128)]")
    if hand_in is not None:
        if hand_in.dtype != torch.float32 or hand_in.shape[0] < M or hand_in.stride(1) != 1 or hand_in.shape[1] < 1:
            raise KernelError("gemm_mid: hand_in must be float32 [M, n]")
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(y) if y is not None else None, y.stride(0) if y is not None else 0,
             epilogue, M, N, K, _ptr(residual) if residual is not None else None,
             residual.stride(0) if residual is not None else 0,
             _ptr(norm_w) if norm_w is not None else None,
             1 if (norm_w is not None and norm_w.dtype == torch.float32) else 0,
             _ptr(xw) if xw is not None else None, xw.stride(0) if xw is not None else 0,
             _ptr(sums_out) if sums_out is not None else None, sums_out.stride(0) if sums_out is not None else 0,
             _ptr(hand_in) if hand_in is not None else None, hand_in.stride(0) if hand_in is not None else 0,
             hand_in.shape[1] if hand_in is not None else 0, float(eps), _ptr(tc_status(x.device)), _stream()),
           "gemm_mid")


# ------------------------------------------------------------------- attention

MAX_HEAD_DIM = 256


def _attn(head_dim: int) -> ctypes.CDLL:
    if head_dim % 16 != 0 or head_dim < 16 or head_dim > MAX_HEAD_DIM:
        raise KernelError(f"attention kernels take head sizes that are multiples of 16 up to "
                          f"{MAX_HEAD_DIM}; got {head_dim}")
    return _lib(f"attention_d{head_dim}", "attention.cu", {"RL_HEAD_DIM": head_dim})


DECODE_PARTITION = 128
PREFILL_TILE_ROWS = 128


def attn_decode(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                block_table: torch.Tensor, items: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                max_parts: int, counters: Optional[torch.Tensor], out: torch.Tensor, nitems: int,
                num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                impl: int = 0) -> None:
    """One query token per item over the paged cache.

    items     int32 [nitems, 4]: (token index of the query, sequence index, context length, 0)
    counters  int32 [nitems * num_kv_heads], zero (the tensor-core kernel needs and keeps them zero)
    impl      0: the best kernel that applies (streaming tensor-core for launches with many partitions,
              one-partition tensor-core, CUDA-core); 1: CUDA-core; 2: one-partition tensor-core or error;
              3: streaming tensor-core or error; 4: one cluster per (item, kv head), partial results
              merged through distributed shared memory (few rows of similar length) or error
    """
    _need_cuda(q, kcache, out)
    f = _fn(_attn(head_dim), "rl_attn_decode",
            [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    need = nitems * num_heads * max_parts
    if part_o.numel() < need * head_dim or part_ml.numel() < need * 2:
        raise KernelError("attn_decode: partition workspace too small")
    if counters is not None and counters.numel() < nitems * num_kv_heads:
        raise KernelError("attn_decode: counter workspace too small")
    if items.data_ptr() % 16 != 0:
        raise KernelError("attn_decode: items must be 16-byte aligned")
    _check(f(_code(q.dtype), _ptr(q), q_stride, _ptr(kcache), _ptr(vcache), _ptr(block_table),
             block_table.shape[1], _ptr(items), _ptr(part_o), _ptr(part_ml), max_parts, _ptr(counters), _ptr(out),
             out.stride(0), nitems, num_heads, num_kv_heads, page_size, window, float(scale), impl, _stream()),
           "attn_decode", 2)


def attn_decode_streams(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                        part_o: torch.Tensor, counters: Optional[torch.Tensor], out: torch.Tensor, max_parts: int,
                        nitems: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                        impl: int = 0) -> bool:
    """Whether ``attn_decode`` with these arguments runs the streaming kernel."""
    if not q.is_cuda or q.dtype != torch.bfloat16 or head_dim not in (64, 128):
        return False
    f = _fn(_attn(head_dim), "rl_attn_decode_streams",
            [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int])
    return bool(f(_code(q.dtype), _ptr(q), q_stride, _ptr(kcache), _ptr(vcache), _ptr(part_o), _ptr(counters),
                  _ptr(out), out.stride(0), max_parts, nitems, num_heads, num_kv_heads, page_size, impl))


_rows_cluster: Dict[Tuple[int, int, int], Tuple[int, int]] = {}
_rows_warps: Dict[int, int] = {}


def attn_decode_rows_cluster(nitems: int, num_kv_heads: int, head_dim: int, device: torch.device) -> Tuple[int, int]:
    """(CTAs per row, clusters resident at once) that ``attn_decode`` with impl 4 would use for a launch of
    ``nitems`` items; (0, 0) if it does not take such a launch (no tensor-core decode kernel for this head
    size).  With fewer resident clusters than rows a cluster takes several rows, one after another."""
    if device.type != "cuda" or head_dim not in (64, 128) or nitems <= 0:
        return 0, 0
    key = (device.index if device.index is not None else torch.cuda.current_device(), nitems * num_kv_heads, head_dim)
    if key not in _rows_cluster:
        f = _fn(_attn(head_dim), "rl_attn_decode_rows_cluster", [c_int, c_int, c_void_p])
        resident = ctypes.c_int(0)
        with torch.cuda.device(key[0]):
            csize = int(f(nitems, num_kv_heads, ctypes.byref(resident)))
        _rows_cluster[key] = (csize, resident.value)
    return _rows_cluster[key]


def attn_decode_rows_pays(nitems: int, num_kv_heads: int, head_dim: int, max_ctx: int, sum_ctx: int, window: int,
                          device: torch.device) -> bool:
    """Whether the decode kernel of one cluster per (item, kv head) (impl 4) is expected to beat the others for
    a launch of ``nitems`` rows of at most ``max_ctx`` and together ``sum_ctx`` keys.  Its time goes with the
    longest row (a row has its cluster's SMs only) times the rows a cluster takes in turn, the streaming
    kernel's with all keys plus the count and merge of its pieces.  The constants are fitted to times on a
    B200 (head size 64, 8 kv heads, batches 1 to 128 at 512 to 8,192 keys): 4.4 us plus, per row a group of
    warps takes, 1.7 us per 32-key sub-block of a warp's run (and 0.7 + 0.25 x turns when it takes more than
    one), but no less than the keys' bytes at 6.2 TB/s; against 8 us plus the keys' bytes at 5.3 TB/s."""
    csize, resident = attn_decode_rows_cluster(nitems, num_kv_heads, head_dim, device)
    if csize <= 0 or resident <= 0 or max_ctx <= 0:
        return False
    if window > 0:
        max_ctx, sum_ctx = min(max_ctx, window), min(sum_ctx, nitems * window)
    if head_dim not in _rows_warps:
        _rows_warps[head_dim] = int(_fn(_attn(head_dim), "rl_attn_decode_rows_warps", [])())
    warps = _rows_warps[head_dim]
    rows = nitems * num_kv_heads
    groups = 1                      # (as the launcher chooses them)
    if rows > resident:
        groups = next((d for d in range(2, warps) if warps % d == 0 and resident * d >= rows), warps)
    turns = (rows + resident * groups - 1) // (resident * groups)
    sub_blocks = (max_ctx + 31) // 32
    per_row = csize * (warps // groups)
    nbytes = sum_ctx * num_kv_heads * head_dim * 4
    per_turn = 1.7 * (head_dim / 64.0) * ((sub_blocks + per_row - 1) // per_row) + (0.7 + 0.25 * turns if turns > 1 else 0.0)
    t_rows = 4.4 + max(turns * per_turn, nbytes / 6.2e6)
    t_stream = 8.0 + nbytes / 5.3e6
    return t_rows < t_stream


def attn_decode_rope_ok(qkv: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                        part_o: torch.Tensor, counters: Optional[torch.Tensor], out: torch.Tensor, max_parts: int,
                        nitems: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                        k_col: int, v_col: int) -> bool:
    """Whether ``attn_decode_rope`` takes a launch with these arguments: bfloat16, head size 64 or 128,
    and one of the two tensor-core decode kernels applies."""
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16 or head_dim not in (64, 128):
        return False
    f = _fn(_attn(head_dim), "rl_attn_decode_rope_ok",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int])
    return bool(f(_ptr(qkv), q_stride, _ptr(kcache), _ptr(vcache), _ptr(part_o), _ptr(counters), _ptr(out),
                  out.stride(0), max_parts, nitems, num_heads, num_kv_heads, page_size, k_col, v_col))


def attn_decode_rope(qkv: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_table: torch.Tensor, items: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                     max_parts: int, counters: torch.Tensor, out: torch.Tensor, nitems: int, num_heads: int,
                     num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                     cos: torch.Tensor, sin: torch.Tensor, k_col: int, v_col: int, status: torch.Tensor,
                     impl: int = 0) -> None:
    """``attn_decode`` by a tensor-core kernel with the rotary encoding and the cache write done in the
    kernel: ``qkv`` holds the UNROTATED rows [q | k | v] of the query tokens (k at column ``k_col``, v at
    ``v_col``); a token's position is its context length - 1; its rotated k and its v are written into the
    cache there.  Only where ``attn_decode_rope_ok`` says so.  impl 0 or 4 as for ``attn_decode``."""
    _need_cuda(qkv, kcache, out)
    f = _fn(_attn(head_dim), "rl_attn_decode_rope",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
             c_void_p, c_int, c_void_p])
    need = nitems * num_heads * max_parts
    if part_o.numel() < need * head_dim or part_ml.numel() < need * 2:
        raise KernelError("attn_decode_rope: partition workspace too small")
    if counters.numel() < nitems * num_kv_heads:
        raise KernelError("attn_decode_rope: counter workspace too small")
    if cos.dtype != torch.float32 or cos.shape[1] != head_dim // 2 or not cos.is_contiguous() or not sin.is_contiguous():
        raise KernelError("attn_decode_rope: cos / sin must be contiguous float32 [positions, head_dim / 2]")
    _check(f(_ptr(qkv), q_stride, _ptr(kcache), _ptr(vcache), _ptr(block_table), block_table.shape[1], _ptr(items),
             _ptr(part_o), _ptr(part_ml), max_parts, _ptr(counters), _ptr(out), out.stride(0), nitems, num_heads,
             num_kv_heads, page_size, window, float(scale), _ptr(cos), _ptr(sin), cos.shape[0], k_col, v_col,
             _ptr(status), impl, _stream()), "attn_decode_rope")


def attn_prefill(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                 block_table: torch.Tensor, tile_seq: torch.Tensor, tile_tok: torch.Tensor,
                 tile_rows: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, tiles: int,
                 num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int,
                 scale: float, impl: int = 0) -> None:
    """Tiles of up to 128 consecutive query tokens of one sequence (tile_seq, tile_tok, tile_rows) over the
    paged cache.  impl 0: the best kernel that applies (bfloat16: tcgen05 at head size 64, mma.sync at
    head size 128; else CUDA cores); 1: CUDA cores; 2: the mma.sync kernel or an error; 3: the tcgen05
    kernel or an error."""
    _need_cuda(q, kcache, out)
    f = _fn(_attn(head_dim), "rl_attn_prefill",
            [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_code(q.dtype), _ptr(q), q_stride, _ptr(kcache), _ptr(vcache), _ptr(block_table),
             block_table.shape[1], _ptr(tile_seq), _ptr(tile_tok), _ptr(tile_rows), _ptr(positions),
             _ptr(out), out.stride(0), tiles, num_heads, num_kv_heads, page_size, window, float(scale), impl,
             _ptr(tc_status(q.device)), _stream()), "attn_prefill")


# -------------------------------------------------------------------- sampling

SAMPLE_CHUNKS = 64


def sample(logits: torch.Tensor, rows: int, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, seed_lo: torch.Tensor, seed_hi: torch.Tensor, position: torch.Tensor,
           out_token: torch.Tensor, out_logprob: Optional[torch.Tensor], stream_id: int = 0,
           scratch: Optional[torch.Tensor] = None) -> None:
    """One token per row of float32 logits.  ``scratch`` (float32, rows * SAMPLE_CHUNKS * 4) lets greedy
    rows use a two-stage arg max over the whole GPU."""
    _need_cuda(logits, out_token)
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    f = _fn(_lib("sampling", "sampling.cu"), "rl_sample",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_uint, c_void_p, c_void_p, c_void_p, c_void_p])
    if scratch is not None and scratch.numel() < rows * SAMPLE_CHUNKS * 4:
        raise KernelError("sample: scratch too small")
    _check(f(_ptr(logits), rows, logits.shape[1], logits.stride(0), _ptr(temperature), _ptr(top_k),
             _ptr(top_p), _ptr(seed_lo), _ptr(seed_hi), _ptr(position), stream_id, _ptr(out_token),
             _ptr(out_logprob), _ptr(scratch), _stream()), "sample", 2 if scratch is not None else 1)


def gather_logprob(logits: torch.Tensor, rows: int, target: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(logits, target, out)
    f = _fn(_lib("sampling", "sampling.cu"), "rl_gather_logprob",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), rows, logits.shape[1], logits.stride(0), _ptr(target), _ptr(out), _stream()),
           "gather_logprob")


def build_all(head_dims=(64, 128), verbose: bool = True) -> None:
    """Compiles every kernel family (attention for the given head sizes) and removes built files of
    these modules that belong to other versions of the sources."""
    built = [
        build.compile_module("elementwise", "elementwise.cu", verbose=verbose),
        build.compile_module("gemm_simt", "gemm_simt.cu", verbose=verbose),
        build.compile_module("gemm_skinny", "gemm_skinny.cu", verbose=verbose),
        build.compile_module("gemm_tc", "gemm_tc.cu", verbose=verbose),
        build.compile_module("gemm_mid", "gemm_mid.cu", verbose=verbose),
        build.compile_module("sampling", "sampling.cu", verbose=verbose),
        build.compile_module("host_core", "host_core.cpp", verbose=verbose),   # host-only: cache manager, batch filler
    ]
    for d in head_dims:
        built.append(build.compile_module(f"attention_d{d}", "attention.cu", {"RL_HEAD_DIM": d}, verbose=verbose))
    build.remove_other_versions(built)
