"""y = x W^T for the linear layers.

* bfloat16 x, bfloat16 W, at most 16 rows (a small decode batch): the package's own
  tensor-core kernel built around the weight stream (csrc/gemm_skinny.cu).
* bfloat16 x, bfloat16 W, more rows: a library matrix product (cuBLAS through torch), as the
  reference uses cuBLASLt for its half-precision products
  (src/cuda/gemm/cublaslt_gemm.cpp:97-111); float32 output for the logits.
* anything with a float32 operand: the package's own CUDA-core kernel, which is a
  true 32-bit product (no TF32, no tensor cores), also for a weight that the
  checkpoint stores in 32-bit next to bfloat16 activations.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import kernels

_mm_f32_out: Optional[bool] = None


def _bf16_mm_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """out (float32) = x (bf16) @ w^T (bf16) with the library, if this torch can."""
    global _mm_f32_out
    if _mm_f32_out is False:
        return False
    try:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        _mm_f32_out = True
        return True
    except (TypeError, RuntimeError):
        if _mm_f32_out is None:
            _mm_f32_out = False
            return False
        raise


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[T, N] = x[T, K] @ w[N, K]^T.  x and out may be row-strided views."""
    if not x.is_cuda:
        raise kernels.KernelError("linear runs on CUDA tensors only; there is no CPU fallback")
    if x.shape[0] == 0:
        return out
    # (a very tall matrix, the head over a large vocabulary, runs at the bandwidth limit in the library)
    if (kernels.skinny_ok(x.shape[0], w, x.dtype) and w.shape[0] <= 32768 and out.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.stride(1) == 1):
        kernels.gemm_skinny(w, out, kernels.EPI_BF16 if out.dtype == torch.bfloat16 else kernels.EPI_F32,
                            x.shape[0], x=x)
        return out
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if out.dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
            return out
        if out.is_contiguous() and _bf16_mm_f32(x, w, out):
            return out
    kernels.gemm_tn_simt(x, w, out)
    return out
