// y[M, N] = x[M, K] . W[N, K]^T with float accumulation on the CUDA cores.
//
// This is the matrix product of the true 32-bit path (float operands, FFMA only,
// no tensor-core or TF32 mode), and the fallback for any mix of float / bfloat16
// operands (a weight stored in 32-bit next to bfloat16 activations, float logits
// from bfloat16 operands at small sizes).  Any M, N, K.  The k loop runs in a
// fixed order for every output element, so a row's result does not depend on how
// many other rows are in the batch.
#include "common.cuh"

namespace rl {

constexpr int kTM = 64, kTN = 64, kTK = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_tn_simt_kernel(const TA* __restrict__ x, const TW* __restrict__ w, TC* __restrict__ y, int M,
                    int N, int K, int ldx, int ldy) {
  pdl_launch();
  pdl_wait();
  __shared__ float xs[kTK][kTM + 4];
  __shared__ float ws[kTK][kTN + 4];
  const int m0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;  // loader: row 0..63, k offset 0,4,8,12
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kTK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int m = m0 + lr, n = n0 + lr;
      xs[lk + e][lr] = (m < M && k < K) ? to_float(x[static_cast<size_t>(m) * ldx + k]) : 0.f;
      ws[lk + e][lr] = (n < N && k < K) ? to_float(w[static_cast<size_t>(n) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) y[static_cast<size_t>(m) * ldy + n] = from_float<TC>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW, typename TC>
int launch(const void* x, const void* w, void* y, int M, int N, int K, int ldx, int ldy,
           cudaStream_t stream) {
  dim3 grid((N + kTN - 1) / kTN, (M + kTM - 1) / kTM);
  launch_kernel(gemm_tn_simt_kernel<TA, TW, TC>, dim3(grid), dim3(256), 0, stream, 
      static_cast<const TA*>(x), static_cast<const TW*>(w), static_cast<TC*>(y), M, N, K, ldx, ldy);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace rl

using namespace rl;

extern "C" {

// dtypes: 0 = float32, 1 = bfloat16.  ldx / ldy: row strides of x and y in elements.
int rl_gemm_tn_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype,
                    int M, int N, int K, int ldx, int ldy, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  const int code = x_dtype * 4 + w_dtype * 2 + y_dtype;
  switch (code) {
    case 0: return launch<float, float, float>(x, w, y, M, N, K, ldx, ldy, stream);
    case 1: return launch<float, float, bf16>(x, w, y, M, N, K, ldx, ldy, stream);
    case 2: return launch<float, bf16, float>(x, w, y, M, N, K, ldx, ldy, stream);
    case 3: return launch<float, bf16, bf16>(x, w, y, M, N, K, ldx, ldy, stream);
    case 4: return launch<bf16, float, float>(x, w, y, M, N, K, ldx, ldy, stream);
    case 5: return launch<bf16, float, bf16>(x, w, y, M, N, K, ldx, ldy, stream);
    case 6: return launch<bf16, bf16, float>(x, w, y, M, N, K, ldx, ldy, stream);
    case 7: return launch<bf16, bf16, bf16>(x, w, y, M, N, K, ldx, ldy, stream);
  }
  return static_cast<int>(cudaErrorInvalidValue);
}

}  // extern "C"
