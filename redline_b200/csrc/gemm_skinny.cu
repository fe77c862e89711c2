// y[M, N] = x[M, K] . W[N, K]^T for few rows (M <= 16, a small decode batch), bfloat16
// operands, float accumulation on the tensor cores.
//
// A decode step reads every weight once and does little arithmetic, so the kernel is
// built around the weight stream: the weights are the MMA's 16-row operand and are
// loaded straight from global memory in 16-byte pieces (no shared-memory stage), the
// few activation rows are the 8-wide operand and sit in shared memory.  One CTA owns
// 16 output features (32 for the gated product: 16 gate rows and their 16 up rows) and
// its warps split K in interleaved 64-wide blocks; partial sums meet in shared memory
// and are added in warp order, so a row's result does not depend on how many other rows
// are in the batch, and not on the run.
//
// Fused around the product:
//   prologue  NORM: x = bfloat16(rmsnorm(residual[rows]) * norm_weight), computed in the
//             CTA from the float32 residual stream (optionally gathered by row index)
//   epilogue  bfloat16 store | float32 store (logits) | residual += y (float32) |
//             SiLU-gated product silu(gate) * up
//
// mma.sync.m16n8k16 is used rather than tcgen05: with at most 16 rows the product is
// bound by the weight stream, a 128-row UMMA tile would be 1/16 full, and mma.sync can
// take its weight fragments from registers without a shared-memory round trip.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rl {

typedef __nv_bfloat16 bf16;

enum Epilogue { kStoreBf16 = 0, kStoreF32 = 1, kAddResidual = 2, kSwiglu = 3 };

struct SkinnyArgs {
  const bf16* w;          // [N, K] (for kSwiglu: [2 * N, K], gate rows then up rows)
  const bf16* x;          // [M, ldx] bfloat16 activations        (NORM = false)
  const float* residual;  // [*, K] float32 residual stream       (NORM = true)
  const void* norm_w;     // [K] norm weight                      (NORM = true)
  int norm_w_f32;         // norm weight is float32 (else bfloat16)
  const int32_t* rows_idx;  // optional: row m of x is residual[rows_idx[m]]
  float eps;
  void* y;                // output (bf16 / float), or the residual stream for kAddResidual
  int M, N, K, ldx, ldy;
  int row_tiles;          // 16-row tiles per CTA (run one after another)
};

__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

constexpr int kSB = 128;  // k per warp iteration (a "super-block": two 64-wide MMA blocks)

// The weights of one super-block as a thread holds them: rows g and g + 8 of the tile,
// four 16-byte pieces each (k = sb * 128 + q * 32 + t * 8 .. + 8, q = 0..3).
struct WFrag {
  uint4 lo[4], hi[4];
};

__device__ __forceinline__ void load_wfrag(WFrag& f, const bf16* w_lo, const bf16* w_hi, int k_first, int K) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int k = k_first + q * 32;
    const bool ok = k < K;               // K is a multiple of 8: a 16-byte piece is in or out whole
    f.lo[q] = ok ? ldg_stream(w_lo + k) : make_uint4(0, 0, 0, 0);
    f.hi[q] = ok ? ldg_stream(w_hi + k) : make_uint4(0, 0, 0, 0);
  }
}

// MT: token rows padded to 8 or 16; WARPS: warps per CTA; EPI: epilogue; NORM: fused norm.
template <int MT, int WARPS, int EPI, bool NORM>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const SkinnyArgs a, int kc) {
  constexpr bool GATED = (EPI == kSwiglu);
  constexpr int NG = MT / 8;           // 8-token groups
  // the gated product has two weight streams (gate rows, up rows): the first half of the
  // warps takes one, the second half the other, and each half splits K among its KW warps
  constexpr int KW = GATED ? WARPS / 2 : WARPS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lds = kc + 32;             // row stride of the staged activations (elements): 64 B off a
                                       // multiple of 128 B, so the 16-byte fragment reads do not collide
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  float* red = reinterpret_cast<float*>(smem_raw);   // reused after the k loop
  __shared__ float inv_rms[MT];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int M = a.M, K = a.K;
  const int kw = warp % KW, stream = warp / KW;
  const int nsb = (K + kSB - 1) / kSB;       // super-blocks in K; warp kw takes kw, kw + KW, ...

  // The first weights are asked for before anything else: they do not depend on the
  // activations, and their latency then hides behind the norm and the staging.
  WFrag cur, nxt;
  const bf16 *w_lo, *w_hi;
  auto set_rows = [&](int n0) {
    const int r_lo = min(n0 + g, a.N - 1), r_hi = min(n0 + g + 8, a.N - 1);   // clamped; stores are predicated
    w_lo = a.w + static_cast<size_t>(stream * a.N + r_lo) * K;
    w_hi = a.w + static_cast<size_t>(stream * a.N + r_hi) * K;
  };
  const int tile0 = blockIdx.x * a.row_tiles;
  set_rows(tile0 * 16);
  load_wfrag(cur, w_lo, w_hi, kw * kSB + t * 8, K);

  if (NORM) {
    for (int m = warp; m < MT; m += WARPS) {
      float ss = 0.f;
      if (m < M) {
        const float* r = a.residual + static_cast<size_t>(a.rows_idx ? a.rows_idx[m] : m) * K;
        for (int k = lane * 4; k < K; k += 128) {
          const float4 v = *reinterpret_cast<const float4*>(r + k);
          ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) inv_rms[m] = rsqrtf(ss / static_cast<float>(K) + a.eps);
    }
    __syncthreads();
  }

  for (int rt = 0; rt < a.row_tiles; ++rt) {
    const int n0 = (tile0 + rt) * 16;
    if (n0 >= a.N) break;
    const bool more_tiles = (rt + 1 < a.row_tiles) && (n0 + 16 < a.N);
    float acc[NG][4];
#pragma unroll
    for (int j = 0; j < NG; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

    for (int k0 = 0; k0 < K; k0 += kc) {
      const int kn = min(kc, K - k0);
      __syncthreads();   // the previous chunk (or the previous tile's reduction) is done with smem
      // ---- stage x[:, k0 : k0 + kn] as bfloat16, zero beyond M and beyond kn (to a multiple of 128)
      const int kpad = (kn + kSB - 1) / kSB * kSB;
      for (int i = tid; i < MT * (kpad / 8); i += WARPS * 32) {
        const int m = i / (kpad / 8), c = (i - m * (kpad / 8)) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < M && c < kn) {
          if (NORM) {
            const float* r = a.residual + static_cast<size_t>(a.rows_idx ? a.rows_idx[m] : m) * K + k0 + c;
            const float4 p = *reinterpret_cast<const float4*>(r), q = *reinterpret_cast<const float4*>(r + 4);
            float wv[8];
            if (a.norm_w_f32) {
              const float* nw = static_cast<const float*>(a.norm_w) + k0 + c;
#pragma unroll
              for (int e = 0; e < 8; ++e) wv[e] = nw[e];
            } else {
              const uint4 nw = *reinterpret_cast<const uint4*>(static_cast<const bf16*>(a.norm_w) + k0 + c);
              const uint32_t ww[4] = {nw.x, nw.y, nw.z, nw.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                wv[2 * e] = __uint_as_float(ww[e] << 16);
                wv[2 * e + 1] = __uint_as_float(ww[e] & 0xFFFF0000u);
              }
            }
            const float s = inv_rms[m];
            const float f[8] = {p.x, p.y, p.z, p.w, q.x, q.y, q.z, q.w};
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * e] * s * wv[2 * e], f[2 * e + 1] * s * wv[2 * e + 1]);
              o[e] = *reinterpret_cast<const uint32_t*>(&h);
            }
            v = make_uint4(o[0], o[1], o[2], o[3]);
          } else {
            v = *reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(m) * a.ldx + k0 + c);
          }
        }
        *reinterpret_cast<uint4*>(xs + m * lds + c) = v;
      }
      __syncthreads();
      // ---- the weight stream: warp kw takes super-blocks kw, kw + KW, ... ; the next one is
      //      in flight while this one is multiplied
      const int sb_end = min((k0 + kc) / kSB, nsb);
      for (int sb = k0 / kSB + kw; sb < sb_end; sb += KW) {
        const int sbn = sb + KW;
        if (sbn < nsb) {
          load_wfrag(nxt, w_lo, w_hi, sbn * kSB + t * 8, K);
        } else if (more_tiles) {         // this tile's stream is done: start the next tile's
          set_rows(n0 + 16);
          load_wfrag(nxt, w_lo, w_hi, kw * kSB + t * 8, K);
        }
        const int kb = sb * kSB - k0;    // within the staged chunk
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int j = 0; j < NG; ++j) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xs + (j * 8 + g) * lds + kb + q * 32 + t * 8);
            mma_bf16(acc[j], cur.lo[q].x, cur.hi[q].x, cur.lo[q].y, cur.hi[q].y, xv.x, xv.y);
            mma_bf16(acc[j], cur.lo[q].z, cur.hi[q].z, cur.lo[q].w, cur.hi[q].w, xv.z, xv.w);
          }
        }
        cur = nxt;
      }
    }
    // a warp that had no super-block in this tile (K shorter than WARPS super-blocks) still holds the
    // tile's first fragment in `cur`: fetch the next tile's instead
    if (kw >= nsb && more_tiles) {
      set_rows(n0 + 16);
      load_wfrag(cur, w_lo, w_hi, kw * kSB + t * 8, K);
    }
    // ---- partial sums of the warps meet in shared memory: red[warp][16][MT]
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NG; ++j) {
      float* r = red + (warp * 16) * MT;
      const int col = j * 8 + t * 2;
      r[g * MT + col] = acc[j][0];
      r[g * MT + col + 1] = acc[j][1];
      r[(g + 8) * MT + col] = acc[j][2];
      r[(g + 8) * MT + col + 1] = acc[j][3];
    }
    __syncthreads();
    for (int i = tid; i < 16 * MT; i += WARPS * 32) {
      // consecutive threads take consecutive features of one token: coalesced stores
      const int m = i / 16, f = i - m * 16;
      const int n = n0 + f;
      if (m >= M || n >= a.N) continue;
      float v = 0.f, u = 0.f;
#pragma unroll
      for (int w = 0; w < KW; ++w) {
        v += red[(w * 16 + f) * MT + m];
        if (GATED) u += red[((KW + w) * 16 + f) * MT + m];
      }
      const size_t o = static_cast<size_t>(m) * a.ldy + n;
      if (EPI == kStoreBf16) {
        static_cast<bf16*>(a.y)[o] = __float2bfloat16_rn(v);
      } else if (EPI == kStoreF32) {
        static_cast<float*>(a.y)[o] = v;
      } else if (EPI == kAddResidual) {
        // the unfused path rounds the product to bfloat16 before the add; so does this one
        static_cast<float*>(a.y)[o] += __bfloat162float(__float2bfloat16_rn(v));
      } else {
        const float gt = __bfloat162float(__float2bfloat16_rn(v)), up = __bfloat162float(__float2bfloat16_rn(u));
        static_cast<bf16*>(a.y)[o] = __float2bfloat16_rn(gt / (1.f + expf(-gt)) * up);
      }
    }
  }
}

template <int MT, int WARPS, int EPI, bool NORM>
int launch_one(const SkinnyArgs& a, int ctas, cudaStream_t stream) {
  // K is staged in equal chunks that are multiples of 64 * WARPS, so that warp w always
  // takes the global 128-wide super-blocks w, w + WARPS, ...: the order of a row's sums does not
  // depend on the chunking, hence not on how many rows the batch has.
  constexpr int kUnit = kSB * (EPI == kSwiglu ? WARPS / 2 : WARPS);
  const int kunits = (a.K + kUnit - 1) / kUnit;
  int max_units = (98304 / (MT * 2) - 32) / kUnit;
  if (max_units < 1) max_units = 1;
  const int chunks = (kunits + max_units - 1) / max_units;
  const int kc = (kunits + chunks - 1) / chunks * kUnit;
  const size_t xbytes = static_cast<size_t>(MT) * (kc + 32) * 2;
  const size_t rbytes = static_cast<size_t>(WARPS) * 16 * MT * 4;
  const size_t smem = xbytes > rbytes ? xbytes : rbytes;
  static size_t set_for = 0;
  if (smem > set_for) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<MT, WARPS, EPI, NORM>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    set_for = smem;
  }
  gemm_skinny_kernel<MT, WARPS, EPI, NORM><<<ctas, WARPS * 32, smem, stream>>>(a, kc);
  return static_cast<int>(cudaGetLastError());
}

template <int EPI, bool NORM>
int launch_mt(const SkinnyArgs& a, int ctas, bool wide, cudaStream_t stream) {
  if (a.M <= 8) return wide ? launch_one<8, 16, EPI, NORM>(a, ctas, stream) : launch_one<8, 8, EPI, NORM>(a, ctas, stream);
  return wide ? launch_one<16, 16, EPI, NORM>(a, ctas, stream) : launch_one<16, 8, EPI, NORM>(a, ctas, stream);
}

}  // namespace rl

using namespace rl;

extern "C" {

int rl_gemm_skinny_max_rows() { return 16; }

// epilogue: 0 bf16 store, 1 float32 store, 2 residual += y, 3 SiLU-gated product (w holds
// N gate rows then N up rows).  norm != 0: x is rmsnorm(residual[rows_idx]) * norm_w.
// Requirements: M <= 16, K a multiple of 8, 16-byte aligned rows.  Returns cudaErrorInvalidValue
// otherwise (the caller then takes another path).
int rl_gemm_skinny(const void* w, const void* x, int ldx, const float* residual, const void* norm_w,
                   int norm_w_f32, const int32_t* rows_idx, float eps, int norm, void* y, int ldy,
                   int epilogue, int M, int N, int K, int sm_count, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K % 8 != 0 || (!norm && ldx % 8 != 0)) return static_cast<int>(cudaErrorInvalidValue);
  SkinnyArgs a;
  a.w = static_cast<const bf16*>(w);
  a.x = static_cast<const bf16*>(x);
  a.residual = residual;
  a.norm_w = norm_w;
  a.norm_w_f32 = norm_w_f32;
  a.rows_idx = rows_idx;
  a.eps = eps;
  a.y = y;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldx = ldx;
  a.ldy = ldy;
  const int tiles = (N + 15) / 16;
  // no more tiles than SMs: one CTA of 16 warps per tile (one CTA fits an SM); more: CTAs of
  // 8 warps (two fit an SM), several tiles per CTA when there are many so that the prologue
  // (staging, norm) is shared
  const bool wide = tiles <= sm_count;
  int rt = 1;
  if (!wide) {
    rt = tiles / (4 * sm_count);
    if (rt < 1) rt = 1;
    if (rt > 8) rt = 8;
  }
  a.row_tiles = rt;
  const int ctas = (tiles + rt - 1) / rt;
  if (norm) {
    switch (epilogue) {
      case kStoreBf16: return launch_mt<kStoreBf16, true>(a, ctas, wide, stream);
      case kStoreF32: return launch_mt<kStoreF32, true>(a, ctas, wide, stream);
      case kSwiglu: return launch_mt<kSwiglu, true>(a, ctas, wide, stream);
    }
  } else {
    switch (epilogue) {
      case kStoreBf16: return launch_mt<kStoreBf16, false>(a, ctas, wide, stream);
      case kStoreF32: return launch_mt<kStoreF32, false>(a, ctas, wide, stream);
      case kAddResidual: return launch_mt<kAddResidual, false>(a, ctas, wide, stream);
      case kSwiglu: return launch_mt<kSwiglu, false>(a, ctas, wide, stream);
    }
  }
  return static_cast<int>(cudaErrorInvalidValue);
}

}  // extern "C"
