// y[M, N] = x[M, K] . W[N, K]^T for few rows (M <= 16, a small decode batch), bfloat16
// operands, float accumulation on the tensor cores.
//
// A decode step reads every weight once and does little arithmetic, so the kernel is
// built around the weight stream: the weights are the MMA's 16-row operand and are
// loaded straight from global memory in 16-byte pieces (no shared-memory stage), two
// 128-wide super-blocks per warp held in registers and refilled in place two steps
// ahead.  The few activation rows are the 8-wide operand: with bfloat16 activations of up
// to 8 rows they too come from global memory, with the weights of the same k; otherwise
// (a fused norm of the float32 stream, or 9 to 16 rows) they are staged in shared memory.
// One CTA owns 16 output features (32 for the gated product: 16 gate rows and their 16 up
// rows) and its warps split K in interleaved 128-wide blocks; partial sums meet in shared
// memory and are added in warp order, so a row's result does not depend on how many other
// rows are in the batch, and not on the run.
//
// Fused around the product:
//   prologue  NORM: x = bfloat16(rmsnorm(residual[rows]) * norm_weight), computed in the
//             CTA from the float32 residual stream (optionally gathered by row index)
//   epilogue  bfloat16 store | float32 store (logits) | residual += y (float32) |
//             SiLU-gated product silu(gate) * up
//   between two products: the RMSNorm after a `residual += y` handed over instead of run as a
//             kernel: the first product also leaves bfloat16(residual * norm_weight) and per-tile
//             sums of residual^2, the second takes that as its x and scales its rows by
//             rsqrt(sum / K + eps)
// What an epilogue needs from global memory (the residual values, the norm weights, the partial
// sums) is copied into shared memory at the kernel's start, so that no round trip is left for the
// kernel's end and no register is held across the k loop, which has none to spare.
//
// mma.sync.m16n8k16 is used rather than tcgen05: with at most 16 rows the product is
// bound by the weight stream, a 128-row UMMA tile would be 1/16 full, and mma.sync can
// take its weight fragments from registers without a shared-memory round trip.
#include "common.cuh"

namespace rl {

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
  // The norm after a `residual += y` handed over to the next product (kAddResidual only; xw == nullptr:
  // not done): xw[m, n] = bfloat16(residual[m, n] * next_w[n]) and, per row and 16-feature tile,
  // ss_out[m * tiles + tile] = the tile's sum of residual^2 (tiles = ceil(N / 16)).
  const void* next_w;
  int next_w_f32;
  bf16* xw;
  int ldxw;
  float* ss_out;
  // ... and taken over (unstaged bfloat16 x of up to 8 rows only; ss_in == nullptr: x is used as it is):
  // x is such an xw, and row m of the product is scaled by rsqrt(sum(ss_in[m, 0 : ss_n]) / K + eps).
  const float* ss_in;
  int ss_n;
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

// 4 bytes from global to shared memory without a register in between (cp.async), and the wait for all
// such copies of the thread
__device__ __forceinline__ void cp_async4(const void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))), "l"(gmem));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

constexpr int kSB = 128;  // k per warp iteration (a "super-block": two 64-wide MMA blocks)

// The weights of one super-block as a thread holds them: rows g and g + 8 of the tile,
// four 16-byte pieces each (k = sb * 128 + q * 32 + t * 8 .. + 8, q = 0..3).
struct WFrag {
  uint4 lo[4], hi[4];
  uint4 x[4];     // XG only: the activations of the same k, row g of the batch
};

// The epilogue `residual += y` that also hands the next norm over (see SkinnyArgs).  A function of its
// own that is not inlined: the kernels with 16 warps have no register to spare in their k loop, and
// whatever this needs must not be kept alive across that loop.  red: the warps' partial sums
// [WARPS][16][MT] in shared memory; the CTA's round begins at feature cta_n0.
template <int MT, int WARPS, int KW>
// early: the round's residual values [TPC * 16 * MT] and norm weights [TPC * 16] staged in shared
// memory at the kernel's start (nullptr: read from global memory here).
__device__ __noinline__ void hand_over_epilogue(const float* red, const float* early, float* y, int ldy, const void* next_w,
                                                int next_w_f32, bf16* xw, int ldxw, float* ss_out, int M, int N,
                                                int cta_n0, int tid) {
  constexpr int TPC = WARPS / KW;
  for (int i = tid; i < TPC * 16 * MT; i += WARPS * 32) {     // a multiple of 32: whole warps
    const int m = i / (TPC * 16), ft = i - m * (TPC * 16);
    const int tl = ft >> 4, f = ft & 15;
    const int n = cta_n0 + ft;
    const bool live = m < M && n < N;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < KW; ++w) v += red[((tl * KW + w) * 16 + f) * MT + m];
    float r = 0.f;
    if (live) {
      const size_t o = static_cast<size_t>(m) * ldy + n;
      r = (early ? early[i] : y[o]) + __bfloat162float(__float2bfloat16_rn(v));
      y[o] = r;
      const float nw = early         ? early[TPC * 16 * MT + ft]
                       : next_w_f32 ? static_cast<const float*>(next_w)[n]
                                    : __bfloat162float(static_cast<const bf16*>(next_w)[n]);
      xw[static_cast<size_t>(m) * ldxw + n] = __float2bfloat16_rn(r * nw);
    }
    float sq = r * r;          // the 16 lanes of a tile (one row m) add up in a fixed order
#pragma unroll
    for (int x = 8; x > 0; x >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, x);
    if (f == 0 && m < M && cta_n0 + tl * 16 < N) ss_out[static_cast<size_t>(m) * ((N + 15) / 16) + (cta_n0 >> 4) + tl] = sq;
  }
}

// MT: token rows padded to 8 or 16; WARPS: warps per CTA; EPI: epilogue; NORM: fused norm.
// MT: token rows padded to 8 or 16; WARPS: warps per CTA; KW: warps that split the K of one
// 16-row weight stream; EPI: epilogue; NORM: fused norm.  The CTA's WARPS / KW groups of warps
// take different streams at the same time: 16-row tiles next to each other and, for the gated
// product, the gate rows and the up rows of a tile.
template <int MT, int WARPS, int KW, int EPI, bool NORM>
__global__ void __launch_bounds__(WARPS * 32, WARPS <= 8 ? 2 : 1)     // (at most 128 registers: two CTAs of 8 warps per SM)
gemm_skinny_kernel(const SkinnyArgs a, int kc, int extra_off) {
  constexpr bool GATED = (EPI == kSwiglu);
  constexpr int NG = MT / 8;                    // 8-token groups
  // XG: with bfloat16 activations and at most 8 rows the activations are not staged in shared memory
  // at all: a thread's activation fragment of a super-block (16 bytes per piece, row g of the batch)
  // comes from global memory (L2) together with the weights of the same k, two steps ahead, and the
  // k loop has no barriers.  The sums are taken in the same order as with staging.
  constexpr bool XG = !NORM && MT == 8;
  constexpr int STREAMS = GATED ? 2 : 1;        // weight streams per tile (gate rows, up rows)
  constexpr int TPC = WARPS / KW / STREAMS;     // tiles a CTA works on at the same time
  static_assert(TPC >= 1 && TPC * KW * STREAMS == WARPS, "bad warp split");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lds = kc + 32;             // row stride of the staged activations (elements): 64 B off a
                                       // multiple of 128 B, so the 16-byte fragment reads do not collide
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  float* red = reinterpret_cast<float*>(smem_raw);   // reused after the k loop
  // Behind both: what the epilogue of the CTA's first round needs from global memory, copied there at the
  // kernel's start so that no round trip is left for the kernel's end (and no register is held for it
  // across the k loop): for `residual +=` the residual values [TPC * 16 * MT] and, with a norm handed
  // over, its weights [TPC * 16]; for a norm taken over, the partial sums [M][ss_n].
  float* early = reinterpret_cast<float*>(smem_raw + extra_off);
  __shared__ float inv_rms[MT];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int M = a.M, K = a.K;
  const int kw = warp % KW, grp = warp / KW;
  const int stream = grp % STREAMS, tile_in_cta = grp / STREAMS;
  const int nsb = (K + kSB - 1) / kSB;       // super-blocks in K; warp kw takes kw, kw + KW, ...

  // The weight stream of a warp is the sequence of its super-blocks over all the tiles of the CTA:
  // (tile 0: kw, kw + KW, ...), (tile 1: kw, ...), ...  Two super-blocks are held in registers, fa
  // for the even steps of the sequence and fb for the odd ones; as soon as a 16-byte piece has been
  // multiplied, the piece in the same place two steps on is asked for into the same registers, so
  // nearly two super-blocks (8 KB per warp) are in flight all the time.  The first two are asked for
  // before anything else: they do not depend on the activations, and their latency then hides behind
  // the wait for the kernels before this one, the norm and the staging.
  WFrag fa, fb;
  const bf16 *w_lo, *w_hi;
  auto set_rows = [&](int n0) {
    const int r_lo = min(n0 + g, a.N - 1), r_hi = min(n0 + g + 8, a.N - 1);   // clamped; stores are predicated
    w_lo = a.w + static_cast<size_t>(stream * a.N + r_lo) * K;
    w_hi = a.w + static_cast<size_t>(stream * a.N + r_hi) * K;
  };
  const int tile0 = blockIdx.x * a.row_tiles * TPC + tile_in_cta;   // then tile0 + TPC, ... (row_tiles rounds)
  // the load cursor: round l_rt of the CTA, super-block l_sb; l_ok: there is such a super-block
  int l_rt = 0, l_sb = kw;
  bool l_ok = kw < nsb && blockIdx.x * a.row_tiles * TPC * 16 < a.N;
  set_rows(tile0 * 16);
  auto load_piece = [&](uint4& lo, uint4& hi, int q) {
    const int k = l_sb * kSB + q * 32 + t * 8;
    const bool ok = l_ok && k < K;        // K is a multiple of 8: a 16-byte piece is in or out whole
    lo = ok ? ldg_stream(w_lo + k) : make_uint4(0, 0, 0, 0);
    hi = ok ? ldg_stream(w_hi + k) : make_uint4(0, 0, 0, 0);
  };
  auto load_x = [&](uint4& xv, int q) {          // (after the wait on the kernels before: they wrote x)
    const int k = l_sb * kSB + q * 32 + t * 8;
    const bool ok = l_ok && k < K && g < M;
    xv = ok ? *reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(g) * a.ldx + k) : make_uint4(0, 0, 0, 0);
  };
  auto load_advance = [&]() {
    l_sb += KW;
    if (l_sb >= nsb) {                     // on to the next round of the CTA
      l_sb = kw;
      ++l_rt;
      l_ok = l_ok && l_rt < a.row_tiles && (blockIdx.x * a.row_tiles + l_rt) * TPC * 16 < a.N;
      if (l_ok) set_rows((tile0 + l_rt * TPC) * 16);
    }
  };
  pdl_launch();
  const int sb0 = l_sb;
  const bool ok0 = l_ok;
#pragma unroll
  for (int q = 0; q < 4; ++q) load_piece(fa.lo[q], fa.hi[q], q);
  load_advance();
  const int sb1 = l_sb;
  const bool ok1 = l_ok;
#pragma unroll
  for (int q = 0; q < 4; ++q) load_piece(fb.lo[q], fb.hi[q], q);
  load_advance();
  int step = 0;       // super-blocks this warp has multiplied
  if (EPI == kAddResidual && a.xw != nullptr && tid < TPC * 16) {
    // the weights of the norm that is handed over (they do not depend on the kernels before this one)
    const int n = blockIdx.x * a.row_tiles * TPC * 16 + tid;
    if (n < a.N)
      early[TPC * 16 * MT + tid] = a.next_w_f32 ? static_cast<const float*>(a.next_w)[n]
                                                : __bfloat162float(static_cast<const bf16*>(a.next_w)[n]);
  }
  pdl_wait();   // everything below reads what earlier kernels of the step wrote
  if (EPI == kAddResidual) {
    const int n00 = blockIdx.x * a.row_tiles * TPC * 16;
    for (int i = tid; i < TPC * 16 * MT; i += WARPS * 32) {
      const int m = i / (TPC * 16), n = n00 + (i - m * (TPC * 16));
      if (m < M && n < a.N) cp_async4(early + i, static_cast<const float*>(a.y) + static_cast<size_t>(m) * a.ldy + n);
    }
  }
  if (XG) {     // the activations of the first two steps (the load cursor is already two steps on)
    const int sb2 = l_sb;
    const bool ok2 = l_ok;
    l_sb = sb0;
    l_ok = ok0;
#pragma unroll
    for (int q = 0; q < 4; ++q) load_x(fa.x[q], q);
    l_sb = sb1;
    l_ok = ok1;
#pragma unroll
    for (int q = 0; q < 4; ++q) load_x(fb.x[q], q);
    l_sb = sb2;
    l_ok = ok2;
  }

  // a norm handed over by the product before: row m's partial sums are added up by warp m after the k loop
  constexpr bool TAKES = XG && EPI != kAddResidual;
  if (TAKES && a.ss_in != nullptr && warp < M) {
#pragma unroll 1
    for (int c = lane; c < a.ss_n; c += 32)
      cp_async4(early + warp * a.ss_n + c, a.ss_in + static_cast<size_t>(warp) * a.ss_n + c);
  }

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
    const int cta_n0 = (blockIdx.x * a.row_tiles + rt) * TPC * 16;   // first feature of the CTA's round
    if (cta_n0 >= a.N) break;
    float acc[NG][4];
#pragma unroll
    for (int j = 0; j < NG; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
    for (int k0 = 0; k0 < K; k0 += kc) {
      const int kn = min(kc, K - k0);
      if (!XG) __syncthreads();   // the previous chunk (or the previous tile's reduction) is done with smem
      // ---- stage x[:, k0 : k0 + kn] as bfloat16, zero beyond M and beyond kn (to a multiple of 128)
      const int kpad = (kn + kSB - 1) / kSB * kSB;
      for (int i = tid; i < (XG ? 0 : MT * (kpad / 8)); i += WARPS * 32) {
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
      if (!XG) __syncthreads();
      // ---- the weight stream: warp kw takes super-blocks kw, kw + KW, ...
      const int sb_end = min((k0 + kc) / kSB, nsb);
      for (int sb = k0 / kSB + kw; sb < sb_end; sb += KW, ++step) {
        const int kb = sb * kSB - k0;    // within the staged chunk
        auto multiply = [&](WFrag& f) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int j = 0; j < NG; ++j) {
              const uint4 xv = XG ? f.x[q] : *reinterpret_cast<const uint4*>(xs + (j * 8 + g) * lds + kb + q * 32 + t * 8);
              mma_bf16(acc[j], f.lo[q].x, f.hi[q].x, f.lo[q].y, f.hi[q].y, xv.x, xv.y);
              mma_bf16(acc[j], f.lo[q].z, f.hi[q].z, f.lo[q].w, f.hi[q].w, xv.z, xv.w);
            }
            load_piece(f.lo[q], f.hi[q], q);     // the same place, two steps on
            if (XG) load_x(f.x[q], q);
          }
          load_advance();
        };
        if (step & 1) multiply(fb); else multiply(fa);
      }
    }
    if (TAKES && a.ss_in != nullptr && rt == 0) {     // (WARPS >= 8 >= M: every row has its warp)
      float ss = 0.f;
      cp_async_wait_all();       // (a lane adds what it copied itself)
      if (warp < M) {
#pragma unroll 1
        for (int c = lane; c < a.ss_n; c += 32) ss += early[warp * a.ss_n + c];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0 && warp < MT) inv_rms[warp] = rsqrtf(ss / static_cast<float>(K) + a.eps);
    }
    if (EPI == kAddResidual) cp_async_wait_all();
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
    if (EPI == kAddResidual && a.xw != nullptr) {       // (the same for the whole CTA)
      hand_over_epilogue<MT, WARPS, KW>(red, rt == 0 ? early : nullptr, static_cast<float*>(a.y), a.ldy, a.next_w,
                                        a.next_w_f32, a.xw, a.ldxw, a.ss_out, M, a.N, cta_n0, tid);
      continue;
    }
    for (int i = tid; i < TPC * 16 * MT; i += WARPS * 32) {
      // consecutive threads take consecutive features of one token: coalesced stores
      const int m = i / (TPC * 16), ft = i - m * (TPC * 16);
      const int tl = ft >> 4, f = ft & 15;             // tile of the CTA's round, feature in the tile
      const int n = cta_n0 + ft;
      if (m >= M || n >= a.N) continue;
      const int w0 = (tl * STREAMS) * KW;              // first warp of the tile's (first) stream
      float v = 0.f, u = 0.f;
#pragma unroll
      for (int w = 0; w < KW; ++w) {
        v += red[((w0 + w) * 16 + f) * MT + m];
        if (GATED) u += red[((w0 + KW + w) * 16 + f) * MT + m];
      }
      if (TAKES && a.ss_in != nullptr) {
        v *= inv_rms[m];
        u *= inv_rms[m];
      }
      const size_t o = static_cast<size_t>(m) * a.ldy + n;
      if (EPI == kStoreBf16) {
        static_cast<bf16*>(a.y)[o] = __float2bfloat16_rn(v);
      } else if (EPI == kStoreF32) {
        static_cast<float*>(a.y)[o] = v;
      } else if (EPI == kAddResidual) {
        // the unfused path rounds the product to bfloat16 before the add; so does this one
        static_cast<float*>(a.y)[o] = (rt == 0 ? early[i] : static_cast<const float*>(a.y)[o]) + __bfloat162float(__float2bfloat16_rn(v));
      } else {
        const float gt = __bfloat162float(__float2bfloat16_rn(v)), up = __bfloat162float(__float2bfloat16_rn(u));
        static_cast<bf16*>(a.y)[o] = __float2bfloat16_rn(gt / (1.f + expf(-gt)) * up);
      }
    }
  }
}

template <int MT, int WARPS, int KW, int EPI, bool NORM>
int launch_one(const SkinnyArgs& a0, int sm_count, cudaStream_t stream) {
  constexpr int STREAMS = (EPI == kSwiglu) ? 2 : 1;
  constexpr int TPC = WARPS / KW / STREAMS;
  SkinnyArgs a = a0;
  const int tiles = (a.N + 15) / 16;
  const int rounds = (tiles + TPC - 1) / TPC;       // CTA-rounds of TPC tiles
  // at most about two CTAs per SM, all resident at once: a second, nearly empty wave would cost
  // as much as the first
  // (one CTA per SM, so that the next product's CTAs could move in beside it, was measured: the decode
  // step is a fifth slower with half the warps streaming)
  int rt = (rounds + 2 * sm_count - 1) / (2 * sm_count);
  if (rt > 16) rt = 16;
  a.row_tiles = rt;
  const int ctas = (rounds + rt - 1) / rt;
  // K is staged in equal chunks that are multiples of 128 * KW, so that warp kw of a stream always
  // takes the global 128-wide super-blocks kw, kw + KW, ...: the order of a row's sums does not
  // depend on the chunking, hence not on how many rows the batch has.
  constexpr int kUnit = kSB * KW;
  const int kunits = (a.K + kUnit - 1) / kUnit;
  int max_units = (98304 / (MT * 2) - 32) / kUnit;
  if (max_units < 1) max_units = 1;
  const int chunks = (kunits + max_units - 1) / max_units;
  const int kc = (kunits + chunks - 1) / chunks * kUnit;
  const size_t xbytes = static_cast<size_t>(MT) * (kc + 32) * 2;
  const size_t rbytes = static_cast<size_t>(WARPS) * 16 * MT * 4;
  constexpr bool XG = !NORM && MT == 8;               // no staging of x: only the reduction uses shared memory
  const size_t base = ((!XG && xbytes > rbytes) ? xbytes : rbytes);
  const size_t extra_off = (base + 15) / 16 * 16;
  const size_t extra = EPI == kAddResidual ? static_cast<size_t>(TPC * 16 * MT + TPC * 16) * 4
                                           : (a.ss_in != nullptr ? static_cast<size_t>(MT) * a.ss_n * 4 : 0);
  const size_t smem = extra_off + extra;
  if (smem > 200 * 1024) return static_cast<int>(cudaErrorInvalidValue);
  static size_t set_for = 0;
  if (smem > set_for) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<MT, WARPS, KW, EPI, NORM>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    set_for = smem;
  }
  launch_kernel(gemm_skinny_kernel<MT, WARPS, KW, EPI, NORM>, dim3(ctas), dim3(WARPS * 32), smem, stream, a, kc,
                static_cast<int>(extra_off));
  return static_cast<int>(cudaGetLastError());
}

// How many warps split the K of one stream: the largest power of two that keeps streams x warps
// at about 16 warps per SM (measured on a B200 over the projection shapes of 1B- to 8B-size
// models: the best split is the one with 1,500 to 2,100 warps in all), at most one warp per
// 128-wide super-block.  Depends on the weight's shape and on the GPU only, never on the
// number of rows.
inline int choose_kw(int N, int K, int streams, int sm_count) {
  const int tiles = (N + 15) / 16, nsb = (K + kSB - 1) / kSB;
  int kw = 1;
  while (kw < 16 && tiles * streams * (kw * 2) <= sm_count * 16 && kw * 2 <= nsb) kw *= 2;
  return kw;
}

template <int MT, int EPI, bool NORM>
int launch_kw(const SkinnyArgs& a, int sm_count, cudaStream_t stream) {
  constexpr int STREAMS = (EPI == kSwiglu) ? 2 : 1;
  int kw = choose_kw(a.N, a.K, STREAMS, sm_count);
  if (STREAMS == 2 && kw > 4) kw = 4;      // 8 warps hold both streams of a tile
  switch (kw) {
    case 1: return launch_one<MT, 8, 1, EPI, NORM>(a, sm_count, stream);
    case 2: return launch_one<MT, 8, 2, EPI, NORM>(a, sm_count, stream);
    case 4: return launch_one<MT, 8, 4, EPI, NORM>(a, sm_count, stream);
    case 8:
      if constexpr (STREAMS == 1) return launch_one<MT, 8, 8, EPI, NORM>(a, sm_count, stream);
    default:
      if constexpr (STREAMS == 1) return launch_one<MT, 16, 16, EPI, NORM>(a, sm_count, stream);
  }
  return static_cast<int>(cudaErrorInvalidValue);
}

template <int EPI, bool NORM>
int launch_mt(const SkinnyArgs& a, int sm_count, cudaStream_t stream) {
  if (a.M <= 8) return launch_kw<8, EPI, NORM>(a, sm_count, stream);
  return launch_kw<16, EPI, NORM>(a, sm_count, stream);
}

}  // namespace rl

using namespace rl;

extern "C" {

int rl_gemm_skinny_max_rows() { return 16; }

// epilogue: 0 bf16 store, 1 float32 store, 2 residual += y, 3 SiLU-gated product (w holds
// N gate rows then N up rows).  norm != 0: x is rmsnorm(residual[rows_idx]) * norm_w.
// Requirements: M <= 16, K a multiple of 8, 16-byte aligned rows.  Returns cudaErrorInvalidValue
// otherwise (the caller then takes another path).
//
// The norm between two products handed over (both optional, see SkinnyArgs): with xw_out, a product with
// epilogue 2 also leaves bfloat16(residual * next_w) and per-tile sums of residual^2 (ss_out, float32
// [M, ceil(N / 16)]); with ss_in, a product of up to 8 rows without the fused norm takes such an x and
// scales its rows by rsqrt(sum / K + eps).
int rl_gemm_skinny_handover(const void* w, const void* x, int ldx, const float* residual, const void* norm_w,
                            int norm_w_f32, const int32_t* rows_idx, float eps, int norm, void* y, int ldy,
                            int epilogue, int M, int N, int K, const void* next_w, int next_w_f32, void* xw_out,
                            int ldxw, float* ss_out, const float* ss_in, int ss_n, int sm_count,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K % 8 != 0 || (!norm && ldx % 8 != 0)) return static_cast<int>(cudaErrorInvalidValue);
  if (xw_out != nullptr && (epilogue != kAddResidual || next_w == nullptr || ss_out == nullptr))
    return static_cast<int>(cudaErrorInvalidValue);
  if (ss_in != nullptr && (norm || M > 8 || ss_n <= 0 || epilogue == kAddResidual))
    return static_cast<int>(cudaErrorInvalidValue);
  SkinnyArgs a;
  a.next_w = next_w;
  a.next_w_f32 = next_w_f32;
  a.xw = static_cast<bf16*>(xw_out);
  a.ldxw = ldxw;
  a.ss_out = ss_out;
  a.ss_in = ss_in;
  a.ss_n = ss_n;
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
  a.row_tiles = 1;
  if (norm) {
    switch (epilogue) {
      case kStoreBf16: return launch_mt<kStoreBf16, true>(a, sm_count, stream);
      case kStoreF32: return launch_mt<kStoreF32, true>(a, sm_count, stream);
      case kSwiglu: return launch_mt<kSwiglu, true>(a, sm_count, stream);
    }
  } else {
    switch (epilogue) {
      case kStoreBf16: return launch_mt<kStoreBf16, false>(a, sm_count, stream);
      case kStoreF32: return launch_mt<kStoreF32, false>(a, sm_count, stream);
      case kAddResidual: return launch_mt<kAddResidual, false>(a, sm_count, stream);
      case kSwiglu: return launch_mt<kSwiglu, false>(a, sm_count, stream);
    }
  }
  return static_cast<int>(cudaErrorInvalidValue);
}

int rl_gemm_skinny(const void* w, const void* x, int ldx, const float* residual, const void* norm_w,
                   int norm_w_f32, const int32_t* rows_idx, float eps, int norm, void* y, int ldy,
                   int epilogue, int M, int N, int K, int sm_count, cudaStream_t stream) {
  return rl_gemm_skinny_handover(w, x, ldx, residual, norm_w, norm_w_f32, rows_idx, eps, norm, y, ldy, epilogue, M, N,
                                 K, nullptr, 0, nullptr, 0, nullptr, nullptr, 0, sm_count, stream);
}

}  // extern "C"
