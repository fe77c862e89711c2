// y[M, N] = x[M, K] . W[N, K]^T for 17 to 128 rows (a decode batch of that many sequences, a short
// prompt portion), bfloat16 operands, on the fifth-generation tensor cores.
//
// With so few rows the product is bound by the weight stream, and a 128-row tile of x would be mostly
// padding.  So the operands are swapped: the 128-row operand of tcgen05.mma is a tile of 128 WEIGHT rows
// (features), the narrow operand (32, 64 or 128 wide) holds the tokens, and the accumulator in tensor
// memory is y transposed: TMEM lane = feature, column = token.  Per 64-wide k block a CTA reads 16 KB of
// weights (from DRAM, once) and at most 16 KB of x (from L2).  N / 128 feature tiles are fewer than the
// SMs for most weight shapes, so K is split: CTA (tile, split) multiplies its share of the k blocks, the
// partial tiles meet in a scratch area in global memory, and the CTA that arrives last at the tile's
// counter adds them up in the order of the splits (the result does not depend on which CTA that is),
// applies the epilogue and writes y.  The counters are left at zero for the next launch.
//
// Warp roles as in gemm_tc.cu: warp 0 issues the TMA loads into a ring of stages (the weight tiles of the
// first stages before the wait on earlier kernels of the step: they do not depend on them), warp 1
// allocates TMEM and issues the MMAs, warps 2-5 read the accumulator and do the rest.  Epilogues:
// bfloat16 store, and the SiLU-gated product (a tile then holds 64 gate rows and their 64 up rows).
// Every wait on an mbarrier is bounded; a wait that runs out sets bit 3 of *status.  No cluster
// multicast anywhere.
//
// State: correct at every shape the tests try, but not yet as fast as the library at 64 rows (a CTA
// has one tile, so its ramp, its stream and its epilogue do not overlap, and the last CTA of a split
// tile reads all partial tiles through L2); the engine does not route products here yet.
#include "umma.cuh"

namespace rl {

constexpr int kMidRows = 128;            // weight rows per tile (the MMA's M)
constexpr int kMidBK = 64, kMidUmmaK = 16;
constexpr int kMidMaxStages = 10;
constexpr int kMidStageA = kMidRows * kMidBK * 2;
// As many stages as fit: the weight stream wants about 100 KB per SM in flight to reach the DRAM's rate.
template <int MB>
struct MidCfg {
  static constexpr int kStages = MB >= 128 ? 6 : (MB >= 64 ? 8 : 10);
};
constexpr int kMidThreads = 192;

enum MidEpilogue { kMidBf16 = 0, kMidSwiglu = 3 };

struct MidShared {
  uint64_t full[kMidMaxStages];
  uint64_t empty[kMidMaxStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int last;                  // this CTA arrived last at its tile's counter
  volatile int abort;
};

struct MidArgs {
  void* y;                   // bfloat16 [M, N]
  int M, N, K, ldy;
  int n_up;                  // kMidSwiglu: row of W where the up rows start
  int tiles, splits;
  float* partial;            // [tiles * splits][MB][128] float32
  int* counters;             // [tiles], zero between launches
  int* status;
};

template <int EPI, int MB>
__global__ void __launch_bounds__(kMidThreads, 1)
gemm_mid_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const MidArgs a) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* base = smem_raw + ((1024u - (raw & 1023u)) & 1023u);      // 128-byte swizzle: 1024-byte alignment
  constexpr int kStageB = MB * kMidBK * 2;
  constexpr int kMidStages = MidCfg<MB>::kStages;
  constexpr int kTmemCols = MB < 32 ? 32 : MB;
  constexpr int kTileN = (EPI == kMidSwiglu) ? kMidRows / 2 : kMidRows;      // features of y per tile
  unsigned char* smem_a = base;
  unsigned char* smem_b = base + kMidStages * kMidStageA;
  MidShared* sh = reinterpret_cast<MidShared*>(base + kMidStages * (kMidStageA + kStageB));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / a.splits, sp = blockIdx.x - tile * a.splits;
  const int nkb_all = (a.K + kMidBK - 1) / kMidBK;
  const int kb0 = static_cast<int>(static_cast<long long>(sp) * nkb_all / a.splits);
  const int kb1 = static_cast<int>(static_cast<long long>(sp + 1) * nkb_all / a.splits);
  const int nkb = kb1 - kb0;                  // >= 1: the host gives no split less than one k block
  const int n0 = tile * kTileN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMidStages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    mbar_init(&sh->acc_full, 1);
    sh->abort = 0;
    sh->last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  pdl_launch();

  if (warp == 0) {
    if (lane == 0) {
      auto load_w = [&](int s, int kb) {
        if (EPI == kMidSwiglu) {
          tma_load_2d(smem_a + s * kMidStageA, &map_w, &sh->full[s], kb * kMidBK, n0);
          tma_load_2d(smem_a + s * kMidStageA + kMidStageA / 2, &map_w, &sh->full[s], kb * kMidBK, a.n_up + n0);
        } else {
          tma_load_2d(smem_a + s * kMidStageA, &map_w, &sh->full[s], kb * kMidBK, n0);
        }
      };
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      const int pre = min(kMidStages, nkb);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&sh->full[i], kMidStageA + kStageB);
        load_w(i, kb0 + i);
      }
      pdl_wait();        // x is written by earlier kernels of the step
      bool ok = true;
      int issued = 0;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % kMidStages;
        if (i >= pre) {
          ok = mbar_wait(&sh->empty[s], ((i / kMidStages) & 1) ^ 1, &sh->abort);
          if (!ok) break;
          mbar_expect_tx(&sh->full[s], kMidStageA + kStageB);
          load_w(s, kb0 + i);
        }
        tma_load_2d(smem_b + s * kStageB, &map_x, &sh->full[s], (kb0 + i) * kMidBK, 0);
        ++issued;
      }
      if (sh->abort) {
        // loads still in flight write shared memory: wait for them (bounded) before the CTA ends
        for (int i2 = max(0, issued - kMidStages); i2 < issued; ++i2) {
          const int s = i2 % kMidStages;
          for (int i = 0; i < kSpinLimit && !mbar_try_wait(&sh->full[s], (i2 / kMidStages) & 1); ++i) {
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kMidRows, MB);
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % kMidStages;
        ok = mbar_wait(&sh->full[s], (i / kMidStages) & 1, &sh->abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem_a + s * kMidStageA), b_addr = smem_u32(smem_b + s * kStageB);
#pragma unroll
        for (int k = 0; k < kMidBK / kMidUmmaK; ++k)
          umma_bf16(tmem, umma_desc(a_addr + k * kMidUmmaK * 2), umma_desc(b_addr + k * kMidUmmaK * 2), idesc, (i | k) != 0);
        umma_commit(&sh->empty[s]);
      }
      if (ok) umma_commit(&sh->acc_full);
    }
  } else {
    // warps 2..5: warp w may touch TMEM lanes 32 * (w % 4) .. + 32; lane of the tile = weight row
    const int q = warp & 3;
    const int nl = q * 32 + lane;                              // row of the tile
    const int et = threadIdx.x - 64;                           // index among the 128 epilogue threads
    pdl_wait();
    const bool ok = mbar_wait(&sh->acc_full, 0, &sh->abort);
    tc_fence_after();
    const uint32_t acc = tmem + (static_cast<uint32_t>(q * 32) << 16);
    bool mine = ok;                                            // this CTA writes y
    if (ok && a.splits > 1) {
      // the partial tile goes to the scratch area as [token][row]: a warp's stores are 128 bytes in a row
      float* part = a.partial + static_cast<size_t>(blockIdx.x) * MB * kMidRows;
#pragma unroll 1
      for (int c = 0; c < MB; c += 32) {
        float v[32];
        tmem_ld32(acc + c, v);
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c + i < a.M) part[(c + i) * kMidRows + nl] = v[i];
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");          // the 128 epilogue threads
      if (et == 0) {
        const int done = atomicAdd(a.counters + tile, 1) + 1;
        sh->last = (done == a.splits) ? 1 : 0;
        if (done == a.splits) a.counters[tile] = 0;            // ready for the next launch
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      mine = sh->last != 0;
      if (mine) __threadfence();
    }
    if (mine && a.splits > 1) {
      // The last CTA adds the partial tiles in the order of the splits.  Here a lane takes four neighbouring
      // rows (features) of one token and a warp every fourth token; four tokens' loads of all splits are
      // asked for together.  Gated: the lane with the gate features n .. n + 3 gets their up features from
      // the lane 16 further on.
      const int wq = warp - 2;                                 // 0..3
      const int nq = lane * 4;                                 // row of the tile
      const float* part0 = a.partial + static_cast<size_t>(tile) * a.splits * MB * kMidRows + nq;
#pragma unroll 1
      for (int m0 = wq; m0 < a.M; m0 += 16) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int s2 = 0; s2 < a.splits; s2 += 4) {
          float4 t[4][4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int m = m0 + 4 * j;
              t[u][j] = (s2 + u < a.splits && m < a.M)
                            ? __ldcg(reinterpret_cast<const float4*>(part0 + (static_cast<size_t>(s2 + u) * MB + m) * kMidRows))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[j].x += t[u][j].x;
              v[j].y += t[u][j].y;
              v[j].z += t[u][j].z;
              v[j].w += t[u][j].w;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int m = m0 + 4 * j;                            // (the same for the whole warp)
          float r[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
          int n = n0 + nq;
          bool store = m < a.M;
          if (EPI == kMidSwiglu) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float up = __bfloat162float(__float2bfloat16_rn(__shfl_down_sync(0xffffffffu, r[e], 16)));
              const float gt = __bfloat162float(__float2bfloat16_rn(r[e]));
              r[e] = gt / (1.f + __expf(-gt)) * up;
            }
            store = store && lane < 16;
          }
          if (store) {
            bf16* out = static_cast<bf16*>(a.y) + static_cast<size_t>(m) * a.ldy + n;
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (n + e < a.N) out[e] = __float2bfloat16_rn(r[e]);
          }
        }
      }
    } else if (mine) {
      // one split: straight from TMEM (lane = row).  Gated: rows 0..63 of the tile are gate features, rows
      // 64..127 their up features; the up half goes through shared memory (the stages are free: every MMA
      // that read them is done) to the gate half
      float* xch = reinterpret_cast<float*>(smem_a);           // [64][33] floats per chunk of 32 tokens
#pragma unroll 1
      for (int c = 0; c < MB; c += 32) {
        float v[32];
        tmem_ld32(acc + c, v);
        if (EPI == kMidSwiglu) {
          if (c > 0) asm volatile("bar.sync 1, 128;" ::: "memory");      // the chunk before has been read
          if (nl >= 64) {
#pragma unroll
            for (int i = 0; i < 32; ++i) xch[(nl - 64) * 33 + i] = v[i];
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (nl < 64) {
            const int n = n0 + nl;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float gt = __bfloat162float(__float2bfloat16_rn(v[i]));
              const float up = __bfloat162float(__float2bfloat16_rn(xch[nl * 33 + i]));
              if (c + i < a.M && n < a.N)
                static_cast<bf16*>(a.y)[static_cast<size_t>(c + i) * a.ldy + n] = __float2bfloat16_rn(gt / (1.f + __expf(-gt)) * up);
            }
          }
        } else {
          const int n = n0 + nl;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c + i < a.M && n < a.N) static_cast<bf16*>(a.y)[static_cast<size_t>(c + i) * a.ldy + n] = __float2bfloat16_rn(v[i]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && sh->abort) atomicOr(a.status, 8);
}

// ---------------------------------------------------------------------------- host side

// A [rows, K] bfloat16 matrix with row pitch ld (elements), tiles of box_rows x 64, 128-byte swizzle;
// rows beyond the matrix read as zero.
static bool mid_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {kMidBK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline int mid_width(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }

// Tiles and splits of a product: as many splits as keep all SMs busy, none with less than two k blocks.
inline void mid_shape(int N, int K, int gated, int sm_count, int* tiles, int* splits) {
  const int tile_n = gated ? kMidRows / 2 : kMidRows;
  *tiles = (N + tile_n - 1) / tile_n;
  const int nkb = (K + kMidBK - 1) / kMidBK;
  int s = sm_count / *tiles;
  if (s > nkb / 2) s = nkb / 2;
  if (s < 1) s = 1;
  *splits = s;
}

template <int EPI, int MB>
static int launch_mid(const CUtensorMap& mw, const CUtensorMap& mx, const MidArgs& a, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(MidCfg<MB>::kStages) * (kMidStageA + MB * kMidBK * 2) + sizeof(MidShared) + 1024;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mid_kernel<EPI, MB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    attr = true;
  }
  launch_kernel(gemm_mid_kernel<EPI, MB>, dim3(a.tiles * a.splits), dim3(kMidThreads), smem, stream, mw, mx, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace rl

using namespace rl;

extern "C" {

int rl_gemm_mid_max_rows() { return 128; }

// Floats of scratch and ints of counters that rl_gemm_mid needs for a product with N features (2 N weight
// rows if gated) and K columns at up to M rows.
int rl_gemm_mid_workspace(int M, int N, int K, int gated, int sm_count, long long* partial_floats, int* counters) {
  int tiles, splits;
  mid_shape(N, K, gated, sm_count, &tiles, &splits);
  *partial_floats = splits > 1 ? static_cast<long long>(tiles) * splits * mid_width(M) * kMidRows : 0;
  *counters = tiles;
  return 0;
}

// epilogue: 0 bfloat16 store, 3 SiLU-gated product (w holds N gate rows then N up rows, y is [M, N]).
// x [M, K] and w are bfloat16 with K a multiple of 8 and 16-byte aligned rows; 1 <= M <= 128.  partial /
// counters: scratch of the sizes rl_gemm_mid_workspace gives (counters zero before the first launch).
// status: device int, bit 3 is set if a wait inside the kernel ran out.  Returns cudaErrorInvalidValue
// for shapes it does not take.
int rl_gemm_mid(const void* x, int ldx, const void* w, void* y, int ldy, int epilogue, int M, int N, int K,
                float* partial, int* counters, int* status, int sm_count, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 128 || K % 8 != 0 || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (epilogue != kMidBf16 && epilogue != kMidSwiglu) || counters == nullptr || status == nullptr)
    return static_cast<int>(cudaErrorInvalidValue);
  const bool gated = epilogue == kMidSwiglu;
  MidArgs a;
  a.y = y;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldy = ldy;
  a.n_up = N;
  mid_shape(N, K, gated ? 1 : 0, sm_count, &a.tiles, &a.splits);
  if (a.splits > 1 && partial == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  a.partial = partial;
  a.counters = counters;
  a.status = status;
  const int mb = mid_width(M);
  CUtensorMap mw, mx;
  if (!mid_map(&mw, w, gated ? 2 * N : N, K, K, gated ? kMidRows / 2 : kMidRows)) return static_cast<int>(cudaErrorNotSupported);
  if (!mid_map(&mx, x, M, K, ldx, mb)) return static_cast<int>(cudaErrorNotSupported);
#define RL_MID_CASE(E)                                                 \
  case E:                                                              \
    if (mb == 32) return launch_mid<E, 32>(mw, mx, a, stream);         \
    if (mb == 64) return launch_mid<E, 64>(mw, mx, a, stream);         \
    return launch_mid<E, 128>(mw, mx, a, stream)
  switch (epilogue) {
    RL_MID_CASE(kMidBf16);
    RL_MID_CASE(kMidSwiglu);
  }
#undef RL_MID_CASE
  return static_cast<int>(cudaErrorInvalidValue);
}

}  // extern "C"
