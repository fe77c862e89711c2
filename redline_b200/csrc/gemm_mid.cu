// y[M, N] = x[M, K] . W[N, K]^T for 17 to 128 rows (a decode batch of that many sequences, a short
// prompt portion), bfloat16 operands, on the fifth-generation tensor cores, with the work that
// surrounds a product in a layer fused into it.
//
// With so few rows the product is bound by the weight stream, and a 128-row tile of x would be mostly
// padding.  So the operands are swapped: the 128-row operand of tcgen05.mma is a tile of 128 WEIGHT rows
// (features), the narrow operand (32, 64 or 128 wide) holds the tokens, and the accumulator in tensor
// memory is y transposed: TMEM lane = feature, column = token.  Per 64-wide k block a CTA reads 16 KB of
// weights (from DRAM, once) and at most 16 KB of x (from L2).
//
// N / 128 feature tiles are fewer than the SMs for most weight shapes, so K is split over the CTAs of a
// thread-block CLUSTER (up to 8): CTA r of a tile's cluster multiplies the r-th share of the k blocks.
// The partial tiles never leave the chip: every CTA puts its own into its shared memory, the cluster
// meets at its hardware barrier, and then CTA r adds up, for every S-th token, the partial results of
// all CTAs of the cluster in the order of k (read through distributed shared memory; the result does not
// depend on timing), applies the epilogue and writes them.  No scratch in global memory, no counters,
// nothing that waits on a flag.
//
// Epilogues: bfloat16 store; `residual += y` on the float32 stream; the SiLU-gated product (a tile then
// holds 64 gate rows and their 64 up rows).  A norm can be handed over between two products as between
// the products for at most 16 rows: the `residual +=` epilogue can also leave
// xw = bfloat16(residual * norm_weight) and, per token and feature tile, the sum of residual^2 ("hand
// out"); a product that reads such an xw as its x scales token m of its result by
// rsqrt(sum of the token's sums / width + eps) ("hand in"), which makes it the product of the normed
// stream without a norm kernel in between.
//
// Warp roles: warp 0 issues the TMA loads into a ring of stages (the weight tiles of the first stages
// before the wait on earlier kernels of the step: they do not depend on them), warp 1 allocates TMEM and
// issues the MMAs, warps 2-5 move the accumulator from TMEM to shared memory; after the cluster's barrier
// all twelve warps add up and write (with four warps that part took as long as the weight stream of a
// small product).  Every wait on an mbarrier is bounded; a wait that runs out sets bit 3 of *status (the
// CTA still goes to the cluster's barriers, so its neighbours are not left waiting).  No load uses
// cluster multicast.
#include <mutex>
#include "umma.cuh"

namespace rl {

constexpr int kMidRows = 128;            // weight rows per tile (the MMA's M)
constexpr int kMidBK = 64, kMidUmmaK = 16;
constexpr int kMidMaxStages = 10;
constexpr int kMidStageA = kMidRows * kMidBK * 2;
constexpr int kMidMaxTokens = 128;
constexpr int kMidMaxSplits = 8;          // the portable cluster size
// As many stages as fit (a ring of 192 KB): with half the ring the gated gate/up shape of a 1B model at
// 64 rows took 18.9 us instead of 16.6.
template <int MB>
struct MidCfg {
  static constexpr int kStages = MB >= 128 ? 6 : (MB >= 64 ? 8 : 10);
};
constexpr int kMidThreads = 384;          // 2 role warps + 4 that read the accumulator; all 12 add up and write
constexpr int kMidWarps = kMidThreads / 32;

enum MidEpilogue { kMidBf16 = 0, kMidResidual = 2, kMidSwiglu = 3 };

struct MidShared {
  uint64_t full[kMidMaxStages];
  uint64_t empty[kMidMaxStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  volatile int abort;
  float scale[kMidMaxTokens];   // hand in: the factor of every token's row
};

struct MidArgs {
  void* y;                   // bfloat16 [M, N] (kMidBf16, kMidSwiglu)
  int ldy;
  float* residual;           // float32 [M, N] (kMidResidual): residual += y
  int ldr;
  // hand out (kMidResidual, xw != nullptr): the norm that is applied to the stream next
  const void* norm_w;        // [N], bfloat16 or float32
  int norm_w_f32;
  bf16* xw;                  // [M, N] = bfloat16(residual * norm_w)
  int ldxw;
  float* sums_out;           // [M, sums_out_ld]: column t = sum over feature tile t of residual^2
  int sums_out_ld;
  // hand in (sums_in != nullptr): x is such an xw; token m of the result is scaled by rsqrt(sum_c sums_in[m][c] / K + eps)
  const float* sums_in;
  int sums_in_ld, sums_in_n;
  float eps;
  int M, N, K;
  int n_up;                  // kMidSwiglu: row of W where the up rows start
  int vec_y, vec_xw;         // every row of y / xw starts 8-byte aligned
  int tiles, splits;         // grid = tiles * splits CTAs in clusters of `splits`
  int* status;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Four floats at a shared-memory address of this CTA's layout, read from CTA `rank` of the cluster.
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t smem_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr), "r"(rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
  return v;
}

// Up to four values as bfloat16 to p: `left` features are left in the row from p on; vec says that every
// such p of the matrix is 8-byte aligned.
__device__ __forceinline__ void store_bf16x4(bf16* p, const float* v, int left, int vec) {
  if (vec && left >= 4) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (e < left) p[e] = __float2bfloat16_rn(v[e]);
  }
}

// The second half of the epilogue for the tokens first, first + step, ... of one warp, U of them at a time:
// a lane has four neighbouring rows (features) of the tile; the partial results of all CTAs of the cluster
// are added in the order of k, then scaled (hand in), gated or added to the stream, and written.  All loads
// of the U tokens are issued before the arithmetic and all stores after it: a token's chain of latencies
// (shared memory of a peer, the stream in global memory, the special-function unit) is several hundred
// cycles long and a warp has nothing else to do meanwhile.
// Gated: the lane with the gate features n .. n + 3 gets their up features from the lane 16 further on.
template <int EPI, int U>
__device__ __forceinline__ void mid_finish(const MidArgs& a, const MidShared* sh, const unsigned char* smem_a,
                                           int first, int step, int S, int sp, int n0, int tile, int lane) {
  const int nq = lane * 4;                                   // row of the tile
  const int n = n0 + nq;
  const uint32_t part_u = smem_u32(smem_a);
  const bool whole = n + 3 < a.N;                            // all four features exist
#pragma unroll 1
  for (int mb = first; mb < a.M; mb += U * step) {           // (the same for the whole warp)
    float r[U][4];
    float4 old[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int m = mb + u * step;
      r[u][0] = r[u][1] = r[u][2] = r[u][3] = 0.f;
      old[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < a.M) {
        if (EPI == kMidResidual && whole)
          old[u] = *reinterpret_cast<const float4*>(a.residual + static_cast<size_t>(m) * a.ldr + n);
        const uint32_t off = static_cast<uint32_t>(m * kMidRows + nq) * 4;
#pragma unroll
        for (int p = 0; p < kMidMaxSplits; ++p)
          if (p < S) {
            const float4 t = p == sp ? *reinterpret_cast<const float4*>(smem_a + off) : ld_cluster_f4(part_u + off, p);
            r[u][0] += t.x;
            r[u][1] += t.y;
            r[u][2] += t.z;
            r[u][3] += t.w;
          }
      }
    }
    float wv[U][4];
    float sq[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int m = mb + u * step;
      sq[u] = 0.f;
      if (m < a.M) {
        if (a.sums_in != nullptr) {
          const float f = sh->scale[m];
#pragma unroll
          for (int e = 0; e < 4; ++e) r[u][e] *= f;
        }
        if (EPI == kMidSwiglu) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float up = __bfloat162float(__float2bfloat16_rn(__shfl_down_sync(0xffffffffu, r[u][e], 16)));
            const float gt = __bfloat162float(__float2bfloat16_rn(r[u][e]));
            r[u][e] = __fdividef(gt, 1.f + __expf(-gt)) * up;
          }
        }
        if (EPI == kMidResidual) {
          if (whole) {
            r[u][0] += old[u].x;
            r[u][1] += old[u].y;
            r[u][2] += old[u].z;
            r[u][3] += old[u].w;
          } else {
            const float* res = a.residual + static_cast<size_t>(m) * a.ldr + n;
#pragma unroll
            for (int e = 0; e < 4; ++e) r[u][e] = n + e < a.N ? r[u][e] + res[e] : 0.f;
          }
          if (a.xw != nullptr) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float w = 0.f;
              if (n + e < a.N)
                w = a.norm_w_f32 ? static_cast<const float*>(a.norm_w)[n + e]
                                 : __bfloat162float(static_cast<const bf16*>(a.norm_w)[n + e]);
              sq[u] += r[u][e] * r[u][e];
              wv[u][e] = w * r[u][e];
            }
            // the tile's share of the token's sum of squares: the 32 lanes hold its 128 features
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq[u] += __shfl_xor_sync(0xffffffffu, sq[u], o);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int m = mb + u * step;
      if (m < a.M) {
        if (EPI == kMidResidual) {
          if (n < a.N) {
            float* res = a.residual + static_cast<size_t>(m) * a.ldr + n;
            if (whole) {
              *reinterpret_cast<float4*>(res) = make_float4(r[u][0], r[u][1], r[u][2], r[u][3]);
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (n + e < a.N) res[e] = r[u][e];
            }
            if (a.xw != nullptr) store_bf16x4(a.xw + static_cast<size_t>(m) * a.ldxw + n, wv[u], a.N - n, a.vec_xw);
          }
          if (a.xw != nullptr && lane == 0) a.sums_out[static_cast<size_t>(m) * a.sums_out_ld + tile] = sq[u];
        } else if ((EPI != kMidSwiglu || lane < 16) && n < a.N) {
          store_bf16x4(static_cast<bf16*>(a.y) + static_cast<size_t>(m) * a.ldy + n, r[u], a.N - n, a.vec_y);
        }
      }
    }
  }
}

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
  static_assert(MB * kMidRows * 4 <= kMidStages * (kMidStageA + kStageB), "the partial tile lies in the ring of stages");
  unsigned char* smem_a = base;
  unsigned char* smem_b = base + kMidStages * kMidStageA;
  MidShared* sh = reinterpret_cast<MidShared*>(base + kMidStages * (kMidStageA + kStageB));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = a.splits;
  const int tile = blockIdx.x / S;
  const int sp = static_cast<int>(cluster_rank());          // = blockIdx.x % S: clusters are S consecutive CTAs
  const int nkb_all = (a.K + kMidBK - 1) / kMidBK;
  const int kb0 = static_cast<int>(static_cast<long long>(sp) * nkb_all / S);
  const int kb1 = static_cast<int>(static_cast<long long>(sp + 1) * nkb_all / S);
  const int nkb = kb1 - kb0;                  // >= 1: the host gives no split less than one k block
  const int n0 = tile * kTileN;

  auto load_w = [&](int s, int kb) {
    if (EPI == kMidSwiglu) {
      tma_load_2d(smem_a + s * kMidStageA, &map_w, &sh->full[s], kb * kMidBK, n0);
      tma_load_2d(smem_a + s * kMidStageA + kMidStageA / 2, &map_w, &sh->full[s], kb * kMidBK, a.n_up + n0);
    } else {
      tma_load_2d(smem_a + s * kMidStageA, &map_w, &sh->full[s], kb * kMidBK, n0);
    }
  };
  const int pre = min(kMidStages, nkb);
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < kMidStages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    mbar_init(&sh->acc_full, 1);
    sh->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // The weight tiles of the first stages depend on nothing that runs before this kernel and on nothing
    // the other warps set up: they are on their way before the CTA has met for the first time.
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(&sh->full[i], kMidStageA + kStageB);
      load_w(i, kb0 + i);
    }
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
        // loads still in flight write shared memory: wait for them (bounded) before the CTA goes on
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
  } else if (warp < 6) {
    // warps 2..5: warp w may touch TMEM lanes 32 * (w % 4) .. + 32; lane of the tile = weight row.
    // The partial tile goes into this CTA's shared memory as [token][row] float32, over the ring of weight
    // stages (every load has landed and every MMA that read them is done when the accumulator is).
    const int q = warp & 3;
    const int nl = q * 32 + lane;                              // row of the tile
    const int et = threadIdx.x - 64;                           // index among the 128 epilogue threads
    pdl_wait();                                                // the stream, the sums handed in
    if (a.sums_in != nullptr && et < a.M) {
      float ss = 0.f;
      for (int c = 0; c < a.sums_in_n; ++c) ss += a.sums_in[static_cast<size_t>(et) * a.sums_in_ld + c];
      sh->scale[et] = rsqrtf(ss / static_cast<float>(a.K) + a.eps);
    }
    const bool ok = mbar_wait(&sh->acc_full, 0, &sh->abort);
    tc_fence_after();
    if (__all_sync(0xffffffffu, ok)) {
      const uint32_t acc = tmem + (static_cast<uint32_t>(q * 32) << 16);
      float* part = reinterpret_cast<float*>(smem_a);
#pragma unroll 1
      for (int c = 0; c < MB; c += 32) {
        float v[32];
        tmem_ld32(acc + c, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) part[(c + j) * kMidRows + nl] = v[j];
      }
    }
  }
  // ---- the cluster's partial tiles are in place
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();
  // CTA r takes the tokens r, r + S, ...; a warp every twelfth of those, four (two, with many peers to read)
  // at a time.
  if (S <= 2)
    mid_finish<EPI, 4>(a, sh, smem_a, sp + warp * S, kMidWarps * S, S, sp, n0, tile, lane);
  else
    mid_finish<EPI, 2>(a, sh, smem_a, sp + warp * S, kMidWarps * S, S, sp, n0, tile, lane);
  // ---- no CTA leaves while a neighbour may still read its shared memory
  cluster_sync_all();
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

// Tiles and splits of a product: the largest cluster size (8 at most) of which as many clusters as there
// are tiles can be resident at once (max_clusters[s], from the occupancy calculator: a cluster lies within
// one GPC, so it is not sm_count / s), none with less than two k blocks.
inline void mid_shape(int N, int K, int gated, const int* max_clusters, int* tiles, int* splits) {
  const int tile_n = gated ? kMidRows / 2 : kMidRows;
  *tiles = (N + tile_n - 1) / tile_n;
  const int nkb = (K + kMidBK - 1) / kMidBK;
  int s = kMidMaxSplits;
  while (s > 1 && (max_clusters[s] < *tiles || s > nkb / 2)) --s;
  *splits = s;
}

constexpr int kMidMaxDevices = 64;

template <int EPI, int MB>
static int launch_mid(const CUtensorMap& mw, const CUtensorMap& mx, MidArgs& a, int gated, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(MidCfg<MB>::kStages) * (kMidStageA + MB * kMidBK * 2) + sizeof(MidShared) + 1024;
  // per device, once: the shared-memory limit of the kernel and how many clusters of each size fit
  static int max_clusters[kMidMaxDevices][kMidMaxSplits + 1];
  static bool ready[kMidMaxDevices] = {};
  static std::mutex lock;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMidMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
  {
    std::lock_guard<std::mutex> g(lock);
    if (!ready[dev]) {
      cudaError_t e = cudaFuncSetAttribute(gemm_mid_kernel<EPI, MB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      for (int s = 1; s <= kMidMaxSplits; ++s) {
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(s);
        q.blockDim = dim3(kMidThreads);
        q.dynamicSmemBytes = smem > (120u << 10) ? smem : (120u << 10);      // as if one CTA had an SM to itself
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = s;
        qa[0].val.clusterDim.y = 1;
        qa[0].val.clusterDim.z = 1;
        q.attrs = qa;
        q.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_mid_kernel<EPI, MB>, &q) != cudaSuccess) {
          cudaGetLastError();
          n = 0;
        }
        max_clusters[dev][s] = n;
      }
      ready[dev] = true;
    }
  }
  mid_shape(a.N, a.K, gated, max_clusters[dev], &a.tiles, &a.splits);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.tiles * a.splits);
  cfg.blockDim = dim3(kMidThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = a.splits;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_mid_kernel<EPI, MB>, mw, mx, a));
}

}  // namespace rl

using namespace rl;

extern "C" {

int rl_gemm_mid_max_rows() { return kMidMaxTokens; }

// Feature tiles of a product with N features that is not gated (the columns of the sums a `residual +=`
// epilogue hands out).
int rl_gemm_mid_tiles(int N) { return (N + kMidRows - 1) / kMidRows; }

// epilogue: 0 bfloat16 store into y [M, N]; 2 residual [M, N] (float32) += the product; 3 SiLU-gated
// product (w holds N gate rows then N up rows, y is [M, N]).  x [M, K] and w are bfloat16 with K a multiple
// of 8 and 16-byte aligned rows; 1 <= M <= 128.
// Hand out (epilogue 2, xw != null): xw [M, N] = bfloat16(residual * norm_w), sums_out [M, sums_out_ld]
// with column t = the sum over feature tile t (128 features) of residual^2, rl_gemm_mid_tiles(N) columns.
// Hand in (sums_in != null): row m of the product is scaled by rsqrt(sum of sums_in[m][0 .. sums_in_n) / K + eps).
// status: device int, bit 3 is set if a wait inside the kernel ran out.  Returns cudaErrorInvalidValue for
// shapes it does not take.
int rl_gemm_mid(const void* x, int ldx, const void* w, void* y, int ldy, int epilogue, int M, int N, int K,
                float* residual, int ldr, const void* norm_w, int norm_w_f32, void* xw, int ldxw, float* sums_out,
                int sums_out_ld, const float* sums_in, int sums_in_ld, int sums_in_n, float eps, int* status,
                cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > kMidMaxTokens || K % 8 != 0 || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(w) & 15) || status == nullptr ||
      (epilogue != kMidBf16 && epilogue != kMidSwiglu && epilogue != kMidResidual))
    return static_cast<int>(cudaErrorInvalidValue);
  if (epilogue == kMidResidual) {
    if (residual == nullptr || ldr % 4 != 0 || (reinterpret_cast<uintptr_t>(residual) & 15))
      return static_cast<int>(cudaErrorInvalidValue);
    if (xw != nullptr && (norm_w == nullptr || sums_out == nullptr || sums_out_ld < rl_gemm_mid_tiles(N)))
      return static_cast<int>(cudaErrorInvalidValue);
  } else if (y == nullptr || xw != nullptr) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (sums_in != nullptr && (sums_in_n <= 0 || sums_in_ld < sums_in_n)) return static_cast<int>(cudaErrorInvalidValue);
  const bool gated = epilogue == kMidSwiglu;
  MidArgs a;
  a.y = y;
  a.ldy = ldy;
  a.residual = residual;
  a.ldr = ldr;
  a.norm_w = norm_w;
  a.norm_w_f32 = norm_w_f32;
  a.xw = static_cast<bf16*>(xw);
  a.ldxw = ldxw;
  a.sums_out = sums_out;
  a.sums_out_ld = sums_out_ld;
  a.sums_in = sums_in;
  a.sums_in_ld = sums_in_ld;
  a.sums_in_n = sums_in_n;
  a.eps = eps;
  a.M = M;
  a.N = N;
  a.K = K;
  a.n_up = N;
  a.vec_y = y != nullptr && ldy % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 7) == 0;
  a.vec_xw = xw != nullptr && ldxw % 4 == 0 && (reinterpret_cast<uintptr_t>(xw) & 7) == 0;
  a.status = status;
  const int mb = mid_width(M);
  CUtensorMap mw, mx;
  if (!mid_map(&mw, w, gated ? 2 * N : N, K, K, gated ? kMidRows / 2 : kMidRows)) return static_cast<int>(cudaErrorNotSupported);
  if (!mid_map(&mx, x, M, K, ldx, mb)) return static_cast<int>(cudaErrorNotSupported);
#define RL_MID_CASE(E)                                                 \
  case E:                                                              \
    if (mb == 32) return launch_mid<E, 32>(mw, mx, a, gated, stream);         \
    if (mb == 64) return launch_mid<E, 64>(mw, mx, a, gated, stream);         \
    return launch_mid<E, 128>(mw, mx, a, gated, stream)
  switch (epilogue) {
    RL_MID_CASE(kMidBf16);
    RL_MID_CASE(kMidResidual);
    RL_MID_CASE(kMidSwiglu);
  }
#undef RL_MID_CASE
  return static_cast<int>(cudaErrorInvalidValue);
}

}  // extern "C"
