// y[M, N] = x[M, K] . W[N, K]^T for many rows (prompt portions), bfloat16 operands, on the
// fifth-generation tensor cores: tcgen05.mma with the accumulator in tensor memory (TMEM),
// operands brought into shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle).
//
// A CTA computes 128 x 256 (or 128 x 128) tiles of y, one after another (persistent: one CTA per SM); the
// epilogue of a tile overlaps the MMAs of the next.  Warp roles:
//   warp 0     producer: one lane issues the TMA loads of the A (x) and B (W) tiles of every
//              64-wide k block into a ring of shared-memory stages and arms the stage's
//              "full" mbarrier with the byte count
//   warp 1     allocates TMEM (two accumulators); one lane issues the MMAs (four of K = 16 per
//              stage) and commits them to the stage's "empty" mbarrier, and after a tile's last
//              block to that accumulator's "full" mbarrier
//   warps 2-5  epilogue: each reads its quarter of the 128 TMEM lanes with tcgen05.ld and
//              writes bfloat16 or float32 rows (or adds into the float32 residual stream, or
//              forms silu(gate) * up when the B tile holds 64 gate rows and their 64 up rows)
// Both operands are K-major (x row-major, W [N, K] row-major), which is how the weights are
// stored.  No cluster multicast is used anywhere.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the CTA raises a flag in
// shared memory, all roles leave their loops, outstanding loads are waited for (again
// bounded), TMEM is freed, and bit 0 of *status is set for the host to read.  The kernel
// never traps and never spins without a limit.
#include <mutex>

#include "umma.cuh"

namespace rl {

constexpr int kBM = 128, kBK = 64, kUmmaK = 16;
constexpr int kMaxStages = 6;
constexpr int kStageBytesA = kBM * kBK * 2;
constexpr int kTcThreads = 192;          // 6 warps
// The tile is 128 x BN with BN = 128 or 256.  Per 64-wide k block the tensor core reads both
// operand tiles from shared memory: 32 KB per 256 clocks at BN = 128, which is all the shared
// memory delivers (128 B/clock), 48 KB per 512 clocks at BN = 256: the wider tile is the one that
// is not bound by shared memory.  Two accumulators live in TMEM: 2 x BN of its 512 columns.
template <int BN>
struct TileCfg {
  static constexpr int kStageBytesB = BN * kBK * 2;
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kTmemCols = 2 * BN;
};

enum TcEpilogue { kTcBf16 = 0, kTcF32 = 1, kTcAddResidual = 2, kTcSwiglu = 3 };

struct TcShared {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];     // the MMAs of a tile are done: the epilogue may read this TMEM buffer
  uint64_t acc_empty[2];    // the epilogue has read it: the next tile's MMAs may overwrite it
  uint32_t tmem_base;
  volatile int abort;
};

struct TcArgs {
  void* y;          // bf16 / float output, or the float32 residual stream
  int M, N, K, ldy;
  int n_up;         // kTcSwiglu: row of W where the up rows start (the number of gate rows)
  int tiles_m, tiles_n;
  int group_n;      // feature tiles per group of the tile order (see tc_tile)
  int* status;
};

// The order of the tiles: groups of group_n feature tiles, every row tile of a group before the next
// group, so that the CTAs that run together (tiles c, c + 1, ...) cover all rows of x and a few tiles of
// the weights: x stays in L2 and the weights are read from DRAM once.  Gives the tile's row tile and
// feature tile.
__device__ __forceinline__ void tc_tile(const TcArgs& a, int tile, int& mt, int& nt) {
  const int per_group = a.group_n * a.tiles_m;
  const int grp = tile / per_group, r = tile - grp * per_group;
  const int n_first = grp * a.group_n;
  const int gn = min(a.group_n, a.tiles_n - n_first);      // the last group may be narrower
  mt = r / gn;
  nt = n_first + r - mt * gn;
}

// The epilogue of one thread: row `row` of y (TMEM lane of `acc`), the tile's kBN accumulator columns from
// feature n0 on: bfloat16 or float32 store, `residual +=`, or silu(gate) * up when the first half of the
// columns are gate features and the second half their up features.
template <int EPI, int kBN>
__device__ __forceinline__ void tc_drain(const TcArgs& a, uint32_t acc, int row, int n0) {
  if (EPI == kTcSwiglu) {
#pragma unroll 1
    for (int c = 0; c < kBN / 2; c += 32) {
      float g[32], u[32], r[32];
      tmem_ld32(acc + c, g);
      tmem_ld32(acc + kBN / 2 + c, u);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float gt = __bfloat162float(__float2bfloat16_rn(g[i])), up = __bfloat162float(__float2bfloat16_rn(u[i]));
        r[i] = __fdividef(gt, 1.f + __expf(-gt)) * up;
      }
      if (row < a.M) {
        bf16* out = static_cast<bf16*>(a.y) + static_cast<size_t>(row) * a.ldy + n0 + c;
        if (n0 + c + 32 <= a.N && (a.ldy % 8 == 0)) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) store16(out + i, r + i);
        } else {
          for (int i = 0; i < 32 && n0 + c + i < a.N; ++i) out[i] = __float2bfloat16_rn(r[i]);
        }
      }
    }
  } else {
#pragma unroll 1
    for (int c = 0; c < kBN; c += 32) {
      float v[32];
      tmem_ld32(acc + c, v);
      if (row < a.M) {
        const size_t o = static_cast<size_t>(row) * a.ldy + n0 + c;
        const bool whole = (n0 + c + 32 <= a.N);
        if (EPI == kTcBf16) {
          bf16* out = static_cast<bf16*>(a.y) + o;
          if (whole && (a.ldy % 8 == 0)) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) store16(out + i, v + i);
          } else {
            for (int i = 0; i < 32 && n0 + c + i < a.N; ++i) out[i] = __float2bfloat16_rn(v[i]);
          }
        } else if (EPI == kTcF32) {
          float* out = static_cast<float*>(a.y) + o;
          if (whole && (a.ldy % 4 == 0)) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) store16(out + i, v + i);
          } else {
            for (int i = 0; i < 32 && n0 + c + i < a.N; ++i) out[i] = v[i];
          }
        } else {
          float* out = static_cast<float*>(a.y) + o;   // residual += bfloat16(product)
          if (whole && (a.ldy % 4 == 0)) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              float r4[4];
              load16(out + i, r4);
#pragma unroll
              for (int e = 0; e < 4; ++e) r4[e] += __bfloat162float(__float2bfloat16_rn(v[i + e]));
              store16(out + i, r4);
            }
          } else {
            for (int i = 0; i < 32 && n0 + c + i < a.N; ++i) out[i] += __bfloat162float(__float2bfloat16_rn(v[i]));
          }
        }
      }
    }
  }
}

// Persistent: CTA c takes tiles c, c + gridDim.x, ... of the order of tc_tile.  TMEM holds two
// accumulators: while the epilogue warps drain one tile, the MMAs of the next tile fill the other.
template <int EPI, int kBN>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcArgs a) {
  extern __shared__ unsigned char smem_raw[];
  // the stages need 1024-byte alignment for the 128-byte swizzle
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* base = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  constexpr int kStages = TileCfg<kBN>::kStages, kStageBytesB = TileCfg<kBN>::kStageBytesB;
  constexpr int kTmemCols = TileCfg<kBN>::kTmemCols;
  unsigned char* smem_a = base;
  unsigned char* smem_b = base + kStages * kStageBytesA;
  TcShared* sh = reinterpret_cast<TcShared*>(base + kStages * (kStageBytesA + kStageBytesB));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kTileN = (EPI == kTcSwiglu) ? kBN / 2 : kBN;   // gated: 64 gate features and their 64 up features
  const int nkb = (a.K + kBK - 1) / kBK;
  const int ntiles = a.tiles_m * a.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->acc_full[b], 1);
      mbar_init(&sh->acc_empty[b], 128);    // every epilogue thread arrives
    }
    sh->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // TMEM allocation is a whole-warp operation
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
      auto load_b = [&](int s, int kb, int n0) {
        if (EPI == kTcSwiglu) {
          tma_load_2d(smem_b + s * kStageBytesB, &map_b, &sh->full[s], kb * kBK, n0);
          tma_load_2d(smem_b + s * kStageBytesB + kStageBytesB / 2, &map_b, &sh->full[s], kb * kBK, a.n_up + n0);
        } else {
          tma_load_2d(smem_b + s * kStageBytesB, &map_b, &sh->full[s], kb * kBK, n0);
        }
      };
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      // The weights do not depend on earlier kernels of the step: the first stages' weight tiles are
      // asked for before the wait on those kernels, the activation tiles after it.
      const int pre = (blockIdx.x < ntiles) ? min(kStages, nkb) : 0;
      int pre_mt = 0, pre_nt = 0;
      if (blockIdx.x < ntiles) tc_tile(a, blockIdx.x, pre_mt, pre_nt);
      const int pre_n0 = pre_nt * kTileN;
      for (int kb = 0; kb < pre; ++kb) {
        mbar_expect_tx(&sh->full[kb], kStageBytesA + kStageBytesB);
        load_b(kb, kb, pre_n0);
      }
      pdl_wait();        // x is written by earlier kernels of the step
      int it = 0, issued = 0;      // it: k blocks over all of this CTA's tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        int mt, nt;
        tc_tile(a, tile, mt, nt);
        const int m0 = mt * kBM, n0 = nt * kTileN;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % kStages;
          if (it < pre) {          // armed above, the weight tile is on its way
            tma_load_2d(smem_a + s * kStageBytesA, &map_a, &sh->full[s], kb * kBK, m0);
            ++issued;
            continue;
          }
          const uint32_t parity = ((it / kStages) & 1) ^ 1;        // a fresh barrier passes a wait on parity 1
          ok = mbar_wait(&sh->empty[s], parity, &sh->abort);
          if (!ok) break;
          mbar_expect_tx(&sh->full[s], kStageBytesA + kStageBytesB);
          tma_load_2d(smem_a + s * kStageBytesA, &map_a, &sh->full[s], kb * kBK, m0);
          load_b(s, kb, n0);
          ++issued;
        }
      }
      if (sh->abort) {
        // loads still in flight write shared memory: wait for them (bounded) before the CTA ends
        for (int i2 = max(0, issued - kStages); i2 < issued; ++i2) {
          const int s = i2 % kStages;
          for (int i = 0; i < kSpinLimit && !mbar_try_wait(&sh->full[s], (i2 / kStages) & 1); ++i) {
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kBM, kBN);
      bool ok = true;
      int it = 0, t = 0;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++t) {
        const int buf = t & 1;
        ok = mbar_wait(&sh->acc_empty[buf], ((t >> 1) & 1) ^ 1, &sh->abort);   // fresh: passes at once
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem + buf * kBN;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % kStages;
          ok = mbar_wait(&sh->full[s], (it / kStages) & 1, &sh->abort);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + s * kStageBytesA), b_addr = smem_u32(smem_b + s * kStageBytesB);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // inside the 128-byte swizzle atom the next 16 k (32 bytes) are 32 bytes further on
            umma_bf16(acc, umma_desc(a_addr + k * kUmmaK * 2), umma_desc(b_addr + k * kUmmaK * 2), idesc,
                      (kb | k) != 0);
          }
          umma_commit(&sh->empty[s]);     // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(&sh->acc_full[buf]);
      }
    }
  } else {
    // epilogue warps 2..5: warp w may touch TMEM lanes 32 * (w % 4) .. + 32
    const int q = warp & 3;
    int t = 0;
    pdl_wait();        // y (or the residual stream) may still be in use by earlier kernels
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++t) {
      const int buf = t & 1;
      int mt, nt;
        tc_tile(a, tile, mt, nt);
        const int m0 = mt * kBM, n0 = nt * kTileN;
      if (!mbar_wait(&sh->acc_full[buf], (t >> 1) & 1, &sh->abort)) break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t acc = tmem + buf * kBN + (static_cast<uint32_t>(q * 32) << 16);
      tc_drain<EPI, kBN>(a, acc, row, n0);
      tc_fence_before();
      mbar_arrive(&sh->acc_empty[buf]);     // this thread is done with the buffer
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && sh->abort) atomicOr(a.status, 1);
}

// ---------------------------------------------------------------------------- CTA pairs
//
// The same product with tcgen05.mma.cta_group::2: two CTAs of a cluster (on two SMs) work on one 256 x 256
// tile of y.  Each loads its own 128 rows of x and HALF of the weight tile (128 of its 256 rows) per k block,
// 32 KB instead of the 48 KB that a CTA alone loads for a 128 x 256 tile, and the tensor cores of both SMs
// read both halves: a third less traffic from L2 into shared memory per operation, which is what bounds the
// kernel above (its tensor pipe is busy two thirds of the time).  The accumulator of CTA r is rows
// 128 r .. 128 r + 127 of the tile, in its own tensor memory.
//
// The even CTA of the pair (the leader) issues the MMAs.  Its "full" barrier of a stage counts the bytes of
// all four loads (the peer's loads name the leader's barrier: cp.async.bulk.tensor with .cta_group::2, no
// multicast); a tcgen05.commit with .multicast::cluster tells both CTAs that a stage is free again or that
// an accumulator is complete; the epilogue threads of both CTAs arrive at the leader's "accumulator drained"
// barrier.  The cluster meets once after the barriers are set up and once before tensor memory is freed.
// Every mbarrier wait is bounded as above.

constexpr int kPairStages = 6;            // 6 x (16 KB of x + 16 KB of weights) per CTA
constexpr int kPairBN = 256;
constexpr int kPairStageBytes = kStageBytesA + kBM * kBK * 2;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared-memory window, of `p` of this CTA's layout in CTA `rank`.
__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// A TMA tile load into this CTA's shared memory whose bytes are counted at a barrier that may be the other
// CTA's of the pair (`cluster_bar`: an address of cluster_addr).  Not a multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// When the MMAs issued so far are done, one arrival at `bar` (this CTA's layout) in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(static_cast<uint16_t>(3))
      : "memory");
}

// Persistent: pair c takes the 256-row tiles c, c + pairs, ... of the order of tc_tile (tiles_m counts
// 256-row tiles here).
template <int EPI>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcArgs a) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* base = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  constexpr int kStageBytesB = kBM * kBK * 2;             // this CTA's half of the weight tile
  constexpr int kTmemCols = 2 * kPairBN;
  unsigned char* smem_a = base;
  unsigned char* smem_b = base + kPairStages * kStageBytesA;
  TcShared* sh = reinterpret_cast<TcShared*>(base + kPairStages * kPairStageBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                // 0: the leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  constexpr int kTileN = (EPI == kTcSwiglu) ? kPairBN / 2 : kPairBN;
  const int nkb = (a.K + kBK - 1) / kBK;
  const int ntiles = a.tiles_m * a.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->acc_full[b], 1);
      mbar_init(&sh->acc_empty[b], 256);    // every epilogue thread of both CTAs arrives (at the leader's)
    }
    sh->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // the same warp of both CTAs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();          // both CTAs' barriers exist before anything arrives at them
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  pdl_launch();

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      // this CTA's half of the weight tile: rows n0 + 128 r; gated: the leader the gate rows, the peer the up rows
      auto b_row = [&](int n0) { return EPI == kTcSwiglu ? (rank ? a.n_up + n0 : n0) : n0 + static_cast<int>(rank) * kBM; };
      // The weights do not depend on earlier kernels of the step: the first stages' weight tiles are
      // asked for before the wait on those kernels, the activation tiles after it.
      const int pre = (pair < ntiles) ? min(kPairStages, nkb) : 0;
      int pre_mt = 0, pre_nt = 0;
      if (pair < ntiles) tc_tile(a, pair, pre_mt, pre_nt);
      for (int kb = 0; kb < pre; ++kb) {
        if (rank == 0) mbar_expect_tx(&sh->full[kb], 2 * kPairStageBytes);
        tma_load_2d_pair(smem_b + kb * kStageBytesB, &map_b, cluster_addr(&sh->full[kb], 0), kb * kBK, b_row(pre_nt * kTileN));
      }
      pdl_wait();        // x is written by earlier kernels of the step
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < ntiles && ok; tile += npairs) {
        int mt, nt;
        tc_tile(a, tile, mt, nt);
        const int m0 = mt * 2 * kBM + static_cast<int>(rank) * kBM, n0 = nt * kTileN;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % kPairStages;
          const uint32_t bar = cluster_addr(&sh->full[s], 0);
          if (it >= pre) {
            const uint32_t parity = ((it / kPairStages) & 1) ^ 1;        // a fresh barrier passes a wait on parity 1
            ok = mbar_wait(&sh->empty[s], parity, &sh->abort);
            if (!ok) break;
            if (rank == 0) mbar_expect_tx(&sh->full[s], 2 * kPairStageBytes);
            tma_load_2d_pair(smem_b + s * kStageBytesB, &map_b, bar, kb * kBK, b_row(n0));
          }
          tma_load_2d_pair(smem_a + s * kStageBytesA, &map_a, bar, kb * kBK, m0);
        }
      }
      if (sh->abort) {
        // loads still in flight write shared memory, and their bytes are counted at the leader: give them
        // time to land (they take microseconds) before the CTA goes to the cluster's last meeting
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(2 * kBM, kPairBN);
      bool ok = true;
      int it = 0, t = 0;
      for (int tile = pair; tile < ntiles && ok; tile += npairs, ++t) {
        const int buf = t & 1;
        ok = mbar_wait(&sh->acc_empty[buf], ((t >> 1) & 1) ^ 1, &sh->abort);   // fresh: passes at once
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem + buf * kPairBN;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % kPairStages;
          ok = mbar_wait(&sh->full[s], (it / kPairStages) & 1, &sh->abort);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + s * kStageBytesA), b_addr = smem_u32(smem_b + s * kStageBytesB);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_bf16_pair(acc, umma_desc(a_addr + k * kUmmaK * 2), umma_desc(b_addr + k * kUmmaK * 2), idesc,
                           (kb | k) != 0);
          umma_commit_pair(&sh->empty[s]);     // both CTAs' stage is free once these MMAs have read it
        }
        if (ok) umma_commit_pair(&sh->acc_full[buf]);
      }
    }
  } else {
    // epilogue warps 2..5 of both CTAs: warp w may touch TMEM lanes 32 * (w % 4) .. + 32 of its own CTA
    const int q = warp & 3;
    int t = 0;
    pdl_wait();        // y (or the residual stream) may still be in use by earlier kernels
    for (int tile = pair; tile < ntiles; tile += npairs, ++t) {
      const int buf = t & 1;
      int mt, nt;
      tc_tile(a, tile, mt, nt);
      const int m0 = mt * 2 * kBM + static_cast<int>(rank) * kBM, n0 = nt * kTileN;
      if (!mbar_wait(&sh->acc_full[buf], (t >> 1) & 1, &sh->abort)) break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t acc = tmem + buf * kPairBN + (static_cast<uint32_t>(q * 32) << 16);
      tc_drain<EPI, kPairBN>(a, acc, row, n0);
      tc_fence_before();
      mbar_arrive_cluster(cluster_addr(&sh->acc_empty[buf], 0));     // this thread is done with the buffer
    }
  }
  // neither CTA leaves (or frees tensor memory) while the other may still read its shared memory or arrive
  // at its barriers
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && sh->abort) atomicOr(a.status, 1);
}

// ---------------------------------------------------------------------------- host side

// A [rows, K] bfloat16 matrix with row pitch ld (elements), tiles of box_rows x 64, 128-byte swizzle.
static bool make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {   // box_rows <= 256
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {kBK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int EPI, int BN>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a0, int sm_count, cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  const size_t smem = static_cast<size_t>(Cfg::kStages) * (kStageBytesA + Cfg::kStageBytesB) + sizeof(TcShared) + 1024;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    attr = true;
  }
  const int tile_n = (EPI == kTcSwiglu) ? BN / 2 : BN;
  TcArgs a = a0;
  a.tiles_n = (a.N + tile_n - 1) / tile_n;
  a.tiles_m = (a.M + kBM - 1) / kBM;
  const int tiles = a.tiles_m * a.tiles_n;
  a.group_n = (sm_count + a.tiles_m / 2) / a.tiles_m;      // a wave of CTAs covers about one group
  if (a.group_n < 1) a.group_n = 1;
  if (a.group_n > a.tiles_n) a.group_n = a.tiles_n;
  dim3 grid(tiles < sm_count ? tiles : sm_count);
  launch_kernel(gemm_tc_kernel<EPI, BN>, grid, dim3(kTcThreads), smem, stream, ma, mb, a);
  return static_cast<int>(cudaGetLastError());
}

constexpr int kTcMaxDevices = 64;

template <int EPI>
static int launch_tc_pair(const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a0, int sm_count, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(kPairStages) * kPairStageBytes + sizeof(TcShared) + 1024;
  // per device, once: the kernel's shared-memory limit and how many pairs can be resident
  static int max_pairs[kTcMaxDevices];
  static bool ready[kTcMaxDevices] = {};
  static std::mutex lock;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kTcMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  {
    std::lock_guard<std::mutex> g(lock);
    if (!ready[dev]) {
      cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      cfg.gridDim = dim3(2);
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<EPI>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      max_pairs[dev] = n;
      ready[dev] = true;
    }
  }
  int pairs = max_pairs[dev] < sm_count / 2 ? max_pairs[dev] : sm_count / 2;
  if (pairs < 1) return static_cast<int>(cudaErrorNotSupported);
  const int tile_n = (EPI == kTcSwiglu) ? kPairBN / 2 : kPairBN;
  TcArgs a = a0;
  a.tiles_n = (a.N + tile_n - 1) / tile_n;
  a.tiles_m = (a.M + 2 * kBM - 1) / (2 * kBM);
  const int tiles = a.tiles_m * a.tiles_n;
  a.group_n = (pairs + a.tiles_m / 2) / a.tiles_m;      // a wave of pairs covers about one group
  if (a.group_n < 1) a.group_n = 1;
  if (a.group_n > a.tiles_n) a.group_n = a.tiles_n;
  cfg.gridDim = dim3(2 * (tiles < pairs ? tiles : pairs));
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<EPI>, ma, mb, a));
}

// 256-wide tiles unless they would leave most SMs without a tile.
static int choose_bn(int M, int N, int epilogue, int sm_count) {
  const int tile_n = epilogue == kTcSwiglu ? 128 : 256;
  const int tiles = ((M + kBM - 1) / kBM) * ((N + tile_n - 1) / tile_n);
  return tiles * 10 >= sm_count * 8 ? 256 : 128;
}

}  // namespace rl

using namespace rl;

extern "C" {

// epilogue: 0 bf16 store, 1 float32 store, 2 residual (float32) += product, 3 SiLU-gated product
// (w holds N gate rows then N up rows; y is [M, N] bfloat16).  x [M, K] and w [N or 2N, K] are
// bfloat16 with K a multiple of 8 and 16-byte aligned rows.  status: device int, bit 0 is set if a
// wait inside the kernel ran out.  force_bn: 0 = choose the tiling; 128 or 256 = one CTA per 128-row tile of
// that width; 512 = CTA pairs (256 x 256 tiles, cta_group::2).
// Returns cudaErrorInvalidValue for shapes it does not take.
int rl_gemm_tc(const void* x, int ldx, const void* w, void* y, int ldy, int epilogue, int M, int N, int K,
               int* status, int sm_count, int force_bn, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0 || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return static_cast<int>(cudaErrorInvalidValue);
  CUtensorMap ma, mb;
  const bool gated = epilogue == kTcSwiglu;
  // pairs from two row tiles on (a single row tile would leave the peer's half of the MMA empty)
  const int bn = force_bn > 0 ? force_bn : (M > kBM ? 512 : choose_bn(M, N, epilogue, sm_count));
  if (bn != 128 && bn != 256 && bn != 512) return static_cast<int>(cudaErrorInvalidValue);
  if (!make_map(&ma, x, M, K, ldx, kBM)) return static_cast<int>(cudaErrorNotSupported);
  if (bn == 512) {
    if (!make_map(&mb, w, gated ? 2 * N : N, K, K, kBM)) return static_cast<int>(cudaErrorNotSupported);
    TcArgs a;
    a.y = y;
    a.M = M;
    a.N = N;
    a.K = K;
    a.ldy = ldy;
    a.n_up = N;
    a.status = status;
    switch (epilogue) {
      case kTcBf16: return launch_tc_pair<kTcBf16>(ma, mb, a, sm_count, stream);
      case kTcF32: return launch_tc_pair<kTcF32>(ma, mb, a, sm_count, stream);
      case kTcAddResidual: return launch_tc_pair<kTcAddResidual>(ma, mb, a, sm_count, stream);
      case kTcSwiglu: return launch_tc_pair<kTcSwiglu>(ma, mb, a, sm_count, stream);
    }
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (!make_map(&mb, w, gated ? 2 * N : N, K, K, gated ? bn / 2 : bn)) return static_cast<int>(cudaErrorNotSupported);
  TcArgs a;
  a.y = y;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldy = ldy;
  a.n_up = N;
  a.status = status;
#define RL_TC_CASE(E)                                                                   \
  case E:                                                                               \
    return bn == 256 ? launch_tc<E, 256>(ma, mb, a, sm_count, stream) : launch_tc<E, 128>(ma, mb, a, sm_count, stream)
  switch (epilogue) {
    RL_TC_CASE(kTcBf16);
    RL_TC_CASE(kTcF32);
    RL_TC_CASE(kTcAddResidual);
    RL_TC_CASE(kTcSwiglu);
  }
#undef RL_TC_CASE
  return static_cast<int>(cudaErrorInvalidValue);
}

}  // extern "C"
