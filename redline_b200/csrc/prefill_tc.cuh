// Prompt-portion attention on the fifth-generation tensor cores (bfloat16, head size 64 or 128).
//
// Included by attention.cu.  An item of work is a tile of up to 128 consecutive query rows of one
// sequence for TWO query heads of one kv head (the last pair of an odd group has one): the two
// heads are the CTA's two "slots", they attend to the same keys and values, so a K tile and a V
// tile are brought into shared memory once for both.  Persistent CTAs (one per SM) take items
// one after another, longest first, and the pipeline runs on across items.  Per item the keys
// come in tiles of 128; for each slot and key tile:
//   S = Q K^T      tcgen05.mma, 128 x 128, k = head size, accumulator in tensor memory
//   softmax        two threads per query row (eight warps per slot, so that every scheduler of the SM
//                  has four row warps to choose from) read the row of S from tensor memory, each
//                  keeps the running maximum of the row and the denominator of its 64 keys in
//                  float32 and writes their P as bfloat16 back into tensor memory
//   O += P V       tcgen05.mma with P as the A operand from tensor memory and V as it lies in the
//                  cache (a key's values contiguous: the B operand in MN-major form); O stays in
//                  tensor memory for the whole item and is accumulated by the tensor core
// The running maximum that P is scaled by is moved (and O and the denominator rescaled, by the
// row's own thread, between two products) only when a warp sees a row's maximum grow by more
// than 2^8 over it: P stays below 256, which bfloat16 holds as well as numbers below 1, and the
// rescaling of O, a round trip through registers, becomes rare after a row's first tiles.  The
// result is the same sum: every term of a row carries the same factor, which the division by
// the denominator takes out.
// While the rows of one slot are in their softmax, the tensor core works on the other slot's
// products.  Tensor memory (512 columns): S0 at column 0, S1 at 128, O0 at 256, O1 at 256 + head
// size.  At head size 64 that leaves 128 columns, and P has columns of its own (P0 at 384, P1 at
// 448): the S product of the next key tile is issued as soon as the rows have READ this tile's S
// into registers, so it is done before they have finished with this tile, and the rows never wait
// for the tensor core.  At head size 128 the columns are all taken: P lies over the first 64
// columns of its S, and the next S product has to wait for the O product that reads P.
// Warp roles: warps 0-7 rows of slot 0, warps 8-15 rows of slot 1 (warp w owns TMEM lanes
// 32 (w % 4) ..), warp 16 brings both Q tiles once per item and the K tiles, warp 17 the V tiles,
// from the paged cache with 16-byte cp.async copies (zero-filled outside the live keys), lane 0
// of warp 18 issues the MMAs of slot 0 and lane 0 of warp 19 those of slot 1 (a slot's products
// never wait for the other slot's rows).  Everything is handed over through mbarriers; every wait is
// bounded (kSpinLimit polls), after which the CTA raises an abort flag, all roles leave their
// loops, the copies in flight are waited for, TMEM is freed and bit 2 of *status is set.
#pragma once

#include "umma.cuh"

namespace rl {

constexpr int kTcRows = 128, kTcKeys = 128;
constexpr int kTcRowWarps = 16;                        // two threads to a row: 8 warps per slot
constexpr int kTcThreads = (kTcRowWarps + 4) * 32;      // the row warps, two loaders, two MMA warps
constexpr int kTcHalves = kD / 64;                      // a head's columns in halves of 64 (128 bytes)
constexpr int kTcHalfBytes = 128 * 128;                 // 128 rows x 64 bfloat16, 128-byte swizzled
constexpr int kTcTileBytes = kTcHalves * kTcHalfBytes;  // a Q, K or V tile
constexpr int kTcStages = kD == 64 ? 3 : 2;             // K and V stages
constexpr int kTcTmemCols = 512;
constexpr int kTcColO = 256;                            // O of slot s at kTcColO + s * kD
constexpr bool kTcOwnP = kD == 64;                      // P has tensor-memory columns of its own (else: over S)
constexpr int kTcColP = 384;                            // with columns of its own: P of slot s at kTcColP + s * 64
constexpr float kTcGrow = 8.f;                          // log2 of the growth of a row's maximum that moves the reference

struct PrefillTcShared {
  uint64_t q_full[2], q_free[2];                  // per slot: Q of an item has landed / its last S product has read it
  uint64_t k_full[kTcStages], k_free[kTcStages];  // loader's arrival / the tile's last S product is done
  uint64_t v_full[kTcStages], v_free[kTcStages];  // loader's arrival / the tile's last O product is done
  uint64_t qk_done[2], pv_done[2];                // per slot, MMA commits: S of the tile is ready / its O product is done
  uint64_t p_ready[2];                            // per slot: its four row warps have written P
  uint64_t s_free[2];                             // per slot: its four row warps have read S (used if P has its own columns)
  uint64_t pair[2][4];                            // per slot and quarter of rows: the two warps that share the rows meet (2 arrivals)
  float l_half[2][2][kTcRows];                    // [slot][half][row]: a thread's part of the row's denominator
  uint64_t o_free[2];                             // per slot: its four row warps have read the item's O
  uint32_t tmem_base;
  volatile int abort;
};
constexpr size_t kPrefillTcSmem = 1024 + (2 + 2 * kTcStages) * kTcTileBytes + sizeof(PrefillTcShared);

// One item of a CTA's work: a tile of query rows for up to two query heads of one kv head.
struct TcItem {
  int seq, tok0, rows, head0, kvh;
  bool two;                            // the second slot has a head (head0 + 1)
  int pos0, k_end, lo0, k_begin, nt;   // first position, keys [lo0, k_end) are live, nt key tiles from k_begin
};

// Item `rem` of a tile of query rows: kv head rem / pairs, pair of heads rem % pairs.
__device__ __forceinline__ TcItem tc_item(const PrefillArgs<bf16>& a, int tile, int rem, int pairs) {
  TcItem w;
  const int G = a.hq / a.hkv;
  w.kvh = rem / pairs;
  const int p = rem - w.kvh * pairs;
  w.head0 = w.kvh * G + 2 * p;
  w.two = 2 * p + 1 < G;
  w.seq = a.tile_seq[tile];
  w.tok0 = a.tile_tok[tile];
  w.rows = a.tile_rows[tile];
  w.pos0 = a.positions[w.tok0];
  w.k_end = w.pos0 + w.rows;
  w.lo0 = (a.window > 0 && w.pos0 + 1 > a.window) ? w.pos0 + 1 - a.window : 0;
  w.k_begin = w.lo0 / kTcKeys * kTcKeys;
  w.nt = (w.k_end - w.k_begin + kTcKeys - 1) / kTcKeys;
  return w;
}

// Shared-memory matrix descriptor of an MN-major tile: 64 elements of the MN dimension contiguous
// (128 bytes), one such row per k, 128-byte swizzled in groups of 8 k (1024 bytes apart).
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);        // start address
  d |= static_cast<uint64_t>(1) << 16;                            // leading byte offset: next 64 of MN (none here)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                    // stride byte offset: 8 k x 128 B
  d |= static_cast<uint64_t>(1) << 46;                            // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;                            // layout: 128-byte swizzle
  return d;
}

// D (tensor memory) += A (tensor memory: a row per lane, two bfloat16 of k per 32-bit column) x B (shared memory).
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 16 consecutive 32-bit columns of this thread's TMEM lane, load (no wait) and store.
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// 64 consecutive 32-bit columns of this thread's TMEM lane in one instruction (no wait).
__device__ __forceinline__ void tmem_ld64_issue(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Two floats in one 64-bit register and the packed arithmetic on them (one instruction for two lanes).
__device__ __forceinline__ uint64_t f32x2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void f32x2_split(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Sets the scores of 64 keys that a row may not see to -inf: key j of them is live if jmin <= j <= jmax.
// Without a window (the same for all threads) there is no lower limit to test.
__device__ __forceinline__ void tc_mask64(uint32_t* sr, int jmax, int jmin, bool window) {
  if (!window) {
#pragma unroll
    for (int j = 0; j < 64; ++j)
      if (j > jmax) sr[j] = 0xff800000u;
  } else {
#pragma unroll
    for (int j = 0; j < 64; ++j)
      if (j > jmax || j < jmin) sr[j] = 0xff800000u;
  }
}

// The items of a CTA: in round k the CTAs take items k G .. k G + G - 1 (G CTAs), in odd rounds in
// reverse order, so that the CTA with the longest item of one round has the shortest of the next.
// Gives the CTA's next item and moves `round` on; -1 when there is none.
__device__ __forceinline__ int tc_next_item(int& round, int n_items) {
  const int G = gridDim.x;
  while (round * G < n_items) {
    const int k = round++;
    const int item = k * G + ((k & 1) ? G - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x));
    if (item < n_items) return item;
  }
  return -1;
}

// A role's walk over the CTA's items.  Every role walks the same list and keeps the same counts:
// `it` items so far, `g` key tiles of all items so far (tile g uses K / V stage g % kTcStages in
// its (g / kTcStages)-th use), and the same two counts for the second slot, which sits out the
// items that have one head only (its barriers then see no phase).
struct TcWalk {
  int round = 0, item = -1;
  int it = 0, g = 0, it1 = 0, g1 = 0;
  TcItem w;
  __device__ __forceinline__ bool first(const PrefillArgs<bf16>& a, int n_items, int pairs, int tiles) {
    item = tc_next_item(round, n_items);
    if (item < 0) return false;
    w = load(a, item, pairs, tiles);
    return true;
  }
  // moves to the CTA's next item; false when there is none
  __device__ __forceinline__ bool next(const PrefillArgs<bf16>& a, int n_items, int pairs, int tiles) {
    ++it;
    g += w.nt;
    if (w.two) {
      ++it1;
      g1 += w.nt;
    }
    return first(a, n_items, pairs, tiles);
  }
  // Items are numbered longest first (a later tile of a sequence attends to more keys), the kv heads and
  // pairs of a tile next to each other, so that CTAs that run together share K and V in L2.
  static __device__ __forceinline__ TcItem load(const PrefillArgs<bf16>& a, int item, int pairs, int tiles) {
    const int per_tile = a.hkv * pairs;
    const int t = item / per_tile;
    return tc_item(a, tiles - 1 - t, item - t * per_tile, pairs);
  }
};

__global__ void __launch_bounds__(kTcThreads, 1)
prefill_attn_tc_kernel(const PrefillArgs<bf16> a, int tiles, int* status) {
  static_assert(kD == 64 || kD == 128, "this kernel is written for head sizes 64 and 128");
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* base = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* q_s = base;                                        // one tile per slot
  unsigned char* k_s = base + 2 * kTcTileBytes;                     // kTcStages tiles
  unsigned char* v_s = base + (2 + kTcStages) * kTcTileBytes;       // kTcStages tiles
  PrefillTcShared* sh = reinterpret_cast<PrefillTcShared*>(base + (2 + 2 * kTcStages) * kTcTileBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pairs = (a.hq / a.hkv + 1) / 2;
  const int n_items = tiles * a.hkv * pairs;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->q_full[s], 1);
      mbar_init(&sh->q_free[s], 1);
      mbar_init(&sh->qk_done[s], 1);
      mbar_init(&sh->pv_done[s], 1);
      mbar_init(&sh->p_ready[s], 8);      // one arrival per row warp of the slot (its lanes meet first)
      mbar_init(&sh->s_free[s], 8);
      mbar_init(&sh->o_free[s], 8);
      for (int qq = 0; qq < 4; ++qq) mbar_init(&sh->pair[s][qq], 2);
    }
    for (int b = 0; b < kTcStages; ++b) {
      mbar_init(&sh->k_full[b], 1);
      mbar_init(&sh->k_free[b], 2);       // one commit per slot (a lone slot commits twice)
      mbar_init(&sh->v_full[b], 1);
      mbar_init(&sh->v_free[b], 2);
    }
    sh->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kTcRowWarps + 2) {   // TMEM allocation is a whole-warp operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)),
                 "r"(kTcTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  pdl_launch();
  pdl_wait();        // q and the newest keys come from the kernels before this one

  if (warp == kTcRowWarps || warp == kTcRowWarps + 1) {
    // ------------------------------------------------------------------ loaders: warp 8 K (and both Q), warp 9 V
    const bool is_v = warp == kTcRowWarps + 1;
    const int ps_shift = __ffs(a.page_size) - 1, ps_mask = a.page_size - 1;
    const size_t head_stride = static_cast<size_t>(a.page_size) * kD;
    constexpr int CPR = kD / 8;                          // 16-byte chunks of a row
    constexpr int RPI = 32 / CPR;                        // rows that the warp's lanes cover at once
    const int c = lane % CPR, rr = lane / CPR;           // chunk of a row, row within a round of RPI rows
    // a row's chunk c lies in half c / 8 at 16-byte position (c % 8) ^ (row % 8) of the row's 128 bytes
    const uint32_t c_half = static_cast<uint32_t>(c >> 3) * kTcHalfBytes;
    const int c7 = c & 7;
    const bf16* cache = is_v ? a.vcache : a.kcache;
    const uint32_t stage0 = smem_u32(is_v ? v_s : k_s);
    uint64_t* full = is_v ? sh->v_full : sh->k_full;
    uint64_t* freed = is_v ? sh->v_free : sh->k_free;
    const int rpp = min(a.page_size, kTcKeys);            // rows of a page that lie in a tile
    const int pages = kTcKeys / rpp;                      // pages per tile (at most eight: pages of 16 keys or more)
    const uint32_t lane_src = static_cast<uint32_t>(rr * kD + c * 8);
    // Before the warp blocks on a stage or a Q buffer, what it has copied so far is handed over: the
    // reader of a stage never waits for a tile that waits for that reader.
    bool ok = true;
    int pending = -1;                                     // a tile copied but not handed over (its stage)
    int q_pending = 0;                                    // bit s: Q of slot s copied but not handed over
    auto hand_over = [&](bool all) {
      if (all) cp_async_wait<0>(); else cp_async_wait<1>();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (q_pending & 1) mbar_arrive(&sh->q_full[0]);
        if (q_pending & 2) mbar_arrive(&sh->q_full[1]);
        if (pending >= 0) mbar_arrive(&full[pending]);
      }
      q_pending = 0;
      pending = -1;
    };
    TcWalk wk;
    for (bool more = wk.first(a, n_items, pairs, tiles); more && ok; more = wk.next(a, n_items, pairs, tiles)) {
      const TcItem& w = wk.w;
      const int32_t* bt = a.block_table + static_cast<size_t>(w.seq) * a.max_blocks;
      if (!is_v) {
        for (int s = 0; s < (w.two ? 2 : 1) && ok; ++s) {
          const int n = s == 0 ? wk.it : wk.it1;          // the slot's items so far
          if (!mbar_try_wait(&sh->q_free[s], (n & 1) ^ 1)) {
            hand_over(true);
            ok = mbar_wait(&sh->q_free[s], (n & 1) ^ 1, &sh->abort);
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (pending >= 0) hand_over(true);              // (keeps the groups of Q and of a tile apart)
          const uint32_t q_u = smem_u32(q_s) + s * kTcTileBytes;
          for (int j = 0; j < kTcRows / RPI; ++j) {
            const int r = j * RPI + rr;
            const bool live = r < w.rows;
            const bf16* src = a.q + static_cast<size_t>(w.tok0 + (live ? r : 0)) * a.q_stride + (w.head0 + s) * kD + c * 8;
            cp_async16_s(q_u + c_half + r * 128 + ((c7 ^ (r & 7)) << 4), src, live);
          }
          cp_async_commit();
          q_pending |= 1 << s;
        }
        if (!ok) break;
      }
      for (int i = 0; i < w.nt; ++i) {
        const int g = wk.g + i;
        const int b = g % kTcStages;
        const uint32_t par = ((g / kTcStages) & 1) ^ 1;   // a fresh barrier passes a wait on parity 1
        const int k0 = w.k_begin + i * kTcKeys;
        // the tile's pages: lane l < pages holds the id of page l, 0 for one without a live key
        int my_page = 0;
        {
          const int pidx = (k0 >> ps_shift) + lane;
          const int first = max(k0, w.lo0) >> ps_shift, last = (min(k0 + kTcKeys, w.k_end) - 1) >> ps_shift;
          if (lane < pages && pidx >= first && pidx <= last) my_page = bt[pidx];
        }
        if (!mbar_try_wait(&freed[b], par)) {
          hand_over(true);
          ok = mbar_wait(&freed[b], par, &sh->abort);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t dst = stage0 + b * kTcTileBytes + c_half;
        const bool whole = k0 >= w.lo0 && k0 + kTcKeys <= w.k_end;    // every key of the tile is live
        const int in_page = k0 & ps_mask;                              // the tile's first row within its page (pages > 128 keys)
        for (int pg = 0; pg < pages; ++pg) {
          const size_t page = static_cast<size_t>(__shfl_sync(0xffffffffu, my_page, pg));
          const bf16* src = cache + (page * a.hkv + w.kvh) * head_stride + static_cast<size_t>(in_page) * kD + lane_src;
          const int row0 = pg * rpp;
          if (whole) {
#pragma unroll 4
            for (int jj = 0; jj < rpp; jj += RPI) {
              const int key = row0 + jj + rr;
              cp_async16_s(dst + key * 128 + ((c7 ^ (key & 7)) << 4), src + jj * kD);
            }
          } else {
#pragma unroll 4
            for (int jj = 0; jj < rpp; jj += RPI) {
              const int key = row0 + jj + rr, ka = k0 + key;
              cp_async16_s(dst + key * 128 + ((c7 ^ (key & 7)) << 4), src + jj * kD, ka < w.k_end && ka >= w.lo0);
            }
          }
        }
        cp_async_commit();
        if (pending >= 0 || q_pending) hand_over(false);   // the tile before (and Q): landed by now, or nearly
        pending = b;
      }
    }
    hand_over(true);
  } else if (warp >= kTcRowWarps + 2) {
    // ------------------------------------------------------------------ MMA issue: lane 0 of warp 10 for slot 0, of warp 11 for slot 1
    // Each slot has an issuing thread of its own, so that neither slot's products ever wait for the
    // other slot's rows.  With columns of its own for P a slot's products go  S(0), S(1), O += P(0) V,
    // S(2), O += P(1) V, ...: the S product runs one key tile ahead of the rows; with P over S:
    // S(0), O += P(0) V, S(1), O += P(1) V, ...
    const int s = warp - (kTcRowWarps + 2);
    if (lane == 0 && blockIdx.x < n_items) {
      const uint32_t idesc_qk = umma_idesc(kTcRows, kTcKeys);
      const uint32_t idesc_pv = umma_idesc(kTcRows, 64) | (1u << 16);          // B (V) is MN-major; 64 columns of O at a time
      const uint32_t q_u = smem_u32(q_s) + s * kTcTileBytes, k_u = smem_u32(k_s), v_u = smem_u32(v_s);
      const uint32_t s_col = tmem + s * kTcKeys, o_col = tmem + kTcColO + s * kD;
      const uint32_t p_col = kTcOwnP ? tmem + kTcColP + s * 64 : s_col;
      // a key tile of an item of this slot: g counts the CTA's key tiles (its K / V stage), n and it the
      // slot's own key tiles and items (the parities of its barriers)
      struct Tile { int g, n, it, i, nt; bool two; };
      bool ok = true;
      auto issue_qk = [&](const Tile& t) {
        const int b = t.g % kTcStages;
        if (t.i == 0) ok = ok && mbar_wait(&sh->q_full[s], t.it & 1, &sh->abort);
        ok = ok && mbar_wait(&sh->k_full[b], (t.g / kTcStages) & 1, &sh->abort);
        if (t.n > 0) {
          if (kTcOwnP)     // the rows have read the S of the tile before
            ok = ok && mbar_wait(&sh->s_free[s], (t.n - 1) & 1, &sh->abort);
          else             // S lies where the slot's P of the tile before was: its O product must be done
            ok = ok && mbar_wait(&sh->pv_done[s], (t.n - 1) & 1, &sh->abort);
        }
        if (!ok) return;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t off = (k >> 2) * kTcHalfBytes + (k & 3) * 32;
          umma_bf16(s_col, umma_desc(q_u + off), umma_desc(k_u + b * kTcTileBytes + off), idesc_qk, k != 0);
        }
        umma_commit(&sh->qk_done[s]);
        umma_commit(&sh->k_free[b]);                                           // this slot has read the K tile;
        if (!t.two) umma_commit(&sh->k_free[b]);                               // and there is no other slot to wait for
        if (t.i == t.nt - 1) umma_commit(&sh->q_free[s]);                      // the item's Q has been read
      };
      auto issue_pv = [&](const Tile& t) {
        const int b = t.g % kTcStages;
        ok = ok && mbar_wait(&sh->p_ready[s], t.n & 1, &sh->abort);
        ok = ok && mbar_wait(&sh->v_full[b], (t.g / kTcStages) & 1, &sh->abort);
        // the first product of an item overwrites O: the rows of the item before must have read theirs
        if (t.i == 0) ok = ok && mbar_wait(&sh->o_free[s], (t.it & 1) ^ 1, &sh->abort);
        if (!ok) return;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kTcKeys / 16; ++k)
#pragma unroll
          for (int h = 0; h < kTcHalves; ++h)
            umma_bf16_ts(o_col + h * 64, p_col + k * 8,
                         umma_desc_mn(v_u + b * kTcTileBytes + h * kTcHalfBytes + k * 2048), idesc_pv,
                         (t.i != 0 || k != 0) ? 1u : 0u);
        umma_commit(&sh->pv_done[s]);
        umma_commit(&sh->v_free[b]);
        if (!t.two) umma_commit(&sh->v_free[b]);
      };
      // the slot's items: slot 1 skips those with one head
      TcWalk wk;
      auto seek = [&](bool more) {
        while (more && s == 1 && !wk.w.two) more = wk.next(a, n_items, pairs, tiles);
        return more;
      };
      auto tile0 = [&]() { return Tile{wk.g, s == 0 ? wk.g : wk.g1, s == 0 ? wk.it : wk.it1, 0, wk.w.nt, wk.w.two}; };
      if (seek(wk.first(a, n_items, pairs, tiles))) {
        Tile cur = tile0();
        issue_qk(cur);
        while (ok) {
          // the tile after cur: of this item, or the first of the slot's next item
          Tile nxt = cur;
          bool more = true;
          ++nxt.g;
          ++nxt.n;
          if (++nxt.i == cur.nt) {
            more = seek(wk.next(a, n_items, pairs, tiles));
            if (more) nxt = tile0();
          }
          if (kTcOwnP) {
            if (more) issue_qk(nxt);
            issue_pv(cur);
          } else {
            issue_pv(cur);
            if (more) issue_qk(nxt);
          }
          if (!more) break;
          cur = nxt;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ the row threads, two to a row
    // Warp w < 16: slot w / 8, half h = (w / 4) % 2, rows 32 (w % 4) .. + 32 of the slot's tile (the TMEM
    // lanes a warp may touch).  A thread has the keys 64 h .. + 64 of every S tile, writes their P, and has
    // the columns h D / 2 .. + D / 2 of O.  Both threads of a row take the maximum over the whole row (the
    // other half is read from tensor memory for that alone, which is cheaper than an exchange), so both
    // come to the same reference and the same decisions; each keeps the denominator of its own keys, and
    // the two are added at the item's end (one exchange through shared memory).
    const int s = warp >> 3, h = (warp >> 2) & 1, q = warp & 3;
    const int r = q * 32 + lane;                         // row of the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t s_addr = tmem + lane_addr + s * kTcKeys;           // S
    const uint32_t p_addr = (kTcOwnP ? tmem + lane_addr + kTcColP + s * 64 : s_addr) + h * 32;   // this thread's 32 columns of P
    const uint32_t o_addr = tmem + lane_addr + kTcColO + s * kD + h * (kD / 2);
    const float sc = a.scale * kLog2e;
    bool ok = true;
    int xphase = 0;                                       // exchanges done so far (parity of the pair's mbarrier)
    TcWalk wk;
    for (bool more = wk.first(a, n_items, pairs, tiles); more && ok; more = wk.next(a, n_items, pairs, tiles)) {
      const TcItem& w = wk.w;
      if (s == 1 && !w.two) continue;                     // this slot sits the item out
      const int g_base = s == 0 ? wk.g : wk.g1;           // the slot's key tiles so far
      const int rows = w.rows, pos0 = w.pos0;
      const int pos_r = pos0 + r;
      const int win_r = (a.window > 0 && pos_r + 1 > a.window) ? pos_r + 1 - a.window : 0;
      const int lim_r = r < rows ? pos_r : -1;             // the row's live keys are win_r .. lim_r (none for a row past the tile's rows)
      float m_ref = -INFINITY, l = 0.f;                   // the maximum that P is scaled by (log2 units), this thread's part of the denominator
      for (int i = 0; i < w.nt && ok; ++i) {
        const int n = g_base + i;
        const int t0 = w.k_begin + i * kTcKeys;
        ok = mbar_wait(&sh->qk_done[s], n & 1, &sh->abort);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // only tiles that reach past the first row's position, before the last row's window or past the
        // tile's rows need the masks (the same for the whole CTA)
        const bool masked = (t0 + kTcKeys - 1 > pos0) || (a.window > 0 && t0 < pos0 + kTcRows - a.window) || (rows < kTcRows);
        float mx0 = -INFINITY, mx1 = -INFINITY;
        uint32_t sr[64];
        {   // the other thread's keys, for the maximum; then this thread's own
          tmem_ld64_issue(s_addr + (h ^ 1) * 64, sr);
          tmem_wait_ld();
          if (masked) tc_mask64(sr, lim_r - (t0 + (h ^ 1) * 64), win_r - (t0 + (h ^ 1) * 64), a.window > 0);
#pragma unroll
          for (int j = 0; j < 64; j += 4) {
            mx0 = max3(mx0, __uint_as_float(sr[j]), __uint_as_float(sr[j + 1]));
            mx1 = max3(mx1, __uint_as_float(sr[j + 2]), __uint_as_float(sr[j + 3]));
          }
        }
        tmem_ld64_issue(s_addr + h * 64, sr);
        tmem_wait_ld();
        if (kTcOwnP) {                                     // S is in registers: the next S product may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh->s_free[s]);
        }
        if (masked) tc_mask64(sr, lim_r - (t0 + h * 64), win_r - (t0 + h * 64), a.window > 0);
#pragma unroll
        for (int j = 0; j < 64; j += 4) {
          mx0 = max3(mx0, __uint_as_float(sr[j]), __uint_as_float(sr[j + 1]));
          mx1 = max3(mx1, __uint_as_float(sr[j + 2]), __uint_as_float(sr[j + 3]));
        }
        const float m_new = fmaxf(m_ref, fmaxf(mx0, mx1) * sc);   // in units of log2 of the scaled scores
        // The reference moves for the whole warp or not at all (the other warp of these rows sees the same
        // maxima and decides the same); the denominator follows at once, the row of O below, when O is at rest.
        float alpha = 1.f;
        bool moved = false;
        if (i == 0) {
          m_ref = m_new;
        } else if (__any_sync(0xffffffffu, m_new > m_ref + kTcGrow)) {
          alpha = m_new == m_ref ? 1.f : ex2_approx(m_ref - m_new);                       // 2^(-inf) = 0
          l *= alpha;
          m_ref = m_new;
          moved = true;
        }
        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;  // a row without a live key so far
        const uint64_t sc2 = f32x2(sc, sc), nm2 = f32x2(-m_use, -m_use);
        uint64_t sum_a = f32x2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
        for (int j = 0; j < 64; j += 4) {
          float x0, x1, x2, x3;
          f32x2_split(fma_f32x2(f32x2(__uint_as_float(sr[j]), __uint_as_float(sr[j + 1])), sc2, nm2), x0, x1);
          f32x2_split(fma_f32x2(f32x2(__uint_as_float(sr[j + 2]), __uint_as_float(sr[j + 3])), sc2, nm2), x2, x3);
          const float p0 = ex2_approx(x0), p1 = ex2_approx(x1), p2 = ex2_approx(x2), p3 = ex2_approx(x3);
          sum_a = add_f32x2(sum_a, f32x2(p0, p1));
          sum_b = add_f32x2(sum_b, f32x2(p2, p3));
          const __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1), hi = __floats2bfloat162_rn(p2, p3);
          sr[j >> 1] = *reinterpret_cast<const uint32_t*>(&lo);       // (columns j / 2: behind the ones still to be read)
          sr[(j >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&hi);
        }
        {
          float s0, s1, s2, s3;
          f32x2_split(sum_a, s0, s1);
          f32x2_split(sum_b, s2, s3);
          l += (s0 + s1) + (s2 + s3);
        }
        if (kTcOwnP && n > 0) {
          // P of the tile before must have been read, and O must be at rest, before this tile's P and a
          // rescaled O are written (long done by now: that product was issued a whole tile ago)
          ok = mbar_wait(&sh->pv_done[s], (n - 1) & 1, &sh->abort);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
        }
        if (!kTcOwnP) {
          // P goes over columns of S that the other thread of the row reads too (its own keys, or this
          // thread's for the maximum): both must have read S before either writes P
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh->pair[s][q]);
          ok = mbar_wait(&sh->pair[s][q], xphase & 1, &sh->abort);
          ++xphase;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
        }
        if (moved) {
          // (with P over S, O is at rest too: the product that made S waited for the O product of the tile before)
#pragma unroll
          for (int c0 = 0; c0 < kD / 2; c0 += 32) {
            uint32_t o[32];
            tmem_ld16_issue(o_addr + c0, o);
            tmem_ld16_issue(o_addr + c0 + 16, o + 16);
            tmem_wait_ld();
#pragma unroll
            for (int d = 0; d < 32; ++d) o[d] = __float_as_uint(__uint_as_float(o[d]) * alpha);
            tmem_st16(o_addr + c0, o);
            tmem_st16(o_addr + c0 + 16, o + 16);
          }
        }
        // P: two keys per 32-bit column; this thread's 64 keys are 32 columns
        tmem_st16(p_addr, sr);
        tmem_st16(p_addr + 16, sr + 16);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->p_ready[s]);
      }
      if (!ok) break;
      // ---- the row's denominator: this thread's part and the other's
      sh->l_half[s][h][r] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->pair[s][q]);        // (release: the values are visible to who sees the phase)
      ok = mbar_wait(&sh->pair[s][q], xphase & 1, &sh->abort);
      ++xphase;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const float l_all = l + sh->l_half[s][h ^ 1][r];
      // ---- the item's rows: O / denominator, once its last product is done
      ok = mbar_wait(&sh->pv_done[s], (g_base + w.nt - 1) & 1, &sh->abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
      bf16* dst = a.out + static_cast<size_t>(w.tok0 + (r < rows ? r : 0)) * a.out_stride + (w.head0 + s) * kD + h * (kD / 2);
#pragma unroll
      for (int c0 = 0; c0 < kD / 2; c0 += 32) {
        uint32_t o[32];
        tmem_ld16_issue(o_addr + c0, o);
        tmem_ld16_issue(o_addr + c0 + 16, o + 16);
        tmem_wait_ld();
        if (r < rows) {
#pragma unroll
          for (int d = 0; d < 32; d += 8) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(o[d + e]) * inv;
            store16(dst + c0 + d, v);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->o_free[s]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kTcRowWarps + 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTcTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && sh->abort) atomicOr(status, 4);
}

}  // namespace rl
