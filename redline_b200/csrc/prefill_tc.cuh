// Prompt-portion attention on the fifth-generation tensor cores (bfloat16, head size 64).
//
// Included by attention.cu.  An item of work is a tile of up to 128 consecutive query rows of one
// sequence for one query head; persistent CTAs (one per SM) take items one after another, longest
// first, and the pipeline below runs on across items (the next item's Q and first keys are on their
// way while the rows of this one finish).  Per item the keys come in tiles of 128:
//   S = Q K^T      tcgen05.mma, 128 x 128, K = 64, accumulator in tensor memory (two S buffers)
//   softmax        two threads per query row read the row of S from TMEM (tcgen05.ld), keep the
//                  running maximum and denominator in float32, writes P as bfloat16 into shared
//                  memory in the K-major 128-byte-swizzled layout that the MMA reads
//   O_tile = P V   tcgen05.mma, 128 x 64, K = 128; V is read as it lies in the cache (a key's 64
//                  values contiguous: the B operand in MN-major form); fresh accumulator per key
//                  tile (two O buffers), which the row's thread adds into its float32 running sum
//                  after scaling that by 2^(old max - new max)
// Warp roles: warps 0-7 are the row threads, two to a row (warp w owns TMEM lanes 32 (w % 4) .., the
// keys 64 (w / 4) .. of an S tile and the columns 32 (w / 4) .. of O), warp 8 brings Q once and
// the K tiles, warp 9 the V tiles, from the paged cache with 16-byte cp.async copies (two stages
// each, zero-filled outside the live keys), lane 0 of warp 10 issues the MMAs, the S product of tile
// i + 1 before the O product of tile i so that the tensor core works while the rows of tile i are
// in their softmax.  Everything is handed over through mbarriers; every wait is bounded
// (kSpinLimit polls), after which the CTA raises an abort flag, all roles leave their loops, the
// copies in flight are waited for, TMEM is freed and bit 2 of *status is set.
#pragma once

#include "umma.cuh"

namespace rl {

constexpr int kTcRows = 128, kTcKeys = 128;
constexpr int kTcThreads = 352;                     // 8 row warps, two loaders, the MMA warp
constexpr int kTcTileBytes = kTcKeys * 128;          // a 128 x 64 bfloat16 tile: K, V, Q or half of P
constexpr int kTcTmemCols = 512;                     // S0 0.., S1 128.., O0 256.., O1 320..

struct PrefillTcShared {
  uint64_t q_full[2], q_free[2];      // Q of an item has landed / its last S product has read it
  uint64_t k_full[2], v_full[2];      // one arrival by the loader warp (after all its lanes' copies have landed)
  uint64_t qk_done[2], pv_done[2];    // MMA commits: S of the tile is ready / K stage free; O of the tile ready / V, P free
  uint64_t s_free[2], o_free[2];      // the 8 row warps have read the buffer
  uint64_t p_ready[2];                // the 8 row warps have written P
  uint64_t pair[4];                   // the two warps of a quarter of rows exchange a value (2 arrivals a phase)
  float xchg[2][2][kTcRows];          // [phase parity][half][row]
  uint32_t tmem_base;
  volatile int abort;
};
constexpr size_t kPrefillTcSmem = 1024 + 10 * kTcTileBytes + sizeof(PrefillTcShared);   // 2 Q, 2 K, 2 V, 2 x 2 P

// One item of a CTA's work: a tile of query rows for one query head.
struct TcItem {
  int seq, tok0, rows, head, kvh;
  int pos0, k_end, lo0, k_begin, nt;   // first position, keys [lo0, k_end) are live, nt key tiles from k_begin
};

// Items are numbered longest first (a later tile of a sequence attends to more keys), the heads of a
// tile next to each other, so that CTAs that run together share K and V in L2.
__device__ __forceinline__ TcItem tc_item(const PrefillArgs<bf16>& a, int item, int tiles) {
  TcItem w;
  const int tile = tiles - 1 - item / a.hq;
  w.head = item - (item / a.hq) * a.hq;
  w.kvh = w.head / (a.hq / a.hkv);
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

__global__ void __launch_bounds__(kTcThreads, 1)
prefill_attn_tc_kernel(const PrefillArgs<bf16> a, int tiles, int* status) {
  static_assert(kD == 64, "this kernel is written for head size 64");
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* base = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* q_s = base;                             // two buffers
  unsigned char* k_s = base + 2 * kTcTileBytes;          // two stages
  unsigned char* v_s = base + 4 * kTcTileBytes;          // two stages
  unsigned char* p_s = base + 6 * kTcTileBytes;          // two buffers of two 64-key halves
  PrefillTcShared* sh = reinterpret_cast<PrefillTcShared*>(base + 10 * kTcTileBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = tiles * a.hq;

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->q_full[b], 1);
      mbar_init(&sh->q_free[b], 1);
      mbar_init(&sh->k_full[b], 1);
      mbar_init(&sh->v_full[b], 1);
      mbar_init(&sh->qk_done[b], 1);
      mbar_init(&sh->pv_done[b], 1);
      mbar_init(&sh->s_free[b], 8);       // one arrival per row warp (its lanes meet first)
      mbar_init(&sh->o_free[b], 8);
      mbar_init(&sh->p_ready[b], 8);
    }
    for (int qq = 0; qq < 4; ++qq) mbar_init(&sh->pair[qq], 2);
    sh->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 10) {   // TMEM allocation is a whole-warp operation
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

  // Every role walks the same list of items (blockIdx.x, + gridDim.x, ...) and counts the key tiles of
  // all its items in one sequence g: tile g uses stage / buffer g & 1 in its ((g >> 1) & 1)-th use, item
  // number `it` of the CTA uses Q buffer it & 1.  A role reads an item's description one item ahead.
  if (warp == 8 || warp == 9) {
    // ------------------------------------------------------------------ loaders: warp 8 K (and Q), warp 9 V
    const bool is_v = warp == 9;
    const int ps_shift = __ffs(a.page_size) - 1, ps_mask = a.page_size - 1;
    const size_t head_stride = static_cast<size_t>(a.page_size) * kD;
    const int c = lane & 7, r4 = lane >> 3;            // chunk of a row, row within a round of four rows
    const bf16* cache = is_v ? a.vcache : a.kcache;
    const uint32_t stage0 = smem_u32(is_v ? v_s : k_s);
    uint64_t* full = is_v ? sh->v_full : sh->k_full;
    uint64_t* freed = is_v ? sh->pv_done : sh->qk_done;   // the product that read the stage two tiles back
    const int rpp = min(a.page_size, kTcKeys);            // rows of a page that lie in a tile
    const int pages = kTcKeys / rpp;                      // pages per tile (at most eight: pages of 16 keys or more)
    const uint32_t lane_src = static_cast<uint32_t>(r4 * kD + c * 8);
    // Before the warp blocks on a stage or a Q buffer, what it has copied so far is handed over: the
    // reader of a stage never waits for a tile that waits for that reader.
    bool ok = true;
    int pending = -1, q_pending = -1;                     // a tile (a Q buffer) copied but not handed over
    auto hand_over = [&](bool all) {
      if (all) cp_async_wait<0>(); else cp_async_wait<1>();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (q_pending >= 0) mbar_arrive(&sh->q_full[q_pending]);
        if (pending >= 0) mbar_arrive(&full[pending & 1]);
      }
      q_pending = -1;
      pending = -1;
    };
    int g = 0, it = 0, round = 0;
    for (int item = tc_next_item(round, n_items); item >= 0 && ok; item = tc_next_item(round, n_items), ++it) {
      const TcItem w = tc_item(a, item, tiles);
      const int32_t* bt = a.block_table + static_cast<size_t>(w.seq) * a.max_blocks;
      if (!is_v) {
        const int qb = it & 1;
        if (!mbar_try_wait(&sh->q_free[qb], ((it >> 1) & 1) ^ 1)) {
          hand_over(true);
          ok = mbar_wait(&sh->q_free[qb], ((it >> 1) & 1) ^ 1, &sh->abort);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (pending >= 0) hand_over(true);                // (keeps the groups of Q and of a tile apart)
        const uint32_t q_u = smem_u32(q_s) + qb * kTcTileBytes;
        for (int j = 0; j < kTcRows / 4; ++j) {
          const int r = j * 4 + r4;
          const bool live = r < w.rows;
          const bf16* src = a.q + static_cast<size_t>(w.tok0 + (live ? r : 0)) * a.q_stride + w.head * kD + c * 8;
          cp_async16_s(q_u + r * 128 + ((c ^ (r & 7)) << 4), src, live);
        }
        cp_async_commit();
        q_pending = qb;
      }
      for (int i = 0; i < w.nt; ++i, ++g) {
        const int b = g & 1;
        const uint32_t par = (((g >> 1) & 1) ^ 1);        // a fresh barrier passes a wait on parity 1
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
        const uint32_t dst = stage0 + b * kTcTileBytes;
        const bool whole = k0 >= w.lo0 && k0 + kTcKeys <= w.k_end;    // every key of the tile is live
        const int in_page = k0 & ps_mask;                              // the tile's first row within its page (pages > 128 keys)
        for (int pg = 0; pg < pages; ++pg) {
          const size_t page = static_cast<size_t>(__shfl_sync(0xffffffffu, my_page, pg));
          const bf16* src = cache + (page * a.hkv + w.kvh) * head_stride + static_cast<size_t>(in_page) * kD + lane_src;
          const int row0 = pg * rpp;
          if (whole) {
#pragma unroll 4
            for (int jj = 0; jj < rpp; jj += 4) {
              const int key = row0 + jj + r4;
              cp_async16_s(dst + key * 128 + ((c ^ (key & 7)) << 4), src + jj * kD);
            }
          } else {
#pragma unroll 4
            for (int jj = 0; jj < rpp; jj += 4) {
              const int key = row0 + jj + r4, ka = k0 + key;
              cp_async16_s(dst + key * 128 + ((c ^ (key & 7)) << 4), src + jj * kD, ka < w.k_end && ka >= w.lo0);
            }
          }
        }
        cp_async_commit();
        if (pending >= 0 || q_pending >= 0) hand_over(false);   // the tile before (and Q): landed by now, or nearly
        pending = g;
      }
    }
    hand_over(true);
  } else if (warp == 10) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0 && blockIdx.x < n_items) {
      const uint32_t idesc_qk = umma_idesc(kTcRows, kTcKeys);
      const uint32_t idesc_pv = umma_idesc(kTcRows, kD) | (1u << 16);          // B (V) is MN-major
      const uint32_t q_u = smem_u32(q_s), k_u = smem_u32(k_s), v_u = smem_u32(v_s), p_u = smem_u32(p_s);
      struct Tile { int item, it, i, nt, g; };                                  // a key tile of an item of this CTA
      bool ok = true;
      auto issue_qk = [&](const Tile& t) {
        const int b = t.g & 1;
        if (t.i == 0) ok = ok && mbar_wait(&sh->q_full[t.it & 1], (t.it >> 1) & 1, &sh->abort);
        ok = ok && mbar_wait(&sh->k_full[b], (t.g >> 1) & 1, &sh->abort) &&
             mbar_wait(&sh->s_free[b], ((t.g >> 1) & 1) ^ 1, &sh->abort);
        if (!ok) return;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kD / 16; ++k)
          umma_bf16(tmem + b * kTcKeys, umma_desc(q_u + (t.it & 1) * kTcTileBytes + k * 32),
                    umma_desc(k_u + b * kTcTileBytes + k * 32), idesc_qk, k != 0);
        umma_commit(&sh->qk_done[b]);
        if (t.i == t.nt - 1) umma_commit(&sh->q_free[t.it & 1]);             // the item's Q has been read
      };
      auto issue_pv = [&](const Tile& t) {
        const int b = t.g & 1;
        ok = ok && mbar_wait(&sh->v_full[b], (t.g >> 1) & 1, &sh->abort) &&
             mbar_wait(&sh->p_ready[b], (t.g >> 1) & 1, &sh->abort) &&
             mbar_wait(&sh->o_free[b], ((t.g >> 1) & 1) ^ 1, &sh->abort);
        if (!ok) return;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kTcKeys / 16; ++k)
          umma_bf16(tmem + 2 * kTcKeys + b * kD,
                    umma_desc(p_u + b * 2 * kTcTileBytes + (k >> 2) * kTcTileBytes + (k & 3) * 32),
                    umma_desc_mn(v_u + b * kTcTileBytes + k * 2048), idesc_pv, k != 0);
        umma_commit(&sh->pv_done[b]);
      };
      // the S product of the next tile (of this item or the next) is issued before the O product of this one
      int round = 0;
      Tile cur;
      cur.item = tc_next_item(round, n_items);
      cur.it = 0;
      cur.i = 0;
      cur.g = 0;
      cur.nt = tc_item(a, cur.item, tiles).nt;
      issue_qk(cur);
      int item_after = -1, nt_after = 0;                  // the item after cur's and its key tiles (read at cur's start)
      while (ok) {
        if (cur.i == 0) {
          item_after = tc_next_item(round, n_items);
          nt_after = item_after >= 0 ? tc_item(a, item_after, tiles).nt : 0;
        }
        Tile nxt = cur;
        ++nxt.g;
        if (++nxt.i == cur.nt) {
          nxt.item = item_after;
          ++nxt.it;
          nxt.i = 0;
          nxt.nt = nt_after;
        }
        const bool more = nxt.item >= 0;
        if (more) issue_qk(nxt);
        issue_pv(cur);
        if (!more) break;
        cur = nxt;
      }
    }
  } else {
    // ------------------------------------------------------------------ the row threads, two to a row
    // Warp w < 8: rows 32 (w % 4) .. + 32 (the TMEM lanes a warp may touch), keys 64 (w / 4) .. + 64 of
    // every S tile and columns 32 (w / 4) .. + 32 of O.  Both threads of a row take the maximum over the
    // whole row; each keeps the denominator of its own keys, and the two are added at the end (one
    // exchange through shared memory, an mbarrier per quarter of rows, 2 arrivals).
    const int q = warp & 3, h = warp >> 2;
    const int r = q * 32 + lane;                         // row of the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const float sc = a.scale * kLog2e;
    const uint32_t p_u = smem_u32(p_s);
    bool ok = true;
    int xphase = 0;                                       // exchanges done so far (parity of the pair's mbarrier)
    auto exchange = [&](float mine) -> float {            // gives the partner's value
      sh->xchg[xphase & 1][h][r] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->pair[q]);           // (release: the values are visible to who sees the phase)
      ok = ok && mbar_wait(&sh->pair[q], xphase & 1, &sh->abort);
      const float other = sh->xchg[xphase & 1][h ^ 1][r];
      ++xphase;
      return other;
    };
    float acc[32];
    auto add_o = [&](int g, float alpha) {                // acc = acc * alpha + O_tile(g), this thread's 32 columns
      const int b = g & 1;
      ok = ok && mbar_wait(&sh->pv_done[b], (g >> 1) & 1, &sh->abort);
      if (!ok) return;
      tc_fence_after();
      float o[32];
      tmem_ld32(tmem + lane_addr + 2 * kTcKeys + b * kD + h * 32, o);
#pragma unroll
      for (int d = 0; d < 32; ++d) acc[d] = fmaf(acc[d], alpha, o[d]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->o_free[b]);
    };
    int g = 0, round = 0;
    int item = tc_next_item(round, n_items);
    TcItem w;
    if (item >= 0) w = tc_item(a, item, tiles);
    for (; item >= 0 && ok;) {
      const int item_next = tc_next_item(round, n_items);
      TcItem w_next = w;
      if (item_next >= 0) w_next = tc_item(a, item_next, tiles);   // on its way during this item
      const int rows = w.rows, pos0 = w.pos0;
      const int pos_r = pos0 + r;
      const int win_r = (a.window > 0 && pos_r + 1 > a.window) ? pos_r + 1 - a.window : 0;
#pragma unroll
      for (int d = 0; d < 32; ++d) acc[d] = 0.f;
      float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
      for (int i = 0; i < w.nt && ok; ++i, ++g) {
        const int b = g & 1;
        const int t0 = w.k_begin + i * kTcKeys;
        const int k0 = t0 + h * 64;                       // this thread's first key of the tile
        ok = mbar_wait(&sh->qk_done[b], (g >> 1) & 1, &sh->abort);
        if (!ok) break;
        tc_fence_after();
        // only tiles that reach past the first row's position, before the last row's window or past the
        // tile's rows need the masks (the same for the whole CTA)
        const bool masked = (t0 + kTcKeys - 1 > pos0) || (a.window > 0 && t0 < pos0 + kTcRows - a.window) || (rows < kTcRows);
        // the row's maximum over all 128 keys: the other thread's half is read too (and dropped), which is
        // cheaper than an exchange between the two threads
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        {
          const int ko = t0 + (h ^ 1) * 64;
#pragma unroll
          for (int c0 = 0; c0 < 64; c0 += 32) {
            float o[32];
            tmem_ld32(tmem + lane_addr + b * kTcKeys + (h ^ 1) * 64 + c0, o);
            if (masked) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int key = ko + c0 + j;
                if (!(key <= pos_r && key >= win_r && r < rows)) o[j] = -INFINITY;
              }
            }
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              mx0 = fmaxf(mx0, o[j]);
              mx1 = fmaxf(mx1, o[j + 1]);
              mx2 = fmaxf(mx2, o[j + 2]);
              mx3 = fmaxf(mx3, o[j + 3]);
            }
          }
        }
        float s[64];
        tmem_ld32(tmem + lane_addr + b * kTcKeys + h * 64, s);
        tmem_ld32(tmem + lane_addr + b * kTcKeys + h * 64 + 32, s + 32);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->s_free[b]);         // S of this tile has been read
        if (masked) {
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            const int key = k0 + j;
            if (!(key <= pos_r && key >= win_r && r < rows)) s[j] = -INFINITY;
          }
        }
#pragma unroll
        for (int j = 0; j < 64; j += 4) {
          mx0 = fmaxf(mx0, s[j]);
          mx1 = fmaxf(mx1, s[j + 1]);
          mx2 = fmaxf(mx2, s[j + 2]);
          mx3 = fmaxf(mx3, s[j + 3]);
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        const float m_new = fmaxf(m, mx * sc);               // in units of log2 of the scaled scores
        const float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row without a live key so far
        const float alpha = ex2_approx(m - m_use);           // 2^(-inf) = 0 the first time
        float sm0 = 0.f, sm1 = 0.f, sm2 = 0.f, sm3 = 0.f;
#pragma unroll
        for (int j = 0; j < 64; j += 4) {
          s[j] = ex2_approx(fmaf(s[j], sc, -m_use));
          s[j + 1] = ex2_approx(fmaf(s[j + 1], sc, -m_use));
          s[j + 2] = ex2_approx(fmaf(s[j + 2], sc, -m_use));
          s[j + 3] = ex2_approx(fmaf(s[j + 3], sc, -m_use));
          sm0 += s[j];
          sm1 += s[j + 1];
          sm2 += s[j + 2];
          sm3 += s[j + 3];
        }
        l = l * alpha + ((sm0 + sm1) + (sm2 + sm3));
        m = m_new;
        // ---- the P buffer must be free: the O product of two tiles back has read it
        ok = mbar_wait(&sh->pv_done[b], ((g >> 1) & 1) ^ 1, &sh->abort);
        if (!ok) break;
        // this thread's 64 keys are the row's eight 16-byte chunks of the 64-key half h
        const uint32_t prow = p_u + b * 2 * kTcTileBytes + h * kTcTileBytes + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t wd[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 hh = __floats2bfloat162_rn(s[c * 8 + 2 * e], s[c * 8 + 2 * e + 1]);
            wd[e] = *reinterpret_cast<const uint32_t*>(&hh);
          }
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(prow + ((c ^ (r & 7)) << 4)), "r"(wd[0]),
                       "r"(wd[1]), "r"(wd[2]), "r"(wd[3])
                       : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->p_ready[b]);
        // ---- while the O product of this tile runs: add the one of the tile before
        if (i > 0) add_o(g - 1, alpha_prev);
        alpha_prev = alpha;
      }
      if (ok && w.nt > 0) add_o(g - 1, alpha_prev);
      const float l_all = l + exchange(l);
      if (ok && r < rows) {
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        bf16* dst = a.out + static_cast<size_t>(w.tok0 + r) * a.out_stride + w.head * kD + h * 32;
#pragma unroll
        for (int d = 0; d < 32; d += 8) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = acc[d + e] * inv;
          store16(dst + d, v);
        }
      }
      w = w_next;
      item = item_next;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 10) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTcTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && sh->abort) atomicOr(status, 4);
}

}  // namespace rl
