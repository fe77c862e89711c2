// Decode attention for launches of few, long rows: one thread-block CLUSTER per (item, kv head).
//
// Included by attention.cu after decode_stream.cuh (bfloat16, head size 64 or 128), whose pipeline it
// shares: every warp moves 32-key sub-blocks through a private two-stage ring of shared memory with
// 16-byte asynchronous copies and does S = Q K^T, the online softmax and O += P V on them with
// mma.sync.m16n8k16.  What differs is who gets which keys and how the partial results meet.  The live keys
// of a row are cut into as many equal runs of sub-blocks as the row's cluster has warps (CTAs of the
// cluster in rank order, warps in order: runs in the order of the keys).  At the end every warp leaves its
// (max, denominator, numerators) in its own, then idle, ring; the CTA adds its warps' in order and puts the
// sums into a slot of its own in the shared memory of the cluster's first CTA (a store through distributed
// shared memory); the cluster meets at its hardware barrier; the first CTA adds the slots in order and
// writes the row.  Nothing goes through global memory, nothing is counted,
// nothing waits on a flag: the streaming kernel spends 8 of its 19 microseconds at batch 8 x 4,096 keys on
// exactly that.
//
// A launch with more rows than clusters can be resident runs clusters of one CTA whose warps form groups,
// a row to each group at the same time (and, if that is still not enough, several one after another); a
// group adds its warps' results at a barrier of its own and writes the row itself.
//
// The cost: a row has its cluster's SMs and no others.  With rows of very different lengths the longest
// one sets the kernel's time, where the streaming kernel shares all keys among all warps; the caller
// chooses (rl_attn_decode, impl 4).
//
// The first copies are issued before the wait on the kernels before this one: keys of earlier steps do not
// depend on them.  With the rotation fused (rope.cos set) the token's own key is not in the cache yet: the
// warp that holds it puts k (rotated) and v from the token's row into the cache and over what the copy
// brought; without, the kernel before has just written it, and the sub-block that holds it is asked for
// after the wait.
#pragma once

namespace rl {

// (13 warps at head size 64, which shared memory has rings for, leave a thread 128 registers: the kernel
// spills and batch 8 x 4,096 keys takes 15.7 us instead of 14.7.)
constexpr int kRowsWarps = kStreamWarps;
constexpr int kRowsThreads = kRowsWarps * 32;

// The largest cluster: what shared memory has room for beside the rings (the first CTA keeps a slot for the
// sums of every other CTA of its cluster).
constexpr int kRowsMaxCluster = (kD == 64) ? 8 : 4;
struct RowsShared {
  float cta_o[kRowsMaxCluster][16][kD];      // slot c: the numerators of CTA c of the cluster, head by head
  float cta_ml[kRowsMaxCluster][16][2];      // (max in log2 units, denominator); an empty CTA leaves (-inf, 0)
};
constexpr int kRowsLd = kD + 4;        // floats per head in a warp's partial result: numerators, max, denominator
static_assert(16 * kRowsLd * 4 <= 2 * kStreamStageBytes, "a warp's partial result lies in its own ring");
constexpr size_t kRowsSmem = static_cast<size_t>(kRowsWarps) * 2 * kStreamStageBytes + sizeof(RowsShared) + 16;

__device__ __forceinline__ uint32_t rows_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t rows_cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void rows_cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Two floats to a shared-memory address of this CTA's layout in CTA `rank` of the cluster.
__device__ __forceinline__ void rows_st_cluster(float* p, uint32_t rank, float2 v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32s(p)), "r"(rank));
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(remote), "f"(v.x), "f"(v.y) : "memory");
}

// HI: groups of more than 8 heads (rows g + 8 of the MMA tile are in use).
template <bool HI>
__global__ void __launch_bounds__(kRowsThreads, 1)
decode_attn_rows_kernel(const DecodeArgs<bf16> a, int nrows, int groups, const DecodeRope rope) {
  constexpr int DB = kD / 32, DG = kD / 64;
  constexpr float kLog2e = 1.4426950408889634f;
  constexpr int CPR = kD / 8;            // 16-byte chunks per row
  constexpr int RPR = 32 / CPR;          // rows that one round of the warp's copies covers
  extern __shared__ __align__(16) unsigned char smem_raw[];
  RowsShared* sh = reinterpret_cast<RowsShared*>(smem_raw + kRowsWarps * 2 * kStreamStageBytes);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = a.hq / a.hkv;
  const int csize = static_cast<int>(rows_cluster_size()), rank = static_cast<int>(rows_cluster_rank());
  // (Like the streaming kernel it does not tell its dependents to launch early: measured in the decode step,
  // at the kernel's start or after the runs, the step then takes 1.18 ms instead of 0.82: the kernels after it
  // move in and wait where this kernel's and the next one's CTAs should run.)
  // The cluster's row.  A launch with more rows than clusters can be resident runs clusters of ONE CTA whose
  // warps form `groups` groups, a row to each at the same time (rows 0 .. CTAs - 1 go to the first groups
  // of the CTAs, the next to their second groups, ...: as many SMs as there are stream), and if that is not
  // enough, a group takes several rows one after another.
  const int gsize = kRowsWarps / groups;                // warps of a group (groups divides kRowsWarps)
  const int gi = warp / gsize, wg = warp - gi * gsize;
  const int nclusters = gridDim.x / csize;
#pragma unroll 1
  for (int rowi = gi * nclusters + blockIdx.x / csize; rowi < nrows; rowi += groups * nclusters) {
  const int item = rowi / a.hkv, kvh = rowi - item * a.hkv;
  // (items and block tables were written before the step's kernels began)
  const int4 info = a.items[item];
  const int tok = info.x, seq = info.y, ctx = info.z;
  if (ctx <= 0) continue;                               // (the same for the whole cluster)
  const int lo = (a.window > 0 && ctx > a.window) ? ctx - a.window : 0;
  const bool fused = rope.cos != nullptr;

  // ---- this warp's run of sub-blocks
  const int sb_first = lo / kSub, n_sb = (ctx - 1) / kSub - sb_first + 1;
  const int W = csize * gsize, wi = rank * gsize + wg;
  const int per = n_sb / W, rem = n_sb - per * W;
  const int my_n = per + (wi < rem ? 1 : 0);
  const int my_sb = sb_first + wi * per + min(wi, rem);
  const int sb_newest = (ctx - 1) / kSub;               // the sub-block of the token's own key

  const int ps = a.page_size;
  const int ps_shift = __ffs(ps) - 1;                   // page sizes are powers of two
  const uint32_t stages = smem_u32s(smem_raw) + warp * 2 * kStreamStageBytes;
  const int g = lane >> 2, t = lane & 3;
  const float sc = a.scale * kLog2e;
  const int crow = lane / CPR, cchunk = lane % CPR;     // this lane's row (of a round) and chunk in the copies
  const int32_t* bt = a.block_table + static_cast<size_t>(seq) * a.max_blocks;

  // the (at most two) pages sub-block sb lies in; a page without a live key reads as page 0
  auto sub_pages = [&](int sb) -> int2 {
    const int a0 = sb * kSub;
    const int first = max(a0, lo), last = min(a0 + kSub, ctx) - 1;     // live keys of the sub-block
    int2 pg;
    const int i0 = a0 >> ps_shift, i1 = (a0 + 16) >> ps_shift;
    pg.x = (first >> ps_shift) <= i0 && i0 <= (last >> ps_shift) ? bt[i0] : 0;
    pg.y = (first >> ps_shift) <= i1 && i1 <= (last >> ps_shift) ? bt[i1] : 0;
    return pg;
  };
  // Copies sub-block sb into stage st with the swizzles of the streaming kernel (K: chunk ^ ((row & 1) << 2),
  // V: chunk ^ (((row >> 1) & 3) << 1)); keys outside [lo, ctx) are zero-filled.
  const uint32_t lane_src = static_cast<uint32_t>(crow * kD + cchunk * 8);                   // elements
  const uint32_t dst_k = static_cast<uint32_t>(crow * (kD * 2) + ((cchunk ^ ((crow & 1) << 2)) << 4));
  const uint32_t dst_v = static_cast<uint32_t>(crow * (kD * 2) + ((cchunk ^ (((crow >> 1) & 3) << 1)) << 4));
  auto issue = [&](int sb, int st, int2 pg) {
    const int a0 = sb * kSub;
    const uint32_t ks = stages + st * kStreamStageBytes + dst_k;
    const uint32_t vs = stages + st * kStreamStageBytes + kStreamKBytes + dst_v;
    // rows 0..15 lie in page pg.x and rows 16..31 in pg.y (the same page when it holds 32 keys or more)
    const long long in_page = a0 & (ps - 1);
    const long long e0 = ((static_cast<long long>(pg.x) * a.hkv + kvh) * ps + in_page) * kD + lane_src;
    const long long e1 = ps == 16 ? ((static_cast<long long>(pg.y) * a.hkv + kvh) * ps - 16) * kD + lane_src : e0;
    const bf16* k0p = a.kcache + e0;
    const bf16* k1p = a.kcache + e1;
    const bf16* v0p = a.vcache + e0;
    const bf16* v1p = a.vcache + e1;
    if (a0 >= lo && a0 + kSub <= ctx) {                 // every key is live
#pragma unroll
      for (int k = 0; k < kSub / RPR; ++k) {
        const int row = RPR * k;                        // + crow
        const uint32_t vx = static_cast<uint32_t>((((row >> 1) & 3) << 1) << 4);
        cp_async16_s(ks + row * (kD * 2), (row < 16 ? k0p : k1p) + row * kD);
        cp_async16_s((vs ^ vx) + row * (kD * 2), (row < 16 ? v0p : v1p) + row * kD);
      }
    } else {
#pragma unroll
      for (int k = 0; k < kSub / RPR; ++k) {
        const int row = RPR * k;
        const uint32_t vx = static_cast<uint32_t>((((row >> 1) & 3) << 1) << 4);
        const int key = a0 + row + crow;
        const bool live = key < ctx && key >= lo;
        cp_async16_s(ks + row * (kD * 2), (row < 16 ? k0p : k1p) + row * kD, live);
        cp_async16_s((vs ^ vx) + row * (kD * 2), (row < 16 ? v0p : v1p) + row * kD, live);
      }
    }
  };

  // ---- the first two sub-blocks: before the wait on the kernels before, unless one of them holds a key
  // that the kernel before has written (the token's own, when this kernel does not rotate)
  int loaded = 0;                                       // sub-blocks of the run that have been asked for
  const bool early = fused || my_n == 0 || my_sb + min(my_n, 2) - 1 < sb_newest;
  if (early) {
#pragma unroll 1
    for (int st = 0; st < 2; ++st) {
      if (loaded < my_n) {
        issue(my_sb + loaded, st, sub_pages(my_sb + loaded));
        ++loaded;
      }
      cp_async_commit();              // one group per sub-block, empty once the work has run out
    }
  }
  pdl_wait();       // q and the newest token's K and V come from the kernels before this one
  if (!early) {
#pragma unroll 1
    for (int st = 0; st < 2; ++st) {
      if (loaded < my_n) {
        issue(my_sb + loaded, st, sub_pages(my_sb + loaded));
        ++loaded;
      }
      cp_async_commit();
    }
  }

  uint4 qlo[DB], qhi[DB];
  float o[DG][8][4];
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
#pragma unroll
  for (int dg = 0; dg < DG; ++dg)
#pragma unroll
    for (int jj = 0; jj < 8; ++jj)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[dg][jj][e] = 0.f;
  if (my_n > 0) {
#pragma unroll
    for (int db = 0; db < DB; ++db) {
      const bf16* qp = a.q + static_cast<size_t>(tok) * a.q_stride + static_cast<size_t>(kvh * G) * kD + db * 32 + t * 8;
      qlo[db] = g < G ? *reinterpret_cast<const uint4*>(qp + g * kD) : make_uint4(0, 0, 0, 0);
      qhi[db] = (HI && g + 8 < G) ? *reinterpret_cast<const uint4*>(qp + (g + 8) * kD) : make_uint4(0, 0, 0, 0);
    }
    if (fused) {     // rotate: the piece db pairs with the piece db + DB / 2 (the same d + D / 2)
      int pos = ctx - 1;
      if (pos >= rope.max_pos) {
        if (lane == 0) atomicOr(rope.status, 2);
        pos = 0;
      }
#pragma unroll
      for (int db = 0; db < DB / 2; ++db) {
        const float* c = rope.cos + static_cast<size_t>(pos) * (kD / 2) + db * 32 + t * 8;
        const float* sn = rope.sin + static_cast<size_t>(pos) * (kD / 2) + db * 32 + t * 8;
        rope_rotate8(qlo[db], qlo[db + DB / 2], c, sn);
        if (HI) rope_rotate8(qhi[db], qhi[db + DB / 2], c, sn);
      }
    }
  }

#pragma unroll 1
  for (int n = 0; n < my_n; ++n) {
    const int st = n & 1;
    const int sb = my_sb + n;
    // the page ids of the sub-block that will be loaded into this stage once it has been read
    int2 pf_pages = make_int2(0, 0);
    if (loaded < my_n) pf_pages = sub_pages(my_sb + loaded);
    cp_async_wait<1>();                                 // this sub-block's copies (all but the newest group)
    __syncwarp();                                       // ... of every lane
    const uint32_t Ks = stages + st * kStreamStageBytes;
    const uint32_t Vs = Ks + kStreamKBytes;
    const int k0 = sb * kSub;
    if (fused && sb == sb_newest) {
      // the token's own key lies in this sub-block: its k (rotated) and v go from the token's row into the
      // cache and over what the copy brought from the cache's not yet written slot
      const int pos_raw = ctx - 1, row = pos_raw - k0;
      const int pos = pos_raw < rope.max_pos ? pos_raw : 0;
      const bf16* trow = a.q + static_cast<size_t>(tok) * a.q_stride;
      const int32_t page = bt[pos_raw >> ps_shift];
      const size_t cache_row = ((static_cast<size_t>(page) * a.hkv + kvh) * ps + (pos_raw & (ps - 1))) * kD;
      constexpr int HC = CPR / 2;                       // chunks in half a row
      if (lane < HC) {
        const bf16* kp = trow + rope.k_col + kvh * kD;
        uint4 x0 = *reinterpret_cast<const uint4*>(kp + lane * 8), x1 = *reinterpret_cast<const uint4*>(kp + (lane + HC) * 8);
        rope_rotate8(x0, x1, rope.cos + static_cast<size_t>(pos) * (kD / 2) + lane * 8,
                     rope.sin + static_cast<size_t>(pos) * (kD / 2) + lane * 8);
        *reinterpret_cast<uint4*>(rope.kcache + cache_row + lane * 8) = x0;
        *reinterpret_cast<uint4*>(rope.kcache + cache_row + (lane + HC) * 8) = x1;
        const uint32_t kr = Ks + row * (kD * 2);
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(kr + ((lane ^ ((row & 1) << 2)) << 4)), "r"(x0.x),
                     "r"(x0.y), "r"(x0.z), "r"(x0.w) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(kr + (((lane + HC) ^ ((row & 1) << 2)) << 4)), "r"(x1.x),
                     "r"(x1.y), "r"(x1.z), "r"(x1.w) : "memory");
      } else if (lane < HC + CPR) {
        const int c = lane - HC;
        const uint4 x = *reinterpret_cast<const uint4*>(trow + rope.v_col + kvh * kD + c * 8);
        *reinterpret_cast<uint4*>(rope.vcache + cache_row + c * 8) = x;
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(Vs + row * (kD * 2) + ((c ^ (((row >> 1) & 3) << 1)) << 4)),
                     "r"(x.x), "r"(x.y), "r"(x.z), "r"(x.w) : "memory");
      }
      __syncwarp();
    }
    const bool whole = k0 >= lo && k0 + kSub <= ctx;               // no key of the sub-block is masked
    constexpr int kdb = kD * 2;                                    // bytes per row

    // ---- S = Q K^T (key = nt * 8 + g)
    float sv[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) sv[nt][e] = 0.f;
      const int key = nt * 8 + g;
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        const int c = db * 4 + t;
        const uint4 kf = lds128(Ks + key * kdb + ((c ^ ((key & 1) << 2)) << 4));
        mma_16816(sv[nt], qlo[db].x, qhi[db].x, qlo[db].y, qhi[db].y, kf.x, kf.y);
        mma_16816(sv[nt], qlo[db].z, qhi[db].z, qlo[db].w, qhi[db].w, kf.z, kf.w);
      }
    }
    // ---- online softmax (rows g and g + 8; the 4 lanes of a row share by shuffles); m in units of log2
    if (!whole) {
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = k0 + nt * 8 + t * 2 + e;
          if (!(key < ctx && key >= lo)) sv[nt][e] = sv[nt][2 + e] = -INFINITY;
        }
    }
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        mx_lo = fmaxf(mx_lo, sv[nt][e]);
        if (HI) mx_hi = fmaxf(mx_hi, sv[nt][2 + e]);
      }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo * sc);          // finite: the sub-block has a live key
    const float al_lo = ex2_approx(m_lo - mn_lo);         // 2^(-inf) = 0 the first time
    float ps_lo = 0.f, ps_hi = 0.f, al_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        sv[nt][e] = ex2_approx(fmaf(sv[nt][e], sc, -mn_lo));
        ps_lo += sv[nt][e];
      }
    ps_lo += __shfl_xor_sync(0xffffffffu, ps_lo, 1);
    ps_lo += __shfl_xor_sync(0xffffffffu, ps_lo, 2);
    l_lo = l_lo * al_lo + ps_lo;
    m_lo = mn_lo;
    if (HI) {
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_hi = fmaxf(m_hi, mx_hi * sc);
      al_hi = ex2_approx(m_hi - mn_hi);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          sv[nt][2 + e] = ex2_approx(fmaf(sv[nt][2 + e], sc, -mn_hi));
          ps_hi += sv[nt][2 + e];
        }
      ps_hi += __shfl_xor_sync(0xffffffffu, ps_hi, 1);
      ps_hi += __shfl_xor_sync(0xffffffffu, ps_hi, 2);
      l_hi = l_hi * al_hi + ps_hi;
      m_hi = mn_hi;
    }
#pragma unroll
    for (int dg = 0; dg < DG; ++dg)
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        o[dg][jj][0] *= al_lo;
        o[dg][jj][1] *= al_lo;
        if (HI) {
          o[dg][jj][2] *= al_hi;
          o[dg][jj][3] *= al_hi;
        }
      }
    // ---- O += P V
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const uint32_t p0 = pack_bf16(sv[2 * ks][0], sv[2 * ks][1]);
      const uint32_t p1 = HI ? pack_bf16(sv[2 * ks][2], sv[2 * ks][3]) : 0u;
      const uint32_t p2 = pack_bf16(sv[2 * ks + 1][0], sv[2 * ks + 1][1]);
      const uint32_t p3 = HI ? pack_bf16(sv[2 * ks + 1][2], sv[2 * ks + 1][3]) : 0u;
      const int kr = ks * 16 + t * 2;                 // rows kr, kr+1, kr+8, kr+9 of the V tile
#pragma unroll
      for (int dg = 0; dg < DG; ++dg) {
        uint4 v4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int row = kr + (q & 1) + (q >> 1) * 8;
          v4[q] = lds128(Vs + row * kdb + (((dg * 8 + g) ^ (((row >> 1) & 3) << 1)) << 4));
        }
        const uint32_t va[4] = {v4[0].x, v4[0].y, v4[0].z, v4[0].w}, vb[4] = {v4[1].x, v4[1].y, v4[1].z, v4[1].w};
        const uint32_t vc[4] = {v4[2].x, v4[2].y, v4[2].z, v4[2].w}, vd[4] = {v4[3].x, v4[3].y, v4[3].z, v4[3].w};
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const uint32_t sel = (jj & 1) ? 0x7632u : 0x5410u;
          mma_16816(o[dg][jj], p0, p1, p2, p3, __byte_perm(va[jj >> 1], vb[jj >> 1], sel),
                    __byte_perm(vc[jj >> 1], vd[jj >> 1], sel));
        }
      }
    }
    __syncwarp();                                       // every lane has read the stage
    if (loaded < my_n) {
      issue(my_sb + loaded, st, pf_pages);
      ++loaded;
    }
    cp_async_commit();
  }
  cp_async_wait<0>();
  __syncwarp();

  // ---- the warp's partial result into its own ring: head r at r * kRowsLd floats, d as the output has it,
  // then (max, denominator).  Thread (g, t) holds, of head g (and g + 8), d = dg*64 + (t*2+e)*8 + jj.
  float* mine = reinterpret_cast<float*>(smem_raw + warp * 2 * kStreamStageBytes);
#pragma unroll
  for (int h = 0; h < (HI ? 2 : 1); ++h) {
    const int r = g + 8 * h;
    if (r >= G) continue;
#pragma unroll
    for (int dg = 0; dg < DG; ++dg)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float* dst = mine + r * kRowsLd + dg * 64 + (t * 2 + e) * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(o[dg][0][2 * h + e], o[dg][1][2 * h + e], o[dg][2][2 * h + e], o[dg][3][2 * h + e]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(o[dg][4][2 * h + e], o[dg][5][2 * h + e], o[dg][6][2 * h + e], o[dg][7][2 * h + e]);
      }
    if (t == 0) *reinterpret_cast<float2*>(mine + r * kRowsLd + kD) = make_float2(h ? m_hi : m_lo, h ? l_hi : l_lo);
  }
  if (csize == 1) {
    // ---- a cluster of one CTA: the group's warps in order, straight to the output (a warp without keys has
    // max -inf and weighs nothing); only the group meets, at a barrier of its own
    const int gthreads = gsize * 32;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(gthreads) : "memory");
    for (int idx = wg * 32 + lane; idx < G * (kD / 2); idx += gthreads) {
      const int r = idx / (kD / 2), d = (idx - r * (kD / 2)) * 2;
      float m = -INFINITY;
      for (int w = gi * gsize; w < (gi + 1) * gsize; ++w)
        m = fmaxf(m, reinterpret_cast<const float*>(smem_raw + w * 2 * kStreamStageBytes)[r * kRowsLd + kD]);
      float den = 0.f, n0 = 0.f, n1 = 0.f;
      for (int w = gi * gsize; w < (gi + 1) * gsize; ++w) {
        const float* pw = reinterpret_cast<const float*>(smem_raw + w * 2 * kStreamStageBytes) + r * kRowsLd;
        const float mw = pw[kD];
        const float f = mw == -INFINITY ? 0.f : ex2_approx(mw - m);
        const float2 v = *reinterpret_cast<const float2*>(pw + d);
        den += f * pw[kD + 1];
        n0 += f * v.x;
        n1 += f * v.y;
      }
      const __nv_bfloat162 hh = __floats2bfloat162_rn(n0 / den, n1 / den);
      *reinterpret_cast<__nv_bfloat162*>(a.out + static_cast<size_t>(tok) * a.out_stride + (kvh * G + r) * kD + d) = hh;
    }
    asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(gthreads) : "memory");     // before the rings are used again
    continue;
  }
  __syncthreads();
  // ---- the CTA's warps in order (a warp without keys has max -inf and weighs nothing)
  for (int idx = threadIdx.x; idx < G * (kD / 2); idx += kRowsThreads) {
    const int r = idx / (kD / 2), d = (idx - r * (kD / 2)) * 2;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kRowsWarps; ++w)
      m = fmaxf(m, reinterpret_cast<const float*>(smem_raw + w * 2 * kStreamStageBytes)[r * kRowsLd + kD]);
    float den = 0.f, n0 = 0.f, n1 = 0.f;
#pragma unroll
    for (int w = 0; w < kRowsWarps; ++w) {
      const float* pw = reinterpret_cast<const float*>(smem_raw + w * 2 * kStreamStageBytes) + r * kRowsLd;
      const float mw = pw[kD];
      const float f = mw == -INFINITY ? 0.f : ex2_approx(mw - m);
      const float2 v = *reinterpret_cast<const float2*>(pw + d);
      den += f * pw[kD + 1];
      n0 += f * v.x;
      n1 += f * v.y;
    }
    // into slot `rank` of the cluster's first CTA (its own slot 0 for that CTA itself)
    if (rank == 0) {
      *reinterpret_cast<float2*>(&sh->cta_o[0][r][d]) = make_float2(n0, n1);
      if (d == 0) *reinterpret_cast<float2*>(&sh->cta_ml[0][r][0]) = make_float2(m, den);
    } else {
      rows_st_cluster(&sh->cta_o[rank][r][d], 0, make_float2(n0, n1));
      if (d == 0) rows_st_cluster(&sh->cta_ml[rank][r][0], 0, make_float2(m, den));
    }
  }
  // ---- the cluster's CTAs in order, by the first one, from its own shared memory (the barrier's release and
  // acquire make the other CTAs' stores visible there); the others are done
  rows_cluster_barrier();
  if (rank == 0) {
    for (int idx = threadIdx.x; idx < G * (kD / 2); idx += kRowsThreads) {
      const int r = idx / (kD / 2), d = (idx - r * (kD / 2)) * 2;
      float m = -INFINITY;
#pragma unroll
      for (int c = 0; c < kRowsMaxCluster; ++c)
        if (c < csize) m = fmaxf(m, sh->cta_ml[c][r][0]);
      float den = 0.f, n0 = 0.f, n1 = 0.f;
#pragma unroll
      for (int c = 0; c < kRowsMaxCluster; ++c)
        if (c < csize) {
          const float mc = sh->cta_ml[c][r][0];
          const float f = mc == -INFINITY ? 0.f : ex2_approx(mc - m);
          const float2 v = *reinterpret_cast<const float2*>(&sh->cta_o[c][r][d]);
          den += f * sh->cta_ml[c][r][1];
          n0 += f * v.x;
          n1 += f * v.y;
        }
      const __nv_bfloat162 hh = __floats2bfloat162_rn(n0 / den, n1 / den);
      *reinterpret_cast<__nv_bfloat162*>(a.out + static_cast<size_t>(tok) * a.out_stride + (kvh * G + r) * kD + d) = hh;
    }
  }
  }
}

}  // namespace rl
