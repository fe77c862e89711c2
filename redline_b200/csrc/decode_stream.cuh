// Decode attention that streams the cache: persistent CTAs (one per SM) of independent warps.
//
// Included by attention.cu (bfloat16, head size 64 or 128).  The unit of work is one (item, kv
// head, 128-key partition); the units of a launch are numbered in one list, an item's kv heads
// one after another and a head's partitions in order, and the list is cut into as many equal
// runs as there are warps at work.  Every warp is its own pipeline: it moves the keys of its run
// through a private two-stage ring of shared memory in sub-blocks of 32 keys; while it computes
// on one sub-block, the 16-byte asynchronous copies (cp.async) of the next are in flight, issued
// by the warp itself.  Per sub-block: S = Q K^T, online softmax, O += P V (mma.sync.m16n8k16
// with the fragment permutations of the kernel above; keys outside the live range are
// zero-filled by the copy).  The running (m, l, O) carries on from partition to partition of
// the same (item, head): a row of partitions that lies in one warp's run goes straight to the
// output; one that is cut by the ends of runs leaves one partial result per run, and the warps
// count those at the end of their runs, when none of their copies are in flight any more (a
// release at device scope waits for those too).  The warp that counts a row's last piece
// queues the merge, and when all warps of the CTA are through with their runs they do the queued
// merges together, pieces in order.  Nothing in the kernel waits on a flag.
//
// The cut of the list depends on how many units the launch has, so the order in which a row's
// keys are summed, and with it the last bits of the result, depends on what else is in the batch.
#pragma once

namespace rl {

constexpr int kStreamWarps = (kD == 64) ? 12 : 6;
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kStreamMaxItems = 512;
constexpr int kSub = 32;                                  // keys per sub-block
constexpr int kStreamKBytes = kSub * kD * 2;              // K (or V) of one sub-block
constexpr int kStreamStageBytes = 2 * kStreamKBytes;
constexpr int kStreamMinUnits = 1024;    // launches that can have fewer units go to the one-partition kernel
constexpr int kStreamQueue = 256;       // merges a CTA can hold for its end (more are done at once, by one warp)

struct StreamShared {
  int units;
  int queued;
  int2 queue[kStreamQueue];
  int start[kStreamMaxItems + 1];      // first unit of every item
  int4 items[kStreamMaxItems];
};
constexpr size_t kStreamSmem = static_cast<size_t>(kStreamWarps) * 2 * kStreamStageBytes + sizeof(StreamShared) + 16;

// The cut of the unit list into runs: run k is [k q + min(k, rem), ...) with q or q + 1 units.
struct StreamCut {
  int warps, q, rem;
  __device__ __forceinline__ int begin(int k) const { return k * q + min(k, rem); }
  __device__ __forceinline__ int run_of(int u) const {
    const int big = rem * (q + 1);
    return u < big ? u / (q + 1) : rem + (u - big) / q;
  }
};

// As few warps as do the work in the same number of rounds, so that every warp has (almost) the same
// number of units: with 2048 units and 1776 warps, 1024 warps take two each.
__device__ __forceinline__ StreamCut stream_cut(int units, int max_warps) {
  StreamCut c;
  const int rounds = (units + max_warps - 1) / max_warps;
  c.warps = rounds > 0 ? (units + rounds - 1) / rounds : 0;
  c.q = c.warps > 0 ? units / c.warps : 0;
  c.rem = c.warps > 0 ? units - c.q * c.warps : 0;
  return c;
}

struct StreamUnit {
  int item, part, kvh;     // part: absolute partition index
  int tok, seq, ctx, lo;
  int p_lo, np;            // the item's first live partition and their number
  int row_begin;           // the unit of (item, kvh, p_lo)
};

// Unit u of the launch.  `hint` is an item that earlier units of the caller lay in: units only move
// forward, and while u still lies in that item no search is needed.
__device__ __forceinline__ StreamUnit stream_unit(const StreamShared* sh, int u, int nitems, int window, int hint) {
  int it = hint;
  if (it < 0 || u >= sh->start[it + 1]) {
    int lo_i = it < 0 ? 0 : it + 1, hi_i = nitems - 1;            // largest i with start[i] <= u
    while (lo_i < hi_i) {
      const int mid = (lo_i + hi_i + 1) >> 1;
      if (sh->start[mid] <= u) lo_i = mid; else hi_i = mid - 1;
    }
    it = lo_i;
  }
  StreamUnit w;
  w.item = it;
  const int4 info = sh->items[it];
  w.tok = info.x;
  w.seq = info.y;
  w.ctx = info.z;
  w.lo = (window > 0 && w.ctx > window) ? w.ctx - window : 0;
  w.p_lo = w.lo / kPart;
  w.np = (w.ctx - 1) / kPart - w.p_lo + 1;
  const int local = u - sh->start[it];
  w.kvh = local / w.np;
  w.part = w.p_lo + local - w.kvh * w.np;
  w.row_begin = sh->start[it] + w.kvh * w.np;
  return w;
}

// Walks the sub-blocks of a warp's run in order.
struct StreamCursor {
  int u, end;              // unit and the end of the run (u >= end: done)
  StreamUnit w;
  int sb, sb_last;         // sub-block of the partition and its last live one
};

__device__ __forceinline__ void cursor_enter(StreamCursor& c, const StreamShared* sh, int nitems, int window) {
  if (c.u >= c.end) return;
  c.w = stream_unit(sh, c.u, nitems, window, c.w.item);
  const int k0 = c.w.part * kPart;
  c.sb = (max(c.w.lo, k0) - k0) / kSub;
  c.sb_last = (min(c.w.ctx, k0 + kPart) - 1 - k0) / kSub;
}
__device__ __forceinline__ void cursor_advance(StreamCursor& c, const StreamShared* sh, int nitems, int window) {
  if (++c.sb > c.sb_last) {
    ++c.u;
    cursor_enter(c, sh, nitems, window);
  }
}

__device__ __forceinline__ float ex2_approx(float x) {      // 2^x; -inf gives 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ int atomic_add_acq_rel(int* p, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}

__device__ __forceinline__ uint32_t smem_u32s(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void cp_async16_s(uint32_t smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem), "l"(gmem));
}
__device__ __forceinline__ void cp_async16_s(uint32_t smem, const void* gmem, bool pred) {
  const int bytes = pred ? 16 : 0;   // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "r"(bytes));
}

// Merges the pieces of (item, kv head) into the output row of each of its heads; `nthreads` threads
// (a warp or the CTA) share the columns, tid being the caller's index among them.  A piece is what
// one run of the cut left of the row; it lies in the slot of its first partition.  Pieces are taken
// sixteen at a time, all their loads in flight together, and folded into a running (max,
// denominator, numerators) in order: the result does not depend on who merges.
__device__ __forceinline__ void stream_merge(const DecodeArgs<bf16>& a, const StreamShared* sh, const StreamCut& cut,
                                             int item, int kvh, int tid, int nthreads) {
  const int G = a.hq / a.hkv;
  const int4 info = sh->items[item];
  const int tok = info.x, ctx = info.z;
  const int lo = (a.window > 0 && ctx > a.window) ? ctx - a.window : 0;
  const int p_lo = lo / kPart, np = (ctx - 1) / kPart - p_lo + 1;
  const int row_begin = sh->start[item] + kvh * np;
  const int k_first = cut.run_of(row_begin), k_last = cut.run_of(row_begin + np - 1);
  const int pieces = k_last - k_first + 1;
  for (int idx = tid; idx < G * (kD / 2); idx += nthreads) {        // a thread takes two neighbouring columns
    const int r = idx / (kD / 2), d = (idx - r * (kD / 2)) * 2;
    const int head = kvh * G + r;
    const size_t row0 = (static_cast<size_t>(item) * a.hq + head) * a.max_parts + p_lo;
    const float2* ml = reinterpret_cast<const float2*>(a.part_ml) + row0;
    const float* po = a.part_o + row0 * kD + d;
    float mrun = -INFINITY, den = 0.f, num0 = 0.f, num1 = 0.f;
    for (int i0 = 0; i0 < pieces; i0 += 16) {
      float2 q[16], v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const bool in = i0 + i < pieces;
        const int slot = in ? max(cut.begin(k_first + i0 + i) - row_begin, 0) : 0;    // the piece's first partition
        q[i] = in ? __ldcg(&ml[slot]) : make_float2(-INFINITY, 0.f);
        v[i] = in ? __ldcg(reinterpret_cast<const float2*>(po + static_cast<size_t>(slot) * kD)) : make_float2(0.f, 0.f);
      }
      float mc = mrun;
#pragma unroll
      for (int i = 0; i < 16; ++i) mc = fmaxf(mc, q[i].x);        // finite: every piece has a live key
      const float f = expf(mrun - mc);                            // exp(-inf) = 0 the first time
      den *= f;
      num0 *= f;
      num1 *= f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float wgt = expf(q[i].x - mc);
        den += wgt * q[i].y;
        num0 += wgt * v[i].x;
        num1 += wgt * v[i].y;
      }
      mrun = mc;
    }
    const __nv_bfloat162 hh = __floats2bfloat162_rn(num0 / den, num1 / den);
    *reinterpret_cast<__nv_bfloat162*>(a.out + static_cast<size_t>(tok) * a.out_stride + head * kD + d) = hh;
  }
}

// HI: groups of more than 8 heads (rows g + 8 of the MMA tile are in use).
template <bool HI>
__global__ void __launch_bounds__(kStreamThreads, 1)
decode_attn_stream_kernel(const DecodeArgs<bf16> a, int nitems, const DecodeRope rope) {
  constexpr int DB = kD / 32, DG = kD / 64;
  constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
  constexpr int CPR = kD / 8;            // 16-byte chunks per row
  constexpr int RPR = 32 / CPR;          // rows that one round of the warp's copies covers
  static_assert(RPR == 2 || RPR == 4, "the swizzle bookkeeping assumes 2 or 4 rows per round");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  StreamShared* sh = reinterpret_cast<StreamShared*>(smem_raw + kStreamWarps * 2 * kStreamStageBytes);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = a.hq / a.hkv;

  // (The kernel does not tell its dependents to launch early: measured in the decode step, the step is a
  // fifth slower when it does, at its beginning or after the runs.)
  // ---- the list of units: items and block tables were written before the step's kernels began,
  // so this part may run while the kernel before this one drains
  for (int i = threadIdx.x; i < nitems; i += kStreamThreads) sh->items[i] = a.items[i];
  __syncthreads();
  if (warp == 0) {
    int run = 0;
    for (int i0 = 0; i0 < nitems; i0 += 32) {
      const int i = i0 + lane;
      int n = 0;
      if (i < nitems) {
        const int ctx = sh->items[i].z;
        if (ctx > 0) {
          const int lo = (a.window > 0 && ctx > a.window) ? ctx - a.window : 0;
          n = ((ctx - 1) / kPart - lo / kPart + 1) * a.hkv;
        }
      }
      int inc = n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += up;
      }
      if (i < nitems) sh->start[i] = run + inc - n;
      run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) {
      sh->start[nitems] = run;
      sh->units = run;
      sh->queued = 0;
    }
  }
  __syncthreads();
  const int units = sh->units;
  const StreamCut cut = stream_cut(units, gridDim.x * kStreamWarps);
  pdl_wait();       // q and the newest token's K and V come from the kernels before this one

  // ---- this warp's pipeline
  const int ps = a.page_size;
  const int ps_shift = __ffs(ps) - 1;                   // page sizes are powers of two
  const uint32_t stages = smem_u32s(smem_raw) + warp * 2 * kStreamStageBytes;
  const int g = lane >> 2, t = lane & 3;
  const float sc = a.scale * kLog2e;
  const int crow = lane / CPR, cchunk = lane % CPR;     // this lane's row (of a round) and chunk in the copies

  // the (at most two) pages a sub-block of cursor c lies in; a page without a live key reads as page 0
  auto sub_pages = [&](const StreamCursor& c) -> int2 {
    const int a0 = c.w.part * kPart + c.sb * kSub;
    const int32_t* bt = a.block_table + static_cast<size_t>(c.w.seq) * a.max_blocks;
    const int first = max(a0, c.w.lo), last = min(a0 + kSub, c.w.ctx) - 1;     // live keys of the sub-block
    int2 pg;
    const int i0 = a0 >> ps_shift, i1 = (a0 + 16) >> ps_shift;
    pg.x = (first >> ps_shift) <= i0 && i0 <= (last >> ps_shift) ? bt[i0] : 0;
    pg.y = (first >> ps_shift) <= i1 && i1 <= (last >> ps_shift) ? bt[i1] : 0;
    return pg;
  };
  // Copies the sub-block into stage st: K rows with the chunk swizzle c ^ ((row & 1) << 2), V rows with
  // c ^ (((row >> 1) & 3) << 1) (the low three bits of the chunk index), which make the fragment reads
  // below free of bank conflicts.  Keys outside [lo, ctx) are zero-filled.  Round k of the copies
  // takes rows crow + RPR k: the row's parity, and so the K swizzle, is the lane's own, and the V
  // swizzle is the lane's own part XOR a part that depends on k alone.
  const uint32_t lane_src = static_cast<uint32_t>(crow * kD + cchunk * 8);                   // elements
  const uint32_t dst_k = static_cast<uint32_t>(crow * (kD * 2) + ((cchunk ^ ((crow & 1) << 2)) << 4));
  const uint32_t dst_v = static_cast<uint32_t>(crow * (kD * 2) + ((cchunk ^ (((crow >> 1) & 3) << 1)) << 4));
  auto issue = [&](const StreamCursor& c, int st, int2 pg) {
    const int a0 = c.w.part * kPart + c.sb * kSub;
    const uint32_t ks = stages + st * kStreamStageBytes + dst_k;
    const uint32_t vs = stages + st * kStreamStageBytes + kStreamKBytes + dst_v;
    // rows 0..15 lie in page pg.x and rows 16..31 in pg.y (the same page when it holds 32 keys or more)
    const long long in_page = a0 & (ps - 1);
    const long long e0 = ((static_cast<long long>(pg.x) * a.hkv + c.w.kvh) * ps + in_page) * kD + lane_src;
    const long long e1 = ps == 16 ? ((static_cast<long long>(pg.y) * a.hkv + c.w.kvh) * ps - 16) * kD + lane_src : e0;
    const bf16* k0p = a.kcache + e0;
    const bf16* k1p = a.kcache + e1;
    const bf16* v0p = a.vcache + e0;
    const bf16* v1p = a.vcache + e1;
    if (a0 >= c.w.lo && a0 + kSub <= c.w.ctx) {         // every key is live
#pragma unroll
      for (int k = 0; k < kSub / RPR; ++k) {
        const int row = RPR * k;                        // + crow
        // ((crow + row) >> 1) & 3 = (crow >> 1) ^ ((row >> 1) & 3): no carry, as row >> 1 is even (RPR = 4) or crow < 2
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
        const bool live = key < c.w.ctx && key >= c.w.lo;
        cp_async16_s(ks + row * (kD * 2), (row < 16 ? k0p : k1p) + row * kD, live);
        cp_async16_s((vs ^ vx) + row * (kD * 2), (row < 16 ? v0p : v1p) + row * kD, live);
      }
    }
  };

  StreamCursor cc, lc;                  // compute and load cursors; the load cursor runs two sub-blocks ahead
  {
    const int k = warp * gridDim.x + blockIdx.x;      // runs of neighbouring numbers go to different SMs
    cc.u = cc.end = 0;
    if (k < cut.warps) {
      cc.u = cut.begin(k);
      cc.end = cut.begin(k + 1);
    }
    cc.w.item = -1;                                   // no item known yet
    cc.sb = cc.sb_last = 0;
    cursor_enter(cc, sh, nitems, a.window);
  }
  const int run_end = cc.end;
  lc = cc;
#pragma unroll 1
  for (int st = 0; st < 2; ++st) {
    if (lc.u < run_end) {
      issue(lc, st, sub_pages(lc));
      cursor_advance(lc, sh, nitems, a.window);
    }
    cp_async_commit();                  // one group per sub-block, empty once the work has run out
  }

  uint4 qlo[DB], qhi[DB];
  float o[DG][8][4];
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  int piece_begin = -1;                 // first unit of the piece of a row that is being summed; -1: none yet
  int2 owed0 = make_int2(-1, 0), owed1 = make_int2(-1, 0);   // rows this warp left a piece of: (item, kv head)
#pragma unroll 1
  for (int n = 0; cc.u < run_end; ++n) {
    const int st = n & 1;
    // the page ids of the sub-block that will be loaded into this stage once it has been read
    int2 pf_pages = make_int2(0, 0);
    if (lc.u < run_end) pf_pages = sub_pages(lc);
    if (piece_begin < 0 || (cc.u == cc.w.row_begin && cc.u != piece_begin)) {     // a new row begins
      piece_begin = cc.u;
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        const bf16* qp = a.q + static_cast<size_t>(cc.w.tok) * a.q_stride + static_cast<size_t>(cc.w.kvh * G) * kD + db * 32 + t * 8;
        qlo[db] = g < G ? *reinterpret_cast<const uint4*>(qp + g * kD) : make_uint4(0, 0, 0, 0);
        qhi[db] = (HI && g + 8 < G) ? *reinterpret_cast<const uint4*>(qp + (g + 8) * kD) : make_uint4(0, 0, 0, 0);
      }
      if (rope.cos != nullptr) {     // rotate: the piece db pairs with the piece db + DB / 2 (the same d + D / 2)
        int pos = cc.w.ctx - 1;
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
#pragma unroll
      for (int dg = 0; dg < DG; ++dg)
#pragma unroll
        for (int jj = 0; jj < 8; ++jj)
#pragma unroll
          for (int e = 0; e < 4; ++e) o[dg][jj][e] = 0.f;
      m_lo = m_hi = -INFINITY;
      l_lo = l_hi = 0.f;
    }
    cp_async_wait<1>();                                 // this sub-block's copies (all but the newest group)
    __syncwarp();                                       // ... of every lane
    const uint32_t Ks = stages + st * kStreamStageBytes;
    const uint32_t Vs = Ks + kStreamKBytes;
    const int k0 = cc.w.part * kPart + cc.sb * kSub;
    if (rope.cos != nullptr && k0 <= cc.w.ctx - 1 && cc.w.ctx - 1 < k0 + kSub) {
      // the token's own key lies in this sub-block: its k (rotated) and v go from the token's row into the
      // cache and over what the copy brought from the cache's not yet written slot
      const int pos_raw = cc.w.ctx - 1, row = pos_raw - k0;
      const int pos = pos_raw < rope.max_pos ? pos_raw : 0;
      const bf16* trow = a.q + static_cast<size_t>(cc.w.tok) * a.q_stride;
      const int32_t page = a.block_table[static_cast<size_t>(cc.w.seq) * a.max_blocks + (pos_raw >> ps_shift)];
      const size_t crow = ((static_cast<size_t>(page) * a.hkv + cc.w.kvh) * ps + (pos_raw & (ps - 1))) * kD;
      constexpr int HC = CPR / 2;                       // chunks in half a row
      if (lane < HC) {
        const bf16* kp = trow + rope.k_col + cc.w.kvh * kD;
        uint4 x0 = *reinterpret_cast<const uint4*>(kp + lane * 8), x1 = *reinterpret_cast<const uint4*>(kp + (lane + HC) * 8);
        rope_rotate8(x0, x1, rope.cos + static_cast<size_t>(pos) * (kD / 2) + lane * 8,
                     rope.sin + static_cast<size_t>(pos) * (kD / 2) + lane * 8);
        *reinterpret_cast<uint4*>(rope.kcache + crow + lane * 8) = x0;
        *reinterpret_cast<uint4*>(rope.kcache + crow + (lane + HC) * 8) = x1;
        const uint32_t kr = Ks + row * (kD * 2);
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(kr + ((lane ^ ((row & 1) << 2)) << 4)), "r"(x0.x),
                     "r"(x0.y), "r"(x0.z), "r"(x0.w) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(kr + (((lane + HC) ^ ((row & 1) << 2)) << 4)), "r"(x1.x),
                     "r"(x1.y), "r"(x1.z), "r"(x1.w) : "memory");
      } else if (lane < HC + CPR) {
        const int c = lane - HC;
        const uint4 x = *reinterpret_cast<const uint4*>(trow + rope.v_col + cc.w.kvh * kD + c * 8);
        *reinterpret_cast<uint4*>(rope.vcache + crow + c * 8) = x;
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(Vs + row * (kD * 2) + ((c ^ (((row >> 1) & 3) << 1)) << 4)),
                     "r"(x.x), "r"(x.y), "r"(x.z), "r"(x.w) : "memory");
      }
      __syncwarp();
    }
    const bool whole = k0 >= cc.w.lo && k0 + kSub <= cc.w.ctx;     // no key of the sub-block is masked
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
          if (!(key < cc.w.ctx && key >= cc.w.lo)) sv[nt][e] = sv[nt][2 + e] = -INFINITY;
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
    if (lc.u < run_end) {
      issue(lc, st, pf_pages);
      cursor_advance(lc, sh, nitems, a.window);
    }
    cp_async_commit();
    // ---- is this the end of the row, or of this warp's piece of it?
    const StreamUnit w = cc.w;
    const bool unit_done = (cc.sb == cc.sb_last);
    cursor_advance(cc, sh, nitems, a.window);
    if (!unit_done) continue;
    const int row_end = w.row_begin + w.np;
    const int u_next = cc.u;                            // the unit after the one just finished
    if (u_next != row_end && u_next != run_end) continue;
    // thread (g, t) holds, of row g (and g + 8), d = dg*64 + (t*2+e)*8 + jj
    const bool whole_row = (piece_begin == w.row_begin && u_next == row_end);
    const int slot = w.p_lo + (piece_begin - w.row_begin);          // the piece's first partition
#pragma unroll
    for (int h = 0; h < (HI ? 2 : 1); ++h) {
      const int r = g + 8 * h;
      if (r >= G) continue;
      const int head = w.kvh * G + r;
      const float l = h ? l_hi : l_lo, m = h ? m_hi : m_lo;
      if (whole_row) {
        const float inv = 1.f / l;
#pragma unroll
        for (int dg = 0; dg < DG; ++dg)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float v[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) v[jj] = o[dg][jj][2 * h + e] * inv;
            store16(a.out + static_cast<size_t>(w.tok) * a.out_stride + head * kD + dg * 64 + (t * 2 + e) * 8, v);
          }
      } else {
        const size_t row = (static_cast<size_t>(w.item) * a.hq + head) * a.max_parts + slot;
#pragma unroll
        for (int dg = 0; dg < DG; ++dg)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float* dst = a.part_o + row * kD + dg * 64 + (t * 2 + e) * 8;
            *reinterpret_cast<float4*>(dst) = make_float4(o[dg][0][2 * h + e], o[dg][1][2 * h + e], o[dg][2][2 * h + e], o[dg][3][2 * h + e]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(o[dg][4][2 * h + e], o[dg][5][2 * h + e], o[dg][6][2 * h + e], o[dg][7][2 * h + e]);
          }
        if (t == 0) *reinterpret_cast<float2*>(a.part_ml + row * 2) = make_float2(m * kLn2, l);   // natural-log units
      }
    }
    // a run has at most two pieces of rows: one at its beginning and one at its end
    if (!whole_row) {
      if (owed0.x < 0) owed0 = make_int2(w.item, w.kvh);
      else owed1 = make_int2(w.item, w.kvh);
    }
  }
  cp_async_wait<0>();
  // ---- count the pieces; the warp that counts a row's last piece queues the merge (or, if the queue is
  // full, merges at once by itself)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int2 ow = i == 0 ? owed0 : owed1;
    if (ow.x < 0) continue;                             // (the same for all lanes)
    const int item = ow.x, kvh = ow.y;
    __syncwarp();
    int slot = -1;
    if (lane == 0) {
      const int4 info = sh->items[item];
      const int lo = (a.window > 0 && info.z > a.window) ? info.z - a.window : 0;
      const int np = (info.z - 1) / kPart - lo / kPart + 1;
      const int row_begin = sh->start[item] + kvh * np;
      const int pieces = cut.run_of(row_begin + np - 1) - cut.run_of(row_begin) + 1;
      int* c = a.counters + item * a.hkv + kvh;
      const int done = atomic_add_acq_rel(c, 1) + 1;
      if (done == pieces) {
        *c = 0;                                          // ready for the next launch
        slot = atomicAdd(&sh->queued, 1);
        if (slot < kStreamQueue) sh->queue[slot] = make_int2(item, kvh);
      }
    }
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot >= kStreamQueue) {
      __threadfence();
      stream_merge(a, sh, cut, item, kvh, lane, 32);
    }
  }
  __syncthreads();
  // The queued merges, several at a time: a merge takes one thread per pair of output columns (the
  // pieces are read with ld.cg from L2, where the counting made them visible).
  const int nq = min(sh->queued, kStreamQueue);
  const int pairs = G * (kD / 2);
  const int per = min(kStreamThreads, (pairs + 31) / 32 * 32), groups = kStreamThreads / per;
  const int grp = threadIdx.x / per;
  if (grp < groups)
    for (int i = grp; i < nq; i += groups) {
      const int2 e = sh->queue[i];
      stream_merge(a, sh, cut, e.x, e.y, threadIdx.x - grp * per, per);
    }
}

}  // namespace rl
