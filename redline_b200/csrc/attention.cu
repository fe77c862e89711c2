// Attention over the paged cache, compiled for one head size (-DRL_HEAD_DIM=D,
// D a multiple of 16 up to 256) and both element types (float, bfloat16).
//
//   rl_attn_decode   one query token per item; the keys are cut into absolute
//                    128-key partitions and all G query heads of a group are computed
//                    from one read of K and V (restates src/cuda/kernels/attention.cu:69-209).
//                    Three kernels: a CUDA-core kernel, one CTA per (partition, kv head,
//                    item), with a second kernel that merges the partitions with
//                    w_i = exp(m_i - m) (any head size, both types); a tensor-core kernel of
//                    the same shape with the merge fused (bfloat16, head size 64 or 128);
//                    and, for launches with many partitions, the streaming kernel of
//                    decode_stream.cuh (persistent CTAs, cp.async rings).
//   rl_attn_prefill  tiles of query rows against tiles of keys with an online softmax; the
//                    keys of a tile come from the cache, so a prompt portion attends to
//                    what earlier portions left there (attention.cu:217-359).  A CUDA-core
//                    kernel (32 x 32 tiles, any head size, both types), an mma.sync kernel
//                    (64 query rows x 64 keys per CTA, bfloat16, head size 64 or 128) and,
//                    at head size 64, the tcgen05 kernel of prefill_tc.cuh.
//
// Scores, the softmax and the P.V sums are float whatever the element type.  A
// window w > 0 keeps only keys with pos - w < key <= pos.  The cache of a layer is
// K [pages, Hkv, page_size, D] and V alike; a token's page comes from its
// sequence's row of the block table.
#include <mutex>

#include "common.cuh"

#ifndef RL_HEAD_DIM
#error "compile with -DRL_HEAD_DIM=<head size>"
#endif

namespace rl {

constexpr int kD = RL_HEAD_DIM;
static_assert(kD % 16 == 0 && kD >= 16 && kD <= 256, "head size must be a multiple of 16, at most 256");
constexpr int kPart = 128;      // keys per decode partition (absolute boundaries)
constexpr int kDecThreads = 128;
constexpr int kLPK = 8;         // lanes that share one key
constexpr int kKeysPerIter = kDecThreads / kLPK;  // 16
constexpr int kGT = 4;          // query heads per pass over the keys
constexpr int kMaxMergeParts = 256;    // the fused merge of the tensor-core kernel holds this many weights

template <typename T>
struct DecodeArgs {
  const T* q;            // [tokens, q_stride], head h at column h * D
  int q_stride;
  const T* kcache;
  const T* vcache;
  const int32_t* block_table;  // [seqs, max_blocks]
  int max_blocks;
  const int4* items;           // [items] (token index of the query, sequence index, context length, 0)
  float* part_o;               // [items, Hq, max_parts, D]
  float* part_ml;              // [items, Hq, max_parts, 2]
  int max_parts;
  int* counters;               // [items, Hkv] zero between launches (tensor-core kernel: fused merge)
  T* out;                      // [tokens, out_stride]
  int out_stride;
  int hq, hkv, page_size, window;
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(kDecThreads)
decode_attn_kernel(const DecodeArgs<T> a) {
  pdl_launch();
  pdl_wait();
  constexpr int VEC = Vec16<T>::N;
  constexpr int CH = kD / VEC;                     // 16-byte chunks per key
  constexpr int CPL = (CH + kLPK - 1) / kLPK;      // chunks per lane
  __shared__ float qs[kGT][kD];
  __shared__ float sc[kGT][kPart];
  __shared__ float red[kDecThreads / 32][kGT][kD];
  __shared__ float stat_m[kGT], stat_l[kGT];

  const int part = blockIdx.x, kvh = blockIdx.y, item = blockIdx.z;
  const int4 info = a.items[item];
  const int tok = info.x, seq = info.y, ctx = info.z;
  const int lo = (a.window > 0 && ctx > a.window) ? ctx - a.window : 0;
  const int j_lo = max(lo, part * kPart), j_hi = min(ctx, (part + 1) * kPart);
  if (j_lo >= j_hi) return;
  const int G = a.hq / a.hkv;
  const int lane8 = threadIdx.x % kLPK, slot = threadIdx.x / kLPK;
  const int warp = threadIdx.x >> 5;
  const int32_t* bt = a.block_table + static_cast<size_t>(seq) * a.max_blocks;
  const int base = part * kPart;

  for (int g0 = 0; g0 < G; g0 += kGT) {
    const int ng = min(kGT, G - g0);
    __syncthreads();
    for (int i = threadIdx.x; i < kGT * kD; i += kDecThreads) {
      const int g = i / kD, d = i - g * kD;
      qs[g][d] = g < ng ? to_float(a.q[static_cast<size_t>(tok) * a.q_stride +
                                       (kvh * G + g0 + g) * kD + d]) * a.scale
                        : 0.f;
    }
    __syncthreads();
    // ---- scores
    // (the trip count is the same for every lane of a warp: the shuffles below need all of them)
    for (int jb = j_lo; jb < j_hi; jb += kKeysPerIter) {
      const int j = jb + slot;
      const bool live = j < j_hi;
      const size_t page = live ? bt[j / a.page_size] : 0;
      const T* kp = a.kcache + ((page * a.hkv + kvh) * a.page_size + j % a.page_size) * kD;
      float dot[kGT];
#pragma unroll
      for (int g = 0; g < kGT; ++g) dot[g] = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int ch = lane8 + c * kLPK;
        if (live && ch < CH) {
          float kf[VEC];
          load16(kp + ch * VEC, kf);
#pragma unroll
          for (int g = 0; g < kGT; ++g) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) dot[g] += kf[e] * qs[g][ch * VEC + e];
          }
        }
      }
#pragma unroll
      for (int g = 0; g < kGT; ++g) {
        float v = dot[g];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        if (lane8 == 0 && live) sc[g][j - base] = v;
      }
    }
    __syncthreads();
    // ---- softmax statistics of this partition, one warp per head
    for (int g = warp; g < ng; g += kDecThreads / 32) {
      float m = -INFINITY;
      for (int j = j_lo + (threadIdx.x & 31); j < j_hi; j += 32) m = fmaxf(m, sc[g][j - base]);
      m = warp_max(m);
      float l = 0.f;
      for (int j = j_lo + (threadIdx.x & 31); j < j_hi; j += 32) {
        const float p = expf(sc[g][j - base] - m);
        sc[g][j - base] = p;
        l += p;
      }
      l = warp_sum(l);
      if ((threadIdx.x & 31) == 0) {
        stat_m[g] = m;
        stat_l[g] = l;
      }
    }
    __syncthreads();
    // ---- P.V
    float acc[kGT][CPL][VEC];
#pragma unroll
    for (int g = 0; g < kGT; ++g)
#pragma unroll
      for (int c = 0; c < CPL; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[g][c][e] = 0.f;
    for (int j = j_lo + slot; j < j_hi; j += kKeysPerIter) {
      const size_t page = bt[j / a.page_size];
      const T* vp = a.vcache + ((page * a.hkv + kvh) * a.page_size + j % a.page_size) * kD;
      float p[kGT];
#pragma unroll
      for (int g = 0; g < kGT; ++g) p[g] = g < ng ? sc[g][j - base] : 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int ch = lane8 + c * kLPK;
        if (ch < CH) {
          float vf[VEC];
          load16(vp + ch * VEC, vf);
#pragma unroll
          for (int g = 0; g < kGT; ++g)
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[g][c][e] += p[g] * vf[e];
        }
      }
    }
    // lanes 8 and 16 apart hold other keys of the same chunk
#pragma unroll
    for (int g = 0; g < kGT; ++g)
#pragma unroll
      for (int c = 0; c < CPL; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          float v = acc[g][c][e];
          v += __shfl_xor_sync(0xffffffffu, v, 8);
          v += __shfl_xor_sync(0xffffffffu, v, 16);
          acc[g][c][e] = v;
        }
    if ((threadIdx.x & 31) < kLPK) {
#pragma unroll
      for (int g = 0; g < kGT; ++g)
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          const int ch = lane8 + c * kLPK;
          if (ch < CH) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) red[warp][g][ch * VEC + e] = acc[g][c][e];
          }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < ng * kD; i += kDecThreads) {
      const int g = i / kD, d = i - g * kD;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kDecThreads / 32; ++w) v += red[w][g][d];
      const int head = kvh * G + g0 + g;
      const size_t row = (static_cast<size_t>(item) * a.hq + head) * a.max_parts + part;
      a.part_o[row * kD + d] = v;
      if (d == 0) {
        a.part_ml[row * 2] = stat_m[g];
        a.part_ml[row * 2 + 1] = stat_l[g];
      }
    }
  }
}

// Merges the partitions of one (item, head): out = sum_i w_i o_i / sum_i w_i l_i.
template <typename T>
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int4* __restrict__ items, T* __restrict__ out,
                                    int out_stride, int hq, int max_parts, int window) {
  pdl_launch();
  pdl_wait();
  const int item = blockIdx.x, head = blockIdx.y;
  const int4 info = items[item];
  const int tok = info.x, ctx = info.z;
  const int lo = (window > 0 && ctx > window) ? ctx - window : 0;
  const int p_lo = lo / kPart, p_hi = (ctx - 1) / kPart;  // inclusive
  const size_t row0 = (static_cast<size_t>(item) * hq + head) * max_parts;
  float m = -INFINITY;
  for (int p = p_lo; p <= p_hi; ++p) m = fmaxf(m, part_ml[(row0 + p) * 2]);
  for (int d = threadIdx.x; d < kD; d += blockDim.x) {
    float num = 0.f, den = 0.f;
    for (int p = p_lo; p <= p_hi; ++p) {
      const float w = expf(part_ml[(row0 + p) * 2] - m);
      num += w * part_o[(row0 + p) * kD + d];
      den += w * part_ml[(row0 + p) * 2 + 1];
    }
    out[static_cast<size_t>(tok) * out_stride + head * kD + d] = from_float<T>(num / den);
  }
}

// ------------------------------------------------- decode on the tensor cores
// The same work as decode_attn_kernel for bfloat16 and head sizes 64 and 128, with mma.sync.m16n8k16: the G query heads of the group are the 16 rows of the
// MMA (rows past G are zero), the keys its 8-wide side.  K and V go from global memory
// straight into MMA fragments in 16-byte pieces: within a 32-wide block of d (for
// Q.K^T) the MMA's k index is permuted so that a thread's two fragment words are
// adjacent in memory, and for P.V the head dimension is permuted so that the eight
// output tiles of a thread come from one 16-byte piece of a V row.  Four warps take 32
// keys each of the CTA's 128-key partition, issue all their loads at once, and merge
// through shared memory; the CTA that finishes last among an item's partitions merges
// those (in partition order, so the result does not depend on which CTA that is).
#if RL_HEAD_DIM == 64 || RL_HEAD_DIM == 128
#define RL_HAVE_MMA_DECODE 1

__device__ __forceinline__ void mma_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// The rotary position encoding and the cache write of the query tokens inside the tensor-core decode
// kernels, instead of in a kernel of their own before them: what such a kernel needs (cos == nullptr:
// not done in the kernel).  The token's unrotated q, k and v
// lie in one row (q at column 0, k at k_col, v at v_col).  A warp rotates the q rows it loads; the one
// warp that takes the token's own key rotates k, writes k and v into the cache for later steps and
// uses them for this one.
struct DecodeRope {
  const float* cos;        // [max_pos, D / 2]
  const float* sin;
  int max_pos;
  int k_col, v_col;
  bf16* kcache;            // writable views of the caches
  bf16* vcache;
  int* status;             // bit 1 is set for a position outside the tables
};

// Rotates the pairs (x0[e], x1[e]) of eight packed bfloat16 each by the angles whose cosines and sines
// start at c and s: y0 = x0 c - x1 s, y1 = x1 c + x0 s in float32, rounded once.
__device__ __forceinline__ void rope_rotate8(uint4& x0, uint4& x1, const float* c, const float* s) {
  float a[8], b[8], cc[8], ss[8];
  const uint32_t w0[4] = {x0.x, x0.y, x0.z, x0.w}, w1[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    a[2 * i] = __uint_as_float(w0[i] << 16);
    a[2 * i + 1] = __uint_as_float(w0[i] & 0xFFFF0000u);
    b[2 * i] = __uint_as_float(w1[i] << 16);
    b[2 * i + 1] = __uint_as_float(w1[i] & 0xFFFF0000u);
  }
  load16(c, cc);
  load16(c + 4, cc + 4);
  load16(s, ss);
  load16(s + 4, ss + 4);
  uint32_t o0[4], o1[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float y00 = a[2 * i] * cc[2 * i] - b[2 * i] * ss[2 * i];
    const float y01 = a[2 * i + 1] * cc[2 * i + 1] - b[2 * i + 1] * ss[2 * i + 1];
    const float y10 = b[2 * i] * cc[2 * i] + a[2 * i] * ss[2 * i];
    const float y11 = b[2 * i + 1] * cc[2 * i + 1] + a[2 * i + 1] * ss[2 * i + 1];
    o0[i] = pack_bf16(y00, y01);
    o1[i] = pack_bf16(y10, y11);
  }
  x0 = make_uint4(o0[0], o0[1], o0[2], o0[3]);
  x1 = make_uint4(o1[0], o1[1], o1[2], o1[3]);
}

__global__ void __launch_bounds__(128)
decode_attn_mma_kernel(const DecodeArgs<bf16> a, const DecodeRope rope) {
  pdl_launch();
  constexpr int DB = kD / 32;   // 32-wide blocks of d for Q.K^T
  constexpr int DG = kD / 64;   // 64-wide groups of d for P.V
  constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
  // a warp's output row as its threads hold it: column c = dg*64 + j*8 + (t*2+e) holds
  // d = dg*64 + (t*2+e)*8 + j; rows are 8 floats longer than D so that the 8-byte stores of a
  // half-warp fall into distinct banks
  constexpr int LDO = kD + 8;
  __shared__ __align__(16) float sm_o[4][16][LDO];
  __shared__ float sm_m[4][16], sm_l[4][16];
  static_assert(16 * (kMaxMergeParts + 1) <= 4 * 16 * LDO, "the merge weights reuse the output rows");
  float (*sm_w)[kMaxMergeParts + 1] = reinterpret_cast<float (*)[kMaxMergeParts + 1]>(&sm_o[0][0][0]);
  __shared__ int sm_last;

  const int part = blockIdx.x, kvh = blockIdx.y, item = blockIdx.z;
  const int4 info = a.items[item];
  const int tok = info.x, seq = info.y, ctx = info.z;
  const int lo = (a.window > 0 && ctx > a.window) ? ctx - a.window : 0;
  if (max(lo, part * kPart) >= min(ctx, (part + 1) * kPart)) return;
  const int G = a.hq / a.hkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int32_t* bt = a.block_table + static_cast<size_t>(seq) * a.max_blocks;
  const size_t head_stride = static_cast<size_t>(a.page_size) * kD;   // one (page, head) box
  const int k0 = part * kPart + warp * 32;                            // this warp's 32 keys
  const int ps_shift = __ffs(a.page_size) - 1, ps_mask = a.page_size - 1;   // page sizes are powers of two

  // ---- every load of the warp is issued up front: K and V (through the block table), then Q.
  // The keys before the token's own were written by earlier steps, and the step's metadata by a copy
  // before its first kernel: their loads are issued BEFORE the wait on the kernels before this one, so
  // that the trip through the block table and the cache's latency pass while the product before drains.
  // The token's own key (ctx - 1) comes after the wait: with rope.cos set it is not in the cache yet and
  // the threads whose fragments hold it take k and v from the token's row (k rotated: a thread's pieces
  // db and db + DB / 2 are the pairs d, d + D / 2) and write them into the cache for later steps; without,
  // the kernel before has just written it there.
  const bool fused = rope.cos != nullptr;
  const int newest = ctx - 1;
  int pos = ctx - 1;
  if (fused && pos >= rope.max_pos) {
    if (threadIdx.x == 0) atomicOr(rope.status, 2);
    pos = 0;
  }
  const bf16* trow = a.q + static_cast<size_t>(tok) * a.q_stride;
  const float* cs = rope.cos + static_cast<size_t>(pos) * (kD / 2) + t * 8;
  const float* sn = rope.sin + static_cast<size_t>(pos) * (kD / 2) + t * 8;
  uint4 kf[4][DB];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int key = k0 + nt * 8 + g;
    const bool live = key < newest;
    const size_t page = live ? bt[key >> ps_shift] : 0;
    const bf16* kp = a.kcache + (page * a.hkv + kvh) * head_stride + static_cast<size_t>(key & ps_mask) * kD + t * 8;
#pragma unroll
    for (int db = 0; db < DB; ++db)
      kf[nt][db] = live ? *reinterpret_cast<const uint4*>(kp + db * 32) : make_uint4(0, 0, 0, 0);
  }
  // V pieces: for each 16-key step the keys t*2, t*2+1, t*2+8, t*2+9, d = dg*64 + g*8 ..
  uint4 vf[2][4][DG];
#pragma unroll
  for (int ks = 0; ks < 2; ++ks)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int key = k0 + ks * 16 + t * 2 + (q & 1) + (q >> 1) * 8;
      const bool live = key < newest;
      const size_t page = live ? bt[key >> ps_shift] : 0;
      const bf16* vp = a.vcache + (page * a.hkv + kvh) * head_stride + static_cast<size_t>(key & ps_mask) * kD + g * 8;
#pragma unroll
      for (int dg = 0; dg < DG; ++dg)
        vf[ks][q][dg] = live ? *reinterpret_cast<const uint4*>(vp + dg * 64) : make_uint4(0, 0, 0, 0);
    }
  pdl_wait();
  if (newest >= k0 && newest < k0 + 32) {          // this warp holds the token's own key
    const size_t page = bt[newest >> ps_shift];
    const size_t at0 = (page * a.hkv + kvh) * head_stride + static_cast<size_t>(newest & ps_mask) * kD;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      if (k0 + nt * 8 + g != newest) continue;
      const size_t at = at0 + t * 8;
      if (fused) {
        const bf16* kp = trow + rope.k_col + kvh * kD + t * 8;
#pragma unroll
        for (int db = 0; db < DB; ++db) kf[nt][db] = *reinterpret_cast<const uint4*>(kp + db * 32);
#pragma unroll
        for (int db = 0; db < DB / 2; ++db) rope_rotate8(kf[nt][db], kf[nt][db + DB / 2], cs + db * 32, sn + db * 32);
#pragma unroll
        for (int db = 0; db < DB; ++db) *reinterpret_cast<uint4*>(rope.kcache + at + db * 32) = kf[nt][db];
      } else {
#pragma unroll
        for (int db = 0; db < DB; ++db) kf[nt][db] = *reinterpret_cast<const uint4*>(a.kcache + at + db * 32);
      }
    }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (k0 + ks * 16 + t * 2 + (q & 1) + (q >> 1) * 8 != newest) continue;
        const size_t at = at0 + g * 8;
        if (fused) {
          const bf16* vp = trow + rope.v_col + kvh * kD + g * 8;
#pragma unroll
          for (int dg = 0; dg < DG; ++dg) {
            vf[ks][q][dg] = *reinterpret_cast<const uint4*>(vp + dg * 64);
            *reinterpret_cast<uint4*>(rope.vcache + at + dg * 64) = vf[ks][q][dg];
          }
        } else {
#pragma unroll
          for (int dg = 0; dg < DG; ++dg) vf[ks][q][dg] = *reinterpret_cast<const uint4*>(a.vcache + at + dg * 64);
        }
      }
  }
  // Q fragments: rows g and g + 8 of the group, all of d
  uint4 qlo[DB], qhi[DB];
#pragma unroll
  for (int db = 0; db < DB; ++db) {
    const bf16* qp = a.q + static_cast<size_t>(tok) * a.q_stride + static_cast<size_t>(kvh * G) * kD + db * 32 + t * 8;
    qlo[db] = g < G ? *reinterpret_cast<const uint4*>(qp + g * kD) : make_uint4(0, 0, 0, 0);
    qhi[db] = g + 8 < G ? *reinterpret_cast<const uint4*>(qp + (g + 8) * kD) : make_uint4(0, 0, 0, 0);
  }
  if (fused) {
#pragma unroll
    for (int db = 0; db < DB / 2; ++db) {
      rope_rotate8(qlo[db], qlo[db + DB / 2], cs + db * 32, sn + db * 32);
      rope_rotate8(qhi[db], qhi[db + DB / 2], cs + db * 32, sn + db * 32);
    }
  }
  float o[DG][8][4];
#pragma unroll
  for (int dg = 0; dg < DG; ++dg)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[dg][j][e] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;   // rows g and g + 8, log2 units
  const float sc = a.scale * kLog2e;

  if (k0 < ctx && k0 + 32 > lo) {      // the warp has a live key (the same for all its lanes)
    // ---- S = Q K^T
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        mma_16816(s[nt], qlo[db].x, qhi[db].x, qlo[db].y, qhi[db].y, kf[nt][db].x, kf[nt][db].y);
        mma_16816(s[nt], qlo[db].z, qhi[db].z, qlo[db].w, qhi[db].w, kf[nt][db].z, kf[nt][db].w);
      }
    }
    // ---- mask and softmax (rows g and g + 8; the 4 lanes of a row share by shuffles)
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = k0 + nt * 8 + t * 2 + e;
        const bool ok = key < ctx && key >= lo;
        s[nt][e] = ok ? s[nt][e] * sc : -INFINITY;
        s[nt][2 + e] = ok ? s[nt][2 + e] * sc : -INFINITY;
        mx_lo = fmaxf(mx_lo, s[nt][e]);
        mx_hi = fmaxf(mx_hi, s[nt][2 + e]);
      }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    m_lo = mx_lo;                       // finite: the warp has a live key
    m_hi = mx_hi;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        s[nt][e] = exp2f(s[nt][e] - m_lo);
        s[nt][2 + e] = exp2f(s[nt][2 + e] - m_hi);
        l_lo += s[nt][e];
        l_hi += s[nt][2 + e];
      }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    // ---- O = P V
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const uint32_t p0 = pack_bf16(s[2 * ks][0], s[2 * ks][1]), p1 = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
      const uint32_t p2 = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]), p3 = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int dg = 0; dg < DG; ++dg) {
        const uint32_t va[4] = {vf[ks][0][dg].x, vf[ks][0][dg].y, vf[ks][0][dg].z, vf[ks][0][dg].w};
        const uint32_t vb[4] = {vf[ks][1][dg].x, vf[ks][1][dg].y, vf[ks][1][dg].z, vf[ks][1][dg].w};
        const uint32_t vc[4] = {vf[ks][2][dg].x, vf[ks][2][dg].y, vf[ks][2][dg].z, vf[ks][2][dg].w};
        const uint32_t vd[4] = {vf[ks][3][dg].x, vf[ks][3][dg].y, vf[ks][3][dg].z, vf[ks][3][dg].w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
          const uint32_t b0 = __byte_perm(va[j >> 1], vb[j >> 1], sel);   // keys t*2, t*2+1 at d = g*8 + j
          const uint32_t b1 = __byte_perm(vc[j >> 1], vd[j >> 1], sel);   // keys t*2+8, t*2+9
          mma_16816(o[dg][j], p0, p1, p2, p3, b0, b1);
        }
      }
    }
  }
  // ---- the four warps merge: row r of warp w has (m, l) and o[r][:]
  if (t == 0) {
    sm_m[warp][g] = m_lo;
    sm_m[warp][g + 8] = m_hi;
    sm_l[warp][g] = l_lo;
    sm_l[warp][g + 8] = l_hi;
  }
#pragma unroll
  for (int dg = 0; dg < DG; ++dg)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = dg * 64 + j * 8 + t * 2;
      *reinterpret_cast<float2*>(&sm_o[warp][g][c]) = make_float2(o[dg][j][0], o[dg][j][1]);
      *reinterpret_cast<float2*>(&sm_o[warp][g + 8][c]) = make_float2(o[dg][j][2], o[dg][j][3]);
    }
  __syncthreads();
  const int p_lo = lo / kPart, p_hi = (ctx - 1) / kPart;     // the item's live partitions, inclusive
  const bool single = (p_lo == p_hi);
  for (int i = threadIdx.x; i < G * kD; i += 128) {
    const int r = i / kD, c = i - r * kD;                     // c: column as stored
    const int d = (c & ~63) + (c & 7) * 8 + ((c & 63) >> 3);
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, sm_m[w][r]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(sm_m[w][r] - m);     // a warp without live keys has m = -inf: weight 0
      acc += f * sm_o[w][r][c];
      l += f * sm_l[w][r];
    }
    const int head = kvh * G + r;
    if (single) {                                  // the only partition: this is the result
      a.out[static_cast<size_t>(tok) * a.out_stride + head * kD + d] = __float2bfloat16_rn(acc / l);
    } else {
      const size_t row = (static_cast<size_t>(item) * a.hq + head) * a.max_parts + part;
      a.part_o[row * kD + d] = acc;
      if (c == 0) {
        a.part_ml[row * 2] = m * kLn2;             // natural-log units
        a.part_ml[row * 2 + 1] = l;
      }
    }
  }
  if (single) return;
  // ---- the CTA that finishes last among the item's partitions (for this kv head) merges them
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* c = a.counters + item * a.hkv + kvh;
    const int done = atomicAdd(c, 1) + 1;
    sm_last = (done == p_hi - p_lo + 1);
    if (sm_last) *c = 0;                           // ready for the next launch
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();          // (every thread is past its reads of sm_o: the barrier above)
  // weights of the partitions, all heads at once: w[r][p] = exp(m_p - max m) (sm_w), and the
  // denominators; then the weighted sums in partition order, so that the result does not
  // depend on which CTA merges
  const int np = p_hi - p_lo + 1;
  for (int r = warp; r < G; r += 4) {
    const size_t row0 = (static_cast<size_t>(item) * a.hq + kvh * G + r) * a.max_parts + p_lo;
    float m = -INFINITY;
    for (int p = lane; p < np; p += 32) m = fmaxf(m, __ldcg(a.part_ml + (row0 + p) * 2));
    m = warp_max(m);
    float den = 0.f;
    for (int p0 = 0; p0 < np; p0 += 32) {          // lanes in partition order, summed in that order below
      const int p = p0 + lane;
      float w = 0.f, l = 0.f;
      if (p < np) {
        w = expf(__ldcg(a.part_ml + (row0 + p) * 2) - m);
        l = __ldcg(a.part_ml + (row0 + p) * 2 + 1);
        sm_w[r][p] = w;
      }
      // ordered sum over the lanes: lane 0 first
      float wl = w * l;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, wl, o);
        if (lane >= o) wl += up;
      }
      den += __shfl_sync(0xffffffffu, wl, 31);
    }
    if (lane == 0) sm_w[r][kMaxMergeParts] = den;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * kD; i += 128) {
    const int r = i / kD, d = i - r * kD;
    const int head = kvh * G + r;
    const size_t row0 = (static_cast<size_t>(item) * a.hq + head) * a.max_parts + p_lo;
    const float* po = a.part_o + row0 * kD + d;
    float num = 0.f;
    int p = 0;
    for (; p + 4 <= np; p += 4) {                  // four loads in flight, added in order
      const float v0 = __ldcg(po + static_cast<size_t>(p) * kD), v1 = __ldcg(po + static_cast<size_t>(p + 1) * kD);
      const float v2 = __ldcg(po + static_cast<size_t>(p + 2) * kD), v3 = __ldcg(po + static_cast<size_t>(p + 3) * kD);
      num += sm_w[r][p] * v0;
      num += sm_w[r][p + 1] * v1;
      num += sm_w[r][p + 2] * v2;
      num += sm_w[r][p + 3] * v3;
    }
    for (; p < np; ++p) num += sm_w[r][p] * __ldcg(po + static_cast<size_t>(p) * kD);
    a.out[static_cast<size_t>(tok) * a.out_stride + head * kD + d] = __float2bfloat16_rn(num / sm_w[r][kMaxMergeParts]);
  }
}
// 16-byte asynchronous copies into shared memory (zero-filled when pred is false)
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = pred ? 16 : 0;   // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

}  // namespace rl
#include "decode_stream.cuh"
#include "decode_rows.cuh"
namespace rl {
#endif  // head size 64 or 128

// ------------------------------------------------------------------ prefill
constexpr int kBQ = 32, kBK = 32, kPreThreads = 128;

template <typename T>
struct PrefillArgs {
  const T* q;
  int q_stride;
  const T* kcache;
  const T* vcache;
  const int32_t* block_table;
  int max_blocks;
  const int32_t* tile_seq;    // [tiles] sequence index
  const int32_t* tile_tok;    // [tiles] first token of the tile (tokens of a tile are consecutive)
  const int32_t* tile_rows;   // [tiles] rows in use (1..128)
  const int32_t* positions;   // [tokens]
  T* out;
  int out_stride;
  int hq, hkv, page_size, window;
  float scale;
};

// One CTA per (tile of 32 consecutive query tokens of one sequence, query head).
// Thread t owns row r = t / 4 and the columns c = t % 4 + 4 i of every tile.
template <typename T>
__global__ void __launch_bounds__(kPreThreads)
prefill_attn_kernel(const PrefillArgs<T> a) {
  pdl_launch();
  pdl_wait();
  constexpr int VEC = Vec16<T>::N;
  constexpr int CH = kD / VEC;
  constexpr int LDQ = kD + 1;
  extern __shared__ float smem[];
  float* Qs = smem;                  // [32][D+1], pre-scaled
  float* Ks = Qs + kBQ * LDQ;        // [32][D+1]
  float* Vs = Ks + kBK * LDQ;        // [32][D]
  float* Ps = Vs + kBK * kD;         // [32][33]

  // the tile list holds tiles of up to 128 rows; this kernel takes them as four quarters of 32
  const int tile = blockIdx.x >> 2, half_tile = blockIdx.x & 3, head = blockIdx.y;
  const int seq = a.tile_seq[tile], tok0 = a.tile_tok[tile] + half_tile * kBQ;
  const int rows = min(a.tile_rows[tile] - half_tile * kBQ, kBQ);
  if (rows <= 0) return;
  const int kvh = head / (a.hq / a.hkv);
  const int pos0 = a.positions[tok0];
  const int32_t* bt = a.block_table + static_cast<size_t>(seq) * a.max_blocks;
  const int r = threadIdx.x >> 2, cq = threadIdx.x & 3;
  const int my_pos = pos0 + r;
  const int my_lo = (a.window > 0 && my_pos + 1 > a.window) ? my_pos + 1 - a.window : 0;
  const int k_end = pos0 + rows;  // exclusive
  const int k_begin = ((a.window > 0 && pos0 + 1 > a.window) ? pos0 + 1 - a.window : 0) / kBK * kBK;

  for (int i = threadIdx.x; i < kBQ * kD; i += kPreThreads) {
    const int rr = i / kD, d = i - rr * kD;
    Qs[rr * LDQ + d] = rr < rows ? to_float(a.q[static_cast<size_t>(tok0 + rr) * a.q_stride + head * kD + d]) * a.scale
                                 : 0.f;
  }
  float m = -INFINITY, l = 0.f;
  float acc[kD / 4];
#pragma unroll
  for (int i = 0; i < kD / 4; ++i) acc[i] = 0.f;

  for (int k0 = k_begin; k0 < k_end; k0 += kBK) {
    __syncthreads();
    for (int i = threadIdx.x; i < kBK * CH; i += kPreThreads) {
      const int key = i / CH, ch = i - key * CH;
      const int j = k0 + key;
      float kf[VEC], vf[VEC];
      if (j < k_end) {
        const size_t page = bt[j / a.page_size];
        const size_t off = ((page * a.hkv + kvh) * a.page_size + j % a.page_size) * kD + ch * VEC;
        load16(a.kcache + off, kf);
        load16(a.vcache + off, vf);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) kf[e] = vf[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        Ks[key * LDQ + ch * VEC + e] = kf[e];
        Vs[key * kD + ch * VEC + e] = vf[e];
      }
    }
    __syncthreads();
    float s[kBK / 4];
#pragma unroll
    for (int i = 0; i < kBK / 4; ++i) s[i] = 0.f;
    for (int d = 0; d < kD; ++d) {
      const float qv = Qs[r * LDQ + d];
#pragma unroll
      for (int i = 0; i < kBK / 4; ++i) s[i] += qv * Ks[(cq + 4 * i) * LDQ + d];
    }
    float tmax = -INFINITY;
#pragma unroll
    for (int i = 0; i < kBK / 4; ++i) {
      const int kp = k0 + cq + 4 * i;
      const bool ok = (r < rows) && kp <= my_pos && kp >= my_lo;
      s[i] = ok ? s[i] : -INFINITY;
      tmax = fmaxf(tmax, s[i]);
    }
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    const float m_new = fmaxf(m, tmax);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_use);
    float psum = 0.f;
#pragma unroll
    for (int i = 0; i < kBK / 4; ++i) {
      const float p = expf(s[i] - m_use);  // exp(-inf) = 0 for masked keys
      Ps[r * (kBK + 1) + cq + 4 * i] = p;
      psum += p;
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    l = l * alpha + psum;
    m = m_new;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < kD / 4; ++i) acc[i] *= alpha;
    for (int c = 0; c < kBK; ++c) {
      const float p = Ps[r * (kBK + 1) + c];
#pragma unroll
      for (int i = 0; i < kD / 4; ++i) acc[i] += p * Vs[c * kD + cq + 4 * i];
    }
  }
  if (r < rows) {
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < kD / 4; ++i)
      a.out[static_cast<size_t>(tok0 + r) * a.out_stride + head * kD + cq + 4 * i] = from_float<T>(acc[i] * inv);
  }
}

// ------------------------------------------------- prefill on the tensor cores
// bfloat16, head size 64 or 128.  A tile of the launch has up to 128 query rows.  One CTA of four
// warps takes 64 MT rows of it for one query head; each warp takes 16 MT consecutive rows, as MT
// blocks of 16 that share every K and V fragment it reads from shared memory (MT = 1, two CTAs to
// a tile, is the default: measured at head size 64, MT = 2 needs 250 registers and is no faster).
// Keys come in tiles of 64 from the paged cache into a two-stage shared-memory ring with
// cp.async; S = Q K^T and O += P V with mma.sync.m16n8k16, online softmax in float32 in the MMA's
// accumulator layout (masks only in the tiles that need them).  Fragments are read from shared
// memory in 16-byte pieces with the same index permutations as the decode kernel (so no ldmatrix
// and no transposes are needed); a 16-byte-chunk XOR swizzle keeps those reads free of bank
// conflicts.
#ifdef RL_HAVE_MMA_DECODE

constexpr int kMK = 64;                        // keys per tile
#ifndef RL_PRE_MT
#define RL_PRE_MT 1
#endif
#ifndef RL_PRE_MINB
#define RL_PRE_MINB 3
#endif
constexpr int kPreMT = RL_PRE_MT;     // 16-row blocks per warp
constexpr int kPreRows = 64 * kPreMT;          // query rows per CTA
constexpr int kPreTile = 128;                  // query rows per tile of the launch

__global__ void __launch_bounds__(128, RL_PRE_MINB)
prefill_attn_mma_kernel(const PrefillArgs<bf16> a) {
  pdl_launch();
  pdl_wait();
  constexpr int MT = kPreMT;
  constexpr int DB = kD / 32, DG = kD / 64, CPR = kD / 8;   // 16-byte chunks per row
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Ks = reinterpret_cast<bf16*>(smem_raw);            // [2][64][D], chunk-swizzled
  bf16* Vs = Ks + 2 * kMK * kD;                            // [2][64][D], chunk-swizzled

  // longest first: a later part of a sequence attends to more keys
  constexpr int kSplit = kPreTile / kPreRows;              // CTAs per tile
  const int cta = gridDim.x - 1 - blockIdx.x, head = blockIdx.y;
  const int tile = cta / kSplit, row0 = (cta % kSplit) * kPreRows;
  const int rows = min(a.tile_rows[tile] - row0, kPreRows);
  if (rows <= 0) return;
  const int seq = a.tile_seq[tile], tok0 = a.tile_tok[tile] + row0;
  const int kvh = head / (a.hq / a.hkv);
  const int pos0 = a.positions[tok0];
  const int32_t* bt = a.block_table + static_cast<size_t>(seq) * a.max_blocks;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ps_shift = __ffs(a.page_size) - 1, ps_mask = a.page_size - 1;
  const size_t head_stride = static_cast<size_t>(a.page_size) * kD;
  const int k_end = pos0 + rows;                                                      // exclusive
  const int lo0 = (a.window > 0 && pos0 + 1 > a.window) ? pos0 + 1 - a.window : 0;   // first key any row sees
  const int k_begin = lo0 / kMK * kMK;
  const int ntiles = (k_end - k_begin + kMK - 1) / kMK;

  auto load_tile = [&](int it, int stage) {
    const int k0 = k_begin + it * kMK;
    bf16* ks = Ks + stage * kMK * kD;
    bf16* vs = Vs + stage * kMK * kD;
    for (int i = threadIdx.x; i < kMK * CPR; i += 128) {
      const int key = i / CPR, c = i - key * CPR;
      const int j = k0 + key;
      const bool live = j < k_end && j >= lo0;
      const size_t page = live ? bt[j >> ps_shift] : 0;
      const size_t off = (page * a.hkv + kvh) * head_stride + static_cast<size_t>(j & ps_mask) * kD + c * 8;
      const int ck = c ^ ((key & 1) << 2);              // K: rows g, g+1 of a read go to different halves
      const int cv = c ^ (key & 7);                     // V: the eight rows of an ldmatrix tile go to eight chunks
      cp_async16(ks + key * kD + ck * 8, a.kcache + off, live);
      cp_async16(vs + key * kD + cv * 8, a.vcache + off, live);
    }
    cp_async_commit();
  };

  load_tile(0, 0);
  // Q fragments of this warp's 16 MT rows (rows past the tile are zero)
  const int wrow0 = warp * 16 * MT;                    // the warp's first row
  uint4 qlo[MT][DB], qhi[MT][DB];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int r_lo = wrow0 + mt * 16 + g, r_hi = r_lo + 8;
#pragma unroll
    for (int db = 0; db < DB; ++db) {
      const bf16* qp = a.q + static_cast<size_t>(tok0) * a.q_stride + head * kD + db * 32 + t * 8;
      qlo[mt][db] = r_lo < rows ? *reinterpret_cast<const uint4*>(qp + static_cast<size_t>(r_lo) * a.q_stride) : make_uint4(0, 0, 0, 0);
      qhi[mt][db] = r_hi < rows ? *reinterpret_cast<const uint4*>(qp + static_cast<size_t>(r_hi) * a.q_stride) : make_uint4(0, 0, 0, 0);
    }
  }
  float o[MT][DG][8][4];
  float m_lo[MT], m_hi[MT], l_lo[MT], l_hi[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_lo[mt] = m_hi[mt] = -INFINITY;
    l_lo[mt] = l_hi[mt] = 0.f;
#pragma unroll
    for (int dg = 0; dg < DG; ++dg)
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[mt][dg][j][e] = 0.f;
  }
  const float sc = a.scale * kLog2e;

  for (int it = 0; it < ntiles; ++it) {
    const int stage = it & 1;
    if (it + 1 < ntiles) {
      load_tile(it + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int k0 = k_begin + it * kMK;
    const bf16* ks = Ks + stage * kMK * kD;
    const bf16* vs = Vs + stage * kMK * kD;
    // a warp whose rows all lie before this tile's keys has nothing to do in it
    const bool warp_live = (k0 <= pos0 + wrow0 + 16 * MT - 1) && (wrow0 < rows);
    if (warp_live) {
      // ---- S = Q K^T: every K fragment serves the warp's MT blocks of rows
      float s[MT][8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[mt][nt][e] = 0.f;
        const int key = nt * 8 + g;
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          const int c = (db * 4 + t) ^ ((key & 1) << 2);
          const uint4 kf = *reinterpret_cast<const uint4*>(ks + key * kD + c * 8);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_16816(s[mt][nt], qlo[mt][db].x, qhi[mt][db].x, qlo[mt][db].y, qhi[mt][db].y, kf.x, kf.y);
            mma_16816(s[mt][nt], qlo[mt][db].z, qhi[mt][db].z, qlo[mt][db].w, qhi[mt][db].w, kf.z, kf.w);
          }
        }
      }
      // ---- online softmax, block by block; m in units of log2 of the scaled scores
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int b0 = wrow0 + mt * 16;                       // the block's first row
        const int r_lo = b0 + g, r_hi = r_lo + 8;
        // only tiles that reach past the first row's position, before the last row's window or past the
        // tile's rows need the masks
        const bool masked = (k0 + kMK - 1 > pos0 + b0) || (a.window > 0 && k0 < pos0 + b0 + 16 - a.window) || (b0 + 16 > rows);
        if (masked) {
          const int pos_lo = pos0 + r_lo, pos_hi = pos0 + r_hi;
          const int win_lo = (a.window > 0 && pos_lo + 1 > a.window) ? pos_lo + 1 - a.window : 0;
          const int win_hi = (a.window > 0 && pos_hi + 1 > a.window) ? pos_hi + 1 - a.window : 0;
#pragma unroll
          for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int kp = k0 + nt * 8 + t * 2 + e;
              const bool ok_lo = kp <= pos_lo && kp >= win_lo && r_lo < rows;
              const bool ok_hi = kp <= pos_hi && kp >= win_hi && r_hi < rows;
              if (!ok_lo) s[mt][nt][e] = -INFINITY;
              if (!ok_hi) s[mt][nt][2 + e] = -INFINITY;
            }
        }
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            mx_lo = fmaxf(mx_lo, s[mt][nt][e]);
            mx_hi = fmaxf(mx_hi, s[mt][nt][2 + e]);
          }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        // a row without a live key so far keeps m = -inf
        const float mn_lo = fmaxf(m_lo[mt], mx_lo * sc), mn_hi = fmaxf(m_hi[mt], mx_hi * sc);
        const float mu_lo = mn_lo == -INFINITY ? 0.f : mn_lo, mu_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float al_lo = ex2_approx(m_lo[mt] - mu_lo), al_hi = ex2_approx(m_hi[mt] - mu_hi);   // 2^(-inf) = 0
        float ps_lo = 0.f, ps_hi = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          s[mt][nt][0] = ex2_approx(fmaf(s[mt][nt][0], sc, -mu_lo));
          s[mt][nt][1] = ex2_approx(fmaf(s[mt][nt][1], sc, -mu_lo));
          s[mt][nt][2] = ex2_approx(fmaf(s[mt][nt][2], sc, -mu_hi));
          s[mt][nt][3] = ex2_approx(fmaf(s[mt][nt][3], sc, -mu_hi));
          ps_lo += s[mt][nt][0] + s[mt][nt][1];
          ps_hi += s[mt][nt][2] + s[mt][nt][3];
        }
        ps_lo += __shfl_xor_sync(0xffffffffu, ps_lo, 1);
        ps_lo += __shfl_xor_sync(0xffffffffu, ps_lo, 2);
        ps_hi += __shfl_xor_sync(0xffffffffu, ps_hi, 1);
        ps_hi += __shfl_xor_sync(0xffffffffu, ps_hi, 2);
        l_lo[mt] = l_lo[mt] * al_lo + ps_lo;
        l_hi[mt] = l_hi[mt] * al_hi + ps_hi;
        m_lo[mt] = mn_lo;
        m_hi[mt] = mn_hi;
#pragma unroll
        for (int dg = 0; dg < DG; ++dg)
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            o[mt][dg][j][0] *= al_lo;
            o[mt][dg][j][1] *= al_lo;
            o[mt][dg][j][2] *= al_hi;
            o[mt][dg][j][3] *= al_hi;
          }
      }
      // ---- O += P V: every V fragment serves the warp's MT blocks of rows
#pragma unroll
      for (int ks16 = 0; ks16 < 4; ++ks16) {
        // S tiles 2 ks and 2 ks + 1 are the two halves of the 16-key step ks of P V
        uint32_t pk[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          pk[mt][0] = pack_bf16(s[mt][2 * ks16][0], s[mt][2 * ks16][1]);
          pk[mt][1] = pack_bf16(s[mt][2 * ks16][2], s[mt][2 * ks16][3]);
          pk[mt][2] = pack_bf16(s[mt][2 * ks16 + 1][0], s[mt][2 * ks16 + 1][1]);
          pk[mt][3] = pack_bf16(s[mt][2 * ks16 + 1][2], s[mt][2 * ks16 + 1][3]);
        }
        // V fragments by ldmatrix.trans: one instruction brings four 8 x 8 tiles, keys (0..7, 8..15) of the
        // step x two 8-wide blocks of d, as the B fragments of two MMAs; lane l gives the address of row
        // l % 8 of tile l / 8
        const int vrow = ks16 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int jp = 0; jp < kD / 16; ++jp) {                // pairs of 8-wide d blocks
          const int c = (jp * 2 + (lane >> 4)) ^ (vrow & 7);
          uint32_t b0, b1, b2, b3;
          const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(vs + vrow * kD + c * 8));
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_16816(o[mt][jp >> 2][(jp & 3) * 2], pk[mt][0], pk[mt][1], pk[mt][2], pk[mt][3], b0, b1);
            mma_16816(o[mt][jp >> 2][(jp & 3) * 2 + 1], pk[mt][0], pk[mt][1], pk[mt][2], pk[mt][3], b2, b3);
          }
        }
      }
    }
    __syncthreads();   // all warps are done with this stage before it is loaded again
  }
  // ---- normalise and store: through shared memory so that rows go out in 16-byte pieces
  bf16* os = Ks;       // [64 MT][D], free now (two stages of [64][D])
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int r_lo = wrow0 + mt * 16 + g, r_hi = r_lo + 8;
    const float inv_lo = l_lo[mt] > 0.f ? 1.f / l_lo[mt] : 0.f, inv_hi = l_hi[mt] > 0.f ? 1.f / l_hi[mt] : 0.f;
#pragma unroll
    for (int dg = 0; dg < DG; ++dg)
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int d = dg * 64 + j * 8 + t * 2 + e;
          os[r_lo * kD + d] = __float2bfloat16_rn(o[mt][dg][j][e] * inv_lo);
          os[r_hi * kD + d] = __float2bfloat16_rn(o[mt][dg][j][2 + e] * inv_hi);
        }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kPreRows * CPR; i += 128) {
    const int r = i / CPR, c = i - r * CPR;
    if (r < rows)
      *reinterpret_cast<uint4*>(a.out + static_cast<size_t>(tok0 + r) * a.out_stride + head * kD + c * 8) =
          *reinterpret_cast<const uint4*>(os + r * kD + c * 8);
  }
}
#endif  // tensor-core prefill

}  // namespace rl
#if RL_HEAD_DIM == 64 || RL_HEAD_DIM == 128
#include "prefill_tc.cuh"
#define RL_HAVE_TC_PREFILL 1
#endif
namespace rl {

}  // namespace rl

using namespace rl;

namespace {

constexpr int kMaxDevices = 64;   // per-device launch set-up is remembered for this many devices

// The rotary tables and columns for a launch that also rotates q and k and writes the token's k and v
// into the cache (streaming kernel only).
struct DecodeRopeHost {
  const float* cos;
  const float* sin;
  int max_pos, k_col, v_col;
  int* status;
};

// Whether a bfloat16 launch goes to the streaming kernel (see rl_attn_decode for impl).
inline bool decode_streams(const void* q, int q_stride, const void* kc, const void* vc, const void* part_o,
                           const void* counters, const void* out, int out_stride, int max_parts, int nitems, int hq,
                           int hkv, int page_size, int impl) {
#ifdef RL_HAVE_MMA_DECODE
  // page sizes that divide a partition and 16-byte aligned rows
  const bool aligned = q_stride % 8 == 0 && out_stride % 8 == 0 &&
                       ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) |
                         reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc) |
                         reinterpret_cast<uintptr_t>(part_o)) & 15) == 0;
  // (with few units the one-partition kernel, four warps to a partition, has the shorter critical path)
  const bool many = static_cast<long long>(nitems) * hkv * max_parts >= static_cast<long long>(kStreamMinUnits);
  return (impl == 3 || (impl == 0 && (many || max_parts > kMaxMergeParts))) && hq / hkv <= 16 && page_size >= 16 &&
         kPart % page_size == 0 && counters != nullptr && nitems <= kStreamMaxItems && aligned;   // (any number of partitions)
#else
  return false;
#endif
}

// Whether a bfloat16 launch that does not stream goes to the one-partition tensor-core kernel.
inline bool decode_one_partition(const void* counters, int max_parts, int hq, int hkv, int page_size, int impl) {
#ifdef RL_HAVE_MMA_DECODE
  // (the kernel finds a key's page with a shift and a mask: pages of a power of two keys)
  return impl != 1 && impl != 3 && hq / hkv <= 16 && page_size >= 16 && (page_size & (page_size - 1)) == 0 &&
         counters != nullptr && max_parts <= kMaxMergeParts;
#else
  return false;
#endif
}

#ifdef RL_HAVE_MMA_DECODE
// Rows kernel (decode_rows.cuh): how many CTAs the cluster of a row gets in a launch of `rows` rows on the
// current device: the largest size up to 8 of which `rows` clusters are resident at once; 1 if not even
// that many clusters of one CTA are (*resident then says how many: each takes several rows); 0 if the kernel
// cannot run at all.  (The occupancy calculator is asked once per device.)
static int rows_cluster_size(int rows, cudaError_t* err, int* resident = nullptr) {
  static int rows_clusters[kMaxDevices][kRowsMaxCluster + 1];
  static bool rows_ready[kMaxDevices] = {};
  static std::mutex rows_lock;
  *err = cudaSuccess;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    *err = e;
    return 0;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    *err = cudaErrorInvalidDevice;
    return 0;
  }
  {
    std::lock_guard<std::mutex> guard(rows_lock);
    if (!rows_ready[dev]) {
      e = cudaFuncSetAttribute(decode_attn_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kRowsSmem));
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(decode_attn_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kRowsSmem));
      if (e != cudaSuccess) {
        *err = e;
        return 0;
      }
      for (int c = 1; c <= kRowsMaxCluster; ++c) {
        cudaLaunchConfig_t qc = {};
        qc.gridDim = dim3(c);
        qc.blockDim = dim3(kRowsThreads);
        qc.dynamicSmemBytes = kRowsSmem;
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = c;
        qa[0].val.clusterDim.y = 1;
        qa[0].val.clusterDim.z = 1;
        qc.attrs = qa;
        qc.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, decode_attn_rows_kernel<false>, &qc) != cudaSuccess) {
          cudaGetLastError();
          n = 0;
        }
        rows_clusters[dev][c] = n;
      }
      rows_ready[dev] = true;
    }
  }
  int cx = kRowsMaxCluster;
  while (cx > 1 && rows_clusters[dev][cx] < rows) --cx;
  if (resident != nullptr) *resident = rows_clusters[dev][cx];
  return rows_clusters[dev][cx] >= 1 ? cx : 0;
}

#endif

template <typename T>
int launch_decode(const void* q, int q_stride, const void* kc, const void* vc, const int32_t* bt,
                  int max_blocks, const int32_t* items, float* part_o, float* part_ml, int max_parts,
                  int* counters, void* out, int out_stride, int nitems, int hq, int hkv, int page_size,
                  int window, float scale, int impl, const DecodeRopeHost* rope, cudaStream_t stream) {
  DecodeArgs<T> a;
  a.q = static_cast<const T*>(q);
  a.q_stride = q_stride;
  a.kcache = static_cast<const T*>(kc);
  a.vcache = static_cast<const T*>(vc);
  a.block_table = bt;
  a.max_blocks = max_blocks;
  a.items = reinterpret_cast<const int4*>(items);
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.max_parts = max_parts;
  a.counters = counters;
  a.out = static_cast<T*>(out);
  a.out_stride = out_stride;
  a.hq = hq;
  a.hkv = hkv;
  a.page_size = page_size;
  a.window = window;
  a.scale = scale;
  dim3 grid(max_parts, hkv, nitems);
#ifdef RL_HAVE_MMA_DECODE
  if constexpr (sizeof(T) == 2) {
    if (impl == 4) {
      // one cluster per (item, kv head): the largest cluster size of which that many clusters are resident
      // (groups of up to 16 heads, pages that divide a partition, 16-byte aligned rows)
      const bool aligned = q_stride % 8 == 0 && out_stride % 8 == 0 &&
                           ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) |
                             reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc)) & 15) == 0;
      if (!(hq / hkv <= 16 && page_size >= 16 && kPart % page_size == 0 && aligned && nitems > 0))
        return static_cast<int>(cudaErrorInvalidValue);
      cudaError_t e = cudaSuccess;
      const int rows = nitems * hkv;
      int resident = 0;
      const int cx = rows_cluster_size(rows, &e, &resident);
      if (e != cudaSuccess) return static_cast<int>(e);
      if (cx < 1) return static_cast<int>(cudaErrorNotSupported);
      const int clusters = rows < resident ? rows : resident;
      // more rows than clusters: the warps of a CTA in as few groups (a divisor of their number) as give
      // every row a group at once, else one warp to a row and several rows in turn
      int groups = 1;
      if (rows > resident) {
        groups = kRowsWarps;
        for (int d = 2; d < kRowsWarps; ++d)
          if (kRowsWarps % d == 0 && static_cast<long long>(resident) * d >= rows) {
            groups = d;
            break;
          }
      }
      DecodeRope sr = {};
      if (rope != nullptr && rope->cos != nullptr) {
        sr.cos = rope->cos;
        sr.sin = rope->sin;
        sr.max_pos = rope->max_pos;
        sr.k_col = rope->k_col;
        sr.v_col = rope->v_col;
        sr.kcache = const_cast<bf16*>(a.kcache);
        sr.vcache = const_cast<bf16*>(a.vcache);
        sr.status = rope->status;
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(clusters * cx);
      cfg.blockDim = dim3(kRowsThreads);
      cfg.dynamicSmemBytes = kRowsSmem;
      cfg.stream = stream;
      cudaLaunchAttribute at[2];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = cx;
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      at[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = at;
      cfg.numAttrs = pdl_enabled() ? 2 : 1;
      if (hq / hkv > 8)
        return static_cast<int>(cudaLaunchKernelEx(&cfg, decode_attn_rows_kernel<true>, a, rows, groups, sr));
      return static_cast<int>(cudaLaunchKernelEx(&cfg, decode_attn_rows_kernel<false>, a, rows, groups, sr));
    }
    if (decode_streams(q, q_stride, kc, vc, part_o, counters, out, out_stride, max_parts, nitems, hq, hkv, page_size,
                       impl)) {
      // (a kernel's shared-memory limit and the SM count belong to a device: looked up once on each)
      static int sms_of[kMaxDevices];
      int dev = 0;
      cudaError_t e = cudaGetDevice(&dev);
      if (e != cudaSuccess) return static_cast<int>(e);
      if (dev < 0 || dev >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
      if (sms_of[dev] == 0) {
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess)
          e = cudaFuncSetAttribute(decode_attn_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kStreamSmem));
        if (e == cudaSuccess)
          e = cudaFuncSetAttribute(decode_attn_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kStreamSmem));
        if (e != cudaSuccess) return static_cast<int>(e);
        sms_of[dev] = n > 0 ? n : 1;
      }
      const int sms = sms_of[dev];
      // no more CTAs than the launch can have units
      const long long most = static_cast<long long>(nitems) * hkv * max_parts;
      const int ctas = static_cast<int>(most < sms ? most : sms);
      DecodeRope sr = {};
      if (rope != nullptr && rope->cos != nullptr) {
        sr.cos = rope->cos;
        sr.sin = rope->sin;
        sr.max_pos = rope->max_pos;
        sr.k_col = rope->k_col;
        sr.v_col = rope->v_col;
        sr.kcache = const_cast<bf16*>(a.kcache);
        sr.vcache = const_cast<bf16*>(a.vcache);
        sr.status = rope->status;
      }
      if (hq / hkv > 8)
        launch_kernel(decode_attn_stream_kernel<true>, dim3(ctas), dim3(kStreamThreads), kStreamSmem, stream, a, nitems, sr);
      else
        launch_kernel(decode_attn_stream_kernel<false>, dim3(ctas), dim3(kStreamThreads), kStreamSmem, stream, a, nitems, sr);
      return static_cast<int>(cudaGetLastError());
    }
    if (impl == 3) return static_cast<int>(cudaErrorInvalidValue);
    // tensor-core kernel: groups of up to 16 heads, pages that hold whole 16-key steps
    if (decode_one_partition(counters, max_parts, hq, hkv, page_size, impl)) {
      DecodeRope sr = {};
      if (rope != nullptr && rope->cos != nullptr) {
        if (q_stride % 8 != 0 || ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc)) & 15) != 0)
          return static_cast<int>(cudaErrorInvalidValue);
        sr.cos = rope->cos;
        sr.sin = rope->sin;
        sr.max_pos = rope->max_pos;
        sr.k_col = rope->k_col;
        sr.v_col = rope->v_col;
        sr.kcache = const_cast<bf16*>(a.kcache);
        sr.vcache = const_cast<bf16*>(a.vcache);
        sr.status = rope->status;
      }
      launch_kernel(decode_attn_mma_kernel, dim3(grid), dim3(128), 0, stream, a, sr);
      return static_cast<int>(cudaGetLastError());
    }
  }
#endif
  if (impl == 2 || impl == 3) return static_cast<int>(cudaErrorInvalidValue);
  if (rope != nullptr && rope->cos != nullptr) return static_cast<int>(cudaErrorInvalidValue);   // only the tensor-core kernels rotate
  launch_kernel(decode_attn_kernel<T>, dim3(grid), dim3(kDecThreads), 0, stream, a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  int th = 32;
  while (th < kD) th <<= 1;
  launch_kernel(decode_merge_kernel<T>, dim3(dim3(nitems, hq)), dim3(th), 0, stream, 
      part_o, part_ml, a.items, static_cast<T*>(out), out_stride, hq, max_parts, window);
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
int launch_prefill(const void* q, int q_stride, const void* kc, const void* vc, const int32_t* bt,
                   int max_blocks, const int32_t* tile_seq, const int32_t* tile_tok,
                   const int32_t* tile_rows, const int32_t* positions, void* out, int out_stride,
                   int tiles, int hq, int hkv, int page_size, int window, float scale, int impl, int* status,
                   cudaStream_t stream) {
  PrefillArgs<T> a;
  a.q = static_cast<const T*>(q);
  a.q_stride = q_stride;
  a.kcache = static_cast<const T*>(kc);
  a.vcache = static_cast<const T*>(vc);
  a.block_table = bt;
  a.max_blocks = max_blocks;
  a.tile_seq = tile_seq;
  a.tile_tok = tile_tok;
  a.tile_rows = tile_rows;
  a.positions = positions;
  a.out = static_cast<T*>(out);
  a.out_stride = out_stride;
  a.hq = hq;
  a.hkv = hkv;
  a.page_size = page_size;
  a.window = window;
  a.scale = scale;
#ifdef RL_HAVE_TC_PREFILL
  if constexpr (sizeof(T) == 2) {
    const bool aligned = q_stride % 8 == 0 && out_stride % 8 == 0 &&
                         ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) |
                           reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc)) & 15) == 0;
    // the tcgen05 kernel: power-of-two pages, 16-byte aligned rows, a status word for its bounded waits
    if ((impl == 0 || impl == 3) && status != nullptr && aligned && (page_size & (page_size - 1)) == 0) {
      static int tsms_of[kMaxDevices];
      int dev = 0;
      cudaError_t e = cudaGetDevice(&dev);
      if (e != cudaSuccess) return static_cast<int>(e);
      if (dev < 0 || dev >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
      if (tsms_of[dev] == 0) {
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess)
          e = cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kPrefillTcSmem));
        if (e != cudaSuccess) return static_cast<int>(e);
        tsms_of[dev] = n > 0 ? n : 1;
      }
      const int tsms = tsms_of[dev];
      const long long items = static_cast<long long>(tiles) * hkv * ((hq / hkv + 1) / 2);   // (tile, kv head, pair of heads)
      const int ctas = static_cast<int>(items < tsms ? items : tsms);      // persistent: one CTA per SM
      launch_kernel(prefill_attn_tc_kernel, dim3(ctas), dim3(kTcThreads), kPrefillTcSmem, stream, a, tiles, status);
      return static_cast<int>(cudaGetLastError());
    }
  }
#endif
  if (impl == 3) return static_cast<int>(cudaErrorInvalidValue);
#ifdef RL_HAVE_MMA_DECODE
  if constexpr (sizeof(T) == 2) {
    if (impl != 1 && page_size >= 16 && (page_size & (page_size - 1)) == 0 && out_stride % 8 == 0 && q_stride % 8 == 0) {
      const size_t msmem = static_cast<size_t>(4) * kMK * kD * sizeof(bf16);
      static bool mattr[kMaxDevices];
      int dev = 0;
      cudaError_t e = cudaGetDevice(&dev);
      if (e != cudaSuccess) return static_cast<int>(e);
      if (dev < 0 || dev >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
      if (!mattr[dev]) {
        e = cudaFuncSetAttribute(prefill_attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(msmem));
        if (e != cudaSuccess) return static_cast<int>(e);
        mattr[dev] = true;
      }
      launch_kernel(prefill_attn_mma_kernel, dim3(dim3(tiles * (kPreTile / kPreRows), hq)), dim3(128), msmem, stream, a);
      return static_cast<int>(cudaGetLastError());
    }
  }
#endif
  if (impl == 2) return static_cast<int>(cudaErrorInvalidValue);
  const size_t smem = sizeof(float) * (kBQ * (kD + 1) + kBK * (kD + 1) + kBK * kD + kBQ * (kBK + 1));
  static bool attr_set[kMaxDevices];  // per instantiation and device: the limit belongs to the function on a device
  {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
    if (!attr_set[dev]) {
      e = cudaFuncSetAttribute(prefill_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      attr_set[dev] = true;
    }
  }
  launch_kernel(prefill_attn_kernel<T>, dim3(dim3(tiles * 4, hq)), dim3(kPreThreads), smem, stream, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

int rl_attn_head_dim() { return kD; }
int rl_attn_partition() { return kPart; }
int rl_attn_tile_rows() { return 4 * kBQ; }

// dtype: 0 = float32, 1 = bfloat16 (type of q, the cache and out).
// items: int32 [nitems, 4] = (token index of the query, sequence index, context length, 0).
// max_parts = ceil(longest context this launch may see / 128); the grid has that many
// partitions per item and CTAs past an item's context return at once.
// counters: int32 [nitems * hkv], zero before the first launch (the kernel leaves them zero).
// impl: 0 = the best kernel that applies: the streaming tensor-core kernel (bfloat16, head size
// 64 or 128, at most 16 heads per group, pages of 16 to 128 keys, at most 512 items), else the
// one-partition-per-CTA tensor-core kernel, else the CUDA-core kernel; 1 = the CUDA-core kernel;
// 2 = the one-partition-per-CTA tensor-core kernel or an error; 3 = the streaming kernel or an error;
// 4 = one cluster per (item, kv head) (decode_rows.cuh: for few rows of similar length) or an error: when the
// launch has more rows than clusters can be resident.
int rl_attn_decode(int dtype, const void* q, int q_stride, const void* kc, const void* vc,
                   const int32_t* bt, int max_blocks, const int32_t* items, float* part_o,
                   float* part_ml, int max_parts, int* counters, void* out, int out_stride, int nitems,
                   int hq, int hkv, int page_size, int window, float scale, int impl, cudaStream_t stream) {
  if (nitems <= 0) return 0;
  if (dtype == 0)
    return launch_decode<float>(q, q_stride, kc, vc, bt, max_blocks, items, part_o, part_ml, max_parts,
                                counters, out, out_stride, nitems, hq, hkv, page_size, window, scale, impl,
                                nullptr, stream);
  return launch_decode<bf16>(q, q_stride, kc, vc, bt, max_blocks, items, part_o, part_ml, max_parts,
                             counters, out, out_stride, nitems, hq, hkv, page_size, window, scale, impl,
                             nullptr, stream);
}

// The cluster size that rl_attn_decode with impl 4 gives a row in a launch of nitems items (0: it refuses the
// launch: a head size without tensor-core decode kernels); *resident: how many such clusters run at once
// (fewer than nitems * hkv: a cluster takes several rows, one after another).
int rl_attn_decode_rows_cluster(int nitems, int hkv, int* resident) {
#ifdef RL_HAVE_MMA_DECODE
  cudaError_t e = cudaSuccess;
  int r = 0;
  const int cx = rows_cluster_size(nitems * hkv, &e, &r);
  if (resident != nullptr) *resident = r;
  return e == cudaSuccess ? cx : 0;
#else
  return 0;
#endif
}

// Warps of a CTA of that kernel (a row's keys are cut into cluster size x this many runs).
int rl_attn_decode_rows_warps() {
#ifdef RL_HAVE_MMA_DECODE
  return kRowsWarps;
#else
  return 0;
#endif
}

// 1 if rl_attn_decode with these arguments runs the streaming kernel (bfloat16 only), else 0.
int rl_attn_decode_streams(int dtype, const void* q, int q_stride, const void* kc, const void* vc, const void* part_o,
                           const void* counters, const void* out, int out_stride, int max_parts, int nitems, int hq,
                           int hkv, int page_size, int impl) {
  if (dtype == 0 || nitems <= 0) return 0;
  return decode_streams(q, q_stride, kc, vc, part_o, counters, out, out_stride, max_parts, nitems, hq, hkv, page_size,
                        impl) ? 1 : 0;
}

// Whether rl_attn_decode_rope takes a launch with these arguments (one of the two tensor-core kernels
// does, and rows are 16-byte aligned).
int rl_attn_decode_rope_ok(const void* q, int q_stride, const void* kc, const void* vc, const void* part_o,
                           const void* counters, const void* out, int out_stride, int max_parts, int nitems, int hq,
                           int hkv, int page_size, int k_col, int v_col) {
  if (nitems <= 0 || k_col % 8 != 0 || v_col % 8 != 0) return 0;
  if (decode_streams(q, q_stride, kc, vc, part_o, counters, out, out_stride, max_parts, nitems, hq, hkv, page_size, 0))
    return 1;
  const bool aligned = q_stride % 8 == 0 && ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kc) |
                                              reinterpret_cast<uintptr_t>(vc)) & 15) == 0;
  return decode_one_partition(counters, max_parts, hq, hkv, page_size, 0) && aligned ? 1 : 0;
}

// rl_attn_decode for launches that a tensor-core kernel takes (rl_attn_decode_rope_ok), with the rotary
// position encoding and the cache write of the query tokens done in the kernel: q points at rows of
// UNROTATED [q | ... k at k_col ... | ... v at v_col ...]; cos / sin are float [max_pos, D / 2] tables; a
// token's position is its context length - 1; its rotated k and its v are written into kc and vc at that
// position (through the block table).  status: device int, bit 1 is set for a position outside the
// tables.  impl: 0 or 4, as for rl_attn_decode.  Returns cudaErrorInvalidValue where no tensor-core kernel
// applies.
int rl_attn_decode_rope(const void* q, int q_stride, void* kc, void* vc, const int32_t* bt, int max_blocks,
                        const int32_t* items, float* part_o, float* part_ml, int max_parts, int* counters, void* out,
                        int out_stride, int nitems, int hq, int hkv, int page_size, int window, float scale,
                        const float* cos_t, const float* sin_t, int max_pos, int k_col, int v_col, int* status,
                        int impl, cudaStream_t stream) {
  if (nitems <= 0) return 0;
  if (cos_t == nullptr || sin_t == nullptr || status == nullptr || k_col % 8 != 0 || v_col % 8 != 0 ||
      (impl != 0 && impl != 4))
    return static_cast<int>(cudaErrorInvalidValue);
  DecodeRopeHost r = {cos_t, sin_t, max_pos, k_col, v_col, status};
  return launch_decode<bf16>(q, q_stride, kc, vc, bt, max_blocks, items, part_o, part_ml, max_parts, counters, out,
                             out_stride, nitems, hq, hkv, page_size, window, scale, impl, &r, stream);
}

int rl_attn_prefill(int dtype, const void* q, int q_stride, const void* kc, const void* vc,
                    const int32_t* bt, int max_blocks, const int32_t* tile_seq,
                    const int32_t* tile_tok, const int32_t* tile_rows, const int32_t* positions,
                    void* out, int out_stride, int tiles, int hq, int hkv, int page_size, int window,
                    float scale, int impl, int* status, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (dtype == 0)
    return launch_prefill<float>(q, q_stride, kc, vc, bt, max_blocks, tile_seq, tile_tok, tile_rows,
                                 positions, out, out_stride, tiles, hq, hkv, page_size, window, scale, impl,
                                 status, stream);
  return launch_prefill<bf16>(q, q_stride, kc, vc, bt, max_blocks, tile_seq, tile_tok, tile_rows,
                              positions, out, out_stride, tiles, hq, hkv, page_size, window, scale, impl,
                              status, stream);
}

}  // extern "C"

// ------------------------------------------------------------------------------------
// The entry point that allocates nothing (declared and explained in attention_noalloc.h).
// ------------------------------------------------------------------------------------
#include <cstdio>
#include <mutex>

#include "attention_noalloc.h"

namespace {

// Scratch of rl_attn_decode_noalloc.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a pointer to pass to a kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[RL_ATTN_NOALLOC_SCRATCH_BYTES];

unsigned char* g_noalloc_ptr[kMaxDevices];   // device address of the array, per device; null until looked up
std::mutex g_noalloc_lock;                   // first calls from several threads look the address up one at a time

}  // namespace

extern "C" int rl_attn_decode_noalloc(int dtype, const void* q, int q_stride, const void* kcache,
                                      const void* vcache, const int32_t* block_table, int max_blocks,
                                      const int32_t* items, int max_parts, void* out, int out_stride,
                                      int nitems, int hq, int hkv, int page_size, int window, float scale,
                                      cudaStream_t stream, char* errbuf, int errbuf_len) {
  if (errbuf && errbuf_len > 0) errbuf[0] = 0;
  if (nitems <= 0) return 0;
  const size_t counter_bytes = (static_cast<size_t>(nitems) * hkv * sizeof(int) + 255) / 256 * 256;
  const size_t rows = static_cast<size_t>(nitems) * hq * max_parts;
  const size_t ml_bytes = (rows * 2 * sizeof(float) + 255) / 256 * 256;
  const size_t need = counter_bytes + ml_bytes + rows * kD * sizeof(float);
  if (need > RL_ATTN_NOALLOC_SCRATCH_BYTES) {
    if (errbuf && errbuf_len > 0) {
      std::snprintf(errbuf, static_cast<size_t>(errbuf_len),
                    "rl_attn_decode_noalloc: %d items x %d heads x %d partitions x head size %d need %zu bytes "
                    "of scratch, the built-in array holds %u; use rl_attn_decode with buffers of your own",
                    nitems, hq, max_parts, kD, need, RL_ATTN_NOALLOC_SCRATCH_BYTES);
    }
    return RL_ATTN_NOALLOC_TOO_LARGE;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> hold(g_noalloc_lock);
    if (g_noalloc_ptr[dev] == nullptr) {
      // set-up, once per device, with that device current: the array's address on this device
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess) return static_cast<int>(e);
      g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
    }
    base = g_noalloc_ptr[dev];
  }
  int* counters = reinterpret_cast<int*>(base);
  float* part_ml = reinterpret_cast<float*>(base + counter_bytes);
  float* part_o = reinterpret_cast<float*>(base + counter_bytes + ml_bytes);
  // the counters must start at zero whatever an earlier call left behind
  e = cudaMemsetAsync(counters, 0, counter_bytes, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dtype == 0)
    return launch_decode<float>(q, q_stride, kcache, vcache, block_table, max_blocks, items, part_o, part_ml,
                                max_parts, counters, out, out_stride, nitems, hq, hkv, page_size, window, scale,
                                0, nullptr, stream);
  return launch_decode<bf16>(q, q_stride, kcache, vcache, block_table, max_blocks, items, part_o, part_ml,
                             max_parts, counters, out, out_stride, nitems, hq, hkv, page_size, window, scale, 0,
                             nullptr, stream);
}
