// Attention over the paged cache, compiled for one head size (-DRL_HEAD_DIM=D,
// D a multiple of 16 up to 256) and both element types (float, bfloat16).
//
//   rl_attn_decode   one query token per item; the keys are cut into absolute
//                    256-key partitions, one CTA per (partition, kv head, item)
//                    computes all G query heads of the group from one read of K
//                    and V and leaves (max, sum, unnormalised output); a second
//                    kernel merges the partitions with w_i = exp(m_i - m).
//                    Restates src/cuda/kernels/attention.cu:69-209.
//   rl_attn_prefill  32-query x 32-key tiles with an online softmax; the keys of a
//                    tile come from the cache, so a prompt portion attends to what
//                    earlier portions left there (attention.cu:217-359).
//
// Scores, the softmax and the P.V sums are float whatever the element type.  A
// window w > 0 keeps only keys with pos - w < key <= pos.  The cache of a layer is
// K [pages, Hkv, page_size, D] and V alike; a token's page comes from its
// sequence's row of the block table.
#include "common.cuh"

#ifndef RL_HEAD_DIM
#error "compile with -DRL_HEAD_DIM=<head size>"
#endif

namespace rl {

constexpr int kD = RL_HEAD_DIM;
static_assert(kD % 16 == 0 && kD >= 16 && kD <= 256, "head size must be a multiple of 16, at most 256");
constexpr int kPart = 256;      // keys per decode partition (absolute boundaries)
constexpr int kDecThreads = 128;
constexpr int kLPK = 8;         // lanes that share one key
constexpr int kKeysPerIter = kDecThreads / kLPK;  // 16
constexpr int kGT = 4;          // query heads per pass over the keys

template <typename T>
struct DecodeArgs {
  const T* q;            // [tokens, q_stride], head h at column h * D
  int q_stride;
  const T* kcache;
  const T* vcache;
  const int32_t* block_table;  // [seqs, max_blocks]
  int max_blocks;
  const int32_t* item_tok;     // [items] token index of the query
  const int32_t* seq_of_token; // [tokens]
  const int32_t* positions;    // [tokens]
  float* part_o;               // [items, Hq, max_parts, D]
  float* part_ml;              // [items, Hq, max_parts, 2]
  int max_parts;
  int hq, hkv, page_size, window;
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(kDecThreads)
decode_attn_kernel(const DecodeArgs<T> a) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int CH = kD / VEC;                     // 16-byte chunks per key
  constexpr int CPL = (CH + kLPK - 1) / kLPK;      // chunks per lane
  __shared__ float qs[kGT][kD];
  __shared__ float sc[kGT][kPart];
  __shared__ float red[kDecThreads / 32][kGT][kD];
  __shared__ float stat_m[kGT], stat_l[kGT];

  const int part = blockIdx.x, kvh = blockIdx.y, item = blockIdx.z;
  const int tok = a.item_tok[item];
  const int seq = a.seq_of_token[tok];
  const int ctx = a.positions[tok] + 1;
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
                                    const int32_t* __restrict__ item_tok,
                                    const int32_t* __restrict__ positions, T* __restrict__ out,
                                    int out_stride, int hq, int max_parts, int window) {
  const int item = blockIdx.x, head = blockIdx.y;
  const int tok = item_tok[item];
  const int ctx = positions[tok] + 1;
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
  const int32_t* tile_rows;   // [tiles] rows in use (1..32)
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
  constexpr int VEC = Vec16<T>::N;
  constexpr int CH = kD / VEC;
  constexpr int LDQ = kD + 1;
  extern __shared__ float smem[];
  float* Qs = smem;                  // [32][D+1], pre-scaled
  float* Ks = Qs + kBQ * LDQ;        // [32][D+1]
  float* Vs = Ks + kBK * LDQ;        // [32][D]
  float* Ps = Vs + kBK * kD;         // [32][33]

  const int tile = blockIdx.x, head = blockIdx.y;
  const int seq = a.tile_seq[tile], tok0 = a.tile_tok[tile], rows = a.tile_rows[tile];
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

}  // namespace rl

using namespace rl;

namespace {

template <typename T>
int launch_decode(const void* q, int q_stride, const void* kc, const void* vc, const int32_t* bt,
                  int max_blocks, const int32_t* item_tok, const int32_t* seq_of_token,
                  const int32_t* positions, float* part_o, float* part_ml, int max_parts, void* out,
                  int out_stride, int items, int hq, int hkv, int page_size, int window, float scale,
                  cudaStream_t stream) {
  DecodeArgs<T> a;
  a.q = static_cast<const T*>(q);
  a.q_stride = q_stride;
  a.kcache = static_cast<const T*>(kc);
  a.vcache = static_cast<const T*>(vc);
  a.block_table = bt;
  a.max_blocks = max_blocks;
  a.item_tok = item_tok;
  a.seq_of_token = seq_of_token;
  a.positions = positions;
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.max_parts = max_parts;
  a.hq = hq;
  a.hkv = hkv;
  a.page_size = page_size;
  a.window = window;
  a.scale = scale;
  dim3 grid(max_parts, hkv, items);
  decode_attn_kernel<T><<<grid, kDecThreads, 0, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  int th = 32;
  while (th < kD) th <<= 1;
  decode_merge_kernel<T><<<dim3(items, hq), th, 0, stream>>>(
      part_o, part_ml, item_tok, positions, static_cast<T*>(out), out_stride, hq, max_parts, window);
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
int launch_prefill(const void* q, int q_stride, const void* kc, const void* vc, const int32_t* bt,
                   int max_blocks, const int32_t* tile_seq, const int32_t* tile_tok,
                   const int32_t* tile_rows, const int32_t* positions, void* out, int out_stride,
                   int tiles, int hq, int hkv, int page_size, int window, float scale,
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
  const size_t smem = sizeof(float) * (kBQ * (kD + 1) + kBK * (kD + 1) + kBK * kD + kBQ * (kBK + 1));
  static bool attr_set = false;  // per instantiation; the attribute belongs to the device function
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attn_kernel<T>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  prefill_attn_kernel<T><<<dim3(tiles, hq), kPreThreads, smem, stream>>>(a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

int rl_attn_head_dim() { return kD; }
int rl_attn_partition() { return kPart; }
int rl_attn_tile_rows() { return kBQ; }

// dtype: 0 = float32, 1 = bfloat16 (type of q, the cache and out).
// max_parts = ceil(longest context this launch may see / 256); the grid has that many
// partitions per item and CTAs past an item's context return at once.
int rl_attn_decode(int dtype, const void* q, int q_stride, const void* kc, const void* vc,
                   const int32_t* bt, int max_blocks, const int32_t* item_tok,
                   const int32_t* seq_of_token, const int32_t* positions, float* part_o,
                   float* part_ml, int max_parts, void* out, int out_stride, int items, int hq,
                   int hkv, int page_size, int window, float scale, cudaStream_t stream) {
  if (items <= 0) return 0;
  if (dtype == 0)
    return launch_decode<float>(q, q_stride, kc, vc, bt, max_blocks, item_tok, seq_of_token, positions,
                                part_o, part_ml, max_parts, out, out_stride, items, hq, hkv, page_size,
                                window, scale, stream);
  return launch_decode<bf16>(q, q_stride, kc, vc, bt, max_blocks, item_tok, seq_of_token, positions,
                             part_o, part_ml, max_parts, out, out_stride, items, hq, hkv, page_size,
                             window, scale, stream);
}

int rl_attn_prefill(int dtype, const void* q, int q_stride, const void* kc, const void* vc,
                    const int32_t* bt, int max_blocks, const int32_t* tile_seq,
                    const int32_t* tile_tok, const int32_t* tile_rows, const int32_t* positions,
                    void* out, int out_stride, int tiles, int hq, int hkv, int page_size, int window,
                    float scale, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (dtype == 0)
    return launch_prefill<float>(q, q_stride, kc, vc, bt, max_blocks, tile_seq, tile_tok, tile_rows,
                                 positions, out, out_stride, tiles, hq, hkv, page_size, window, scale,
                                 stream);
  return launch_prefill<bf16>(q, q_stride, kc, vc, bt, max_blocks, tile_seq, tile_tok, tile_rows,
                              positions, out, out_stride, tiles, hq, hkv, page_size, window, scale,
                              stream);
}

}  // extern "C"
