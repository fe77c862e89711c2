// Row-wise kernels of the decoder: embedding gather, residual add + RMSNorm,
// row gather + RMSNorm for the logits rows, SiLU-gated product, rotary
// embedding fused with the write of keys and values into the paged cache.
//
// Activations are float (32-bit path) or bfloat16; the residual stream, sums of
// squares, rotation and SiLU are always computed in float.  Formulas follow the
// reference's kernels (src/cuda/kernels/elementwise.cu:19-89,
// src/cuda/kernels/rope_kv.cu:13-87) but the residual stream stays in float
// here instead of being rounded to the activation type after every layer.
#include "common.cuh"

namespace rl {

// ---------------------------------------------------------- token feed
// ids[i] = src[i] >= 0 ? sampled[src[i]] : ids[i]: a decode token whose value is
// still on the device (sampled by the step before, not yet read by the host) is
// taken from that step's output (reference: elementwise.cu:12-16).
__global__ void resolve_ids_kernel(int32_t* __restrict__ ids, const int32_t* __restrict__ src,
                                   const int32_t* __restrict__ sampled, int n) {
  pdl_launch();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && src[i] >= 0) ids[i] = sampled[src[i]];
}

// ---------------------------------------------------------------- embedding
// out[t, :] = float(table[ids[t], :]); `out` is the float residual stream.
// A token id outside [0, vocab) sets bit 0 of *status and yields a zero row.
template <typename TW>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab, int* status) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + static_cast<size_t>(t) * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, 1);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = 0.f;
    return;
  }
  const TW* row = table + static_cast<size_t>(id) * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = to_float(row[c]);
}

// ------------------------------------------------------- add + RMSNorm
// residual[r, :] += delta[r, :] (if delta), then
// out[r, :] = residual[r, :] * rsqrt(mean(residual^2) + eps) * w   (elementwise.cu:29-64).
// `rows_idx` (optional) selects which rows are normalised: out row i comes from
// row rows_idx[i] of residual (+ delta); the sum is then not written back (a row
// may be asked for twice), which is what the logits rows after the last layer need.
template <typename TA, typename TD, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   const TW* __restrict__ weight, TA* __restrict__ out,
                                   const int32_t* __restrict__ rows_idx, int hidden, float eps) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows_idx ? rows_idx[r] : r;
  float* res = residual + static_cast<size_t>(src) * hidden;
  const TD* d = delta ? delta + static_cast<size_t>(src) * hidden : nullptr;
  const bool write_back = (d != nullptr) && (rows_idx == nullptr);
  TA* o = out + static_cast<size_t>(r) * hidden;
  float ss = 0.f;
  if (hidden == static_cast<int>(blockDim.x) * 8) {
    // the row is exactly eight columns per thread: they stay in registers between the sum and the scaling
    const int c = threadIdx.x * 8;
    float v[8], w[8], y[8];
    load16(res + c, v);
    load16(res + c + 4, v + 4);
    if (sizeof(TW) == 2) {
      load16(weight + c, w);
    } else {
      load16(weight + c, w);
      load16(weight + c + 4, w + 4);
    }
    if (d) {
      float dv[8];
      if (sizeof(TD) == 2) {
        load16(d + c, dv);
      } else {
        load16(d + c, dv);
        load16(d + c + 4, dv + 4);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += dv[e];
      if (write_back) {
        store16(res + c, v);
        store16(res + c + 4, v + 4);
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = v[e] * inv * w[e];
    if (sizeof(TA) == 2) {
      store16(o + c, y);
    } else {
      store16(o + c, y);
      store16(o + c + 4, y + 4);
    }
    return;
  }
  if (hidden % 8 == 0) {
    // eight columns per thread and step: 16-byte pieces of every operand that is 16 bits wide,
    // two of every operand that is 32 bits wide
    for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
      float v[8];
      load16(res + c, v);
      load16(res + c + 4, v + 4);
      if (d) {
        float dv[8];
        if (sizeof(TD) == 2) {
          load16(d + c, dv);
        } else {
          load16(d + c, dv);
          load16(d + c + 4, dv + 4);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += dv[e];
        if (write_back) {
          store16(res + c, v);
          store16(res + c + 4, v + 4);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
    for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
      float v[8], w[8], y[8];
      load16(res + c, v);
      load16(res + c + 4, v + 4);
      if (d && !write_back) {
        float dv[8];
        if (sizeof(TD) == 2) {
          load16(d + c, dv);
        } else {
          load16(d + c, dv);
          load16(d + c + 4, dv + 4);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += dv[e];
      }
      if (sizeof(TW) == 2) {
        load16(weight + c, w);
      } else {
        load16(weight + c, w);
        load16(weight + c + 4, w + 4);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = v[e] * inv * w[e];
      if (sizeof(TA) == 2) {
        store16(o + c, y);
      } else {
        store16(o + c, y);
        store16(o + c + 4, y + 4);
      }
    }
    return;
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = res[c];
    if (d) v += to_float(d[c]);
    if (write_back) res[c] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = res[c];
    if (d && !write_back) v += to_float(d[c]);
    o[c] = from_float<TA>(v * inv * to_float(weight[c]));
  }
}

// residual[r, :] += delta[r, :] only (after the last layer when nothing follows).
template <typename TD>
__global__ void add_residual_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                    size_t n) {
  pdl_launch();
  pdl_wait();
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) residual[i] += to_float(delta[i]);
}

// --------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gu[t, i]) * gu[t, inter + i], silu(g) = g / (1 + exp(-g))
// (elementwise.cu:66-82), computed in float and rounded once.
template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int inter) {
  pdl_launch();
  pdl_wait();
  constexpr int VEC = Vec16<TA>::N;
  const int t = blockIdx.y;
  const TA* row = gu + static_cast<size_t>(t) * 2 * inter;
  TA* o = out + static_cast<size_t>(t) * inter;
  if (inter % VEC == 0) {                       // 16-byte pieces
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (i >= inter) return;
    float g[VEC], u[VEC], r[VEC];
    load16(row + i, g);
    load16(row + inter + i, u);
#pragma unroll
    for (int e = 0; e < VEC; ++e) r[e] = g[e] / (1.f + expf(-g[e])) * u[e];
    store16(o + i, r);
  } else {
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * VEC, e = 0; e < VEC && i + e < inter; ++e) {
      const float g = to_float(row[i + e]), u = to_float(row[inter + i + e]);
      o[i + e] = from_float<TA>(g / (1.f + expf(-g)) * u);
    }
  }
}

// ------------------------------------------------------------- add bias
template <typename TA, typename TW>
__global__ void add_bias_kernel(TA* __restrict__ x, const TW* __restrict__ bias, int n, size_t total) {
  pdl_launch();
  pdl_wait();
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < total) x[i] = from_float<TA>(to_float(x[i]) + to_float(bias[i % n]));
}

// ------------------------------------------------- RoPE + paged KV write
// qkv [T, (Hq + 2 Hkv) * D]: rotates every q and k head in place by the angle of
// the token's position (pairs (i, i + D/2), cos/sin tables [max_pos, D/2] in
// float: rope_kv.cu:26-51), then writes k and v of every kv head to the cache
// slot of the token: page = slot / page_size, offset = slot % page_size, cache
// layout [pages, Hkv, page_size, D] (rope_kv.cu:60-70).  A negative slot skips
// the write (a call that reads another call's cache).  cos == nullptr: no rotation.
// A slot at or beyond num_slots (pages of the pool times page_size) is not written either and
// sets bit 4 of the status word.
template <typename TA>
__global__ void rope_kv_write_kernel(TA* __restrict__ qkv, const int32_t* __restrict__ positions,
                                     const int32_t* __restrict__ slots,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     TA* __restrict__ kcache, TA* __restrict__ vcache, int hq, int hkv,
                                     int d, int page_size, int max_pos, long long num_slots, int* status) {
  pdl_launch();
  pdl_wait();
  constexpr int VEC = Vec16<TA>::N;    // head sizes are multiples of 16, so D / 2 is a multiple of VEC
  const int t = blockIdx.x;
  const int half = d >> 1;
  const int pos = positions[t];
  TA* row = qkv + static_cast<size_t>(t) * (hq + 2 * hkv) * d;
  int slot = slots ? slots[t] : -1;
  const bool bad_pos = (pos < 0 || pos >= max_pos);
  if (bad_pos && threadIdx.x == 0) atomicOr(status, 2);
  if (slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, 4);
    slot = -1;
  }
  const float* c = cos_t ? cos_t + static_cast<size_t>(bad_pos ? 0 : pos) * half : nullptr;
  const float* s = sin_t ? sin_t + static_cast<size_t>(bad_pos ? 0 : pos) * half : nullptr;
  const size_t page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot % page_size : 0;
  const int rot_heads = hq + hkv;
  const int vec_per_head = half / VEC;
  // One item per thread and round: a (head, run of VEC pairs (i, i + D/2)) of the q and k heads, or a
  // 16-byte piece of v for the cache.  Both kinds are in one loop, so that all of a token's loads are in
  // flight together.
  const int n_rot = rot_heads * vec_per_head;
  const int n_v = slot >= 0 ? hkv * d / VEC : 0;
  for (int idx = threadIdx.x; idx < n_rot + n_v; idx += blockDim.x) {
    if (idx >= n_rot) {
      const int e0 = (idx - n_rot) * VEC;
      const int h = e0 / d, i = e0 - h * d;
      const TA* vrow = row + (hq + hkv) * d;
      *reinterpret_cast<uint4*>(vcache + ((page * hkv + h) * page_size + off) * d + i) =
          *reinterpret_cast<const uint4*>(vrow + e0);
      continue;
    }
    const int h = idx / vec_per_head, i = (idx - h * vec_per_head) * VEC;
    TA* v = row + h * d;
    float x0[VEC], x1[VEC];
    load16(v + i, x0);
    load16(v + i + half, x1);
    if (c) {
      float cv[VEC], sv[VEC];
#pragma unroll
      for (int e = 0; e < VEC; e += 4) {          // (half is a multiple of 8: 16-byte aligned pieces)
        load16(c + i + e, cv + e);
        load16(s + i + e, sv + e);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float cc = cv[e], sn = sv[e];
        const float y0 = x0[e] * cc - x1[e] * sn;
        const float y1 = x1[e] * cc + x0[e] * sn;
        x0[e] = y0;
        x1[e] = y1;
      }
    }
    store16(v + i, x0);
    store16(v + i + half, x1);
    if (h >= hq && slot >= 0) {
      TA* dst = kcache + ((page * hkv + (h - hq)) * page_size + off) * d;
      store16(dst + i, x0);
      store16(dst + i + half, x1);
    }
  }
}

}  // namespace rl

using namespace rl;

static inline int row_threads(int n) {
  int t = 32;
  while (t < n && t < 512) t <<= 1;
  return t;
}

// dtype codes shared with the Python side: 0 = float32, 1 = bfloat16.
#define RL_F32 0
#define RL_BF16 1

extern "C" {

int rl_resolve_ids(int32_t* ids, const int32_t* src, const int32_t* sampled, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  launch_kernel(resolve_ids_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, ids, src, sampled, n);
  RL_LAUNCH_END();
}

int rl_embedding(const int32_t* ids, const void* table, int table_dtype, float* out, int tokens,
                 int hidden, int vocab, int* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int th = row_threads(hidden);
  if (table_dtype == RL_F32) {
    launch_kernel(embedding_kernel<float>, dim3(tokens), dim3(th), 0, stream, ids, static_cast<const float*>(table), out,
                                                       hidden, vocab, status);
  } else {
    launch_kernel(embedding_kernel<bf16>, dim3(tokens), dim3(th), 0, stream, ids, static_cast<const bf16*>(table), out,
                                                      hidden, vocab, status);
  }
  RL_LAUNCH_END();
}

// act_dtype: type of `delta` and `out`; w_dtype: type of `weight`.
int rl_add_rmsnorm(float* residual, const void* delta, const void* weight, int w_dtype, void* out,
                   int act_dtype, const int32_t* rows_idx, int rows, int hidden, float eps,
                   cudaStream_t stream) {
  if (rows <= 0) return 0;
  // eight columns per thread where the row allows it (then, up to 4,096 columns, the row stays in registers)
  const int th = hidden % 8 == 0 ? row_threads(hidden / 8) : row_threads(hidden);
#define RL_NORM_CASE(TA, TW)                                                                 \
  launch_kernel(add_rmsnorm_kernel<TA, TA, TW>, dim3(rows), dim3(th), 0, stream,                                    \
      residual, static_cast<const TA*>(delta), static_cast<const TW*>(weight),               \
      static_cast<TA*>(out), rows_idx, hidden, eps)
  if (act_dtype == RL_F32 && w_dtype == RL_F32) RL_NORM_CASE(float, float);
  else if (act_dtype == RL_F32) RL_NORM_CASE(float, bf16);
  else if (w_dtype == RL_F32) RL_NORM_CASE(bf16, float);
  else RL_NORM_CASE(bf16, bf16);
#undef RL_NORM_CASE
  RL_LAUNCH_END();
}

int rl_add_residual(float* residual, const void* delta, int act_dtype, long long n,
                    cudaStream_t stream) {
  if (n <= 0) return 0;
  const int th = 256;
  const unsigned blocks = static_cast<unsigned>((n + th - 1) / th);
  if (act_dtype == RL_F32)
    launch_kernel(add_residual_kernel<float>, dim3(blocks), dim3(th), 0, stream, residual, static_cast<const float*>(delta), n);
  else
    launch_kernel(add_residual_kernel<bf16>, dim3(blocks), dim3(th), 0, stream, residual, static_cast<const bf16*>(delta), n);
  RL_LAUNCH_END();
}

int rl_swiglu(const void* gu, void* out, int act_dtype, int tokens, int inter, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int th = 256;
  const int per_block = th * (act_dtype == RL_F32 ? 4 : 8);   // a thread takes one 16-byte piece
  dim3 grid((inter + per_block - 1) / per_block, tokens);
  if (act_dtype == RL_F32)
    launch_kernel(swiglu_kernel<float>, dim3(grid), dim3(th), 0, stream, static_cast<const float*>(gu), static_cast<float*>(out), inter);
  else
    launch_kernel(swiglu_kernel<bf16>, dim3(grid), dim3(th), 0, stream, static_cast<const bf16*>(gu), static_cast<bf16*>(out), inter);
  RL_LAUNCH_END();
}

int rl_add_bias(void* x, int act_dtype, const void* bias, int b_dtype, int rows, int n,
                cudaStream_t stream) {
  const size_t total = static_cast<size_t>(rows) * n;
  if (total == 0) return 0;
  const int th = 256;
  const unsigned blocks = static_cast<unsigned>((total + th - 1) / th);
#define RL_BIAS_CASE(TA, TW)                                                               \
  launch_kernel(add_bias_kernel<TA, TW>, dim3(blocks), dim3(th), 0, stream, static_cast<TA*>(x),                  \
                                                     static_cast<const TW*>(bias), n, total)
  if (act_dtype == RL_F32 && b_dtype == RL_F32) RL_BIAS_CASE(float, float);
  else if (act_dtype == RL_F32) RL_BIAS_CASE(float, bf16);
  else if (b_dtype == RL_F32) RL_BIAS_CASE(bf16, float);
  else RL_BIAS_CASE(bf16, bf16);
#undef RL_BIAS_CASE
  RL_LAUNCH_END();
}

int rl_rope_kv_write(void* qkv, int act_dtype, const int32_t* positions, const int32_t* slots,
                     const float* cos_t, const float* sin_t, void* kcache, void* vcache, int tokens,
                     int hq, int hkv, int d, int page_size, int max_pos, long long num_slots, int* status,
                     cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int th = 256;
  if (act_dtype == RL_F32)
    launch_kernel(rope_kv_write_kernel<float>, dim3(tokens), dim3(th), 0, stream, 
        static_cast<float*>(qkv), positions, slots, cos_t, sin_t, static_cast<float*>(kcache),
        static_cast<float*>(vcache), hq, hkv, d, page_size, max_pos, num_slots, status);
  else
    launch_kernel(rope_kv_write_kernel<bf16>, dim3(tokens), dim3(th), 0, stream, 
        static_cast<bf16*>(qkv), positions, slots, cos_t, sin_t, static_cast<bf16*>(kcache),
        static_cast<bf16*>(vcache), hq, hkv, d, page_size, max_pos, num_slots, status);
  RL_LAUNCH_END();
}

}  // extern "C"
