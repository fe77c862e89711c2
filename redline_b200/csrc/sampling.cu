// Token sampling on the GPU: one CTA per row of float logits.
//
//   temperature <= 0   greedy: the arg max, the smaller index on ties
//   temperature  > 0   temperature, then top-k (ties at the k-th value kept), then
//                      top-p over what top-k kept, then one draw by the Gumbel-max
//                      trick: argmax_i (l_i - max) / T - log(-log(u_i)), u_i from
//                      Philox4x32-10 keyed by the request's seed with the counter
//                      (token index, position of the token being drawn, stream),
//                      so a draw does not depend on what else is in the batch.
//
// The thresholds of top-k and top-p are found without a sort by four 8-bit radix
// passes over order-preserving integer keys of the logits, counting tokens (top-k)
// or probability mass (top-p).  Mass is summed as 40-bit fixed point in integer
// atomics, so the result does not depend on the order in which threads arrive.
//
// What is the reference's and what is this file's own: the threshold search follows the
// reference's radix selection pass for pass (src/cuda/kernels/sampling.cu:53-127, including
// its rule for a target that rounding left out of reach: keep all that remains), and the
// Philox round, its counter layout and the constant 0x52444C4E in the counter are the
// reference's (src/cuda/kernels/common.cuh:105-140), as they must be for a seed to draw the
// same token in both engines.  The fixed-point mass in integer atomics, the two-stage arg max
// over chunks of a row and the kernels' organisation are this file's.
#include <cfloat>

#include "common.cuh"

namespace rl {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u >> 31) ? ~u : (u | 0x80000000u);
}

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ Best block_best(Best x, Best* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  Best r = lane < (blockDim.x >> 5) ? scratch[lane] : Best{-FLT_MAX, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = better(r, y);
  }
  return r;
}

__device__ __forceinline__ uint4 philox_4x32_10(uint4 c, uint2 k) {
  const uint32_t m0 = 0xD2511F53u, m1 = 0xCD9E8D57u;
  for (int round = 0; round < 10; ++round) {
    const uint32_t h0 = __umulhi(m0, c.x), l0 = m0 * c.x;
    const uint32_t h1 = __umulhi(m1, c.z), l1 = m1 * c.z;
    c = make_uint4(h1 ^ c.y ^ k.x, l1, h0 ^ c.w ^ k.y, l0);
    k.x += 0x9E3779B9u;
    k.y += 0xBB67AE85u;
  }
  return c;
}

// Uniform in the open interval (0, 1): 24 bits of the first Philox word, centred.
__device__ __forceinline__ float uniform_open01(uint32_t seed_lo, uint32_t seed_hi, uint32_t position,
                                                uint32_t stream, uint32_t index) {
  const uint4 r = philox_4x32_10(make_uint4(index, position, stream, 0x52444C4Eu),
                                 make_uint2(seed_lo, seed_hi));
  return (static_cast<float>(r.x >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

struct SampleSmem {
  float fscratch[32];
  Best bscratch[32];
  unsigned long long hist[256];
  uint32_t prefix;
  unsigned long long remaining;
};

constexpr float kMassScale = 1099511627776.0f;  // 2^40

// Key of the k-th largest logit.
__device__ uint32_t select_top_k(const float* l, int vocab, int k, SampleSmem& sh) {
  uint32_t prefix = 0, mask = 0;
  unsigned long long want = static_cast<unsigned long long>(k);
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) sh.hist[b] = 0ull;
    __syncthreads();
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const uint32_t key = order_key(l[i]);
      if ((key & mask) == prefix) atomicAdd(&sh.hist[(key >> shift) & 255u], 1ull);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long above = 0;
      int b = 255;
      for (; b > 0; --b) {
        if (above + sh.hist[b] >= want) break;
        above += sh.hist[b];
      }
      sh.prefix = prefix | (static_cast<uint32_t>(b) << shift);
      sh.remaining = want - above;
    }
    __syncthreads();
    prefix = sh.prefix;
    want = sh.remaining;
    mask |= 255u << shift;
  }
  return prefix;
}

// Largest key t such that the mass of {key >= t} among {key >= floor_key} reaches `target`
// (fixed point, scaled by 2^40 relative to the largest term).
__device__ uint32_t select_top_p(const float* l, int vocab, float mx, float inv_t, uint32_t floor_key,
                                 unsigned long long target, SampleSmem& sh) {
  uint32_t prefix = 0, mask = 0;
  unsigned long long want = target;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) sh.hist[b] = 0ull;
    __syncthreads();
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const uint32_t key = order_key(l[i]);
      if (key >= floor_key && (key & mask) == prefix) {
        const unsigned long long q =
            static_cast<unsigned long long>(expf((l[i] - mx) * inv_t) * kMassScale);
        atomicAdd(&sh.hist[(key >> shift) & 255u], q);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long above = 0;
      int chosen = -1, lowest = 0;
      for (int b = 255; b >= 0; --b) {
        const unsigned long long c = sh.hist[b];
        if (c == 0ull) continue;
        lowest = b;
        if (above + c >= want) {
          chosen = b;
          break;
        }
        above += c;
      }
      if (chosen < 0) {  // rounding left the target out of reach: keep all that remains
        chosen = lowest;
        sh.remaining = 0ull;
      } else {
        sh.remaining = want - above;
      }
      sh.prefix = prefix | (static_cast<uint32_t>(chosen) << shift);
    }
    __syncthreads();
    prefix = sh.prefix;
    want = sh.remaining;
    mask |= 255u << shift;
  }
  return prefix;
}

// First stage for greedy rows: the row is cut into pieces (kSampleChunks of them, or a quarter as many
// when the launch has many rows: CTAs of 2,000 values each are mostly start and end), one CTA each, which
// leave (max, arg max, sum of exp(l - max)) of their piece.  sample_kernel combines them.
constexpr int kSampleChunks = 64;

struct ChunkStat {
  float mx;
  int idx;
  float sumexp;
  float pad;
};

template <int kSampleHeld>
__global__ void __launch_bounds__(256)
sample_partial_kernel(const float* __restrict__ logits, int vocab, int ld, ChunkStat* __restrict__ stats, int chunks) {
  pdl_launch();
  pdl_wait();
  __shared__ Best bscratch[32];
  __shared__ float fscratch[32];
  const int row = blockIdx.x, chunk = blockIdx.y;
  const int per = (vocab + chunks - 1) / chunks;
  const int lo = chunk * per, hi = min(vocab, lo + per);
  const float* l = logits + static_cast<size_t>(row) * ld;
  // (the second stage reads kSampleChunks slots a row: those beyond this launch's pieces are marked empty)
  if (chunk == 0 && threadIdx.x < kSampleChunks - chunks)
    stats[row * kSampleChunks + chunks + threadIdx.x] = ChunkStat{-FLT_MAX, 0x7fffffff, 0.f, 0.f};
  // A thread's first kSampleHeld values stay in registers (all their loads are in flight together, and the
  // piece is read once); a piece longer than 256 * kSampleHeld goes on through memory.
  float v[kSampleHeld];
#pragma unroll
  for (int j = 0; j < kSampleHeld; ++j) {
    const int i = lo + threadIdx.x + j * 256;
    v[j] = i < hi ? l[i] : -FLT_MAX;
  }
  Best b{-FLT_MAX, 0x7fffffff};
#pragma unroll
  for (int j = 0; j < kSampleHeld; ++j) {
    const int i = lo + threadIdx.x + j * 256;
    if (i < hi) b = better(b, Best{v[j], i});
  }
  for (int i = lo + threadIdx.x + kSampleHeld * 256; i < hi; i += 256) b = better(b, Best{l[i], i});
  b = block_best(b, bscratch);
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < kSampleHeld; ++j) {
    const int i = lo + threadIdx.x + j * 256;
    if (i < hi) s += expf(v[j] - b.v);
  }
  for (int i = lo + threadIdx.x + kSampleHeld * 256; i < hi; i += 256) s += expf(l[i] - b.v);
  s = block_sum(s, fscratch);
  if (threadIdx.x == 0) stats[row * kSampleChunks + chunk] = ChunkStat{b.v, b.i, s, 0.f};
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int vocab, int ld, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const float* __restrict__ top_p,
              const uint32_t* __restrict__ seed_lo, const uint32_t* __restrict__ seed_hi,
              const int32_t* __restrict__ position, uint32_t stream_id, int32_t* __restrict__ out_token,
              float* __restrict__ out_logprob, const ChunkStat* __restrict__ stats) {
  pdl_launch();
  pdl_wait();
  __shared__ SampleSmem sh;
  const int row = blockIdx.x;
  const float* l = logits + static_cast<size_t>(row) * ld;
  if (stats != nullptr && temperature[row] <= 0.f) {
    // greedy row with first-stage statistics: combine the pieces (smaller index wins ties)
    if (threadIdx.x < 32) {
      Best b{-FLT_MAX, 0x7fffffff};
      for (int c = threadIdx.x; c < kSampleChunks; c += 32) {
        const ChunkStat st = stats[row * kSampleChunks + c];
        if (st.idx != 0x7fffffff) b = better(b, Best{st.mx, st.idx});
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, b.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, b.i, o);
        b = better(b, y);
      }
      float sum = 0.f;
      for (int c = threadIdx.x; c < kSampleChunks; c += 32) {
        const ChunkStat st = stats[row * kSampleChunks + c];
        if (st.idx != 0x7fffffff) sum += st.sumexp * expf(st.mx - b.v);
      }
      sum = warp_sum(sum);
      if (threadIdx.x == 0) {
        out_token[row] = b.i;
        if (out_logprob) out_logprob[row] = l[b.i] - (b.v + logf(sum));
      }
    }
    return;
  }

  Best b{-FLT_MAX, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) b = better(b, Best{l[i], i});
  b = block_best(b, sh.bscratch);
  const float mx = b.v;
  float s = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) s += expf(l[i] - mx);
  s = block_sum(s, sh.fscratch);
  const float lse = mx + logf(s);

  int token = b.i;
  const float temp = temperature[row];
  if (temp > 0.f) {
    const float inv_t = 1.f / temp;
    uint32_t thr = 0;
    const int k = top_k[row];
    if (k > 0 && k < vocab) thr = select_top_k(l, vocab, k, sh);
    const float p = top_p[row];
    if (p < 1.f) {
      // total mass of what top-k kept, in the same fixed point
      unsigned long long part = 0;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        if (order_key(l[i]) >= thr)
          part += static_cast<unsigned long long>(expf((l[i] - mx) * inv_t) * kMassScale);
      }
      __syncthreads();
      if (threadIdx.x == 0) sh.remaining = 0ull;
      __syncthreads();
      atomicAdd(&sh.remaining, part);
      __syncthreads();
      const unsigned long long total = sh.remaining;
      __syncthreads();
      const unsigned long long target =
          static_cast<unsigned long long>(static_cast<double>(p) * static_cast<double>(total));
      const uint32_t thr_p = select_top_p(l, vocab, mx, inv_t, thr, target > 0 ? target : 1ull, sh);
      thr = max(thr, thr_p);
    }
    Best g{-FLT_MAX, 0x7fffffff};
    const uint32_t slo = seed_lo[row], shi = seed_hi[row];
    const uint32_t pos = static_cast<uint32_t>(position[row]);
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      if (order_key(l[i]) < thr) continue;
      const float u = uniform_open01(slo, shi, pos, stream_id, static_cast<uint32_t>(i));
      g = better(g, Best{(l[i] - mx) * inv_t - logf(-logf(u)), i});
    }
    g = block_best(g, sh.bscratch);
    if (g.i != 0x7fffffff) token = g.i;
  }
  if (threadIdx.x == 0) {
    out_token[row] = token;
    if (out_logprob) out_logprob[row] = l[token] - lse;
  }
}

// out[r] = log_softmax(logits[r, :])[target[r]]   (sampling.cu:288-300)
__global__ void __launch_bounds__(512)
gather_logprob_kernel(const float* __restrict__ logits, int vocab, int ld,
                      const int32_t* __restrict__ target, float* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const float* l = logits + static_cast<size_t>(blockIdx.x) * ld;
  float m = -FLT_MAX;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, l[i]);
  m = block_max(m, scratch);
  float s = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) s += expf(l[i] - m);
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) out[blockIdx.x] = l[target[blockIdx.x]] - (m + logf(s));
}

}  // namespace rl

using namespace rl;

extern "C" {

int rl_sample_chunks() { return kSampleChunks; }

// scratch: optional [rows * rl_sample_chunks() * 4] floats.  With it, rows whose temperature is <= 0
// are served by a two-stage arg max that uses the whole GPU instead of one CTA per row.
int rl_sample(const float* logits, int rows, int vocab, int ld, const float* temperature,
              const int32_t* top_k, const float* top_p, const uint32_t* seed_lo,
              const uint32_t* seed_hi, const int32_t* position, unsigned stream_id,
              int32_t* out_token, float* out_logprob, float* scratch, cudaStream_t stream) {
  if (rows <= 0) return 0;
  ChunkStat* stats = reinterpret_cast<ChunkStat*>(scratch);
  if (stats != nullptr) {
    if (rows >= 16)
      launch_kernel(sample_partial_kernel<32>, dim3(rows, kSampleChunks / 4), dim3(256), 0, stream, logits, vocab, ld,
                    stats, kSampleChunks / 4);
    else
      launch_kernel(sample_partial_kernel<8>, dim3(rows, kSampleChunks), dim3(256), 0, stream, logits, vocab, ld,
                    stats, kSampleChunks);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  launch_kernel(sample_kernel, dim3(rows), dim3(kSampleThreads), 0, stream, logits, vocab, ld, temperature, top_k, top_p,
                                                     seed_lo, seed_hi, position, stream_id, out_token,
                                                     out_logprob, stats);
  RL_LAUNCH_END();
}

int rl_gather_logprob(const float* logits, int rows, int vocab, int ld, const int32_t* target,
                      float* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  launch_kernel(gather_logprob_kernel, dim3(rows), dim3(512), 0, stream, logits, vocab, ld, target, out);
  RL_LAUNCH_END();
}

}  // extern "C"
