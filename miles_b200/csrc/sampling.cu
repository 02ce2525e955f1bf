// Token sampling for the rollout engine: temperature, top-k, top-p and a counter-based RNG, one CTA
// per request row. The sampled token's log-probability is reported under the temperature-scaled
// *full* distribution (what the trainer recomputes), independent of the top-k/top-p truncation.
//
// Unrestricted rows (top_k <= 0, top_p >= 1) take a single fused sweep: online log-sum-exp plus the
// Gumbel-max trick (argmax of x/T + G, G = -log(-log u)), which draws exactly from softmax(x/T).
// Restricted rows first find a logit threshold by bisection on the order-preserving integer image of
// the float (<= 32 counting sweeps for top-k, <= 32 mass sweeps for top-p over the L2-resident row),
// then run the same Gumbel sweep over the surviving tokens.
//
// Reference counterpart: the sgl-kernel / flashinfer samplers behind SGLang's /generate
// (miles/rollout/generate_utils/generate_endpoint_utils.py:52-77 builds the sampling params).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "launchers.h"

namespace mb {
namespace {

using bf16 = __nv_bfloat16;
constexpr int THREADS = 1024;

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
// uniform in (0, 1)
__device__ __forceinline__ float uniform01(uint64_t seed, uint32_t step, uint32_t idx) {
  const uint64_t h = splitmix64(seed ^ splitmix64((static_cast<uint64_t>(step) << 32) | idx));
  return (static_cast<float>(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ uint32_t ordered(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float unordered(uint32_t o) {
  const uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
  return __uint_as_float(u);
}

template <typename T>
__device__ __forceinline__ float ldf(const T* p, int i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, int i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<bf16>(const bf16* p, int i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < THREADS / 32 ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) red[32] = t;
  }
  __syncthreads();
  const float r = red[32];
  __syncthreads();
  return r;
}

template <typename T>
__global__ void __launch_bounds__(THREADS) sample_kernel(const T* __restrict__ logits, int V, long long ld,
                                                         const float* __restrict__ temperature,
                                                         const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                         const unsigned long long* __restrict__ seeds,
                                                         const int* __restrict__ step, int* __restrict__ out_token,
                                                         float* __restrict__ out_logprob, int restricted_only) {
  __shared__ float red[33];
  __shared__ float s_m[32], s_s[32], s_best[32];
  __shared__ int s_idx[32];
  const int row = blockIdx.x;
  const T* x = logits + static_cast<long long>(row) * ld;
  float temp = temperature ? temperature[row] : 1.f;
  const bool greedy = temp <= 0.f;
  if (greedy) temp = 1.f;
  const float inv_t = 1.f / temp;
  const int k = top_k ? top_k[row] : 0;
  if (restricted_only) {  // the split kernel has already handled every unrestricted row
    const float pp = top_p ? top_p[row] : 1.f;
    if (greedy || !((k > 0 && k < V) || pp < 1.f)) return;
  }
  const float p = top_p ? top_p[row] : 1.f;
  const uint64_t seed = seeds ? seeds[row] : 0x1234ull + row;
  const uint32_t stp = step ? static_cast<uint32_t>(step[row]) : 0u;

  // ---- sweep 1: max and sum exp of x/T
  float m = -FLT_MAX, s = 0.f;
  for (int i = threadIdx.x; i < V; i += THREADS) {
    const float v = ldf<T>(x, i) * inv_t;
    if (v > m) {
      s = s * __expf(m - v) + 1.f;
      m = v;
    } else {
      s += __expf(v - m);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = s * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
  }
  if ((threadIdx.x & 31) == 0) {
    s_m[threadIdx.x >> 5] = m;
    s_s[threadIdx.x >> 5] = s;
  }
  __syncthreads();
  float gm = -FLT_MAX, gs = 0.f;
  for (int w = 0; w < THREADS / 32; ++w) {
    const float nm = fmaxf(gm, s_m[w]);
    gs = gs * __expf(gm - nm) + s_s[w] * __expf(s_m[w] - nm);
    gm = nm;
  }
  const float lse = gm + logf(gs);
  __syncthreads();

  // ---- threshold (in scaled-logit space) from top-k / top-p
  float thr = -FLT_MAX;
  if (!greedy && k > 0 && k < V) {
    uint32_t lo = 0u, hi = 0xffffffffu;  // largest o with count(x >= o) >= k
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1) + 1u;
      float c = 0.f;
      for (int i = threadIdx.x; i < V; i += THREADS) c += (ordered(ldf<T>(x, i) * inv_t) >= mid) ? 1.f : 0.f;
      c = block_reduce_sum(c, red);
      if (c >= static_cast<float>(k)) lo = mid; else hi = mid - 1u;
    }
    thr = unordered(lo);
  }
  if (!greedy && p < 1.f) {
    // mass of the top-k set, then the largest threshold whose tail mass reaches p of it
    float base = 0.f;
    for (int i = threadIdx.x; i < V; i += THREADS) {
      const float v = ldf<T>(x, i) * inv_t;
      if (v >= thr) base += __expf(v - gm);
    }
    base = block_reduce_sum(base, red);
    const float need = p * base;
    uint32_t lo = ordered(thr == -FLT_MAX ? -FLT_MAX : thr), hi = ordered(gm);
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1) + 1u;
      float c = 0.f;
      for (int i = threadIdx.x; i < V; i += THREADS) {
        const float v = ldf<T>(x, i) * inv_t;
        if (ordered(v) >= mid) c += __expf(v - gm);
      }
      c = block_reduce_sum(c, red);
      if (c >= need) lo = mid; else hi = mid - 1u;
    }
    thr = fmaxf(thr, unordered(lo));
  }

  // ---- Gumbel-max over the surviving tokens (plain argmax when greedy)
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += THREADS) {
    const float v = ldf<T>(x, i) * inv_t;
    if (v < thr) continue;
    float key = v;
    if (!greedy) {
      const float u = uniform01(seed, stp, static_cast<uint32_t>(i));
      key = v - __logf(-__logf(u));
    }
    if (key > best || (key == best && i < best_i)) {
      best = key;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    s_best[threadIdx.x >> 5] = best;
    s_idx[threadIdx.x >> 5] = best_i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < THREADS / 32; ++w) {
      if (s_best[w] > best || (s_best[w] == best && s_idx[w] < best_i)) {
        best = s_best[w];
        best_i = s_idx[w];
      }
    }
    if (best_i < 0 || best_i >= V) best_i = 0;
    out_token[row] = best_i;
    if (out_logprob) out_logprob[row] = ldf<T>(x, best_i) * inv_t - lse;
  }
}

// ---- unrestricted rows, split over SPLITS CTAs per row -------------------------------------------------
// One sweep per CTA over its slice: online log-sum-exp and the Gumbel arg-max together. The last CTA of a row to
// finish (a self-resetting arrival counter) merges the SPLITS partial results. One CTA per row leaves most of the
// GPU idle at decode batch sizes, and the vocabulary sweep then costs more than the LM head that feeds it.
constexpr int SPLITS = 32;
constexpr int SPLIT_THREADS = 256;
constexpr int SPLIT_MAX_ROWS = 1024;
__device__ float g_part[SPLIT_MAX_ROWS][SPLITS][4];  // m, s, best key, best index (as int bits)
__device__ unsigned int g_arrive[SPLIT_MAX_ROWS];

__device__ __forceinline__ bool row_is_restricted(const int* top_k, const float* top_p, const float* temperature, int row,
                                                  int V) {
  const int k = top_k ? top_k[row] : 0;
  const float p = top_p ? top_p[row] : 1.f;
  const bool greedy = temperature && temperature[row] <= 0.f;
  return !greedy && ((k > 0 && k < V) || p < 1.f);
}

template <typename T>
__global__ void __launch_bounds__(SPLIT_THREADS) sample_split_kernel(const T* __restrict__ logits, int V, long long ld,
                                                                     const float* __restrict__ temperature,
                                                                     const int* __restrict__ top_k,
                                                                     const float* __restrict__ top_p,
                                                                     const unsigned long long* __restrict__ seeds,
                                                                     const int* __restrict__ step,
                                                                     int* __restrict__ out_token,
                                                                     float* __restrict__ out_logprob) {
  __shared__ float s_m[8], s_s[8], s_best[8];
  __shared__ int s_idx[8];
  __shared__ bool s_last;
  const int row = blockIdx.x, split = blockIdx.y;
  if (row_is_restricted(top_k, top_p, temperature, row, V)) return;  // handled by sample_kernel
  const T* x = logits + static_cast<long long>(row) * ld;
  float temp = temperature ? temperature[row] : 1.f;
  const bool greedy = temp <= 0.f;
  if (greedy) temp = 1.f;
  const float inv_t = 1.f / temp;
  const uint64_t seed = seeds ? seeds[row] : 0x1234ull + row;
  const uint32_t stp = step ? static_cast<uint32_t>(step[row]) : 0u;
  const int per = (V + SPLITS - 1) / SPLITS;
  const int lo = split * per, hi = min(V, lo + per);
  float m = -FLT_MAX, s = 0.f, best = -FLT_MAX;
  int best_i = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += SPLIT_THREADS) {
    const float v = ldf<T>(x, i) * inv_t;
    if (v > m) {
      s = s * __expf(m - v) + 1.f;
      m = v;
    } else {
      s += __expf(v - m);
    }
    float key = v;
    if (!greedy) key = v - __logf(-__logf(uniform01(seed, stp, static_cast<uint32_t>(i))));
    if (key > best || (key == best && i < best_i)) {
      best = key;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = s * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    s_m[warp] = m;
    s_s[warp] = s;
    s_best[warp] = best;
    s_idx[warp] = best_i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < SPLIT_THREADS / 32; ++w) {
      const float nm = fmaxf(m, s_m[w]);
      s = s * __expf(m - nm) + s_s[w] * __expf(s_m[w] - nm);
      m = nm;
      if (s_best[w] > best || (s_best[w] == best && s_idx[w] < best_i)) {
        best = s_best[w];
        best_i = s_idx[w];
      }
    }
    float* part = g_part[row][split];
    part[0] = m;
    part[1] = s;
    part[2] = best;
    part[3] = __int_as_float(best_i);
    __threadfence();
    const unsigned int prev = atomicAdd(&g_arrive[row], 1u);
    s_last = (prev == SPLITS - 1);
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x < 32) {
    __threadfence();
    const volatile float* part = g_part[row][threadIdx.x];  // SPLITS == 32: one partial per lane
    m = part[0];
    s = part[1];
    best = part[2];
    best_i = __float_as_int(part[3]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = s * __expf(m - nm) + os * __expf(om - nm);
      m = nm;
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) {
        best = ob;
        best_i = oi;
      }
    }
    if (threadIdx.x == 0) {
      if (best_i < 0 || best_i >= V) best_i = 0;
      out_token[row] = best_i;
      if (out_logprob) out_logprob[row] = ldf<T>(x, best_i) * inv_t - (m + logf(s));
      g_arrive[row] = 0u;  // ready for the next launch on this stream
    }
  }
}

}  // namespace

void sample_rows(const void* logits, bool fp32, int T, int V, long long ld, const float* temperature, const int* top_k,
                 const float* top_p, const unsigned long long* seeds, const int* step, int* out_token, float* out_logprob,
                 cudaStream_t s) {
  if (T <= 0) return;
  // Unrestricted rows go to the split kernel (calls on different streams must not overlap: its partial results
  // live in one device array); rows with top-k / top-p, if the request tensors are given, to the bisection kernel.
  const bool split = T <= SPLIT_MAX_ROWS;
  const bool may_restrict = top_k != nullptr || top_p != nullptr;
  if (split) {
    if (fp32)
      sample_split_kernel<float><<<dim3(T, SPLITS), SPLIT_THREADS, 0, s>>>(static_cast<const float*>(logits), V, ld,
                                                                          temperature, top_k, top_p, seeds, step,
                                                                          out_token, out_logprob);
    else
      sample_split_kernel<bf16><<<dim3(T, SPLITS), SPLIT_THREADS, 0, s>>>(static_cast<const bf16*>(logits), V, ld,
                                                                         temperature, top_k, top_p, seeds, step,
                                                                         out_token, out_logprob);
    if (!may_restrict) return;
  }
  if (fp32)
    sample_kernel<float><<<T, THREADS, 0, s>>>(static_cast<const float*>(logits), V, ld, temperature, top_k, top_p, seeds,
                                               step, out_token, out_logprob, split ? 1 : 0);
  else
    sample_kernel<bf16><<<T, THREADS, 0, s>>>(static_cast<const bf16*>(logits), V, ld, temperature, top_k, top_p, seeds,
                                              step, out_token, out_logprob, split ? 1 : 0);
}

}  // namespace mb
