// Fused log-probability + entropy over a row of vocabulary logits, forward and backward.
//
// One CTA per row computes, in a single online-softmax sweep over the (bf16 or fp32) logits scaled by
// 1/temperature: log-sum-exp, sum_v p_v x_v, the target's log-probability and the entropy
// H = lse - sum_v p_v x_v. The [T, V] fp32 probabilities are never materialised. The backward pass
// writes dL/dlogits as bf16 (in place for bf16 logits) so the LM-head GEMMs can consume it directly.
//
// Reference counterparts: Megatron fused_vocab_parallel_cross_entropy and _VocabParallelEntropy
// (miles/backends/training_utils/loss_hub/math_utils.py:280-299,397-433).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>

#include "launchers.h"

namespace mb {
namespace {

using bf16 = __nv_bfloat16;

struct Stat {
  float m, s, sx;  // running max, sum exp(x-m), sum exp(x-m)*x
};

__device__ __forceinline__ void stat_add(Stat& a, float x) {
  if (x > a.m) {
    const float c = __expf(a.m - x);
    a.s = a.s * c + 1.f;
    a.sx = a.sx * c + x;
    a.m = x;
  } else {
    const float e = __expf(x - a.m);
    a.s += e;
    a.sx += e * x;
  }
}
__device__ __forceinline__ Stat stat_merge(const Stat& a, const Stat& b) {
  Stat r;
  r.m = fmaxf(a.m, b.m);
  const float ca = a.m == -FLT_MAX ? 0.f : __expf(a.m - r.m);
  const float cb = b.m == -FLT_MAX ? 0.f : __expf(b.m - r.m);
  r.s = a.s * ca + b.s * cb;
  r.sx = a.sx * ca + b.sx * cb;
  return r;
}

template <typename T>
__device__ __forceinline__ float ld(const T* p, long long i);
template <>
__device__ __forceinline__ float ld<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }

template <typename T, int THREADS>
__global__ void logprob_fwd_kernel(const T* __restrict__ logits, const int* __restrict__ targets,
                                   float* __restrict__ logprob, float* __restrict__ entropy, float* __restrict__ lse_out,
                                   float* __restrict__ psumx_out, int V, long long ld_, float inv_temp) {
  __shared__ Stat red[THREADS / 32];
  const long long row = blockIdx.x;
  const T* x = logits + row * ld_;
  Stat st{-FLT_MAX, 0.f, 0.f};
  constexpr int VEC = 16 / sizeof(T);
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  int v0 = 0;
  if (aligned) {
    const int nvec = V / VEC;
    for (int i = threadIdx.x; i < nvec; i += THREADS) {
      const uint4 raw = reinterpret_cast<const uint4*>(x)[i];
      if constexpr (sizeof(T) == 2) {
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(b[j]);
          stat_add(st, f.x * inv_temp);
          stat_add(st, f.y * inv_temp);
        }
      } else {
        const float* f = reinterpret_cast<const float*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) stat_add(st, f[j] * inv_temp);
      }
    }
    v0 = nvec * VEC;
  }
  for (int i = v0 + threadIdx.x; i < V; i += THREADS) stat_add(st, ld<T>(x, i) * inv_temp);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Stat other;
    other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
    other.sx = __shfl_xor_sync(0xffffffffu, st.sx, o);
    st = stat_merge(st, other);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = st;
  __syncthreads();
  if (threadIdx.x == 0) {
    Stat tot = red[0];
    for (int w = 1; w < THREADS / 32; ++w) tot = stat_merge(tot, red[w]);
    const float lse = tot.m + logf(tot.s);
    const float px = tot.sx / tot.s;
    if (lse_out) lse_out[row] = lse;
    if (psumx_out) psumx_out[row] = px;
    if (entropy) entropy[row] = lse - px;
    if (logprob) {
      const int t = targets[row];
      logprob[row] = (t >= 0 && t < V) ? ld<T>(x, t) * inv_temp - lse : 0.f;
    }
  }
}

template <typename T, int THREADS>
__global__ void logprob_bwd_kernel(const T* __restrict__ logits, const int* __restrict__ targets,
                                   const float* __restrict__ lse, const float* __restrict__ psumx,
                                   const float* __restrict__ dlogprob, const float* __restrict__ dentropy,
                                   bf16* __restrict__ dlogits, int V, long long ld_, long long ld_out, float inv_temp) {
  const long long row = blockIdx.x;
  const T* x = logits + row * ld_;
  bf16* dx = dlogits + row * ld_out;
  const float l = lse[row];
  const float px = psumx[row];
  const float dlp = dlogprob ? dlogprob[row] : 0.f;
  const float dh = dentropy ? dentropy[row] : 0.f;
  const int t = targets[row];
  for (int i = blockIdx.y * THREADS + threadIdx.x; i < V; i += gridDim.y * THREADS) {
    const float xs = ld<T>(x, i) * inv_temp;
    const float p = __expf(xs - l);
    float g = -dlp * p - dh * p * (xs - px);
    if (i == t) g += dlp;
    g *= inv_temp;
    dx[i] = __float2bfloat16(g);
  }
}

}  // namespace

void logprob_entropy_fwd(const void* logits, bool fp32, const int* targets, float* logprob, float* entropy, float* lse,
                         float* psum_x, int T, int V, long long ld, float inv_temp, cudaStream_t s) {
  if (T <= 0) return;
  if (fp32)
    logprob_fwd_kernel<float, 512><<<T, 512, 0, s>>>(static_cast<const float*>(logits), targets, logprob, entropy, lse,
                                                     psum_x, V, ld, inv_temp);
  else
    logprob_fwd_kernel<bf16, 512><<<T, 512, 0, s>>>(static_cast<const bf16*>(logits), targets, logprob, entropy, lse,
                                                    psum_x, V, ld, inv_temp);
}

void logprob_entropy_bwd(const void* logits, bool fp32, const int* targets, const float* lse, const float* psum_x,
                         const float* dlogprob, const float* dentropy, void* dlogits, int T, int V, long long ld,
                         long long ld_out, float inv_temp, cudaStream_t s) {
  if (T <= 0) return;
  int bx = (V + 256 * 8 - 1) / (256 * 8);
  if (bx < 1) bx = 1;
  dim3 grid(T, bx);
  if (fp32)
    logprob_bwd_kernel<float, 256><<<grid, 256, 0, s>>>(static_cast<const float*>(logits), targets, lse, psum_x,
                                                        dlogprob, dentropy, static_cast<bf16*>(dlogits), V, ld, ld_out, inv_temp);
  else
    logprob_bwd_kernel<bf16, 256><<<grid, 256, 0, s>>>(static_cast<const bf16*>(logits), targets, lse, psum_x, dlogprob,
                                                       dentropy, static_cast<bf16*>(dlogits), V, ld, ld_out, inv_temp);
}

}  // namespace mb
