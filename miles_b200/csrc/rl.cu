// Generalised advantage estimation as a reverse linear recurrence, one warp per sequence.
//
//   delta_t = r_t + gamma * V_{t+1} - V_t ;  A_t = delta_t + (gamma*lambda) * A_{t+1}
//
// The warp walks the sequence backwards 32 tokens at a time; inside a chunk the recurrence
// a_j = x_j + w * a_{j-1} is solved with a log-step shuffle scan (coefficients are powers of w) and the
// carry of the previous chunk is injected with w^(lane+1). Inputs are flat over trainable tokens with
// cumulative sequence lengths.
//
// Reference counterpart: chunked_gae in
// miles/backends/training_utils/loss_hub/math_utils.py:792-932 (a [*,128]x[128,128] GEMM plus a carry).
#include <cuda_runtime.h>

#include "launchers.h"

namespace mb {
namespace {

__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                           const int* __restrict__ cu, float* __restrict__ adv, float* __restrict__ ret, int num_seqs,
                           float gamma, float lam) {
  const int seq = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (seq >= num_seqs) return;
  const int lo = cu[seq], hi = cu[seq + 1];
  const float w = gamma * lam;
  float wp[5];  // w^1, w^2, w^4, w^8, w^16
  wp[0] = w;
#pragma unroll
  for (int i = 1; i < 5; ++i) wp[i] = wp[i - 1] * wp[i - 1];
  float wl = 1.f;  // w^(lane+1)
  for (int i = 0; i <= lane; ++i) wl *= w;
  float carry = 0.f;
  for (int end = hi; end > lo; end -= 32) {
    const int t = end - 1 - lane;  // lane 0 handles the latest token of the chunk
    const bool valid = t >= lo;
    float x = 0.f, v = 0.f;
    if (valid) {
      v = values[t];
      const float nxt = (t + 1 < hi) ? values[t + 1] : 0.f;
      x = rewards[t] + gamma * nxt - v;
    }
#pragma unroll
    for (int s = 0; s < 5; ++s) {
      const float up = __shfl_up_sync(0xffffffffu, x, 1 << s);
      if (lane >= (1 << s)) x += wp[s] * up;
    }
    x += wl * carry;
    if (valid) {
      adv[t] = x;
      ret[t] = x + v;
    }
    carry = __shfl_sync(0xffffffffu, x, 31);
  }
}

}  // namespace

void gae_reverse_scan(const float* rewards, const float* values, const int* cu_seqlens, float* adv, float* ret,
                      int num_seqs, float gamma, float lam, cudaStream_t s) {
  if (num_seqs <= 0) return;
  const int threads = 128;
  const int blocks = (num_seqs * 32 + threads - 1) / threads;
  gae_kernel<<<blocks, threads, 0, s>>>(rewards, values, cu_seqlens, adv, ret, num_seqs, gamma, lam);
}

}  // namespace mb
