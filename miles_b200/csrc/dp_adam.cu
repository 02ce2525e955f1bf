// Data-parallel optimizer step over NVLink peer memory: gradient reduce-scatter, partitioned Adam and parameter
// all-gather without a library collective.
//
// Every data-parallel rank keeps the flat gradient buffer (fp32) and the flat parameter buffer (bf16) of the
// replicated parameters in symmetric memory that all peers map. Rank r owns the element range [lo, hi) of the flat
// buffers: it keeps Adam moments (and the fp32 master copy) for that range only.
//
//   dp_reduce_shard : reduced[i - lo] = sum_d grad_d[i] for i in [lo, hi), reading every peer's gradient buffer with
//                     16-byte loads over NVLink (the reduce-scatter), plus per-block partial sums of squares for the
//                     global gradient norm (added up in block order, so the norm is reproducible).
//   dp_adam_push    : Adam on (a weight-decay segment of) the owned range with the reduced gradient, scaled by the
//                     device-side clip coefficient; the new bf16 parameters are stored into EVERY rank's parameter
//                     buffer (the all-gather).
//   peer_signal     : raises this rank's flag on every peer ("my gradients are final" before the reduce, "my part of
//                     your parameters has landed" after the pushes); consumers wait with the bounded flag wait of
//                     ep_comm.cu before they touch peer-written memory.
//
// Reference counterpart: Megatron's distributed optimizer: NCCL reduce-scatter of the gradient buckets, TE FusedAdam
// on the owned shard, NCCL all-gather of the updated parameters
// (miles/backends/megatron_utils/arguments.py:15-17, model.py:720-736).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launchers.h"

namespace mb {
namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__global__ void peer_signal_kernel(DpPeers peers, int me, int nranks, unsigned long long* ctrl, int which, int second) {
  const unsigned long long epoch = ctrl[which] + 1;
  __threadfence_system();
  if (threadIdx.x < nranks) st_release_sys_u64((second ? peers.flags2[threadIdx.x] : peers.flags[threadIdx.x]) + me, epoch);
  __syncthreads();
  if (threadIdx.x == 0) ctrl[which] = epoch;
}

// n4 = number of float4 groups in the shard; partial[blockIdx.x] receives the block's sum of squares.
__global__ void __launch_bounds__(256) dp_reduce_shard_kernel(DpPeers peers, int nranks, long long lo4, long long n4,
                                                              float4* __restrict__ reduced, float* __restrict__ partial) {
  __shared__ float red[8];
  float ss = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int d = 0; d < nranks; ++d) {  // fixed rank order: every step adds in the same order
      const float4 g = reinterpret_cast<const float4*>(peers.grad[d])[lo4 + i];
      acc.x += g.x;
      acc.y += g.y;
      acc.z += g.z;
      acc.w += g.w;
    }
    reduced[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}

// Groups of 8 elements (16 bytes of bf16 parameters) starting at absolute group index lo8; the state pointers are
// already offset to the first element of the piece. One call per weight-decay segment of the owned range.
template <typename MT>
__global__ void __launch_bounds__(256) dp_adam_push_kernel(DpPeers peers, int me, int nranks, long long lo8, long long n8,
                                                           const float* __restrict__ reduced, float* __restrict__ master,
                                                           MT* __restrict__ m, MT* __restrict__ v, float lr, float b1,
                                                           float b2, float eps, float wd, float bc1, float bc2,
                                                           const float* __restrict__ grad_scale,
                                                           const float* __restrict__ skip_flag) {
  const bool skip = skip_flag && *skip_flag != 0.f;
  const float gs = grad_scale ? *grad_scale : 1.f;
  const bf16* own = static_cast<const bf16*>(peers.param[me]);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 packed = reinterpret_cast<const uint4*>(own)[lo8 + i];
    if (!skip) {
      const bf16* pw = reinterpret_cast<const bf16*>(&packed);
      __align__(16) bf16 nw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const long long e = i * 8 + j;
        const float grad = reduced[e] * gs;
        float w = master ? master[e] : __bfloat162float(pw[j]);
        float mi = static_cast<float>(m[e]);
        float vi = static_cast<float>(v[e]);
        mi = b1 * mi + (1.f - b1) * grad;
        vi = b2 * vi + (1.f - b2) * grad * grad;
        const float upd = (mi / bc1) / (sqrtf(vi / bc2) + eps);
        w = w - lr * (upd + wd * w);
        m[e] = static_cast<MT>(mi);
        v[e] = static_cast<MT>(vi);
        if (master) master[e] = w;
        nw[j] = __float2bfloat16(w);
      }
      packed = *reinterpret_cast<const uint4*>(nw);
    }
    for (int d = 0; d < nranks; ++d) reinterpret_cast<uint4*>(peers.param[d])[lo8 + i] = packed;  // the all-gather
  }
}

int blocks_for(long long items) {
  long long b = (items + 255) / 256;
  if (b < 1) b = 1;
  return static_cast<int>(b < 148 * 8 ? b : 148 * 8);
}

}  // namespace

void peer_signal(const DpPeers& peers, int me, int nranks, unsigned long long* ctrl, int which, bool second, cudaStream_t s) {
  peer_signal_kernel<<<1, 32, 0, s>>>(peers, me, nranks, ctrl, which, second ? 1 : 0);
}

int dp_reduce_shard_blocks(long long shard_elems) { return blocks_for(shard_elems / 4); }

void dp_reduce_shard(const DpPeers& peers, int nranks, long long lo, long long shard_elems, float* reduced, float* partial,
                     cudaStream_t s) {
  if (shard_elems <= 0) return;
  dp_reduce_shard_kernel<<<blocks_for(shard_elems / 4), 256, 0, s>>>(peers, nranks, lo / 4, shard_elems / 4,
                                                                    reinterpret_cast<float4*>(reduced), partial);
}

void dp_adam_push(const DpPeers& peers, int me, int nranks, long long lo, long long n, const float* reduced, float* master,
                  void* m, void* v, bool mv_bf16, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                  const float* grad_scale, const float* skip_flag, cudaStream_t s) {
  if (n <= 0) return;
  const int grid = blocks_for(n / 8);
  if (mv_bf16)
    dp_adam_push_kernel<bf16><<<grid, 256, 0, s>>>(peers, me, nranks, lo / 8, n / 8, reduced, master, static_cast<bf16*>(m),
                                                   static_cast<bf16*>(v), lr, b1, b2, eps, wd, bc1, bc2, grad_scale, skip_flag);
  else
    dp_adam_push_kernel<float><<<grid, 256, 0, s>>>(peers, me, nranks, lo / 8, n / 8, reduced, master, static_cast<float*>(m),
                                                    static_cast<float*>(v), lr, b1, b2, eps, wd, bc1, bc2, grad_scale,
                                                    skip_flag);
}

}  // namespace mb
