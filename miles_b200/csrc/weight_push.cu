// Trainer -> engine weight update as one kernel per bucket: reshard, optionally quantise, store into the engines'
// weight buffers on every destination GPU over NVLink peer memory, then raise a version flag.
//
// The host describes a bucket as a table of 2-D slabs. A slab is `rows x cols` bf16 elements of the trainer's local
// shard (`src_off`, leading dimension `src_ld`) that lands at position (`dst_row0`, `dst_col0`) of destination tensor
// `tensor` on every rank named in `peer_mask`. Row slices (expert ranges, query-head groups, vocabulary ranges),
// column slices (the input dimension of the output / down projections) and interleaved pieces (gate and up rows of
// one tensor-parallel shard) are all slabs, so any (tensor, expert) layout of the trainer maps onto any layout of
// the engine with one table that is built once.
//
// Destination formats, per tensor table entry:
//   bf16  : the element lands at `val_off + (row * ld + col) * 2` of the destination region.
//   MXFP8 : 32-element blocks along the row; E4M3 values at `val_off + row * K + col`, one E8M0 scale per block
//           (the smallest power of two that keeps amax / scale <= 448) written straight into the scale-factor atom
//           layout the block-scaled tensor-core GEMM reads (csrc/gemm_mx.cu: atoms of 128 rows x 4 scales, 512 bytes).
//   NVFP4 : 16-element blocks; E2M1 pairs at `val_off + (row * K + col) / 2`, E4M3 block scales in the same atom
//           layout, with the per-tensor encode scale 448 * 6 / amax taken from `amax[amax_slot]`: tensors that must
//           share one scale (gate and up, all experts of a layer) name the same slot; the slots are reduced over the
//           trainer's ranks before the launch.
//
// Every thread owns 8 consecutive elements (one 16-byte load), quantises them in registers with the lanes that share
// its block (shuffles), and issues one store per destination rank, so a shard is read once however many engines
// take it. The last CTA to finish publishes `version` into `flags[me]` of every rank in `flag_mask` with a
// system-scope release; `weight_push_wait` is the consumer side: a bounded wait (global timer) on the flags of the
// expected sources that records ERR_WAIT_PEER in the status word and returns when a source never arrives.
//
// Reference counterpart: the per-bucket gather + HF conversion + quantise + broadcast / RDMA write loop of
// miles/backends/megatron_utils/update_weight/update_weight_from_distributed/broadcast.py:201-291 with
// processors/quantizer_mxfp8.py:6-116 and quantizer_nvfp4.py:36-203.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "launchers.h"
#include "ptx.cuh"
#include "quant_math.cuh"

namespace mb {
namespace {

using namespace qmath;
using bf16 = __nv_bfloat16;

__device__ __forceinline__ unsigned long long wp_ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void wp_st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// byte offset of scale `s` of row `r` inside the scale-factor atoms of a tensor with `S` scales per row
__device__ __forceinline__ long long atom_offset(long long r, int s, int S) {
  const long long s4 = (S + 3) / 4;
  const long long atom = (r / 128) * s4 + s / 4;
  const int rr = static_cast<int>(r % 128);
  return atom * 512 + (rr % 32) * 16 + (rr / 32) * 4 + (s % 4);
}

__global__ void __launch_bounds__(256) weight_push_kernel(const bf16* __restrict__ src, const WeightPushSeg* __restrict__ segs,
                                                          int nseg, const WeightPushTensor* __restrict__ tensors,
                                                          const float* __restrict__ amax, WeightPushPeers peers, int me,
                                                          unsigned flag_mask, unsigned long long version,
                                                          unsigned int* __restrict__ counter) {
  const int lane = threadIdx.x & 31;
  for (int si = blockIdx.y; si < nseg; si += gridDim.y) {
    const WeightPushSeg sg = segs[si];
    const WeightPushTensor tn = tensors[sg.tensor];
    const int vec_per_row = static_cast<int>(sg.cols >> 3);
    const long long nvec = static_cast<long long>(sg.rows) * vec_per_row;
    float genc = 1.f;
    if (tn.mode == 2) {
      const float a = amax[tn.amax_slot];
      genc = (448.f * 6.f) / a;
      if (!(genc < FLT_MAX)) genc = FLT_MAX;
      if (genc == 0.f || a == 0.f) genc = 1.f;
    }
    // whole warps iterate together (the shuffles below need every lane): round the trip count up to a warp
    const long long nvec_w = (nvec + 31) & ~31LL;
    for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec_w;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
      const bool valid = v < nvec;
      const long long r = valid ? v / vec_per_row : 0;
      const int cv = valid ? static_cast<int>(v - r * vec_per_row) : 0;
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (valid) raw = __ldg(reinterpret_cast<const uint4*>(src + sg.src_off + r * sg.src_ld + cv * 8));
      const long long R = sg.dst_row0 + r;
      const int Ccol = static_cast<int>(sg.dst_col0) + cv * 8;
      if (tn.mode == 0) {
        if (!valid) continue;
        const long long off = tn.val_off + (R * tn.ld + Ccol) * 2;
#pragma unroll
        for (int p = 0; p < 8; ++p)
          if ((sg.peer_mask >> p) & 1u) *reinterpret_cast<uint4*>(peers.base[p] + off) = raw;
        continue;
      }
      float f[8];
      {
        const bf16* h = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(h[j]);
      }
      float am = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(f[j]));
      if (tn.mode == 1) {
        // 4 lanes share a 32-element block; 16 lanes (128 elements) share one 4-byte group of scales
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
        const uint8_t e = e8m0_ceil(am / 448.f);
        const float inv = 1.f / e8m0_to_float(e);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) lo |= static_cast<uint32_t>(to_e4m3(f[j] * inv)) << (8 * j);
#pragma unroll
        for (int j = 0; j < 4; ++j) hi |= static_cast<uint32_t>(to_e4m3(f[4 + j] * inv)) << (8 * j);
        uint32_t sc4 = e;
        sc4 |= static_cast<uint32_t>(__shfl_down_sync(0xffffffffu, static_cast<uint32_t>(e), 4)) << 8;
        sc4 |= static_cast<uint32_t>(__shfl_down_sync(0xffffffffu, static_cast<uint32_t>(e), 8)) << 16;
        sc4 |= static_cast<uint32_t>(__shfl_down_sync(0xffffffffu, static_cast<uint32_t>(e), 12)) << 24;
        if (!valid) continue;
        const long long qoff = tn.val_off + R * tn.ld + Ccol;
        const bool lead = (lane & 15) == 0;  // cols % 128 == 0 and dst_col0 % 128 == 0: a scale group never straddles rows
        const long long aoff = tn.sf_off + atom_offset(R, Ccol >> 5, static_cast<int>(tn.ld >> 5));
#pragma unroll
        for (int p = 0; p < 8; ++p)
          if ((sg.peer_mask >> p) & 1u) {
            *reinterpret_cast<uint2*>(peers.base[p] + qoff) = make_uint2(lo, hi);
            if (lead) *reinterpret_cast<uint32_t*>(peers.base[p] + aoff) = sc4;
          }
      } else {
        // NVFP4: 2 lanes share a 16-element block; 8 lanes (64 elements) share one 4-byte group of scales
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        const uint8_t sf8 = to_e4m3(am / 6.f * genc);
        const float sf = from_e4m3(sf8);
        const float enc = sf > 0.f ? genc / sf : 0.f;
        uint32_t q = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) q |= static_cast<uint32_t>(to_e2m1(f[j] * enc)) << (4 * j);
        uint32_t sc4 = sf8;
        sc4 |= static_cast<uint32_t>(__shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sf8), 2)) << 8;
        sc4 |= static_cast<uint32_t>(__shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sf8), 4)) << 16;
        sc4 |= static_cast<uint32_t>(__shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sf8), 6)) << 24;
        if (!valid) continue;
        const long long qoff = tn.val_off + ((R * tn.ld + Ccol) >> 1);
        const bool lead = (lane & 7) == 0;
        const long long aoff = tn.sf_off + atom_offset(R, Ccol >> 4, static_cast<int>(tn.ld >> 4));
#pragma unroll
        for (int p = 0; p < 8; ++p)
          if ((sg.peer_mask >> p) & 1u) {
            *reinterpret_cast<uint32_t*>(peers.base[p] + qoff) = q;
            if (lead) *reinterpret_cast<uint32_t*>(peers.base[p] + aoff) = sc4;
          }
      }
    }
  }
  // publish: every thread's peer stores are ordered before the flag by a system fence, the last CTA raises the flags
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y;
    const unsigned done = atomicAdd(counter, 1u) + 1u;
    if (done == total) {
      *counter = 0;
      __threadfence_system();
#pragma unroll
      for (int p = 0; p < 8; ++p)
        if ((flag_mask >> p) & 1u)
          wp_st_release_sys(reinterpret_cast<unsigned long long*>(peers.base[p] + peers.flag_off) + me, version);
    }
  }
}

__global__ void weight_push_wait_kernel(const unsigned long long* __restrict__ flags, unsigned src_mask,
                                        unsigned long long version, unsigned long long wait_ns, int* __restrict__ status) {
  const int p = threadIdx.x;
  if (p >= 8 || !((src_mask >> p) & 1u)) return;
  const unsigned long long t0 = globaltimer_ns();
  while (wp_ld_acquire_sys(flags + p) < version) {
    if (globaltimer_ns() - t0 > wait_ns) {
      atomicCAS(status, 0, ERR_WAIT_PEER);
      return;
    }
    __nanosleep(200);
  }
}

}  // namespace

int weight_push(const void* src, const WeightPushSeg* segs, int nseg, const WeightPushTensor* tensors, const float* amax,
                const WeightPushPeers& peers, int me, unsigned flag_mask, unsigned long long version, unsigned int* counter,
                long long total_vecs, cudaStream_t s) {
  if (nseg <= 0) return 0;
  const int gy = nseg < 8 ? nseg : 8;
  long long per_seg = (total_vecs / nseg + 255) / 256;
  int gx = static_cast<int>(per_seg < 1 ? 1 : (per_seg > 148 ? 148 : per_seg));
  weight_push_kernel<<<dim3(gx, gy), 256, 0, s>>>(static_cast<const bf16*>(src), segs, nseg, tensors, amax, peers, me, flag_mask,
                                                  version, counter);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

void weight_push_wait(const unsigned long long* flags, unsigned src_mask, unsigned long long version, double wait_ms, int* status,
                      cudaStream_t s) {
  weight_push_wait_kernel<<<1, 32, 0, s>>>(flags, src_mask, version, static_cast<unsigned long long>(wait_ms * 1e6), status);
}

}  // namespace mb
