// Expert-parallel token exchange over NVLink peer memory (no NCCL on this path).
//
// Every rank owns two symmetric regions that all peers map: a receive region
// `xrecv[src][cap][H]` (+ per-row metadata, per-source row counts and arrival flags) into which the
// *senders* store routed token rows with plain 16-byte P2P stores, and a return region `yback[T*K][H]`
// into which the expert owners store the processed rows of this rank's (token, slot) pairs.
//
//   dispatch : for each (token, slot) -> owner rank d, position p (stable rank among the entries bound for
//              d): store the row into peer d's xrecv[me][p], its metadata (local expert, source slot), and
//              finally — from the last CTA to finish, after a system-scope fence — the row count and the
//              arrival flag of this epoch.
//   wait     : spin (bounded, acquire loads) until the flags of all sources reach this epoch.
//   return   : the owner stores row j of its result into the source's yback[slot] and raises the return flag.
//
// Epoch counters live in device memory and are advanced by the kernels themselves, so the sequence can
// be captured in a CUDA graph and replayed. All waits are bounded; on expiry a status word is set and
// the kernel returns.
//
// Reference counterpart: Megatron's all-to-all token dispatcher over NCCL
// (forced in miles/utils/arguments.py:2715-2720; DeepEP is the optional fused backend,
// scripts/run_qwen3_30b_a3b.py:331-358).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "launchers.h"

namespace mb {
namespace {

constexpr unsigned long long kWaitNs = 5000000000ull;  // 5 s

__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// ctrl layout (unsigned long long): [0] send epoch, [1] wait epoch, [2] return-send epoch, [3] return-wait epoch,
//                                   [4] done counter (dispatch), [5] done counter (return)
__global__ void ep_dispatch_kernel(const uint4* __restrict__ x, const int* __restrict__ ids,
                                   const int* __restrict__ dest_row, const int* __restrict__ offsets, EpPeers peers,
                                   int me, int nranks, int experts_per_rank, int n_entries, int row_div, int vec_per_row,
                                   int cap, unsigned long long* ctrl, int* status) {
  const unsigned long long epoch = ctrl[0] + 1;
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < n_entries; i += gridDim.x * wpb) {
    const int e = ids[i];
    if (e < 0) continue;
    const int d = e / experts_per_rank;
    if (d >= nranks) continue;
    const int pos = dest_row[i] - offsets[d];
    if (pos < 0 || pos >= cap) {
      if (lane == 0) atomicCAS(status, 0, 7);  // capacity overflow
      continue;
    }
    const uint4* src = x + static_cast<long long>(i / row_div) * vec_per_row;
    uint4* dst = reinterpret_cast<uint4*>(peers.xrecv[d]) + (static_cast<long long>(me) * cap + pos) * vec_per_row;
    for (int c = lane; c < vec_per_row; c += 32) dst[c] = src[c];
    if (lane == 0) {
      int2 m;
      m.x = e - d * experts_per_rank;
      m.y = i;
      reinterpret_cast<int2*>(peers.meta[d])[static_cast<long long>(me) * cap + pos] = m;
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    const unsigned long long done = atomicAdd(&ctrl[4], 1ull);
    is_last = (done == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence_system();
    if (threadIdx.x < nranks) {
      const int d = threadIdx.x;
      int cnt = offsets[d + 1] - offsets[d];
      // offsets are padded to 128; the true count is the number of entries bound for d
      cnt = peers.send_counts ? peers.send_counts[d] : cnt;
      peers.counts[d][me] = cnt < cap ? cnt : cap;
      __threadfence_system();
      st_release_sys(peers.flags[d] + me, epoch);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      ctrl[4] = 0;
      ctrl[0] = epoch;
    }
  }
}

__global__ void ep_wait_kernel(const unsigned long long* __restrict__ flags, int nranks, unsigned long long* ctrl,
                               int which, int* status) {
  const unsigned long long epoch = ctrl[which] + 1;
  if (threadIdx.x < nranks) {
    const unsigned long long t0 = gtimer();
    unsigned int it = 0;
    while (ld_acquire_sys(flags + threadIdx.x) < epoch) {
      if (((++it) & 0x3ff) == 0 && gtimer() - t0 > kWaitNs) {
        atomicCAS(status, 0, 5);  // a peer never arrived
        break;
      }
    }
  }
  __syncthreads();
  __threadfence_system();
  if (threadIdx.x == 0) ctrl[which] = epoch;
}

// Owner side: row j of the receive region (valid when its permuted row >= 0) goes back to its source.
__global__ void ep_return_kernel(const uint4* __restrict__ yp, const int* __restrict__ recv_dest_row,
                                 const int2* __restrict__ meta, const int* __restrict__ counts, EpPeers peers, int me,
                                 int nranks, int cap, int vec_per_row, unsigned long long* ctrl, int* status) {
  const unsigned long long epoch = ctrl[2] + 1;
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(nranks) * cap;
  for (long long j = blockIdx.x * wpb + (threadIdx.x >> 5); j < total; j += static_cast<long long>(gridDim.x) * wpb) {
    const int src = j / cap;
    const int pos = j - static_cast<long long>(src) * cap;
    if (pos >= counts[src]) continue;
    const int row = recv_dest_row[j];
    if (row < 0) continue;
    const int slot = meta[j].y;
    const uint4* s = yp + static_cast<long long>(row) * vec_per_row;
    uint4* d = reinterpret_cast<uint4*>(peers.yback[src]) + static_cast<long long>(slot) * vec_per_row;
    for (int c = lane; c < vec_per_row; c += 32) d[c] = s[c];
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    const unsigned long long done = atomicAdd(&ctrl[5], 1ull);
    is_last = (done == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence_system();
    if (threadIdx.x < nranks) st_release_sys(peers.flags2[threadIdx.x] + me, epoch);
    __syncthreads();
    if (threadIdx.x == 0) {
      ctrl[5] = 0;
      ctrl[2] = epoch;
    }
  }
}

// Destination address of every expert-sorted row: row r holds receive-slot j = row_src[r] (source rank j / cap),
// whose result belongs at yback[source][meta[j].y]. 0 marks padding rows. The grouped GEMM that produces the rows
// stores them there directly (its epilogue is the return transfer).
__global__ void ep_row_ptrs_kernel(const int* __restrict__ row_src, const int2* __restrict__ meta, EpPeers peers, int cap,
                                   long long row_bytes, int max_rows, unsigned long long* __restrict__ out) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= max_rows) return;
  const int j = row_src[r];
  unsigned long long p = 0ull;
  if (j >= 0) {
    const int src = j / cap;
    p = reinterpret_cast<unsigned long long>(peers.yback[src]) + static_cast<unsigned long long>(meta[j].y) * row_bytes;
  }
  out[r] = p;
}

// out[i] = (residual[i] +) sum_d slots[d][i] in fp32, slots d = 0..n-1 at stride `slot_elems` (the tensor-parallel
// partial sums pushed by the peers' GEMM epilogues). Fixed summation order: every rank gets bit-identical results.
__global__ void sum_slots_kernel(const uint4* __restrict__ slots, long long slot_vecs, int n, const uint4* __restrict__ residual,
                                 uint4* __restrict__ out, long long vecs) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int d = 0; d < n; ++d) {
      const uint4 v = slots[d * slot_vecs + i];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (residual) {
      const uint4 v = residual[i];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    out[i] = o;
  }
}

}  // namespace

void sum_slots(const void* slots, long long slot_elems, int n, const void* residual, void* out, long long elems,
               cudaStream_t s) {
  const long long vecs = elems / 8;
  if (vecs <= 0) return;
  long long blocks = (vecs + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  sum_slots_kernel<<<static_cast<int>(blocks), 256, 0, s>>>(static_cast<const uint4*>(slots), slot_elems / 8, n,
                                                            static_cast<const uint4*>(residual), static_cast<uint4*>(out), vecs);
}

void ep_row_ptrs(const int* row_src, const int* meta, const EpPeers& peers, int cap, int H, int max_rows,
                 unsigned long long* out, cudaStream_t s) {
  if (max_rows <= 0) return;
  ep_row_ptrs_kernel<<<(max_rows + 255) / 256, 256, 0, s>>>(row_src, reinterpret_cast<const int2*>(meta), peers, cap,
                                                            static_cast<long long>(H) * 2, max_rows, out);
}

void ep_dispatch(const void* x, const int* ids, const int* dest_row, const int* offsets, const EpPeers& peers, int me,
                 int nranks, int experts_per_rank, int n_entries, int row_div, int H, int cap, unsigned long long* ctrl,
                 int* status, cudaStream_t s) {
  const int wpb = 8;
  int blocks = (n_entries + wpb - 1) / wpb;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 4) blocks = 148 * 4;
  ep_dispatch_kernel<<<blocks, wpb * 32, 0, s>>>(static_cast<const uint4*>(x), ids, dest_row, offsets, peers, me, nranks,
                                                 experts_per_rank, n_entries, row_div, H / 8, cap, ctrl, status);
}

void ep_wait(const unsigned long long* flags, int nranks, unsigned long long* ctrl, int which, int* status, cudaStream_t s) {
  ep_wait_kernel<<<1, 32, 0, s>>>(flags, nranks, ctrl, which, status);
}

void ep_return(const void* yp, const int* recv_dest_row, const int* meta, const int* counts, const EpPeers& peers, int me,
               int nranks, int cap, int H, unsigned long long* ctrl, int* status, cudaStream_t s) {
  const int wpb = 8;
  long long rows = static_cast<long long>(nranks) * cap;
  long long blocks = (rows + wpb - 1) / wpb;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  ep_return_kernel<<<static_cast<int>(blocks), wpb * 32, 0, s>>>(static_cast<const uint4*>(yp), recv_dest_row,
                                                                reinterpret_cast<const int2*>(meta), counts, peers, me,
                                                                nranks, cap, H / 8, ctrl, status);
}

// ---------------------------------------------------------------------- symmetric allocations (CUDA IPC)
int symm_alloc(size_t nbytes, void** ptr, char* handle64) {
  cudaError_t e = cudaMalloc(ptr, nbytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaMemset(*ptr, 0, nbytes);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) return static_cast<int>(e);
  static_assert(sizeof(h) == 64, "unexpected IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
int symm_open(const char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
int symm_close(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }
int symm_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }

}  // namespace mb
