// Low-latency expert-parallel MoE exchange for decode steps (a few rows per rank), over NVLink peer memory.
//
// Every rank keeps its own sequences (attention is data parallel) and owns E / R of the experts. With top-8 routing
// over a handful of ranks a token needs most ranks anyway, so the exchange is a gather of rows rather than a
// per-(token, expert) scatter, and the way back carries one partial sum per (token, owner) instead of one row per
// (token, expert):
//
//   send    : one CTA per local row: RMSNorm, softmax top-k of the router logits, then plain 16-byte stores of the
//             normalised row into the gather buffer `xg[me][row]` of every rank that owns one of its experts, and
//             of its expert ids and gate weights into `ig/wg[me][row]` of every rank; the last CTA raises
//             `flag_a[me]` on every peer (release, system scope).
//   plan    : one CTA: waits for the R arrival flags, then sorts the (row, k) pairs whose expert is local by expert
//             (same output as moe.cu's permutation: offsets, destination rows, row sources, 128-row GEMM tiles).
//   (permute, grouped GEMM, SwiGLU, grouped GEMM: the kernels every other MoE path uses)
//   return  : one warp per gathered row: the gate-weighted sum of this rank's expert outputs for the row, stored
//             into `yb[me][row]` of the row's source rank; the last CTA raises `flag_b[me]` on every peer.
//   combine : one CTA per local row: waits for the R return flags, adds the partial sums of the ranks that own one
//             of the row's experts (rank order, fp32) to the residual.
//
// Flags carry a device-side epoch that the kernels advance themselves, so a decode step replays from a CUDA graph.
// Every wait is bounded by `wait_ns` of the global timer; on expiry the kernel records a status code, treats the
// missing peer as having sent nothing and returns, so the context stays usable. Buffers are reused every layer
// without double buffering: a rank can only start the next layer after every owner has returned this layer's
// rows, and an owner returns them only after it has consumed its gather buffer.
//
// Reference counterpart: the DeepEP low-latency dispatch / combine the reference's expert-parallel engines use
// (scripts/run_qwen3_30b_a3b.py:331-358).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "launchers.h"

namespace mb {
namespace {

using bf16 = __nv_bfloat16;

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
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Bounded wait until the epoch half of *flag reaches `epoch`. Returns the flag (0 when the wait ran out).
__device__ __forceinline__ unsigned long long wait_flag(const unsigned long long* flag, unsigned long long epoch,
                                                        unsigned long long wait_ns, int* status, int code) {
  const unsigned long long t0 = gtimer();
  unsigned int it = 0;
  for (;;) {
    const unsigned long long v = ld_acquire_sys(flag);
    if ((v >> 32) >= epoch) return v;
    if (((++it) & 0xff) == 0 && gtimer() - t0 > wait_ns) {
      atomicCAS(status, 0, code);
      return 0ull;
    }
  }
}

// ctrl (unsigned long long): [0] send epoch, [1] plan epoch, [2] return epoch, [3] combine epoch,
//                            [4] send done counter, [5] return done counter, [6] combine done counter
constexpr int kSendThreads = 256;

__global__ void __launch_bounds__(kSendThreads)
ep_ll_send_kernel(const bf16* __restrict__ x, const bf16* __restrict__ ln_w, float eps, const float* __restrict__ logits,
                  const int* __restrict__ active, EpLLPeers peers, EpLLLayout L, int me, int T, int E, int renorm,
                  int* __restrict__ ids_out, float* __restrict__ w_out, unsigned long long* ctrl) {
  __shared__ float red[kSendThreads / 32];
  __shared__ int s_ids[16];
  __shared__ float s_w[16];
  __shared__ int s_last;
  const unsigned long long epoch = ctrl[0] + 1;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = L.K, H = L.H, R = L.R, el = E / R;
  const int vec = H / 8;
  const bool live = active == nullptr || active[row] != 0;
  // ---- normalised row, eight elements per thread per pass (H <= 8 * 256 * 4)
  uint4 raw[4];
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int c = tid + p * kSendThreads;
    raw[p] = make_uint4(0, 0, 0, 0);
    if (c < vec) {
      raw[p] = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * H)[c];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw[p]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  if (ln_w != nullptr) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kSendThreads / 32; ++w) tot += red[w];
    const float rstd = rsqrtf(tot / H + eps);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int c = tid + p * kSendThreads;
      if (c < vec) {
        const uint4 wv = reinterpret_cast<const uint4*>(ln_w)[c];
        const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
        __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&raw[p]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(b[j]);
          const float2 g = __bfloat1622float2(wb[j]);
          b[j] = __floats2bfloat162_rn(f.x * rstd * g.x, f.y * rstd * g.y);
        }
      }
    }
  }
  // ---- router: softmax over E <= 256 logits, top-k (ties to the lower index), optional renormalisation
  if (warp == 0) {
    float p[8], mx = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane + 32 * i;
      p[i] = e < E ? logits[static_cast<long long>(row) * E + e] : -FLT_MAX;
      mx = fmaxf(mx, p[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      p[i] = (lane + 32 * i) < E ? __expf(p[i] - mx) : 0.f;
      sum += p[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = (lane + 32 * i) < E ? p[i] * inv : -1.f;
    float wsum = 0.f;
    for (int k = 0; k < K; ++k) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        if (q[i] > best || (q[i] == best && e < best_e)) {
          best = q[i];
          best_e = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      if (lane == 0) {
        s_ids[k] = best_e;
        s_w[k] = best;
      }
      wsum += best;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (lane + 32 * i == best_e) q[i] = -2.f;
    }
    __syncwarp();
    if (lane < K) {
      const float r = renorm ? 1.f / fmaxf(wsum, 1e-20f) : 1.f;
      const float wv = s_w[lane] * r;
      s_w[lane] = wv;
      ids_out[static_cast<long long>(row) * K + lane] = s_ids[lane];
      w_out[static_cast<long long>(row) * K + lane] = wv;
    }
  }
  __syncthreads();
  // ---- stores: ids and weights to every rank (a padding row announces "no expert"), the row to the owners
  unsigned owners = 0;
  if (live)
    for (int k = 0; k < K; ++k) owners |= 1u << (s_ids[k] / el);
  const long long slot = static_cast<long long>(me) * L.Bm + row;
  for (int d = 0; d < R; ++d) {
    char* base = peers.base[d];
    if (tid < K) {
      reinterpret_cast<int*>(base + L.off_ig)[slot * K + tid] = live ? s_ids[tid] : -1;
      reinterpret_cast<float*>(base + L.off_wg)[slot * K + tid] = s_w[tid];
    }
    if (owners & (1u << d)) {
      uint4* dst = reinterpret_cast<uint4*>(base + L.off_xg) + slot * vec;
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const int c = tid + p * kSendThreads;
        if (c < vec) dst[c] = raw[p];
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) s_last = (atomicAdd(&ctrl[4], 1ull) == gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (tid < R)
      st_release_sys(reinterpret_cast<unsigned long long*>(peers.base[tid] + L.off_flag_a) + me,
                     (epoch << 32) | static_cast<unsigned long long>(T));
    __syncthreads();
    if (tid == 0) {
      ctrl[4] = 0;
      ctrl[0] = epoch;
    }
  }
}

// Single CTA: wait for every source, then the expert-sorted row plan of the local picks. Entry index i =
// (source * Bm + row) * K + k over the rows every source announced; rows a source did not send count as "no expert".
__global__ void __launch_bounds__(1024)
ep_ll_plan_kernel(char* __restrict__ local, EpLLLayout L, int me, int E, int max_rows, int max_tiles, int align,
                  int* __restrict__ src_rows, int* __restrict__ counts_out, int* __restrict__ offsets,
                  int* __restrict__ dest_row, int* __restrict__ row_src, int* __restrict__ tiles,
                  int* __restrict__ totals, unsigned long long* ctrl, unsigned long long wait_ns, int* status) {
  extern __shared__ int sm[];  // cnt[el], off[el+1], tstart[el+1], rows[R], sid[n]
  const int R = L.R, K = L.K, Bm = L.Bm, el = E / R;
  int* cnt = sm;
  int* off = sm + el;
  int* tstart = off + el + 1;
  int* rows = tstart + el + 1;
  int* sid = rows + R;
  const int n = R * Bm * K;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const unsigned long long epoch = ctrl[1] + 1;
  if (threadIdx.x < R) {
    const unsigned long long v = wait_flag(reinterpret_cast<const unsigned long long*>(local + L.off_flag_a) + threadIdx.x,
                                           epoch, wait_ns, status, 5);
    int r = static_cast<int>(v & 0xffffffffull);
    rows[threadIdx.x] = r < Bm ? r : Bm;
  }
  for (int i = threadIdx.x; i < el; i += blockDim.x) cnt[i] = 0;
  for (int i = threadIdx.x; i < max_rows; i += blockDim.x) row_src[i] = -1;
  __syncthreads();
  if (threadIdx.x < R) src_rows[threadIdx.x] = rows[threadIdx.x];
  const int* ig = reinterpret_cast<const int*>(local + L.off_ig);
  const int lo_e = me * el;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int s = i / (Bm * K);
    const int j = (i - s * Bm * K) / K;
    int e = -1;
    if (j < rows[s]) {
      e = __ldcg(ig + i) - lo_e;  // written by a peer: read past L1
      if (e < 0 || e >= el) e = -1;
    }
    sid[i] = e;
    if (e >= 0) atomicAdd(&cnt[e], 1);
    dest_row[i] = -1;
  }
  __syncthreads();
  if (warp == 0) {
    // exclusive scans by one warp (lane l owns experts [l*per, (l+1)*per)): padded row offsets clamped to the
    // capacity, then the 128-row tile starts of the clamped ranges
    const int per = (el + 31) / 32;
    const int e0 = min(el, lane * per), e1 = min(el, e0 + per);
    const int cap = (max_rows / align) * align;
    int local_rows = 0;
    for (int e = e0; e < e1; ++e) local_rows += ((cnt[e] + align - 1) / align) * align;
    int incl = local_rows;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - local_rows;
    int tl = 0;
    for (int e = e0; e < e1; ++e) {
      const int s0 = min(run, cap);
      run += ((cnt[e] + align - 1) / align) * align;
      const int s1 = min(run, cap);
      off[e] = s0;
      tl += (s1 - s0 + 127) / 128;
      tstart[e] = s1 - s0;
    }
    const int total_rows = min(__shfl_sync(0xffffffffu, incl, 31), cap);
    int tincl = tl;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, tincl, o);
      if (lane >= o) tincl += v;
    }
    int trun = tincl - tl;
    for (int e = e0; e < e1; ++e) {
      const int r = tstart[e];
      tstart[e] = trun;
      trun += (r + 127) / 128;
    }
    const int total_tiles = __shfl_sync(0xffffffffu, tincl, 31);
    if (lane == 0) {
      off[el] = total_rows;
      tstart[el] = total_tiles < max_tiles ? total_tiles : max_tiles;
      totals[0] = tstart[el];
      totals[1] = total_rows;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= el; e += blockDim.x) {
    offsets[e] = off[e];
    if (e < el) counts_out[e] = cnt[e];
  }
  for (int e = warp; e < el; e += nwarps) {
    const int rows_e = off[e + 1] - off[e];
    for (int j = lane; tstart[e] + j < tstart[e + 1] && tstart[e] + j < max_tiles; j += 32) {
      int* t = tiles + 4 * (tstart[e] + j);
      t[0] = e;
      t[1] = off[e] + 128 * j;
      t[2] = min(128, rows_e - 128 * j);
      t[3] = 0;
    }
    if (cnt[e] == 0) continue;
    int base = 0;
    for (int s = 0; s < R && base < cnt[e]; ++s) {
      const int lim = rows[s] * K;  // entries of source s that can hold an expert
      const int first = s * Bm * K;
      for (int start = 0; start < lim; start += 32) {
        const int i = first + start + lane;
        const bool hit = start + lane < lim && sid[i] == e;
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (hit) {
          const int rank = base + __popc(m & ((1u << lane) - 1u));
          if (rank < rows_e) {
            dest_row[i] = off[e] + rank;
            row_src[off[e] + rank] = i;
          }
        }
        base += __popc(m);
      }
    }
  }
  if (threadIdx.x == 0) ctrl[1] = epoch;
}

// One warp per gathered row: partial = sum over the local picks of gate weight x expert output, stored at the source.
__global__ void __launch_bounds__(256)
ep_ll_return_kernel(const bf16* __restrict__ yp, const int* __restrict__ dest_row, const int* __restrict__ src_rows,
                    EpLLPeers peers, EpLLLayout L, int me, unsigned long long* ctrl) {
  __shared__ int s_last;
  const unsigned long long epoch = ctrl[2] + 1;
  const int R = L.R, K = L.K, Bm = L.Bm, H = L.H;
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int vec = H / 8;
  const char* local = peers.base[me];
  const float* wg = reinterpret_cast<const float*>(local + L.off_wg);
  for (int g = blockIdx.x * wpb + (threadIdx.x >> 5); g < R * Bm; g += gridDim.x * wpb) {
    const int s = g / Bm, j = g - s * Bm;
    if (j >= src_rows[s]) continue;
    int dr[16];
    float wk[16];
    int any = 0;
    for (int k = 0; k < K; ++k) {
      dr[k] = dest_row[g * K + k];
      wk[k] = dr[k] >= 0 ? __ldcg(wg + g * K + k) : 0.f;
      any |= dr[k] >= 0;
    }
    if (!any) continue;
    uint4* dst = reinterpret_cast<uint4*>(peers.base[s] + L.off_yb) + (static_cast<long long>(me) * Bm + j) * vec;
    for (int c = lane; c < vec; c += 32) {
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      for (int k = 0; k < K; ++k) {
        if (dr[k] < 0) continue;
        const uint4 v = reinterpret_cast<const uint4*>(yp + static_cast<long long>(dr[k]) * H)[c];
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(b[q]);
          acc[2 * q] += wk[k] * f.x;
          acc[2 * q + 1] += wk[k] * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) ob[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      dst[c] = o;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&ctrl[5], 1ull) == gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < R)
      st_release_sys(reinterpret_cast<unsigned long long*>(peers.base[threadIdx.x] + L.off_flag_b) + me, epoch << 32);
    __syncthreads();
    if (threadIdx.x == 0) {
      ctrl[5] = 0;
      ctrl[2] = epoch;
    }
  }
}

// One CTA per local row: out = residual + sum over owner ranks (rank order) of their partial sums.
__global__ void __launch_bounds__(kSendThreads)
ep_ll_combine_kernel(const char* __restrict__ local, EpLLLayout L, const int* __restrict__ ids, const int* __restrict__ active,
                     const bf16* __restrict__ residual, bf16* __restrict__ out, int E, unsigned long long* ctrl,
                     unsigned long long wait_ns, int* status) {
  __shared__ unsigned s_ok;
  __shared__ int s_last;
  const unsigned long long epoch = ctrl[3] + 1;
  const int row = blockIdx.x, tid = threadIdx.x;
  const int R = L.R, K = L.K, Bm = L.Bm, H = L.H, el = E / R;
  const int vec = H / 8;
  if (tid == 0) s_ok = 0;
  __syncthreads();
  if (tid < R) {
    const unsigned long long v = wait_flag(reinterpret_cast<const unsigned long long*>(local + L.off_flag_b) + tid, epoch,
                                           wait_ns, status, 6);
    if (v != 0ull) atomicOr(&s_ok, 1u << tid);
  }
  __syncthreads();
  unsigned owners = 0;
  if (active == nullptr || active[row] != 0)
    for (int k = 0; k < K; ++k) owners |= 1u << (ids[static_cast<long long>(row) * K + k] / el);
  owners &= s_ok;  // a peer that never answered contributes nothing (status 6 is set)
  const uint4* yb = reinterpret_cast<const uint4*>(local + L.off_yb);
  for (int c = tid; c < vec; c += kSendThreads) {
    float acc[8];
    {
      const uint4 v = reinterpret_cast<const uint4*>(residual + static_cast<long long>(row) * H)[c];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(b[q]);
        acc[2 * q] = f.x;
        acc[2 * q + 1] = f.y;
      }
    }
    for (int d = 0; d < R; ++d) {
      if (!(owners & (1u << d))) continue;
      const uint4 v = __ldcg(yb + (static_cast<long long>(d) * Bm + row) * vec + c);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(b[q]);
        acc[2 * q] += f.x;
        acc[2 * q + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) ob[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    reinterpret_cast<uint4*>(out + static_cast<long long>(row) * H)[c] = o;
  }
  __syncthreads();
  if (tid == 0) s_last = (atomicAdd(&ctrl[6], 1ull) == gridDim.x - 1);
  __syncthreads();
  if (s_last && tid == 0) {
    ctrl[6] = 0;
    ctrl[3] = epoch;
  }
}

}  // namespace

size_t ep_ll_plan_smem(const EpLLLayout& L, int E) {
  const int el = E / L.R;
  return sizeof(int) * (static_cast<size_t>(el) + 2 * (el + 1) + L.R + static_cast<size_t>(L.R) * L.Bm * L.K);
}

int ep_ll_send(const void* x, const void* ln_w, float eps, const float* logits, const int* active, const EpLLPeers& peers,
               const EpLLLayout& L, int me, int T, int E, bool renorm, int* ids_out, float* w_out, unsigned long long* ctrl,
               cudaStream_t s) {
  if (T <= 0 || T > L.Bm || L.K > 16 || E > 256 || L.H % 8 != 0 || L.H > 8 * kSendThreads * 4 || E % L.R != 0) return 1;
  ep_ll_send_kernel<<<T, kSendThreads, 0, s>>>(static_cast<const bf16*>(x), static_cast<const bf16*>(ln_w), eps, logits, active,
                                               peers, L, me, T, E, renorm ? 1 : 0, ids_out, w_out, ctrl);
  return 0;
}

int ep_ll_plan(char* local, const EpLLLayout& L, int me, int E, int max_rows, int max_tiles, int align, int* src_rows,
               int* counts, int* offsets, int* dest_row, int* row_src, int* tiles, int* totals, unsigned long long* ctrl,
               unsigned long long wait_ns, int* status, cudaStream_t s) {
  const size_t smem = ep_ll_plan_smem(L, E);
  if (smem > 200 * 1024) return 1;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(ep_ll_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  ep_ll_plan_kernel<<<1, 1024, smem, s>>>(local, L, me, E, max_rows, max_tiles, align, src_rows, counts, offsets, dest_row,
                                          row_src, tiles, totals, ctrl, wait_ns, status);
  return 0;
}

void ep_ll_return(const void* yp, const int* dest_row, const int* src_rows, const EpLLPeers& peers, const EpLLLayout& L, int me,
                  int rows_hint, unsigned long long* ctrl, cudaStream_t s) {
  int blocks = (L.R * (rows_hint > 0 ? rows_hint : L.Bm) + 7) / 8;
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (blocks < 1) blocks = 1;
  ep_ll_return_kernel<<<blocks, 256, 0, s>>>(static_cast<const bf16*>(yp), dest_row, src_rows, peers, L, me, ctrl);
}

void ep_ll_combine(const char* local, const EpLLLayout& L, const int* ids, const int* active, const void* residual, void* out,
                   int T, int E, unsigned long long* ctrl, unsigned long long wait_ns, int* status, cudaStream_t s) {
  if (T <= 0) return;
  ep_ll_combine_kernel<<<T, kSendThreads, 0, s>>>(local, L, ids, active, static_cast<const bf16*>(residual),
                                                  static_cast<bf16*>(out), E, ctrl, wait_ns, status);
}

}  // namespace mb
