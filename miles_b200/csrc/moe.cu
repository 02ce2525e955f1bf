// MoE routing and token permutation kernels.
//
//   router_topk        : softmax over E experts, top-k (k <= 8), optional renormalisation; with a replay
//                        table the expert choice comes from the rollout engine (rollout routing replay)
//                        and only the gate weights are recomputed from the current logits.
//   build_permutation  : deterministic counting sort of (token, slot) pairs by expert; each expert's rows
//                        are padded to a multiple of `align` (64 for training so that the weight-gradient
//                        contraction blocks stay inside one expert, 1 for inference) and cut into GEMM row
//                        tiles of at most 128 rows that never straddle experts.
//   permute / combine  : gather rows into expert order / weighted gather-sum back to token order, with
//                        their backward passes. All gathers are index-driven (no atomics), so results are
//                        bitwise reproducible.
//
// Reference counterparts: Megatron TopKRouter + token dispatcher (scripts/models/qwen3-30B-A3B.py:29-41),
// the replay hook in miles/utils/replay_base.py:14-237 and the Triton fused-MoE align/sort stage in
// miles/backends/fsdp_utils/kernels/fused_experts.py:15-379.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "launchers.h"

namespace mb {
namespace {

using bf16 = __nv_bfloat16;
constexpr int kMaxK = 16;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per token, E <= 256 (8 values per lane).
__global__ void router_topk_kernel(const float* __restrict__ logits, const int* __restrict__ replay_ids,
                                   int* __restrict__ topk_ids, float* __restrict__ topk_w,
                                   float* __restrict__ probs_out, int T, int E, int K, int renorm) {
  const int wpb = blockDim.x >> 5;
  const int t = blockIdx.x * wpb + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float p[8];
  float mx = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? logits[static_cast<long long>(t) * E + e] : -FLT_MAX;
    mx = fmaxf(mx, p[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? __expf(p[i] - mx) : 0.f;
    sum += p[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    p[i] *= inv;
    const int e = lane + 32 * i;
    if (probs_out && e < E) probs_out[static_cast<long long>(t) * E + e] = p[i];
  }
  int ids[kMaxK];
  float ws[kMaxK];
  if (replay_ids) {
    for (int k = 0; k < K; ++k) {
      int e = replay_ids[static_cast<long long>(t) * K + k];
      e = (e < 0 || e >= E) ? 0 : e;
      // fetch p[e] from the owning lane
      const int owner = e & 31, slot = e >> 5;
      float v = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (slot == i) v = p[i];
      ids[k] = e;
      ws[k] = __shfl_sync(0xffffffffu, v, owner);
    }
  } else {
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = (lane + 32 * i) < E ? p[i] : -1.f;
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
      ids[k] = best_e;
      ws[k] = best;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (lane + 32 * i == best_e) q[i] = -2.f;
    }
  }
  if (renorm) {
    float s = 0.f;
    for (int k = 0; k < K; ++k) s += ws[k];
    const float r = 1.f / fmaxf(s, 1e-20f);
    for (int k = 0; k < K; ++k) ws[k] *= r;
  }
  if (lane == 0) {
    for (int k = 0; k < K; ++k) {
      topk_ids[static_cast<long long>(t) * K + k] = ids[k];
      topk_w[static_cast<long long>(t) * K + k] = ws[k];
    }
  }
}

// dlogits for: p = softmax(logits); w_k = p[id_k] (/ sum_j p[id_j] when renorm).
__global__ void router_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ topk_ids,
                                  const float* __restrict__ topk_w, const float* __restrict__ dtopk_w,
                                  float* __restrict__ dlogits, int T, int E, int K, int renorm) {
  const int wpb = blockDim.x >> 5;
  const int t = blockIdx.x * wpb + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  // dL/dp[e] for the selected experts
  float dp[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float s_sel = 1.f, dot = 0.f;
  if (renorm) {
    s_sel = 0.f;
    for (int k = 0; k < K; ++k) {
      const int e = topk_ids[static_cast<long long>(t) * K + k];
      s_sel += probs[static_cast<long long>(t) * E + e];
      dot += dtopk_w[static_cast<long long>(t) * K + k] * topk_w[static_cast<long long>(t) * K + k];
    }
    s_sel = fmaxf(s_sel, 1e-20f);
  }
  for (int k = 0; k < K; ++k) {
    const int e = topk_ids[static_cast<long long>(t) * K + k];
    const float g = dtopk_w[static_cast<long long>(t) * K + k];
    const float v = renorm ? (g - dot) / s_sel : g;  // d w_k / d p_j = (delta_kj - w_k) / s
    if ((e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if ((e >> 5) == i) dp[i] += v;
    }
  }
  // softmax backward: dlogit = p * (dp - sum_j p_j dp_j)
  float pv[8];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    pv[i] = e < E ? probs[static_cast<long long>(t) * E + e] : 0.f;
    acc += pv[i] * dp[i];
  }
  acc = warp_sum(acc);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    if (e < E) dlogits[static_cast<long long>(t) * E + e] = pv[i] * (dp[i] - acc);
  }
}

// ---------------------------------------------------------------- permutation
// Pass 1: one CTA per expert counts its entries.
__global__ void count_kernel(const int* __restrict__ ids, int n, int* __restrict__ counts) {
  __shared__ int red[32];
  const int e = blockIdx.x;
  int c = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) c += (ids[i] == e);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x < 32) {
    int v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) counts[e] = v;
  }
}

// Pass 2: single CTA: exclusive scan of the per-expert row counts padded to `align`, the list of GEMM row
// tiles (expert, first row, rows to compute; a tile never straddles experts and is at most 128 rows), the
// number of tiles and the number of live rows. tiles[t] = {expert, row0, rows, 0}; totals = {num tiles, live rows}.
__global__ void scan_kernel(const int* __restrict__ counts, int E, int max_rows, int max_tiles, int align,
                            int* __restrict__ offsets, int* __restrict__ tiles, int* __restrict__ totals) {
  extern __shared__ int tile_start[];  // [E+1]
  if (threadIdx.x == 0) {
    int off = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = off;
      tile_start[e] = t;
      int padded = ((counts[e] + align - 1) / align) * align;
      if (off + padded > max_rows) padded = max_rows - off > 0 ? ((max_rows - off) / align) * align : 0;
      off += padded;
      t += (padded + 127) / 128;
    }
    offsets[E] = off;
    tile_start[E] = t < max_tiles ? t : max_tiles;
    totals[0] = tile_start[E];
    totals[1] = off;
  }
  __syncthreads();
  for (int e = 0; e < E; ++e) {
    const int rows_e = offsets[e + 1] - offsets[e];
    for (int j = threadIdx.x; tile_start[e] + j < tile_start[e + 1] && tile_start[e] + j < max_tiles; j += blockDim.x) {
      int* t = tiles + 4 * (tile_start[e] + j);
      t[0] = e;
      t[1] = offsets[e] + 128 * j;
      t[2] = min(128, rows_e - 128 * j);
      t[3] = 0;
    }
  }
}

// Pass 3: one CTA per expert assigns stable ranks (ascending entry index) to its entries.
__global__ void assign_kernel(const int* __restrict__ ids, int n, const int* __restrict__ offsets,
                              int* __restrict__ dest_row, int* __restrict__ row_src) {
  __shared__ int warp_tot[32];
  __shared__ int base_s;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (threadIdx.x == 0) base_s = 0;
  __syncthreads();
  const int cap = offsets[e + 1] - offsets[e];
  for (int start = 0; start < n; start += blockDim.x) {
    const int i = start + threadIdx.x;
    const bool hit = i < n && ids[i] == e;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    const int in_warp = __popc(m & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[w] = __popc(m);
    __syncthreads();
    int before = 0;
    for (int j = 0; j < w; ++j) before += warp_tot[j];
    const int rank = base_s + before + in_warp;
    if (hit) {
      if (rank < cap) {
        dest_row[i] = offsets[e] + rank;
        row_src[offsets[e] + rank] = i;
      } else {
        dest_row[i] = -1;  // capacity overflow: dropped (only if max_rows was under-provisioned)
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int j = 0; j < nw; ++j) tot += warp_tot[j];
      base_s += tot;
    }
    __syncthreads();
  }
}

// Single-CTA variant for small problems (decode steps): counts, scan, tile list and the stable assignment
// in one launch. Also initialises row_src / dest_row, so the caller needs no memset or fill kernels.
__global__ void __launch_bounds__(1024)
build_small_kernel(const int* __restrict__ ids, int n, int E, int max_rows, int max_tiles, int align,
                   int* __restrict__ counts_out, int* __restrict__ offsets, int* __restrict__ dest_row,
                   int* __restrict__ row_src, int* __restrict__ tiles, int* __restrict__ totals) {
  extern __shared__ int sm[];  // counts[E], off[E+1], tile_start[E+1], ids[n]
  int* cnt = sm;
  int* off = sm + E;
  int* tstart = off + E + 1;
  int* sid = tstart + E + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < E; i += blockDim.x) cnt[i] = 0;
  for (int i = threadIdx.x; i < max_rows; i += blockDim.x) row_src[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {  // the only global read of the ids
    const int e = ids[i];
    sid[i] = e;
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    else dest_row[i] = -1;
  }
  __syncthreads();
  if (warp == 0) {
    // Exclusive scans by one warp: lane l owns experts [l*per, (l+1)*per). First the padded row offsets, clamped to
    // the capacity (offsets are multiples of `align`, so clamping both ends of an expert's range equals shrinking the
    // expert that overflows and giving the later ones nothing), then the 128-row tile starts of the clamped ranges.
    const int per = (E + 31) / 32;
    const int e0 = lane * per, e1 = min(E, e0 + per);
    const int cap = (max_rows / align) * align;
    int local = 0;
    for (int e = e0; e < e1; ++e) local += ((cnt[e] + align - 1) / align) * align;
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - local;
    int tl = 0;
    for (int e = e0; e < e1; ++e) {
      const int s0 = min(run, cap);
      run += ((cnt[e] + align - 1) / align) * align;
      const int s1 = min(run, cap);
      off[e] = s0;
      tl += (s1 - s0 + 127) / 128;
      tstart[e] = s1 - s0;  // rows of the expert for now; turned into a tile start below
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
      const int rows = tstart[e];
      tstart[e] = trun;
      trun += (rows + 127) / 128;
    }
    const int total_tiles = __shfl_sync(0xffffffffu, tincl, 31);
    if (lane == 0) {
      off[E] = total_rows;
      tstart[E] = total_tiles < max_tiles ? total_tiles : max_tiles;
      totals[0] = tstart[E];
      totals[1] = total_rows;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = off[e];
    if (e < E) counts_out[e] = cnt[e];
  }
  // tiles and stable ranks: one warp per expert, ids read from shared memory
  for (int e = warp; e < E; e += nwarps) {
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
    for (int start = 0; start < n; start += 32) {
      const int i = start + lane;
      const bool hit = i < n && sid[i] == e;
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int rank = base + __popc(m & ((1u << lane) - 1u));
        if (rank < rows_e) {
          dest_row[i] = off[e] + rank;
          row_src[off[e] + rank] = i;
        } else {
          dest_row[i] = -1;
        }
      }
      base += __popc(m);
      if (base >= cnt[e]) break;  // all entries of this expert placed (warp-uniform)
    }
  }
}

struct alignas(16) V8 {
  uint4 v;
};

// x_perm[row] = x[row_src[row] / K] or zeros for padding rows. One warp per row chunk.
__global__ void permute_kernel(const bf16* __restrict__ x, const int* __restrict__ row_src,
                               const int* __restrict__ num_m_tiles, bf16* __restrict__ x_perm, int max_rows, int H,
                               int K) {
  const int live_rows = min(num_m_tiles[1], max_rows);
  const int vec_per_row = H / 8;
  const long long total = static_cast<long long>(live_rows) * vec_per_row;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = idx / vec_per_row;
    const int c = idx - static_cast<long long>(row) * vec_per_row;
    const int src = row_src[row];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (src >= 0) v = reinterpret_cast<const uint4*>(x + static_cast<long long>(src / K) * H)[c];
    reinterpret_cast<uint4*>(x_perm + static_cast<long long>(row) * H)[c] = v;
  }
}

__device__ __forceinline__ void acc8(const uint4& raw, float w, float (&a)[8]) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(b[i]);
    a[2 * i] += w * f.x;
    a[2 * i + 1] += w * f.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&a)[8]) {
  uint4 r;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn(a[0], a[1]); r.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(a[2], a[3]); r.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(a[4], a[5]); r.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(a[6], a[7]); r.w = *reinterpret_cast<uint32_t*>(&t);
  return r;
}

// out[t] = sum_k w[t,k] * y_perm[dest_row[t,k]]; with w == nullptr the weights are 1 (permute backward).
__global__ void combine_kernel(const bf16* __restrict__ y_perm, const int* __restrict__ dest_row,
                               const float* __restrict__ topk_w, const bf16* __restrict__ residual,
                               bf16* __restrict__ out, int T, int K, int H) {
  const int vec_per_row = H / 8;
  const long long total = static_cast<long long>(T) * vec_per_row;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = idx / vec_per_row;
    const int c = idx - static_cast<long long>(t) * vec_per_row;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (residual) acc8(reinterpret_cast<const uint4*>(residual + static_cast<long long>(t) * H)[c], 1.f, a);
    for (int k = 0; k < K; ++k) {
      const int row = dest_row[static_cast<long long>(t) * K + k];
      if (row < 0) continue;
      const float w = topk_w ? topk_w[static_cast<long long>(t) * K + k] : 1.f;
      acc8(reinterpret_cast<const uint4*>(y_perm + static_cast<long long>(row) * H)[c], w, a);
    }
    reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H)[c] = pack8(a);
  }
}

// One warp per permuted row: dy_perm[row] = w * dout[token]; dw[entry] = <dout[token], y_perm[row]>.
__global__ void combine_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ y_perm,
                                   const int* __restrict__ row_src, const int* __restrict__ num_m_tiles,
                                   const float* __restrict__ topk_w, bf16* __restrict__ dy_perm,
                                   float* __restrict__ dtopk_w, int max_rows, int K, int H) {
  const int live_rows = min(num_m_tiles[1], max_rows);
  const int wpb = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < live_rows; row += gridDim.x * wpb) {
    const int src = row_src[row];
    uint4* dst = reinterpret_cast<uint4*>(dy_perm + static_cast<long long>(row) * H);
    if (src < 0) {
      for (int c = lane; c < H / 8; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const float w = topk_w[src];
    const uint4* g = reinterpret_cast<const uint4*>(dout + static_cast<long long>(src / K) * H);
    const uint4* y = reinterpret_cast<const uint4*>(y_perm + static_cast<long long>(row) * H);
    float dot = 0.f;
    for (int c = lane; c < H / 8; c += 32) {
      const uint4 gr = g[c];
      float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      acc8(gr, w, a);
      dst[c] = pack8(a);
      if (dtopk_w) {
        const uint4 yr = y[c];
        const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gr);
        const __nv_bfloat162* yb = reinterpret_cast<const __nv_bfloat162*>(&yr);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 gf = __bfloat1622float2(gb[i]), yf = __bfloat1622float2(yb[i]);
          dot += gf.x * yf.x + gf.y * yf.y;
        }
      }
    }
    if (dtopk_w) {
      dot = warp_sum(dot);
      if (lane == 0) dtopk_w[src] = dot;
    }
  }
}

int grid_for(long long items, int threads, int cap = 148 * 8) {
  long long b = (items + threads - 1) / threads;
  if (b < 1) b = 1;
  return static_cast<int>(b < cap ? b : cap);
}

}  // namespace

void moe_router_topk(const float* logits, const int* replay_ids, int* topk_ids, float* topk_w, float* probs_out,
                     int T, int E, int K, bool renorm, cudaStream_t s) {
  if (T <= 0) return;
  const int wpb = 4;
  router_topk_kernel<<<(T + wpb - 1) / wpb, wpb * 32, 0, s>>>(logits, replay_ids, topk_ids, topk_w, probs_out, T, E, K,
                                                              renorm ? 1 : 0);
}

void moe_router_bwd(const float* probs, const int* topk_ids, const float* topk_w, const float* dtopk_w, float* dlogits,
                    int T, int E, int K, bool renorm, cudaStream_t s) {
  if (T <= 0) return;
  const int wpb = 4;
  router_bwd_kernel<<<(T + wpb - 1) / wpb, wpb * 32, 0, s>>>(probs, topk_ids, topk_w, dtopk_w, dlogits, T, E, K,
                                                             renorm ? 1 : 0);
}

void moe_build_permutation(const int* topk_ids, int T, int K, int E, int max_rows, int max_tiles, int align,
                           int* expert_counts, int* expert_offsets, int* dest_row, int* row_src, int* tile_group,
                           int* num_m_tiles, cudaStream_t s) {
  const int n = T * K;
  if (n <= 4096 && max_rows <= 16384 && E <= 512) {
    build_small_kernel<<<1, n <= 128 ? 256 : 1024, (3 * E + 2 + n) * sizeof(int), s>>>(topk_ids, n, E, max_rows, max_tiles, align, expert_counts,
                                                                   expert_offsets, dest_row, row_src, tile_group, num_m_tiles);
    return;
  }
  cudaMemsetAsync(dest_row, 0xff, sizeof(int) * static_cast<size_t>(n), s);
  cudaMemsetAsync(row_src, 0xff, sizeof(int) * static_cast<size_t>(max_rows), s);
  count_kernel<<<E, 512, 0, s>>>(topk_ids, n, expert_counts);
  scan_kernel<<<1, 256, (E + 1) * sizeof(int), s>>>(expert_counts, E, max_rows, max_tiles, align, expert_offsets, tile_group,
                                                     num_m_tiles);
  assign_kernel<<<E, 512, 0, s>>>(topk_ids, n, expert_offsets, dest_row, row_src);
}

void moe_permute(const void* x, const int* row_src, const int* num_m_tiles, void* x_perm, int max_rows, int H, int K,
                 cudaStream_t s) {
  if (max_rows <= 0) return;
  permute_kernel<<<grid_for(static_cast<long long>(max_rows) * (H / 8), 256), 256, 0, s>>>(
      static_cast<const bf16*>(x), row_src, num_m_tiles, static_cast<bf16*>(x_perm), max_rows, H, K);
}

void moe_combine(const void* y_perm, const int* dest_row, const float* topk_w, const void* residual, void* out, int T,
                 int K, int H, cudaStream_t s) {
  if (T <= 0) return;
  combine_kernel<<<grid_for(static_cast<long long>(T) * (H / 8), 256), 256, 0, s>>>(
      static_cast<const bf16*>(y_perm), dest_row, topk_w, static_cast<const bf16*>(residual), static_cast<bf16*>(out), T, K, H);
}

void moe_unpermute_sum(const void* dx_perm, const int* dest_row, void* dx, int T, int K, int H, cudaStream_t s) {
  moe_combine(dx_perm, dest_row, nullptr, nullptr, dx, T, K, H, s);
}

void moe_combine_bwd(const void* dout, const void* y_perm, const int* row_src, const int* num_m_tiles,
                     const float* topk_w, void* dy_perm, float* dtopk_w, int max_rows, int K, int H, cudaStream_t s) {
  if (max_rows <= 0) return;
  const int wpb = 8;
  combine_bwd_kernel<<<grid_for(max_rows, wpb), wpb * 32, 0, s>>>(
      static_cast<const bf16*>(dout), static_cast<const bf16*>(y_perm), row_src, num_m_tiles, topk_w,
      static_cast<bf16*>(dy_perm), dtopk_w, max_rows, K, H);
}

}  // namespace mb
