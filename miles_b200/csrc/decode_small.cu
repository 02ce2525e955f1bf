// Light kernels for decode steps of at most 8 tokens.
//
// small_gemv_direct: y[T,N] = (norm?)(x) W^T (+ residual) for weight matrices of a few tens of MB (qkv, o, router):
// one CTA per 16 weight rows, k split across up to 32 warps so that every load of the CTA is issued before the
// first MMA. It starts faster than the persistent streaming kernel of decode_stream.cu (no ring to fill), which
// wins once the matrix is large enough to keep that ring busy. Same MMA scheme: 8 tokens = N of mma.m16n8k16, k
// permuted so that a lane reads 16 contiguous bytes per row, RMSNorm folded in.
//
// router_small: softmax -> top-k (+renorm) over the fp32 router logits and the per-expert (token, slot) lists that
// the weight-streaming MoE kernels consume instead of a sorted permutation.
//
// Reference counterpart: the top-k softmax routing inside SGLang's fused MoE
// (miles/backends/sglang_utils/sglang_engine.py:73-152 launches those engines).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "launchers.h"

namespace mb {
namespace {

typedef __nv_bfloat16 bf16;
constexpr int TOK = 8;  // tokens per step handled by this path

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg16(const bf16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// streaming load for weights that are read once per step: do not keep them in L1
__device__ __forceinline__ uint4 ldg16_stream(const bf16* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ float sumsq_bf16x2(uint32_t a) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&a));
  return f.x * f.x + f.y * f.y;
}

// Activation fragment of one 32-wide k chunk for this lane's token column: 8 values x[t][k0 + c*8 ..], scaled by
// the norm weight when NORM, with the running sum of squares of the raw values.
template <bool NORM>
__device__ __forceinline__ uint4 load_act(const bf16* xrow, const bf16* g, int k, bool live, float& ss) {
  uint4 xv = make_uint4(0u, 0u, 0u, 0u);
  if (live) xv = ldg16(xrow + k);
  if (NORM) {
    ss += sumsq_bf16x2(xv.x) + sumsq_bf16x2(xv.y) + sumsq_bf16x2(xv.z) + sumsq_bf16x2(xv.w);
    const uint4 gv = ldg16(g + k);
    xv.x = mul_bf16x2(xv.x, gv.x);
    xv.y = mul_bf16x2(xv.y, gv.y);
    xv.z = mul_bf16x2(xv.z, gv.z);
    xv.w = mul_bf16x2(xv.w, gv.w);
  }
  return xv;
}

// One warp: acc[16 rows x 8 tokens] += W[rows r, r+8][k range] . x. `w0`/`w1` point at column 0 of rows r and r+8.
template <bool NORM, int UNROLL>
__device__ __forceinline__ void warp_dot(float (&acc)[4], const bf16* w0, const bf16* w1, const bf16* xrow, const bf16* g,
                                         bool live, int k_begin, int k_end, int c, float& ss) {
  int k = k_begin + c * 8;
  for (; k + (UNROLL - 1) * 32 < k_end; k += UNROLL * 32) {
    uint4 a0[UNROLL], a1[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      a0[u] = ldg16_stream(w0 + k + u * 32);
      a1[u] = ldg16_stream(w1 + k + u * 32);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const uint4 xv = load_act<NORM>(xrow, g, k + u * 32, live, ss);
      mma16816(acc, a0[u].x, a1[u].x, a0[u].y, a1[u].y, xv.x, xv.y);
      mma16816(acc, a0[u].z, a1[u].z, a0[u].w, a1[u].w, xv.z, xv.w);
    }
  }
  for (; k < k_end; k += 32) {
    const uint4 a0 = ldg16_stream(w0 + k), a1 = ldg16_stream(w1 + k);
    const uint4 xv = load_act<NORM>(xrow, g, k, live, ss);
    mma16816(acc, a0.x, a1.x, a0.y, a1.y, xv.x, xv.y);
    mma16816(acc, a0.z, a1.z, a0.w, a1.w, xv.z, xv.w);
  }
}

__device__ __forceinline__ float quad_sum(float v) {  // over the 4 lanes that share a token column
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}


// Latency, not bandwidth, is what a skinny product has to beat: a warp that walks a long k range pays one DRAM
// round trip per loop iteration. So every kernel below splits k across the warps of a CTA until each warp owns
// about 128 k-values (4 chunks: all of its loads are issued before the first MMA), one CTA per 16-row block of the
// weights, and the warps reduce through shared memory. `KW` = k-values per warp.
constexpr int KW = 128;
constexpr int MAX_WARPS = 32;

__host__ __device__ inline int warps_for(int K) {
  int w = (K + KW - 1) / KW;
  return w < 1 ? 1 : (w > MAX_WARPS ? MAX_WARPS : w);
}
__device__ __forceinline__ void k_range(int K, int warp, int nwarps, int& k_begin, int& k_end) {
  const int kq = ((K / 32 + nwarps - 1) / nwarps) * 32;
  k_begin = min(K, warp * kq);
  k_end = min(K, k_begin + kq);
}

// ---------------------------------------------------------------------------------------------- small_gemv
template <bool NORM>
__global__ void __launch_bounds__(1024) small_gemv_kernel(const bf16* __restrict__ x, int T, const bf16* __restrict__ g,
                                                          float eps, const bf16* __restrict__ W, int N, int K,
                                                          const bf16* __restrict__ residual, void* __restrict__ out,
                                                          int out_fp32) {
  __shared__ float red[MAX_WARPS][16][TOK];
  __shared__ float ssq[MAX_WARPS][TOK];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * 16;
  int k_begin, k_end;
  k_range(K, warp, nwarps, k_begin, k_end);
  const bool live = r < T;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float ss = 0.f;
  warp_dot<NORM, 4>(acc, W + static_cast<long long>(n0 + r) * K, W + static_cast<long long>(n0 + r + 8) * K,
                    x + static_cast<long long>(r) * K, g, live, k_begin, k_end, c, ss);
  red[warp][r][2 * c] = acc[0];
  red[warp][r][2 * c + 1] = acc[1];
  red[warp][r + 8][2 * c] = acc[2];
  red[warp][r + 8][2 * c + 1] = acc[3];
  if (NORM) {
    ss = quad_sum(ss);
    if (c == 0) ssq[warp][r] = ss;
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    const int row = threadIdx.x >> 3, t = threadIdx.x & 7;
    if (t < T) {
      float v = 0.f, q = 0.f;
      for (int w = 0; w < nwarps; ++w) {
        v += red[w][row][t];
        if (NORM) q += ssq[w][t];
      }
      if (NORM) v *= rsqrtf(q / static_cast<float>(K) + eps);
      const long long o = static_cast<long long>(t) * N + n0 + row;
      if (residual) v += __bfloat162float(residual[o]);
      if (out_fp32)
        static_cast<float*>(out)[o] = v;
      else
        static_cast<bf16*>(out)[o] = __float2bfloat16(v);
    }
  }
}


// ---------------------------------------------------------------------------------------------- small_gemv, 9..64 tokens
// Same scheme with G groups of 8 token columns: the weight fragments of a chunk are loaded once and multiplied with
// every group (G MMAs per fragment pair), the activations come from L1/L2. Used for the dense projections of decode
// steps with up to 64 rows, where a 128-row tcgen05 tile is mostly padding and its fixed cost (tensor-map prefetch,
// TMEM allocation, pipeline fill) is a multiple of the 3-6 us the weights take to stream.
template <int G>
__global__ void __launch_bounds__(256) small_gemv_multi_kernel(const bf16* __restrict__ x, int T, const bf16* __restrict__ W,
                                                               int N, int K, const bf16* __restrict__ residual,
                                                               void* __restrict__ out, int out_fp32) {
  __shared__ float red[8][16][TOK * G];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * 16;
  int k_begin, k_end;
  k_range(K, warp, nwarps, k_begin, k_end);
  float acc[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
  const bf16* w0 = W + static_cast<long long>(n0 + r) * K;
  const bf16* w1 = W + static_cast<long long>(n0 + r + 8) * K;
  constexpr int UNROLL = 4;
  int k = k_begin + c * 8;
  for (; k + (UNROLL - 1) * 32 < k_end; k += UNROLL * 32) {
    uint4 a0[UNROLL], a1[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      a0[u] = ldg16_stream(w0 + k + u * 32);
      a1[u] = ldg16_stream(w1 + k + u * 32);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int t = g * TOK + r;
        uint4 xv = make_uint4(0u, 0u, 0u, 0u);
        if (t < T) xv = ldg16(x + static_cast<long long>(t) * K + k + u * 32);
        mma16816(acc[g], a0[u].x, a1[u].x, a0[u].y, a1[u].y, xv.x, xv.y);
        mma16816(acc[g], a0[u].z, a1[u].z, a0[u].w, a1[u].w, xv.z, xv.w);
      }
    }
  }
  for (; k < k_end; k += 32) {
    const uint4 a0 = ldg16_stream(w0 + k), a1 = ldg16_stream(w1 + k);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int t = g * TOK + r;
      uint4 xv = make_uint4(0u, 0u, 0u, 0u);
      if (t < T) xv = ldg16(x + static_cast<long long>(t) * K + k);
      mma16816(acc[g], a0.x, a1.x, a0.y, a1.y, xv.x, xv.y);
      mma16816(acc[g], a0.z, a1.z, a0.w, a1.w, xv.z, xv.w);
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    red[warp][r][g * TOK + 2 * c] = acc[g][0];
    red[warp][r][g * TOK + 2 * c + 1] = acc[g][1];
    red[warp][r + 8][g * TOK + 2 * c] = acc[g][2];
    red[warp][r + 8][g * TOK + 2 * c + 1] = acc[g][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 16 * TOK * G; i += blockDim.x) {
    const int row = i / (TOK * G), t = i - row * (TOK * G);
    if (t >= T) continue;
    float v = 0.f;
    for (int w = 0; w < nwarps; ++w) v += red[w][row][t];
    const long long o = static_cast<long long>(t) * N + n0 + row;
    if (residual) v += __bfloat162float(residual[o]);
    if (out_fp32)
      static_cast<float*>(out)[o] = v;
    else
      static_cast<bf16*>(out)[o] = __float2bfloat16(v);
  }
}

// ---------------------------------------------------------------------------------------------- router_small
// One CTA of 8 warps over the fp32 router logits [T, E] (a small_gemv with the norm folded in produces them).
// Outputs: topk_ids[T,K], topk_w[T,K], and for the MoE kernels the compact list of active experts with, per
// expert, the (token, slot) pairs routed to it: active[0] = count, active[1..] = expert ids, pair_count[E],
// pair_list[E][TOK] (pair = t*K + k; a token picks an expert at most once).
__global__ void __launch_bounds__(256) router_small_kernel(const float* __restrict__ logits, int T, int E, int K,
                                                           int renorm, int* __restrict__ topk_ids,
                                                           float* __restrict__ topk_w, int* __restrict__ active,
                                                           int* __restrict__ pair_count, int* __restrict__ pair_list) {
  __shared__ int ids_s[TOK][32];
  __shared__ int cnt_s[1024];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < T) {
    const float* lg = logits + static_cast<long long>(warp) * E;
    float m = -FLT_MAX;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, lg[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
    for (int e = lane; e < E; e += 32) s += __expf(lg[e] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float inv = 1.f / s;
    float wsum = 0.f, my_w = 0.f;
    int my_id = 0;
    for (int k = 0; k < K; ++k) {
      float best = -FLT_MAX;
      int bi = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        bool taken = false;
        for (int j = 0; j < k; ++j) taken |= (ids_s[warp][j] == e);
        const float v = lg[e];
        if (!taken && (v > best || (v == best && e < bi))) {
          best = v;
          bi = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) {
          best = ob;
          bi = oi;
        }
      }
      if (lane == 0) ids_s[warp][k] = bi;
      __syncwarp();
      const float pw = __expf(best - m) * inv;
      wsum += pw;
      if (lane == k) {
        my_w = pw;
        my_id = bi;
      }
    }
    if (lane < K) {
      topk_ids[warp * K + lane] = my_id;
      topk_w[warp * K + lane] = renorm ? my_w / wsum : my_w;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int n = 0;
    for (int t = 0; t < T; ++t)
      for (int k = 0; k < K; ++k)
        if (ids_s[t][k] == e) pair_list[e * TOK + n++] = t * K + k;
    pair_count[e] = n;
    cnt_s[e] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = 0;
    for (int e = 0; e < E; ++e)
      if (cnt_s[e] > 0) active[1 + n++] = e;
    active[0] = n;
  }
}

}  // namespace

void small_gemv_direct(const void* x, int T, const void* norm_w, float eps, const void* W, int N, int K,
                       const void* residual, void* out, bool out_fp32, cudaStream_t s) {
  if (T > TOK) {  // 9..64 rows: token groups (no folded norm on this path)
    int warps = (K + 255) / 256;
    warps = warps < 4 ? 4 : (warps > 8 ? 8 : warps);
    const bf16* xb = static_cast<const bf16*>(x);
    const bf16* wb = static_cast<const bf16*>(W);
    const bf16* rb = static_cast<const bf16*>(residual);
    const int f32 = out_fp32 ? 1 : 0;
    if (T <= 16) small_gemv_multi_kernel<2><<<N / 16, 32 * warps, 0, s>>>(xb, T, wb, N, K, rb, out, f32);
    else if (T <= 32) small_gemv_multi_kernel<4><<<N / 16, 32 * warps, 0, s>>>(xb, T, wb, N, K, rb, out, f32);
    else small_gemv_multi_kernel<8><<<N / 16, 32 * warps, 0, s>>>(xb, T, wb, N, K, rb, out, f32);
    return;
  }
  const int threads = 32 * (warps_for(K) < 4 ? 4 : warps_for(K));  // the epilogue needs 128 threads
  if (norm_w)
    small_gemv_kernel<true><<<N / 16, threads, 0, s>>>(static_cast<const bf16*>(x), T, static_cast<const bf16*>(norm_w),
                                                       eps, static_cast<const bf16*>(W), N, K,
                                                       static_cast<const bf16*>(residual), out, out_fp32 ? 1 : 0);
  else
    small_gemv_kernel<false><<<N / 16, threads, 0, s>>>(static_cast<const bf16*>(x), T, nullptr, eps,
                                                        static_cast<const bf16*>(W), N, K,
                                                        static_cast<const bf16*>(residual), out, out_fp32 ? 1 : 0);
}

void router_small(const float* logits, int T, int E, int K, bool renorm, int* topk_ids, float* topk_w, int* active,
                  int* pair_count, int* pair_list, cudaStream_t s) {
  router_small_kernel<<<1, 256, 0, s>>>(logits, T, E, K, renorm ? 1 : 0, topk_ids, topk_w, active, pair_count, pair_list);
}

}  // namespace mb
