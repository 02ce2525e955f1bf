// Weight-streaming matrix products for decode steps of at most 8 tokens (the long tail of a rollout).
//
// With a handful of tokens every projection is bound by the bytes of the weights it reads, and what decides
// the speed is how many of those bytes are in flight per SM. Register-destination loads cap that at the size of
// the register file and stall on every dependent step; here one persistent CTA per SM keeps a ring of
// shared-memory stages (about 190 KB) filled by bulk asynchronous copies (`cp.async.bulk`, one per weight row,
// completion counted on an mbarrier), so the copy engine streams continuously while eight consumer warps
// multiply the stage that has landed.
//
// The 8 tokens form the N=8 operand of `mma.sync.m16n8k16` and 16 weight rows the M operand (a 128-row tcgen05
// tile would carry 8 useful rows and its TMEM/descriptor set-up). A dot product does not depend on the order of
// its terms, so k is permuted such that a lane reads 16 contiguous bytes per row (8 k-values that feed two MMAs)
// from the stage and from the activations with the same addressing.
//
// One kernel serves every small-batch product:
//   dense    y[T, N]      = (norm?)(x) W^T (+ residual)           qkv / o / router logits / dense MLP
//   MoE up   gu[pair, 2I] = W1[e] norm(x[token of pair])          for the active experts only
//   MoE down y[pair, H]   = W2[e] (silu(gate) * up)[pair]         SwiGLU applied while gu is loaded
// RMSNorm is folded in: y = rstd[t] * sum_k W[n,k] (g[k] x[t,k]); sum_k x^2 comes from the activation chunks the
// warps read anyway. Work items are (expert, 16-row tile), dealt round-robin to the CTAs; the number of active
// experts is read from device memory, so the launch shape is fixed and the kernel can sit in a CUDA graph.
//
// Reference counterpart: SGLang's fused-MoE / decode kernels used by the rollout engines
// (miles/backends/sglang_utils/sglang_engine.py:73-152 launches them as servers).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launchers.h"
#include "ptx.cuh"

namespace mb {
namespace {

typedef __nv_bfloat16 bf16;
constexpr int TOK = 8;       // token columns of one MMA
constexpr int ROWS = 16;     // weight rows per tile
constexpr int CWARPS = 8;    // consumer warps; each owns an eighth of a stage's k range
constexpr int MAX_KC = 2048; // k-values per stage
constexpr int SKEW = 64;     // bytes added to the shared-memory row pitch
constexpr int THREADS = 32 * (1 + CWARPS);
constexpr int RING_BYTES = 200 * 1024;
constexpr int MAX_STAGES = 8;

struct StreamArgs {
  const bf16* W;        // [groups, rows, K] row-major
  int rows, K;          // rows per group (multiple of 16), contraction length (multiple of 32)
  int kc, n_kc, stages, chunks_per_warp;
  const bf16* x;        // activations: [T, K] (mode 0) or gu [pairs, 2K] (mode 1)
  long long x_ld;
  int T;
  const bf16* norm_w;   // RMSNorm weight or null
  float eps;
  const int* active;    // null: dense (one group, token column j = token j)
  const int* pair_count;
  const int* pair_list;
  int top_k;
  int act_mode;         // 0: x[token]; 1: silu(gu[pair, k]) * gu[pair, K + k]
  void* out;
  long long out_ld;
  int out_fp32;
  const bf16* residual; // dense mode only, same layout as out
  int* status;
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 ldg16(const bf16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ float sumsq_bf16x2(uint32_t a) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&a));
  return f.x * f.x + f.y * f.y;
}
__device__ __forceinline__ uint32_t swiglu_bf16x2(uint32_t gp, uint32_t up) {
  const float2 gf = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&gp));
  const float2 uf = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&up));
  __nv_bfloat162 o = __floats2bfloat162_rn(gf.x / (1.f + __expf(-gf.x)) * uf.x, gf.y / (1.f + __expf(-gf.y)) * uf.y);
  return *reinterpret_cast<uint32_t*>(&o);
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * CWARPS) : "memory"); }

// CPW: 32-wide k chunks per consumer warp and stage; RT: 16-row tiles per stage (items are sized to 48-64 KB so that
// the per-item barrier traffic and epilogue stay small next to the copy); EXACT: the stage is exactly
// CWARPS * CPW chunks wide and K fits one stage, so the inner loop carries no bounds checks. Stage, phase, group
// and tile indices advance by increments: integer divisions per item had made the consumers issue-bound.
template <int CPW, int RT, bool EXACT>
__global__ void __launch_bounds__(THREADS, 1) stream_kernel(const StreamArgs a) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ float red[RT][CWARPS][ROWS][TOK];
  __shared__ float ssq[CWARPS][TOK];
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;
  const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
  // One k chunk (K <= MAX_KC): an item is RT*16 whole rows, contiguous in memory, and travels as ONE bulk copy.
  // The reads then see a 2-way bank conflict, which is cheap. Several chunks: rows are copied one by one into a
  // skewed layout.
  const int pitch = a.n_kc == 1 ? a.kc * 2 : a.kc * 2 + SKEW;
  const int stage_bytes = RT * ROWS * (a.kc * 2 + SKEW);
  const uint32_t bars = base + a.stages * stage_bytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), CWARPS);
    }
    fence_barrier_init();
  }
  __syncthreads();
  const int n_groups = a.active ? a.active[0] : 1;
  const int tiles = a.rows / (ROWS * RT);
  const int total = n_groups * tiles;
  // contiguous ranges: a CTA stays inside one expert for most of its items, so the activation fragments and the
  // index chain behind them are reloaded once or twice per launch, not once per tile
  const int per_cta = (total + gridDim.x - 1) / gridDim.x;
  const int L_begin = min(total, static_cast<int>(blockIdx.x) * per_cta), L_end = min(total, L_begin + per_cta);
  int g = L_begin / tiles, t = L_begin - g * tiles;
  int stage = 0;
  uint32_t phase = 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer warp
    bool ok = true;
    for (int L = L_begin; ok && L < L_end; ++L) {
      const int e = a.active ? a.active[1 + g] : 0;
      const bf16* wbase = a.W + (static_cast<long long>(e) * a.rows + t * (ROWS * RT)) * a.K;
      for (int kc = 0; kc < a.n_kc; ++kc) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, a.status, ERR_WAIT_EMPTY)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const int kcols = min(a.kc, a.K - kc * a.kc);
        const uint32_t bytes = static_cast<uint32_t>(kcols) * 2u;
        if (lane == 0) mbar_expect_tx(full_bar(stage), RT * ROWS * bytes);
        __syncwarp();
        if (a.n_kc == 1) {
          if (lane == 0) bulk_g2s(base + stage * stage_bytes, wbase, RT * ROWS * bytes, full_bar(stage));
        } else if (lane < ROWS) {  // RT == 1 on this path
          bulk_g2s(base + stage * stage_bytes + lane * pitch, wbase + static_cast<long long>(lane) * a.K + kc * a.kc, bytes,
                   full_bar(stage));
        }
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (++t == tiles) {
        t = 0;
        ++g;
      }
    }
    if (!ok) {  // give copies already in flight a bounded chance to land before shared memory is released
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) {
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int cw = warp - 1;
    const int r = lane >> 2, c = lane & 3;
    const int ct = threadIdx.x - 32;             // 0..255
    const int ep_row = ct >> 3, ep_j = ct & 7;   // epilogue role of the first 128 consumer threads
    int cur_g = -1, m = 0, e = 0, ep_out_row = -1;
    const bf16* xrow = a.x;
    bool live = false;
    uint4 xa[CPW];
    float ss = 0.f;
    bool ok = true;
    const int k_warp = cw * CPW * 32;  // first k of this warp inside a stage
    for (int L = L_begin; L < L_end; ++L) {
      const bool new_group = g != cur_g;
      if (new_group) {
        cur_g = g;
        if (a.active) {
          e = a.active[1 + g];
          m = a.pair_count[e];
          live = r < m;
          const int pair = live ? a.pair_list[e * TOK + r] : 0;
          xrow = a.x + static_cast<long long>(a.act_mode == 0 ? pair / a.top_k : pair) * a.x_ld;
          ep_out_row = (ct < 128 && ep_j < m) ? a.pair_list[e * TOK + ep_j] : -1;
        } else {
          m = a.T;
          live = r < m;
          xrow = a.x + static_cast<long long>(r) * a.x_ld;
          ep_out_row = (ct < 128 && ep_j < m) ? ep_j : -1;
        }
      }
      const bool reload = new_group || a.n_kc > 1;
      if (reload) ss = 0.f;
      float acc[RT][4];
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) acc[rt][0] = acc[rt][1] = acc[rt][2] = acc[rt][3] = 0.f;
      for (int kc = 0; kc < a.n_kc; ++kc) {
        const int kcols = EXACT ? CWARPS * CPW * 32 : min(a.kc, a.K - kc * a.kc);
        if (reload) {
#pragma unroll
          for (int u = 0; u < CPW; ++u) {
            const int kl = k_warp + u * 32;
            xa[u] = make_uint4(0u, 0u, 0u, 0u);
            if ((EXACT || kl < kcols) && live) {
              const int k = kc * a.kc + kl + c * 8;
              if (a.act_mode == 0) {
                uint4 xv = ldg16(xrow + k);
                if (a.norm_w) {
                  ss += sumsq_bf16x2(xv.x) + sumsq_bf16x2(xv.y) + sumsq_bf16x2(xv.z) + sumsq_bf16x2(xv.w);
                  const uint4 gv = ldg16(a.norm_w + k);
                  xv.x = mul_bf16x2(xv.x, gv.x);
                  xv.y = mul_bf16x2(xv.y, gv.y);
                  xv.z = mul_bf16x2(xv.z, gv.z);
                  xv.w = mul_bf16x2(xv.w, gv.w);
                }
                xa[u] = xv;
              } else {
                const uint4 gv = ldg16(xrow + k), uv = ldg16(xrow + a.K + k);
                xa[u].x = swiglu_bf16x2(gv.x, uv.x);
                xa[u].y = swiglu_bf16x2(gv.y, uv.y);
                xa[u].z = swiglu_bf16x2(gv.z, uv.z);
                xa[u].w = swiglu_bf16x2(gv.w, uv.w);
              }
            }
          }
        }
        if (ok && !mbar_wait(full_bar(stage), phase, abort_flag, a.status, ERR_WAIT_FULL)) ok = false;
        if (ok) {
          const uint32_t s0 = base + stage * stage_bytes + r * pitch + (k_warp + c * 8) * 2;
#pragma unroll
          for (int rt = 0; rt < RT; ++rt) {
            const uint32_t sa = s0 + rt * ROWS * pitch, sb = sa + 8 * pitch;
#pragma unroll
            for (int u = 0; u < CPW; ++u) {
              if (EXACT || k_warp + u * 32 < kcols) {  // warp-uniform
                const uint4 w0 = lds16(sa + u * 64), w1 = lds16(sb + u * 64);
                mma16816(acc[rt], w0.x, w1.x, w0.y, w1.y, xa[u].x, xa[u].y);
                mma16816(acc[rt], w0.z, w1.z, w0.w, w1.w, xa[u].z, xa[u].w);
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_bar(stage));
        }
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      // ---- reduce the eight k slices and store RT*16 rows x m token columns
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        red[rt][cw][r][2 * c] = acc[rt][0];
        red[rt][cw][r][2 * c + 1] = acc[rt][1];
        red[rt][cw][r + 8][2 * c] = acc[rt][2];
        red[rt][cw][r + 8][2 * c + 1] = acc[rt][3];
      }
      if (a.norm_w) {
        float q = ss;
        q += __shfl_xor_sync(0xffffffffu, q, 1);
        q += __shfl_xor_sync(0xffffffffu, q, 2);
        if (c == 0) ssq[cw][r] = q;
      }
      consumer_sync();
      if (ok && ep_out_row >= 0) {
        float rs = 1.f;
        if (a.norm_w) {
          float q = 0.f;
#pragma unroll
          for (int w = 0; w < CWARPS; ++w) q += ssq[w][ep_j];
          rs = rsqrtf(q / static_cast<float>(a.K) + a.eps);
        }
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < CWARPS; ++w) v += red[rt][w][ep_row][ep_j];
          v *= rs;
          const long long o = static_cast<long long>(ep_out_row) * a.out_ld + (t * RT + rt) * ROWS + ep_row;
          if (a.residual) v += __bfloat162float(a.residual[o]);
          if (a.out_fp32)
            static_cast<float*>(a.out)[o] = v;
          else
            static_cast<bf16*>(a.out)[o] = __float2bfloat16(v);
        }
      }
      consumer_sync();
      if (++t == tiles) {
        t = 0;
        ++g;
      }
    }
  }
}

template <int CPW, int RT, bool EXACT>
int launch_variant(const StreamArgs& a, int grid, int smem, cudaStream_t s) {
  auto kern = stream_kernel<CPW, RT, EXACT>;
  // the attribute belongs to the (function, device) pair: set on every launch rather than once per process
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, RING_BYTES + 1024) != cudaSuccess) return -1;
  kern<<<grid, THREADS, smem, s>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int g_sms = 0;

int launch_stream(StreamArgs a, int max_groups, cudaStream_t s) {
  a.kc = a.K < MAX_KC ? a.K : MAX_KC;
  a.n_kc = (a.K + a.kc - 1) / a.kc;
  const int chunks = a.kc / 32;
  // rows per item: 2 or 4 tiles when a 16-row tile is far below 64 KB (and the row count allows it)
  int rt = 1;
  if (a.n_kc == 1 && chunks % CWARPS == 0) {
    const int tile_bytes = ROWS * a.kc * 2;
    if (tile_bytes * 4 <= 64 * 1024 && a.rows % (ROWS * 4) == 0) rt = 4;
    else if (tile_bytes * 2 <= 64 * 1024 && a.rows % (ROWS * 2) == 0) rt = 2;
  }
  const int stage_bytes = rt * ROWS * (a.kc * 2 + SKEW);
  a.stages = RING_BYTES / stage_bytes;
  if (a.stages > MAX_STAGES) a.stages = MAX_STAGES;
  a.chunks_per_warp = (chunks + CWARPS - 1) / CWARPS;
  const int smem = a.stages * stage_bytes + 8 * 2 * MAX_STAGES + 128;
  if (g_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long items = static_cast<long long>(max_groups) * (a.rows / (ROWS * rt));
  const int grid = static_cast<int>(items < g_sms ? items : g_sms);
  const bool exact = a.n_kc == 1 && chunks % CWARPS == 0;
  const int cpw = a.chunks_per_warp;
  if (exact && cpw == 8 && rt == 1) return launch_variant<8, 1, true>(a, grid, smem, s);   // K = 2048
  if (exact && cpw == 4 && rt == 2) return launch_variant<4, 2, true>(a, grid, smem, s);   // K = 1024
  if (exact && cpw == 3 && rt == 2) return launch_variant<3, 2, true>(a, grid, smem, s);   // K = 768
  if (exact && cpw == 2 && rt == 4) return launch_variant<2, 4, true>(a, grid, smem, s);   // K = 512
  if (exact && cpw == 1 && rt == 4) return launch_variant<1, 4, true>(a, grid, smem, s);   // K = 256
  // generic: any K that is a multiple of 32, one 16-row tile per item, bounds checks in the inner loop
  if (rt != 1) {
    rt = 1;
    const int sb = ROWS * (a.kc * 2 + SKEW);
    a.stages = RING_BYTES / sb > MAX_STAGES ? MAX_STAGES : RING_BYTES / sb;
    const long long it1 = static_cast<long long>(max_groups) * (a.rows / ROWS);
    return launch_variant<8, 1, false>(a, static_cast<int>(it1 < g_sms ? it1 : g_sms), a.stages * sb + 8 * 2 * MAX_STAGES + 128, s);
  }
  return launch_variant<8, 1, false>(a, grid, smem, s);
}

}  // namespace

void small_gemv_direct(const void* x, int T, const void* norm_w, float eps, const void* W, int N, int K,
                       const void* residual, void* out, bool out_fp32, cudaStream_t s);  // decode_small.cu

void small_gemv(const void* x, int T, const void* norm_w, float eps, const void* W, int N, int K, const void* residual,
                void* out, bool out_fp32, int* status, cudaStream_t s) {
  StreamArgs a = {};
  a.W = static_cast<const bf16*>(W);
  a.rows = N;
  a.K = K;
  a.x = static_cast<const bf16*>(x);
  a.x_ld = K;
  a.T = T;
  a.norm_w = static_cast<const bf16*>(norm_w);
  a.eps = eps;
  a.out = out;
  a.out_ld = N;
  a.out_fp32 = out_fp32 ? 1 : 0;
  a.residual = static_cast<const bf16*>(residual);
  a.status = status;
  if (T > TOK || static_cast<long long>(N) * K * 2 < (48ll << 20)) {  // small matrix or 9..64 rows: the direct kernels
    small_gemv_direct(x, T, norm_w, eps, W, N, K, residual, out, out_fp32, s);
    return;
  }
  launch_stream(a, 1, s);
}

void moe_small_up(const void* x, const void* norm_w, float eps, const void* W1, const int* active, const int* pair_count,
                  const int* pair_list, int max_active, int H, int I, int K, void* gu, int* status, cudaStream_t s) {
  StreamArgs a = {};
  a.W = static_cast<const bf16*>(W1);
  a.rows = 2 * I;
  a.K = H;
  a.x = static_cast<const bf16*>(x);
  a.x_ld = H;
  a.norm_w = static_cast<const bf16*>(norm_w);
  a.eps = eps;
  a.active = active;
  a.pair_count = pair_count;
  a.pair_list = pair_list;
  a.top_k = K;
  a.act_mode = 0;
  a.out = gu;
  a.out_ld = 2 * I;
  a.status = status;
  launch_stream(a, max_active, s);
}

void moe_small_down(const void* gu, const void* W2, const int* active, const int* pair_count, const int* pair_list,
                    int max_active, int H, int I, void* y, int* status, cudaStream_t s) {
  StreamArgs a = {};
  a.W = static_cast<const bf16*>(W2);
  a.rows = H;
  a.K = I;
  a.x = static_cast<const bf16*>(gu);
  a.x_ld = 2 * I;
  a.active = active;
  a.pair_count = pair_count;
  a.pair_list = pair_list;
  a.top_k = 1;
  a.act_mode = 1;
  a.out = y;
  a.out_ld = H;
  a.status = status;
  launch_stream(a, max_active, s);
}

}  // namespace mb
