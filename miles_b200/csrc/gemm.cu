// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   warp 0      : TMA producer (cp.async.bulk.tensor, 128B swizzle, no multicast)
//   warp 1      : TMEM allocator + single-thread tcgen05.mma issuer
//   warps 2..5  : epilogue (tcgen05.ld -> registers -> global), one TMEM lane quadrant each
//
// The accumulator is double-buffered in TMEM (2 x BLOCK_N fp32 columns) so the epilogue of tile
// i overlaps the main loop of tile i+1. One kernel covers dense GEMMs, the MoE grouped GEMMs
// (row tiles tagged with an expert id) and the MoE weight-gradient GEMM (contraction over the rows
// of each expert); both operands may be K-major or MN-major, which gives forward (x.W^T), dgrad
// (dy.W) and wgrad (dy^T.x) without materialising a transpose.
//
// Counterpart in the reference stack: TransformerEngine's cuBLASLt GEMM and TEGroupedLinear used by
// the Megatron trainer (miles/backends/megatron_utils/model.py:560-570).
#include "gemm.h"

#include <cuda.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <string>

#include "ptx.cuh"

namespace mb {

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;  // 64 bf16 = 128 B = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int A_STAGE_BYTES = BLOCK_M * BLOCK_K * 2;

struct KArgs {
  int mode;
  int M, N, K;
  int num_groups;
  int max_tiles;
  const int* tile_group;
  const int* num_m_tiles;
  const int* group_offsets;
  void* c;
  long long ldc;
  long long c_group_stride;
  int accumulate;
  int out_fp32;
  int vec_ok;
  int* status;
  const unsigned long long* row_ptrs;
  unsigned long long* sig_ctrl;
  unsigned long long* sig_flags[8];
  int sig_nranks, sig_me;
  void* dest[8];
  int n_dest;
};

struct Tile {
  int a_mn0, b_mn0;  // M/N coordinates in the operand tensors
  int a_k0, b_k0;    // first contraction coordinate in each operand tensor
  int k_iters;
  int c_row0, c_col0;
  int row_end;  // rows >= row_end are not stored
  long long c_base;
};

template <int BLOCK_N, bool B_MN>
__device__ __forceinline__ int num_tiles_of(const KArgs& p) {
  const int n_tiles = (p.N + BLOCK_N - 1) / BLOCK_N;
  if (p.mode == GEMM_DENSE) return ((p.M + BLOCK_M - 1) / BLOCK_M) * n_tiles;
  if (p.mode == GEMM_GROUPED_ROWS) {
    int live = *p.num_m_tiles;
    const int cap = p.max_tiles;
    live = live < 0 ? 0 : (live > cap ? cap : live);
    return live * n_tiles;
  }
  return p.num_groups * ((p.M + BLOCK_M - 1) / BLOCK_M) * n_tiles;
}

template <int BLOCK_N, bool B_MN>
__device__ __forceinline__ Tile decode_tile(const KArgs& p, int t) {
  Tile r;
  const int n_tiles = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int m_tiles = (p.M + BLOCK_M - 1) / BLOCK_M;
  if (p.mode == GEMM_DENSE) {
    // Rasterise in bands of 8 row tiles so that concurrently running CTAs share B tiles in L2.
    constexpr int BAND = 8;
    const int per_band = BAND * n_tiles;
    const int band = t / per_band;
    const int first_m = band * BAND;
    const int band_rows = (m_tiles - first_m) < BAND ? (m_tiles - first_m) : BAND;
    const int in_band = t - band * per_band;
    const int mt = first_m + in_band % band_rows;
    const int nt = in_band / band_rows;
    r.a_mn0 = mt * BLOCK_M;
    r.b_mn0 = nt * BLOCK_N;
    r.a_k0 = 0;
    r.b_k0 = 0;
    r.k_iters = (p.K + BLOCK_K - 1) / BLOCK_K;
    r.c_row0 = r.a_mn0;
    r.c_col0 = r.b_mn0;
    r.row_end = p.M;
    r.c_base = 0;
  } else if (p.mode == GEMM_GROUPED_ROWS) {
    const int mt = t / n_tiles;
    const int nt = t - mt * n_tiles;
    const int4 td = reinterpret_cast<const int4*>(p.tile_group)[mt];
    int g = td.x;
    g = g < 0 ? 0 : (g >= p.num_groups ? p.num_groups - 1 : g);
    r.a_mn0 = td.y < 0 ? 0 : td.y;
    r.row_end = min(p.M, r.a_mn0 + max(0, min(td.z, BLOCK_M)));
    r.a_k0 = 0;
    if (B_MN) {
      r.b_mn0 = nt * BLOCK_N;
      r.b_k0 = g * p.K;
    } else {
      r.b_mn0 = g * p.N + nt * BLOCK_N;
      r.b_k0 = 0;
    }
    r.k_iters = (p.K + BLOCK_K - 1) / BLOCK_K;
    r.c_row0 = r.a_mn0;
    r.c_col0 = nt * BLOCK_N;
    r.c_base = 0;
  } else {
    const int per_group = m_tiles * n_tiles;
    const int g = t / per_group;
    const int rem = t - g * per_group;
    const int mt = rem / n_tiles;
    const int nt = rem - mt * n_tiles;
    const int k_lo = p.group_offsets[g];
    const int k_hi = p.group_offsets[g + 1];
    r.a_mn0 = mt * BLOCK_M;
    r.b_mn0 = nt * BLOCK_N;
    r.a_k0 = k_lo;
    r.b_k0 = k_lo;
    r.k_iters = k_hi > k_lo ? (k_hi - k_lo + BLOCK_K - 1) / BLOCK_K : 0;
    r.c_row0 = r.a_mn0;
    r.c_col0 = r.b_mn0;
    r.row_end = p.M;
    r.c_base = static_cast<long long>(g) * p.c_group_stride;
  }
  return r;
}

__device__ __forceinline__ void store_chunk(const KArgs& p, const Tile& t, int row, int col,
                                            const uint32_t (&acc)[32], bool zero) {
  if (row >= t.row_end) return;
  if (p.row_ptrs) {
    // scattered bf16 rows (possibly in a peer GPU's memory): N % 8 == 0 and 16-byte aligned rows are checked on the host
    const unsigned long long base = p.row_ptrs[row];
    if (base == 0ull) return;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(base) + col;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (col + 8 * i + 8 <= p.N) {
        uint4 v;
        v.x = zero ? 0u : pack_bf16(__uint_as_float(acc[8 * i + 0]), __uint_as_float(acc[8 * i + 1]));
        v.y = zero ? 0u : pack_bf16(__uint_as_float(acc[8 * i + 2]), __uint_as_float(acc[8 * i + 3]));
        v.z = zero ? 0u : pack_bf16(__uint_as_float(acc[8 * i + 4]), __uint_as_float(acc[8 * i + 5]));
        v.w = zero ? 0u : pack_bf16(__uint_as_float(acc[8 * i + 6]), __uint_as_float(acc[8 * i + 7]));
        *reinterpret_cast<uint4*>(dst + 8 * i) = v;
      }
    }
    return;
  }
  const long long off = t.c_base + static_cast<long long>(row) * p.ldc + col;
  const bool full = (col + 32 <= p.N) && p.vec_ok;
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(p.c) + off;
    if (full) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 v;
        v.x = zero ? 0.f : __uint_as_float(acc[4 * i + 0]);
        v.y = zero ? 0.f : __uint_as_float(acc[4 * i + 1]);
        v.z = zero ? 0.f : __uint_as_float(acc[4 * i + 2]);
        v.w = zero ? 0.f : __uint_as_float(acc[4 * i + 3]);
        if (p.accumulate) {
          const float4 o = *reinterpret_cast<const float4*>(dst + 4 * i);
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
        *reinterpret_cast<float4*>(dst + 4 * i) = v;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (col + i < p.N) {
          float v = zero ? 0.f : __uint_as_float(acc[i]);
          if (p.accumulate) v += dst[i];
          dst[i] = v;
        }
      }
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + off;
    if (full) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = zero ? 0.f : __uint_as_float(acc[8 * i + j]);
        if (p.accumulate) {
          const uint4 o = *reinterpret_cast<const uint4*>(dst + 8 * i);
          const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 of = __bfloat1622float2(ob[j]);
            f[2 * j] += of.x;
            f[2 * j + 1] += of.y;
          }
        }
        uint4 v;
        v.x = pack_bf16(f[0], f[1]);
        v.y = pack_bf16(f[2], f[3]);
        v.z = pack_bf16(f[4], f[5]);
        v.w = pack_bf16(f[6], f[7]);
        *reinterpret_cast<uint4*>(dst + 8 * i) = v;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (col + i < p.N) {
          float v = zero ? 0.f : __uint_as_float(acc[i]);
          if (p.accumulate) v += __bfloat162float(dst[i]);
          dst[i] = __float2bfloat16(v);
        }
      }
    }
  }
}

template <int BLOCK_N, bool A_MN, bool B_MN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const KArgs p) {
  constexpr int B_STAGE_BYTES = BLOCK_N * BLOCK_K * 2;
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;  // 256 or 512: a power of two >= 32
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_smem = smem_base;
  const uint32_t b_smem = a_smem + STAGES * A_STAGE_BYTES;
  const uint32_t bar_base = b_smem + STAGES * B_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  const uint32_t stage_buf = (bar_base + 8u * (2 * STAGES + 5) + 15u) & ~15u;  // epilogue staging (BLOCK_N == 128 only)
  (void)stage_buf;
  __shared__ int abort_flag_s;
  __shared__ uint32_t tmem_base_s;
  volatile int* abort_flag = &abort_flag_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);  // one arrive per epilogue warp
    }
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(tmem_slot));
    tmem_base_s = v;
  }
  __syncthreads();
  const uint32_t tmem_base = tmem_base_s;

  const int total_tiles = num_tiles_of<BLOCK_N, B_MN>(p);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const Tile tl = decode_tile<BLOCK_N, B_MN>(p, t);
        for (int kb = 0; kb < tl.k_iters; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(full_bar(stage), A_STAGE_BYTES + B_STAGE_BYTES);
          const uint32_t a_dst = a_smem + stage * A_STAGE_BYTES;
          const uint32_t b_dst = b_smem + stage * B_STAGE_BYTES;
          const int ka = tl.a_k0 + kb * BLOCK_K;
          const int kbb = tl.b_k0 + kb * BLOCK_K;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BLOCK_M / 64; ++i)
              tma_load_2d(a_dst + i * (BLOCK_K * 128), &tma_a, full_bar(stage), tl.a_mn0 + 64 * i, ka);
          } else {
            tma_load_2d(a_dst, &tma_a, full_bar(stage), ka, tl.a_mn0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BLOCK_N / 64; ++i)
              tma_load_2d(b_dst + i * (BLOCK_K * 128), &tma_b, full_bar(stage), tl.b_mn0 + 64 * i, kbb);
          } else {
            tma_load_2d(b_dst, &tma_b, full_bar(stage), kbb, tl.b_mn0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Give copies that are already in flight a bounded chance to land before smem is released.
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_bf16(BLOCK_M, BLOCK_N, A_MN, B_MN);
    int stage = 0;
    uint32_t phase = 0;
    int iter = 0;  // counts only tiles that use an accumulator, so both roles stay in phase
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const Tile tl = decode_tile<BLOCK_N, B_MN>(p, t);
      if (tl.k_iters == 0) continue;  // epilogue writes zeros without touching TMEM
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
      for (int kb = 0; kb < tl.k_iters; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, ERR_WAIT_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = a_smem + stage * A_STAGE_BYTES;
          const uint32_t b_addr = b_smem + stage * B_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(a_addr + k * UMMA_K * 128, BLOCK_K * 128, 1024)
                                        : make_smem_desc(a_addr + k * UMMA_K * 2, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_addr + k * UMMA_K * 128, BLOCK_K * 128, 1024)
                                        : make_smem_desc(b_addr + k * UMMA_K * 2, 16, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok && lane == 0) umma_commit(tfull_bar(acc));
      __syncwarp();
      ++iter;
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const Tile tl = decode_tile<BLOCK_N, B_MN>(p, t);
      const int row = tl.c_row0 + quad * 32 + lane;
      uint32_t acc_regs[32];
      if (tl.k_iters == 0) {
        if (!p.accumulate) {
#pragma unroll 1
          for (int c = 0; c < BLOCK_N / 32; ++c)
            if (tl.c_col0 + c * 32 < p.N) store_chunk(p, tl, row, tl.c_col0 + c * 32, acc_regs, true);
        }
        continue;
      }
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * BLOCK_N + (static_cast<uint32_t>(quad * 32) << 16);
      if (BLOCK_N == 128 && p.n_dest > 0) {
        // Replicated tile (tensor-parallel partial sums): same staging, every row segment goes to each destination.
        const uint32_t stg = stage_buf + static_cast<uint32_t>(quad) * (32 * 256);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          tmem_ld_32x32(t_addr + c * 32, acc_regs);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t v0 = pack_bf16(__uint_as_float(acc_regs[8 * i + 0]), __uint_as_float(acc_regs[8 * i + 1]));
            const uint32_t v1 = pack_bf16(__uint_as_float(acc_regs[8 * i + 2]), __uint_as_float(acc_regs[8 * i + 3]));
            const uint32_t v2 = pack_bf16(__uint_as_float(acc_regs[8 * i + 4]), __uint_as_float(acc_regs[8 * i + 5]));
            const uint32_t v3 = pack_bf16(__uint_as_float(acc_regs[8 * i + 6]), __uint_as_float(acc_regs[8 * i + 7]));
            const uint32_t chunk = static_cast<uint32_t>(c * 4 + i) ^ static_cast<uint32_t>(lane & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + lane * 256 + chunk * 16), "r"(v0), "r"(v1),
                         "r"(v2), "r"(v3)
                         : "memory");
          }
        }
        __syncwarp();
#pragma unroll 1
        for (int it = 0; it < 16; ++it) {
          const int rl = it * 2 + (lane >> 4);
          const int ch = lane & 15;
          uint4 v;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                       : "r"(stg + rl * 256 + ((ch ^ (rl & 7)) * 16)));
          const int grow = tl.c_row0 + quad * 32 + rl;
          const int col = tl.c_col0 + ch * 8;
          if (grow < tl.row_end && col + 8 <= p.N) {
            const long long off = static_cast<long long>(grow) * p.ldc + col;
            for (int d = 0; d < p.n_dest; ++d) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.dest[d]) + off) = v;
          }
        }
        __syncwarp();
      } else if (BLOCK_N == 128 && p.row_ptrs) {
        // Scattered rows (expert-parallel return): pass the warp's 32 x 128 block through shared memory so that
        // every store instruction writes two whole 256-byte row segments instead of thirty-two 64-byte pieces;
        // over NVLink the size of a write decides how much of the link carries payload.
        const uint32_t stg = stage_buf + static_cast<uint32_t>(quad) * (32 * 256);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          tmem_ld_32x32(t_addr + c * 32, acc_regs);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t v0 = pack_bf16(__uint_as_float(acc_regs[8 * i + 0]), __uint_as_float(acc_regs[8 * i + 1]));
            const uint32_t v1 = pack_bf16(__uint_as_float(acc_regs[8 * i + 2]), __uint_as_float(acc_regs[8 * i + 3]));
            const uint32_t v2 = pack_bf16(__uint_as_float(acc_regs[8 * i + 4]), __uint_as_float(acc_regs[8 * i + 5]));
            const uint32_t v3 = pack_bf16(__uint_as_float(acc_regs[8 * i + 6]), __uint_as_float(acc_regs[8 * i + 7]));
            const uint32_t chunk = static_cast<uint32_t>(c * 4 + i) ^ static_cast<uint32_t>(lane & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + lane * 256 + chunk * 16), "r"(v0), "r"(v1),
                         "r"(v2), "r"(v3)
                         : "memory");
          }
        }
        const unsigned long long my_ptr = (row < tl.row_end) ? p.row_ptrs[row] : 0ull;
        __syncwarp();
#pragma unroll 1
        for (int it = 0; it < 16; ++it) {
          const int rl = it * 2 + (lane >> 4);
          const int ch = lane & 15;
          const unsigned long long base = __shfl_sync(0xffffffffu, my_ptr, rl);
          uint4 v;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                       : "r"(stg + rl * 256 + ((ch ^ (rl & 7)) * 16)));
          const int col = tl.c_col0 + ch * 8;
          if (base != 0ull && col + 8 <= p.N) *reinterpret_cast<uint4*>(base + static_cast<unsigned long long>(col) * 2) = v;
        }
        __syncwarp();
      } else {
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / 32; ++c) {
          if (tl.c_col0 + c * 32 >= p.N) break;  // warp-uniform
          tmem_ld_32x32(t_addr + c * 32, acc_regs);
          tmem_ld_wait();
          store_chunk(p, tl, row, tl.c_col0 + c * 32, acc_regs, false);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      ++iter;
    }
    if (p.row_ptrs || p.n_dest > 0) __threadfence_system();  // peer stores are visible before the CTA reports in
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (p.sig_ctrl && threadIdx.x == 0) {
    __threadfence_system();
    const unsigned long long done = atomicAdd(&p.sig_ctrl[5], 1ull);
    if (done == gridDim.x - 1) {  // every CTA has stored and fenced: raise the return flags of this epoch
      __threadfence_system();
      const unsigned long long epoch = p.sig_ctrl[2] + 1;
      for (int d = 0; d < p.sig_nranks; ++d)
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.sig_flags[d] + p.sig_me), "l"(epoch) : "memory");
      p.sig_ctrl[5] = 0;
      p.sig_ctrl[2] = epoch;
    }
  }
}

// ---------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

std::string g_err;
EncodeTiledFn g_encode = nullptr;
std::once_flag g_once;

EncodeTiledFn get_encode() {
  std::call_once(g_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  return g_encode;
}

int fail(const std::string& m) {
  g_err = m;
  return -1;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with a [box_rows, 64] box.
int make_map(CUtensorMap* map, const GemmOperand& op, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail("cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(op.ptr) & 15) != 0) return fail("operand base must be 16-byte aligned");
  if ((op.ld * 2) % 16 != 0) return fail("operand row pitch must be a multiple of 16 bytes");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(op.cols), static_cast<cuuint64_t>(op.rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(op.ld) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(op.ptr), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return 0;
}

template <int BLOCK_N, bool A_MN, bool B_MN>
int launch(const GemmProblem& p, const KArgs& ka, cudaStream_t stream) {
  // the 128-wide variant gives one pipeline stage to a 32 KB staging buffer for scattered (peer) output rows
  constexpr int STAGES = BLOCK_N == 256 ? 4 : (BLOCK_N == 128 ? 5 : 8);
  constexpr int B_STAGE_BYTES = BLOCK_N * BLOCK_K * 2;
  constexpr int SMEM = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 8 * (2 * STAGES + 5) + 1024 +
                       (BLOCK_N == 128 ? 4 * 32 * 256 + 16 : 0);
  CUtensorMap ma, mb_;
  if (make_map(&ma, p.a, A_MN ? BLOCK_K : BLOCK_M)) return -1;
  if (make_map(&mb_, p.b, B_MN ? BLOCK_K : BLOCK_N)) return -1;
  auto kern = gemm_bf16_kernel<BLOCK_N, A_MN, B_MN, STAGES>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)  // per (function, device)
    return fail("cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long m_tiles = (p.M + BLOCK_M - 1) / BLOCK_M;
  const long long n_tiles = (p.N + BLOCK_N - 1) / BLOCK_N;
  long long tiles = (p.mode == GEMM_GROUPED_ROWS ? static_cast<long long>(p.max_tiles) : m_tiles) * n_tiles *
                    (p.mode == GEMM_GROUPED_CONTR ? p.num_groups : 1);
  int grid = static_cast<int>(tiles < sms ? tiles : sms);
  if (p.max_ctas > 0 && grid > p.max_ctas) grid = p.max_ctas;
  if (grid <= 0) return 0;
  kern<<<grid, kThreads, SMEM, stream>>>(ma, mb_, ka);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(std::string("gemm launch failed: ") + cudaGetErrorString(e));
  return 0;
}

}  // namespace

const char* gemm_last_error() { return g_err.c_str(); }

int gemm_bf16_launch(const GemmProblem& p, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0) return 0;
  if (p.mode != GEMM_GROUPED_CONTR && p.K <= 0) return fail("K must be positive");
  if (p.mode == GEMM_GROUPED_ROWS && (!p.tile_group || !p.num_m_tiles)) return fail("grouped-rows GEMM needs tile_group and num_m_tiles");
  if (p.mode == GEMM_GROUPED_ROWS && p.b.mn_major && p.K % BLOCK_K != 0) return fail("grouped-rows GEMM with an MN-major B needs K % 64 == 0");
  if (p.mode == GEMM_GROUPED_CONTR && (!p.group_offsets || !p.a.mn_major || !p.b.mn_major)) return fail("grouped-contraction GEMM needs MN-major operands and group_offsets");
  KArgs ka;
  memset(&ka, 0, sizeof(ka));
  ka.mode = p.mode;
  ka.M = p.M;
  ka.N = p.N;
  ka.K = p.K;
  ka.num_groups = p.num_groups;
  ka.max_tiles = p.max_tiles;
  ka.tile_group = p.tile_group;
  ka.num_m_tiles = p.num_m_tiles;
  ka.group_offsets = p.group_offsets;
  ka.c = p.c;
  ka.ldc = p.ldc;
  ka.c_group_stride = p.c_group_stride;
  ka.accumulate = p.accumulate ? 1 : 0;
  ka.out_fp32 = p.out_fp32 ? 1 : 0;
  ka.status = p.status;
  ka.row_ptrs = p.row_ptrs;
  ka.sig_ctrl = (p.row_ptrs || p.n_dest > 0) ? p.sig_ctrl : nullptr;
  ka.n_dest = p.n_dest;
  for (int i = 0; i < 8; ++i) ka.dest[i] = p.dest[i];
  if (p.n_dest > 0 && (p.out_fp32 || p.accumulate || p.N % 8 != 0 || p.mode != GEMM_DENSE || p.n_dest > 8 || p.ldc % 8 != 0))
    return fail("replicated output needs a dense bf16 problem without accumulation, N % 8 == 0 and ldc % 8 == 0");
  for (int i = 0; i < 8; ++i) ka.sig_flags[i] = p.sig_flags[i];
  ka.sig_nranks = p.sig_nranks;
  ka.sig_me = p.sig_me;
  if (p.row_ptrs && (p.out_fp32 || p.accumulate || p.N % 8 != 0 || p.mode == GEMM_GROUPED_CONTR))
    return fail("scattered output needs bf16, no accumulation, N % 8 == 0 and a row-major problem");
  const int esz = p.out_fp32 ? 4 : 2;
  const int vec = 16 / esz;
  ka.vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0 && p.ldc % vec == 0 && p.c_group_stride % vec == 0) ? 1 : 0;

  int bn = p.block_n;
  const bool amn = p.a.mn_major, bmn = p.b.mn_major;
  if (bn == 0) {
    const int sms = 148;
    const long long m_tiles = p.mode == GEMM_GROUPED_ROWS ? p.max_tiles : (p.M + BLOCK_M - 1) / BLOCK_M;
    const long long groups = p.mode == GEMM_GROUPED_CONTR ? p.num_groups : 1;
    auto tiles = [&](int b) { return m_tiles * ((p.N + b - 1) / b) * groups; };
    // Prefer the 128x256 tile unless it leaves most SMs idle or wastes a large share of the tile.
    const bool waste256 = (p.N % 256) != 0 && (p.N % 256) <= 128;
    bn = (tiles(256) >= sms && !waste256) || (p.N >= 256 && tiles(256) >= 2 * sms) ? 256 : 128;
    if (p.N <= 128) bn = 128;
    // Skinny problems (decode projections): narrower tiles spread the weight stream over more SMs.
    if (!amn && !bmn && tiles(bn) < sms) {
      if (bn == 256 && tiles(128) <= sms) bn = 128;
      if (bn == 128 && tiles(128) < sms / 2 && p.N >= 64) bn = 64;
      if (bn == 64 && tiles(64) < sms / 2 && p.N >= 32) bn = 32;
    }
  }
  if (p.row_ptrs || p.n_dest > 0) bn = 128;  // the staged scatter epilogue lives in the 128-wide variant
  if (bn != 32 && bn != 64 && bn != 128 && bn != 256) return fail("block_n must be 32, 64, 128 or 256");
  if ((bn == 32 || bn == 64) && (amn || bmn)) return fail("narrow tiles support K-major operands only");
  if (bn == 32) return launch<32, false, false>(p, ka, stream);
  if (bn == 64) return launch<64, false, false>(p, ka, stream);
#define MB_DISPATCH(BN)                                                     \
  if (!amn && !bmn) return launch<BN, false, false>(p, ka, stream);         \
  if (!amn && bmn) return launch<BN, false, true>(p, ka, stream);           \
  if (amn && !bmn) return launch<BN, true, false>(p, ka, stream);           \
  return launch<BN, true, true>(p, ka, stream);
  if (bn == 256) {
    MB_DISPATCH(256)
  } else {
    MB_DISPATCH(128)
  }
#undef MB_DISPATCH
}

}  // namespace mb
