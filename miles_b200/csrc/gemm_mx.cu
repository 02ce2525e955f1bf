// Block-scaled low-precision GEMMs for sm_100a: MXFP8 (E4M3 values, one E8M0 scale per 32 elements along K) and
// NVFP4 (E2M1 values packed two per byte, one UE4M3 scale per 16 elements along K, per-tensor fp32 scales folded into
// `alpha`). C[M,N] (bf16) = alpha * (A . B^T) with both operands K-major.
//
// The tensor core applies the block scales itself (`tcgen05.mma ... .block_scale`): values travel global -> shared
// memory by TMA (128-byte swizzle) as for the bf16 kernel, scale factors travel as 512-byte "atoms" by bulk copy,
// are moved shared memory -> TMEM with `tcgen05.cp.32x128b.warpx4` by the MMA thread and are named to the MMA by
// their TMEM column.
//
// Scale-factor atom (the layout the instruction reads from TMEM, written once by `sf_swizzle`): one atom covers 128
// rows x 4 consecutive scale factors of each row; byte (r % 32) * 16 + (r / 32) * 4 + j holds scale j of row r. Atoms
// are stored [row tile][group of 4 scales along K][512 bytes]. For MXFP8 one atom serves four MMAs (K = 32 each, the
// MMA picks byte j through the scale-id field of the instruction descriptor); for NVFP4 one atom serves one MMA
// (K = 64, all four bytes).
//
//   warp 0 : producer (TMA tiles + bulk copies of the scale atoms)      warp 1 : TMEM allocator, tcgen05.cp + mma issuer
//   warps 2..5 : epilogue (tcgen05.ld -> bf16 -> global), accumulators double-buffered in TMEM
//
// Reference counterpart: TransformerEngine's MXFP8 / NVFP4 GEMMs behind the low-precision recipes
// (miles/utils/mxfp8.py:8-35, miles/utils/nvfp4.py:19-145, miles/backends/megatron_utils/model.py:560-570).
#include <cuda.h>
#include <string.h>

#include <mutex>
#include <string>

#include "gemm.h"
#include "launchers.h"
#include "ptx.cuh"

namespace mb {
namespace {

constexpr int BM = 128;
constexpr int STAGE_K_BYTES = 128;  // one 128-byte swizzle row of packed values per operand row
constexpr int TILE_BYTES = BM * STAGE_K_BYTES;
constexpr int ATOM_BYTES = 512;
constexpr int kThreads = 192;

struct MxArgs {
  int mode;  // GEMM_DENSE or GEMM_GROUPED_ROWS
  int M, N, K;
  int num_groups, max_tiles;
  const int* tile_group;
  const int* num_m_tiles;
  const uint8_t* sfa;  // atoms [row tile of A][K group][512]
  const uint8_t* sfb;  // atoms [row tile of B (over all groups)][K group][512]
  __nv_bfloat16* c;
  long long ldc;
  float alpha;
  const float* alpha_dev;  // optional device scalar multiplied into alpha (keeps per-tensor scales off the host)
  long long b_rows;
  int* status;
};

struct MxTile {
  int a_row0, b_row0, c_col0, row_end;
};

template <int BN>
__device__ __forceinline__ int mx_num_tiles(const MxArgs& p) {
  const int n_tiles = (p.N + BN - 1) / BN;
  if (p.mode == GEMM_DENSE) return ((p.M + BM - 1) / BM) * n_tiles;
  int live = *p.num_m_tiles;
  live = live < 0 ? 0 : (live > p.max_tiles ? p.max_tiles : live);
  return live * n_tiles;
}

template <int BN>
__device__ __forceinline__ MxTile mx_decode(const MxArgs& p, int t) {
  MxTile r;
  const int n_tiles = (p.N + BN - 1) / BN;
  int mt = t / n_tiles, nt = t - mt * n_tiles;
  if (p.mode == GEMM_DENSE) {
    // bands of 8 row tiles, column tiles outermost within a band: CTAs running together share B tiles in L2
    constexpr int BAND = 8;
    const int m_tiles = (p.M + BM - 1) / BM;
    const int per_band = BAND * n_tiles;
    const int band = t / per_band;
    const int first_m = band * BAND;
    const int band_rows = (m_tiles - first_m) < BAND ? (m_tiles - first_m) : BAND;
    const int in_band = t - band * per_band;
    mt = first_m + in_band % band_rows;
    nt = in_band / band_rows;
    r.a_row0 = mt * BM;
    r.b_row0 = nt * BN;
    r.row_end = p.M;
  } else {
    const int4 td = reinterpret_cast<const int4*>(p.tile_group)[mt];
    int g = td.x;
    g = g < 0 ? 0 : (g >= p.num_groups ? p.num_groups - 1 : g);
    r.a_row0 = td.y < 0 ? 0 : (td.y & ~(BM - 1));  // row tiles start on 128-row boundaries (checked on the host side of the layout)
    r.row_end = min(p.M, r.a_row0 + max(0, min(td.z, BM)));
    r.b_row0 = g * p.N + nt * BN;
  }
  r.c_col0 = nt * BN;
  return r;
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Unswizzled K-major descriptor of a 32-row x 16-byte block: four 8-row core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>(1) << 16;          // leading byte offset 16 (a single core matrix along K)
  d |= static_cast<uint64_t>(128 >> 4) << 32;   // stride between 8-row core matrices
  d |= 1ull << 46;
  return d;
}

__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

template <int KIND>
__device__ __forceinline__ void umma_block_scaled(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  if (KIND == 0) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}

// Instruction descriptor of the block-scaled kinds: value formats at bits 7 and 10 (E4M3 = 0 for mxf8f6f4, E2M1 = 1
// for mxf4nvf4), N >> 3 at bit 17, scale format at bit 23 (1 = E8M0, 0 = UE4M3), M >> 4 at bit 24; the scale ids of
// B (bit 4) and A (bit 29) pick the byte of the 32-bit scale column.
template <int KIND, int BN>
__device__ __forceinline__ constexpr uint32_t mx_idesc() {
  return (KIND == 0 ? 0u : ((1u << 7) | (1u << 10))) | (static_cast<uint32_t>(BN >> 3) << 17) |
         ((KIND == 0 ? 1u : 0u) << 23) | (static_cast<uint32_t>(BM >> 4) << 24);
}

template <int KIND, int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const MxArgs p) {
  constexpr int SF_ATOMS = KIND == 0 ? 1 : 4;            // atoms per operand per stage
  constexpr int SF_BYTES = SF_ATOMS * ATOM_BYTES;
  constexpr int K_PER_STAGE = KIND == 0 ? 128 : 256;     // elements of K per stage
  constexpr int NB = BN / 128;                           // 128-row scale tiles of B per stage
  constexpr int B_TILE_BYTES = BN * STAGE_K_BYTES;
  constexpr int SFB_BYTES = SF_BYTES * NB;
  constexpr uint32_t SFA_COLS = 4 * SF_ATOMS;            // TMEM columns of A's scales for one stage
  constexpr uint32_t SFB_COLS = 4 * SF_ATOMS * NB;
  constexpr int ACC_BUFS = BN == 256 ? 1 : 2;            // 256 accumulator columns either way; the rest holds scales
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_smem = smem_base;
  const uint32_t b_smem = a_smem + STAGES * TILE_BYTES;
  const uint32_t sfa_smem = b_smem + STAGES * B_TILE_BYTES;
  const uint32_t sfb_smem = sfa_smem + STAGES * SF_BYTES;
  const uint32_t bar_base = sfb_smem + STAGES * SFB_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
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
    for (int a = 0; a < 2; ++a) {  // the second pair is unused with a single accumulator
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
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
  const int total_tiles = mx_num_tiles<BN>(p);
  const int k_iters = (p.K + K_PER_STAGE - 1) / K_PER_STAGE;
  const long long k_groups = static_cast<long long>(k_iters) * SF_ATOMS;  // atoms along K per row tile

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const MxTile tl = mx_decode<BN>(p, t);
        const uint8_t* sfa_row = p.sfa + static_cast<long long>(tl.a_row0 / BM) * k_groups * ATOM_BYTES;
        const uint8_t* sfb_row = p.sfb + static_cast<long long>(tl.b_row0 / 128) * k_groups * ATOM_BYTES;
        for (int kb = 0; kb < k_iters; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          // the second 128-row scale tile of a 256-wide B tile may lie past the end of B (its columns are never stored)
          const int nb_live = (NB == 2 && tl.b_row0 + 128 < p.b_rows) ? 2 : 1;
          mbar_expect_tx(full_bar(stage), TILE_BYTES + B_TILE_BYTES + SF_BYTES + nb_live * SF_BYTES);
          tma_load_2d(a_smem + stage * TILE_BYTES, &tma_a, full_bar(stage), kb * STAGE_K_BYTES, tl.a_row0);
          tma_load_2d(b_smem + stage * B_TILE_BYTES, &tma_b, full_bar(stage), kb * STAGE_K_BYTES, tl.b_row0);
          bulk_g2s(sfa_smem + stage * SF_BYTES, sfa_row + static_cast<long long>(kb) * SF_BYTES, SF_BYTES, full_bar(stage));
          for (int j = 0; j < nb_live; ++j)
            bulk_g2s(sfb_smem + stage * SFB_BYTES + j * SF_BYTES,
                     sfb_row + (j * k_groups * ATOM_BYTES) + static_cast<long long>(kb) * SF_BYTES, SF_BYTES, full_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc0 = mx_idesc<KIND, BN>();
    const uint32_t sf_tmem = tmem_base + 256;  // scale columns after the two accumulators
    int stage = 0;
    uint32_t phase = 0;
    int iter = 0;
    uint32_t kcount = 0;  // alternates the scale columns between consecutive stages
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const int acc = iter % ACC_BUFS;
      const uint32_t acc_phase = (iter / ACC_BUFS) & 1u;
      if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < k_iters; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, ERR_WAIT_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = a_smem + stage * TILE_BYTES;
          const uint32_t b_addr = b_smem + stage * B_TILE_BYTES;
          const uint32_t sfa_t = sf_tmem + (kcount & 1u) * (SFA_COLS + SFB_COLS);
          const uint32_t sfb_t = sfa_t + SFA_COLS;
          // scales of MMA k: A in columns [4k, 4k+4) (NVFP4) or byte k of columns [0, 4) (MXFP8); B likewise with
          // 4 columns per 128 rows of the tile
#pragma unroll
          for (int a = 0; a < SF_ATOMS; ++a) {
            tmem_cp_sf(sfa_t + 4 * a, make_sf_desc(sfa_smem + stage * SF_BYTES + a * ATOM_BYTES));
#pragma unroll
            for (int j = 0; j < NB; ++j)
              tmem_cp_sf(sfb_t + 4 * NB * a + 4 * j, make_sf_desc(sfb_smem + stage * SFB_BYTES + j * SF_BYTES + a * ATOM_BYTES));
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t adesc = make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = make_smem_desc(b_addr + k * 32, 16, 1024);
            const uint32_t idesc = KIND == 0 ? (idesc0 | (static_cast<uint32_t>(k) << 29) | (static_cast<uint32_t>(k) << 4)) : idesc0;
            const uint32_t sa = KIND == 0 ? sfa_t : sfa_t + 4 * k;
            const uint32_t sb = KIND == 0 ? sfb_t : sfb_t + 4 * NB * k;
            umma_block_scaled<KIND>(d_tmem, adesc, bdesc, idesc, sa, sb, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
        }
        __syncwarp();
        ++kcount;
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
    const int quad = warp & 3;
    int iter = 0;
    bool ok = true;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(p.c) & 15) == 0 && p.ldc % 8 == 0;
    const float alpha = p.alpha_dev ? p.alpha * __ldg(p.alpha_dev) : p.alpha;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const MxTile tl = mx_decode<BN>(p, t);
      const int row = tl.a_row0 + quad * 32 + lane;
      const int acc = iter % ACC_BUFS;
      const uint32_t acc_phase = (iter / ACC_BUFS) & 1u;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      uint32_t r[32];
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col = tl.c_col0 + c * 32;
        if (col >= p.N) break;
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        if (row < tl.row_end) {
          __nv_bfloat16* dst = p.c + static_cast<long long>(row) * p.ldc + col;
          if (vec_ok && col + 32 <= p.N) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(r[8 * i + 0]) * alpha, __uint_as_float(r[8 * i + 1]) * alpha);
              v.y = pack_bf16(__uint_as_float(r[8 * i + 2]) * alpha, __uint_as_float(r[8 * i + 3]) * alpha);
              v.z = pack_bf16(__uint_as_float(r[8 * i + 4]) * alpha, __uint_as_float(r[8 * i + 5]) * alpha);
              v.w = pack_bf16(__uint_as_float(r[8 * i + 6]) * alpha, __uint_as_float(r[8 * i + 7]) * alpha);
              *reinterpret_cast<uint4*>(dst + 8 * i) = v;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < p.N) dst[i] = __float2bfloat16(__uint_as_float(r[i]) * alpha);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      ++iter;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// scales [rows, S] row-major -> atoms [ceil(rows/128)][ceil(S/4)][512]; the output is zero-filled first by the caller.
__global__ void sf_swizzle_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, long long rows, int S) {
  const long long n = rows * S;
  const long long s4 = (S + 3) / 4;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / S;
    const int s = static_cast<int>(i - r * S);
    const long long atom = (r / 128) * s4 + s / 4;
    const int rr = static_cast<int>(r % 128);
    out[atom * ATOM_BYTES + (rr % 32) * 16 + (rr / 32) * 4 + (s % 4)] = in[i];
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::string g_mx_err;
EncodeTiledFn g_mx_encode = nullptr;
std::once_flag g_mx_once;

int mx_fail(const std::string& m) {
  g_mx_err = m;
  return -1;
}

// byte matrix [rows, row_bytes] with a [128 rows, 128 bytes] box, 128-byte swizzle
int make_byte_map(CUtensorMap* map, const void* ptr, long long rows, long long row_bytes, long long pitch_bytes, int box_rows) {
  std::call_once(g_mx_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_mx_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  if (!g_mx_encode) return mx_fail("cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || pitch_bytes % 16 != 0) return mx_fail("operand must be 16-byte aligned with a 16-byte pitch");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(STAGE_K_BYTES), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = g_mx_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mx_fail("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return 0;
}

template <int KIND, int BN>
int launch_mx(const MxGemmProblem& q, cudaStream_t stream) {
  constexpr int STAGES = BN == 256 ? 4 : (KIND == 0 ? 6 : 5);
  constexpr int SF_BYTES = (KIND == 0 ? 1 : 4) * ATOM_BYTES;
  constexpr int NB = BN / 128;
  constexpr int SMEM = STAGES * ((1 + NB) * TILE_BYTES + (1 + NB) * SF_BYTES) + 8 * (2 * STAGES + 5) + 1024;
  const long long kbytes = KIND == 0 ? q.K : q.K / 2;
  CUtensorMap ma, mb_;
  if (make_byte_map(&ma, q.a, q.a_rows, kbytes, q.a_pitch_bytes, BM)) return -1;
  if (make_byte_map(&mb_, q.b, q.b_rows, kbytes, q.b_pitch_bytes, BN)) return -1;
  auto kern = gemm_mx_kernel<KIND, BN, STAGES>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)  // per (function, device)
    return mx_fail("cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
  MxArgs ka;
  memset(&ka, 0, sizeof(ka));
  ka.mode = q.mode;
  ka.M = q.M;
  ka.N = q.N;
  ka.K = q.K;
  ka.num_groups = q.num_groups;
  ka.max_tiles = q.max_tiles;
  ka.tile_group = q.tile_group;
  ka.num_m_tiles = q.num_m_tiles;
  ka.sfa = q.sfa;
  ka.sfb = q.sfb;
  ka.c = static_cast<__nv_bfloat16*>(q.c);
  ka.ldc = q.ldc;
  ka.alpha = q.alpha;
  ka.alpha_dev = q.alpha_dev;
  ka.b_rows = q.b_rows;
  ka.status = q.status;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long m_tiles = q.mode == GEMM_GROUPED_ROWS ? q.max_tiles : (q.M + BM - 1) / BM;
  const long long tiles = m_tiles * ((q.N + BN - 1) / BN);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  if (grid <= 0) return 0;
  kern<<<grid, kThreads, SMEM, stream>>>(ma, mb_, ka);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return mx_fail(std::string("block-scaled gemm launch failed: ") + cudaGetErrorString(e));
  return 0;
}

}  // namespace

const char* gemm_mx_last_error() { return g_mx_err.c_str(); }

int gemm_mx_launch(const MxGemmProblem& q, cudaStream_t stream) {
  if (q.M <= 0 || q.N <= 0) return 0;
  if (q.kind != 0 && q.kind != 1) return mx_fail("kind must be 0 (MXFP8) or 1 (NVFP4)");
  const int kstep = q.kind == 0 ? 128 : 256;
  if (q.K <= 0 || q.K % kstep != 0) return mx_fail("K must be a positive multiple of 128 (MXFP8) or 256 (NVFP4)");
  if (q.mode != GEMM_DENSE && q.mode != GEMM_GROUPED_ROWS) return mx_fail("block-scaled GEMM supports the dense and grouped-rows modes");
  if (q.mode == GEMM_GROUPED_ROWS && (!q.tile_group || !q.num_m_tiles || q.N % 128 != 0))
    return mx_fail("grouped-rows block-scaled GEMM needs tile_group, num_m_tiles and N % 128 == 0");
  if (!q.sfa || !q.sfb) return mx_fail("scale-factor atoms are required");
  if ((reinterpret_cast<uintptr_t>(q.sfa) & 15) != 0 || (reinterpret_cast<uintptr_t>(q.sfb) & 15) != 0)
    return mx_fail("scale-factor atoms must be 16-byte aligned");
  // The 256-wide tile halves the shared-memory traffic per flop (these kinds are otherwise bound by it); it has one
  // accumulator, so it is used when its tiles still fill the GPU and waste no columns.
  const long long m_tiles = q.mode == GEMM_GROUPED_ROWS ? q.max_tiles : (q.M + BM - 1) / BM;
  int bn = q.block_n;
  if (bn == 0) bn = (q.N % 256 == 0 && m_tiles * (q.N / 256) >= 148) ? 256 : 128;
  if (bn != 128 && bn != 256) return mx_fail("block_n must be 128 or 256");
  if (bn == 256) return q.kind == 0 ? launch_mx<0, 256>(q, stream) : launch_mx<1, 256>(q, stream);
  return q.kind == 0 ? launch_mx<0, 128>(q, stream) : launch_mx<1, 128>(q, stream);
}

void sf_swizzle(const uint8_t* in, uint8_t* out, long long rows, int S, cudaStream_t s) {
  if (rows * S <= 0) return;
  long long b = (rows * S + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  sf_swizzle_kernel<<<static_cast<int>(b), 256, 0, s>>>(in, out, rows, S);
}

}  // namespace mb
