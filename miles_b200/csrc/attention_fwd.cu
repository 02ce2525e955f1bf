// Causal variable-length flash attention forward on tcgen05 (training forward, log-prob passes, prefill).
//
// One CTA computes one (128-query tile, query head) pair and walks the KV sequence in blocks of 128:
//
//   warp 0     : TMA producer — Q once, then K_j / V_j into 2-stage rings (128B-swizzled boxes, no multicast)
//   warp 1     : TMEM allocator + MMA issuer — S_j = Q K_j^T (operands K-major) into one of two TMEM score
//                buffers, then O_j = P_j V_j (P from shared memory, V as an MN-major operand) into a TMEM buffer
//   warps 2..9 : softmax — two threads per query row (64 score columns each; the pair sits in two warps that
//                share a TMEM lane quadrant): tcgen05.ld of the scores, online max / sum with ex2, P_j written
//                as bf16 in the swizzled K-major layout the MMA expects. The output accumulates in TMEM across
//                blocks; it is rescaled in place only when a row maximum grows by more than 2^8 (the stale
//                maximum keeps P within bf16 range), which after the first blocks is rare.
//
// QK^T of block j+1 and P.V of block j-1 run while the softmax of block j computes, so the tensor core and the
// exp/FMA work overlap. GQA is handled by indexing the KV head as q_head / group. Log-sum-exp per (head, token) is written
// for the backward pass. Every mbarrier wait is bounded (see ptx.cuh).
//
// Reference counterpart: flash-attn 2 / FA4 varlen attention selected by `--attention-backend flash`
// (scripts/run_qwen3_30b_a3b.py:206).
#include <cuda.h>
#include <float.h>
#include <stdio.h>

#include <mutex>
#include <string>

#include "launchers.h"
#include "ptx.cuh"

namespace mb {
namespace {

constexpr int BM = 128;   // query rows per tile
constexpr int BN = 128;   // kv rows per block
constexpr int HD = 128;   // head dim
constexpr int ATOM_BYTES = 128 * 128;        // 128 rows x 128 B (one swizzle atom column)
constexpr int TILE_BYTES = 2 * ATOM_BYTES;   // 128 x 128 bf16
constexpr int KV_STAGES = 2;
constexpr int FA_THREADS = 320;
constexpr int FA_SMEM = TILE_BYTES * (2 + 2 * KV_STAGES) + 256 + 1024;  // Q, P, K ring, V ring, barriers, alignment

struct FaArgs {
  const int4* tiles;   // {q_row0 (global token index), q_rows, kv_row0 (sequence start), q_pos0 (position of q_row0 in its sequence)}
  int num_tiles;
  int Hq, Hk;
  __nv_bfloat16* out;  // [T, Hq, 128]
  float* lse;          // [Hq, T]
  long long T;
  float scale_log2;
  int* status;
};

__device__ __forceinline__ uint32_t swz_off(int row, int chunk16) {  // byte offset inside a 128x128B atom
  return static_cast<uint32_t>(row * 128 + ((chunk16 ^ (row & 7)) << 4));
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(FA_THREADS, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, const FaArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base;
  const uint32_t p_s = q_s + TILE_BYTES;
  const uint32_t k_s = p_s + TILE_BYTES;
  const uint32_t v_s = k_s + KV_STAGES * TILE_BYTES;
  const uint32_t bars = v_s + KV_STAGES * TILE_BYTES;
  // barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full, pv_done, pair[4]
  auto BAR = [&](int i) { return bars + 8u * i; };
  constexpr int B_QF = 0, B_KF = 1, B_KE = 3, B_VF = 5, B_VE = 7, B_SF = 9, B_PF = 11, B_PVD = 12, B_PAIR = 13;
  const uint32_t tmem_slot = bars + 8u * 17;
  __shared__ int abort_s;
  __shared__ float xch[2][2][BM];  // [buffer][column half][row]: values the two threads of a row exchange
  __shared__ uint32_t tmem_base_s;
  volatile int* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int4 tile = p.tiles[blockIdx.x];
  const int hq = blockIdx.y;
  const int hk = hq / (p.Hq / p.Hk);
  const int q_row0 = tile.x, q_rows = tile.y, kv_row0 = tile.z, q_pos0 = tile.w;
  const int kv_len = q_pos0 + q_rows;               // causal: keys up to the last query of the tile
  const int n_blocks = (kv_len + BN - 1) / BN;

  if (threadIdx.x == 0) {
    abort_s = 0;
    mbar_init(BAR(B_QF), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(BAR(B_KF + s), 1);
      mbar_init(BAR(B_KE + s), 1);
      mbar_init(BAR(B_VF + s), 1);
      mbar_init(BAR(B_VE + s), 1);
      mbar_init(BAR(B_SF + s), 1);
    }
    mbar_init(BAR(B_PF), 8);
    mbar_init(BAR(B_PVD), 1);
    for (int s = 0; s < 4; ++s) mbar_init(BAR(B_PAIR + s), 2);
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
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
  const uint32_t tmem = tmem_base_s;
  auto T_S = [&](int b) { return tmem + static_cast<uint32_t>(b) * 128u; };  // two score buffers
  const uint32_t t_O = tmem + 256;                                             // output accumulator
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(BAR(B_QF), TILE_BYTES);
      tma_load_2d(q_s, &map_q, BAR(B_QF), hq * HD, q_row0);
      tma_load_2d(q_s + ATOM_BYTES, &map_q, BAR(B_QF), hq * HD + 64, q_row0);
      auto load_k = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(BAR(B_KE + st), ((j >> 1) & 1) ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) return false;
        mbar_expect_tx(BAR(B_KF + st), TILE_BYTES);
        const uint32_t dst = k_s + st * TILE_BYTES;
        tma_load_2d(dst, &map_k, BAR(B_KF + st), hk * HD, kv_row0 + j * BN);
        tma_load_2d(dst + ATOM_BYTES, &map_k, BAR(B_KF + st), hk * HD + 64, kv_row0 + j * BN);
        return true;
      };
      auto load_v = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(BAR(B_VE + st), ((j >> 1) & 1) ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) return false;
        mbar_expect_tx(BAR(B_VF + st), TILE_BYTES);
        const uint32_t dst = v_s + st * TILE_BYTES;
        tma_load_2d(dst, &map_v, BAR(B_VF + st), hk * HD, kv_row0 + j * BN);
        tma_load_2d(dst + ATOM_BYTES, &map_v, BAR(B_VF + st), hk * HD + 64, kv_row0 + j * BN);
        return true;
      };
      ok = load_k(0);
      for (int j = 0; ok && j < n_blocks; ++j) {
        if (j + 1 < n_blocks) ok = load_k(j + 1);
        if (ok) ok = load_v(j);
      }
      if (!ok) {  // give copies in flight a bounded chance to land before shared memory is released
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_qk = make_idesc_bf16(BM, BN, false, false);  // S = Q K^T, both K-major over d
    constexpr uint32_t idesc_pv = make_idesc_bf16(BM, HD, false, true);   // O = P V, V is N(d)-contiguous
    bool ok = mbar_wait(BAR(B_QF), 0, abort_flag, p.status, ERR_WAIT_FULL);
    auto issue_qk = [&](int j) -> bool {
      const int st = j & 1;
      if (!mbar_wait(BAR(B_KF + st), (j >> 1) & 1, abort_flag, p.status, ERR_WAIT_FULL)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t kb = k_s + st * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * ATOM_BYTES + (k & 3) * 32;
          umma_f16(T_S(j & 1), make_smem_desc(q_s + off, 16, 1024), make_smem_desc(kb + off, 16, 1024), idesc_qk,
                   k > 0 ? 1u : 0u);
        }
        umma_commit(BAR(B_KE + st));
        umma_commit(BAR(B_SF + (j & 1)));
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int j = 0; ok && j < n_blocks; ++j) {
      // S[(j+1)&1] was last read for block j-1, whose softmax finished before p_full(j-1) was observed below.
      if (j + 1 < n_blocks) ok = issue_qk(j + 1);
      if (!ok) break;
      const int st = j & 1;
      if (!mbar_wait(BAR(B_PF), j & 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY) ||
          !mbar_wait(BAR(B_VF + st), (j >> 1) & 1, abort_flag, p.status, ERR_WAIT_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t vb = v_s + st * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint64_t adesc = make_smem_desc(p_s + (k >> 2) * ATOM_BYTES + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc(vb + k * 2048, ATOM_BYTES, 1024);
          umma_f16(t_O, adesc, bdesc, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(BAR(B_VE + st));
        umma_commit(BAR(B_PVD));
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ softmax (warps 2..9)
    const int quad = warp & 3;           // TMEM lane quadrant this warp may access
    const int half = (warp - 2) >> 2;    // which 64 score / output columns this thread owns
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t pair_bar = BAR(B_PAIR + quad);
    const int qpos = q_pos0 + row;
    float m_used = -INFINITY, l = 0.f;
    uint32_t sr[64];
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      const int b = j & 1;
      if (!mbar_wait(BAR(B_SF + b), (j >> 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t s_addr = T_S(b) + lane_addr + half * 64;
      tmem_ld_32x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
      tmem_ld_32x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
      tmem_ld_wait();
      float mx = -INFINITY;
      const int col0 = j * BN + half * 64;
      if (j * BN + BN - 1 > q_pos0) {  // block reaches past the first query of the tile: apply the causal mask
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          float s = __uint_as_float(sr[i]) * p.scale_log2;
          s = (col0 + i > qpos) ? -INFINITY : s;
          sr[i] = __float_as_uint(s);
          mx = fmaxf(mx, s);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float s = __uint_as_float(sr[i]) * p.scale_log2;
          sr[i] = __float_as_uint(s);
          mx = fmaxf(mx, s);
        }
      }
      // exchange the half-row maxima with the thread that owns the other 64 columns of this row
      xch[b][half][row] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(pair_bar);
      if (!mbar_wait(pair_bar, j & 1, abort_flag, p.status, ERR_WAIT_PEER)) {
        ok = false;
        break;
      }
      mx = fmaxf(mx, xch[b][half ^ 1][row]);
      const float m_new = fmaxf(m_used, mx);
      const bool grow = m_new > m_used + 8.f;  // also true on the first finite maximum
      const bool any_grow = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      if (any_grow) {
        alpha = (m_new == -INFINITY) ? 1.f : ex2(m_used - m_new);
        m_used = m_new;
        l *= alpha;
      }
      const float base_m = (m_used == -INFINITY) ? 0.f : m_used;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p0 = ex2(__uint_as_float(sr[2 * i]) - base_m);
        const float p1 = ex2(__uint_as_float(sr[2 * i + 1]) - base_m);
        sum += p0 + p1;
        sr[i] = pack_bf16(p0, p1);
      }
      l += sum;
      if (j > 0) {
        // P.V of the previous block must have finished: it reads the P buffer and accumulates into O.
        if (!mbar_wait(BAR(B_PVD), (j - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (any_grow) {
          uint32_t o[32];
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            const uint32_t o_addr = t_O + lane_addr + half * 64 + c * 32;
            tmem_ld_32x32(o_addr, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(o_addr, o);
          }
          tmem_st_wait();
        }
      }
      const uint32_t p_row = p_s + half * ATOM_BYTES;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + swz_off(row, c)), "r"(sr[4 * c]),
                     "r"(sr[4 * c + 1]), "r"(sr[4 * c + 2]), "r"(sr[4 * c + 3])
                     : "memory");
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(B_PF));
    }
    // ---- epilogue: O / l -> bf16, log-sum-exp
    if (ok && n_blocks > 0) ok = mbar_wait(BAR(B_PVD), (n_blocks - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      const int b = n_blocks & 1;
      xch[b][half][row] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(pair_bar);
      ok = mbar_wait(pair_bar, n_blocks & 1, abort_flag, p.status, ERR_WAIT_PEER);
      if (ok) {
        const float l_tot = l + xch[b][half ^ 1][row];
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        const bool live = row < q_rows;
        __nv_bfloat16* dst = p.out + (static_cast<long long>(q_row0 + row) * p.Hq + hq) * HD + half * 64;
        uint32_t o[32];
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          tmem_ld_32x32(t_O + lane_addr + half * 64 + c * 32, o);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
              v.y = pack_bf16(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
              v.z = pack_bf16(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
              v.w = pack_bf16(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = v;
            }
          }
        }
        if (live && half == 0 && p.lse)
          p.lse[static_cast<long long>(hq) * p.T + q_row0 + row] =
              l_tot > 0.f ? (m_used + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::string g_fa_err;
EncodeTiledFn g_fa_encode = nullptr;
std::once_flag g_fa_once;

int fa_fail(const std::string& m) {
  g_fa_err = m;
  return -1;
}

// bf16 [rows, heads*128] view with an arbitrary row pitch; box = 64 columns x 128 rows, 128-byte swizzle.
int fa_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld) {
  std::call_once(g_fa_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_fa_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  if (!g_fa_encode) return fa_fail("cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return fa_fail("attention operand base must be 16-byte aligned");
  if ((ld * 2) % 16 != 0) return fa_fail("attention operand row pitch must be a multiple of 16 bytes");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64u, 128u};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = g_fa_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fa_fail("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return 0;
}

}  // namespace

const char* flash_attn_last_error() { return g_fa_err.c_str(); }

int flash_attn_fwd(const void* q, long long q_ld, const void* k, long long k_ld, const void* v, long long v_ld,
                   void* out, float* lse, const int* tiles, int num_tiles, long long Tq, long long Tkv, int Hq, int Hk,
                   int head_dim, float scale, int* status, cudaStream_t stream) {
  if (head_dim != HD) return fa_fail("flash_attn_fwd supports head_dim 128 only");
  if (Hq % Hk != 0) return fa_fail("query heads must be a multiple of kv heads");
  if (num_tiles == 0) return 0;
  CUtensorMap mq, mk, mv;
  if (fa_make_map(&mq, q, Tq, static_cast<long long>(Hq) * HD, q_ld)) return -1;
  if (fa_make_map(&mk, k, Tkv, static_cast<long long>(Hk) * HD, k_ld)) return -1;
  if (fa_make_map(&mv, v, Tkv, static_cast<long long>(Hk) * HD, v_ld)) return -1;
  if (cudaFuncSetAttribute(fa_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM) != cudaSuccess)  // per device
    return fa_fail("cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed for attention");
  FaArgs a;
  a.tiles = reinterpret_cast<const int4*>(tiles);
  a.num_tiles = num_tiles;
  a.Hq = Hq;
  a.Hk = Hk;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.T = Tq;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  fa_fwd_kernel<<<dim3(num_tiles, Hq), FA_THREADS, FA_SMEM, stream>>>(mq, mk, mv, a);
  if (cudaGetLastError() != cudaSuccess) return fa_fail("attention forward launch failed");
  return 0;
}

}  // namespace mb
