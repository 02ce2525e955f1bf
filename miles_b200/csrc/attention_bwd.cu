// Causal variable-length flash attention backward on tcgen05 (training).
//
// One CTA owns one block of 128 keys of one sequence and one KV head. Its dK / dV accumulate in TMEM over every
// query tile (64 rows) at or after the block and over the G = Hq / Hk query heads that share the KV head, so K, V
// stay in shared memory for the whole CTA and dK / dV leave the chip once. Everything is computed transposed
// (keys on the TMEM lanes), which makes P^T and dS^T row-per-thread:
//
//   S^T  = K Q^T            [128 keys x 64 q]   A = K (K-major over d),  B = Q  (K-major over d)
//   dP^T = V dO^T           [128 keys x 64 q]   A = V,                   B = dO
//   P^T  = exp2(S^T * scale*log2e - lse*log2e), dS^T = P^T o (dP^T - D)        (256 threads, two per key row)
//   dV  += P^T  dO          [128 keys x 128 d]  A = P^T  (smem, K-major over q), B = dO (smem, d contiguous)
//   dK  += dS^T Q           [128 keys x 128 d]  A = dS^T (smem, K-major over q), B = Q  (smem, d contiguous)
//   dQ^T = K^T dS^T         [128 d x 64 q]      A = K (d contiguous),           B = dS^T (q contiguous)
//
// dQ is accumulated across key blocks with fp32 `red.global.add` into a scratch tensor (one warp covers 32
// consecutive d of one query row per instruction) and converted to bf16 by a second kernel; D = rowsum(dO o O)
// and lse * log2e come from a first one.
//
//   warp 0      : TMA producer: K, V once; then (Q, dO) tiles into a 3-stage ring, with the tile's lse / D rows
//   warp 1      : TMEM allocator + MMA issuer
//   warps 2..9  : P^T / dS^T math, two threads per key row (32 query columns each); dK / dV epilogue
//   warps 10..13: dQ^T read-out and global accumulation (one thread per d)
//
// TMEM columns: S^T 0..63, dP^T 64..127, dV 128..255, dK 256..383, dQ^T 384..447. Every mbarrier wait is bounded
// (ptx.cuh): on expiry the CTA records a status code, leaves its loops, frees TMEM and returns.
//
// Reference counterpart: the flash-attention backward behind `--attention-backend flash`
// (scripts/run_qwen3_30b_a3b.py:203).
#include <cuda.h>
#include <float.h>

#include <mutex>
#include <string>

#include "launchers.h"
#include "ptx.cuh"

namespace mb {
namespace {

constexpr int BQ = 64;    // query rows per tile
constexpr int BK = 128;   // keys per CTA
constexpr int HD = 128;
constexpr int ATOM_K = BK * 128;     // 128 rows x 128 B
constexpr int ATOM_Q = BQ * 128;     // 64 rows x 128 B
constexpr int KTILE = 2 * ATOM_K;    // K or V block
constexpr int QTILE = 2 * ATOM_Q;    // Q or dO tile
constexpr int PTILE = ATOM_K;        // P^T or dS^T: 128 keys x 64 q
constexpr int STAGES = 3;
constexpr int BWD_THREADS = 14 * 32;
constexpr int BWD_SMEM = 2 * KTILE + 2 * PTILE + STAGES * 2 * QTILE + STAGES * 2 * BQ * 4 + 256 + 1024;

struct FaBwdArgs {
  const int4* blocks;  // {kv_row0 (global token index of the block's first key), kv_rows, kv_pos0 (its position in the
                       //  sequence), seq_end (global token index one past the sequence)}
  int Hq, Hk;
  const float* lse2;   // [Hq, T] log-sum-exp * log2(e)
  const float* dsum;   // [Hq, T] rowsum(dO o O)
  float* dq_acc;       // [T, Hq, 128] fp32, zeroed by the caller
  __nv_bfloat16* dk;   // [T, Hk, 128]
  __nv_bfloat16* dv;
  long long T;
  float scale, scale_log2;
  int* status;
};

__device__ __forceinline__ uint32_t swz_off(int row, int chunk16) {
  return static_cast<uint32_t>(row * 128 + ((chunk16 ^ (row & 7)) << 4));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void red_add_f32(float* p, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

__global__ void __launch_bounds__(BWD_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
              const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const FaBwdArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t k_s = base;
  const uint32_t v_s = k_s + KTILE;
  const uint32_t pt_s = v_s + KTILE;
  const uint32_t ds_s = pt_s + PTILE;
  const uint32_t ring = ds_s + PTILE;                      // per stage: Q tile, dO tile
  const uint32_t stats = ring + STAGES * 2 * QTILE;        // per stage: lse2[64], dsum[64]
  const uint32_t bars = stats + STAGES * 2 * BQ * 4;
  auto BAR = [&](int i) { return bars + 8u * i; };
  constexpr int B_KVF = 0, B_QF = 1, B_QE = 4, B_SF = 7, B_PF = 8, B_DQF = 9, B_DQE = 10, B_FIN = 11;
  const uint32_t tmem_slot = bars + 8u * 12;
  __shared__ int abort_s;
  __shared__ uint32_t tmem_base_s;
  volatile int* abort_flag = &abort_s;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));   // generic pointer to the aligned base
  float* stats_g = reinterpret_cast<float*>(gen + (stats - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int4 blk = p.blocks[blockIdx.x];
  const int hk = blockIdx.y;
  const int G = p.Hq / p.Hk;
  const int kv_row0 = blk.x, kv_rows = blk.y, kv_pos0 = blk.z, seq_end = blk.w;
  // query rows at or after the block's first key (positions kv_pos0 ..): global rows kv_row0 .. seq_end - 1
  const int q_total = seq_end - kv_row0;
  const int n_qt = (q_total + BQ - 1) / BQ;
  const int n_it = n_qt * G;

  if (threadIdx.x == 0) {
    abort_s = 0;
    mbar_init(BAR(B_KVF), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(BAR(B_QF + s), 1);
      mbar_init(BAR(B_QE + s), 1);
    }
    mbar_init(BAR(B_SF), 1);
    mbar_init(BAR(B_PF), 8);
    mbar_init(BAR(B_DQF), 1);
    mbar_init(BAR(B_DQE), 4);
    mbar_init(BAR(B_FIN), 1);
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_do);
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
  const uint32_t t_S = tmem, t_dP = tmem + 64, t_dV = tmem + 128, t_dK = tmem + 256, t_dQ = tmem + 384;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    bool ok = true;
    if (lane == 0) {
      mbar_expect_tx(BAR(B_KVF), 2 * KTILE);
      tma_load_2d(k_s, &map_k, BAR(B_KVF), hk * HD, kv_row0);
      tma_load_2d(k_s + ATOM_K, &map_k, BAR(B_KVF), hk * HD + 64, kv_row0);
      tma_load_2d(v_s, &map_v, BAR(B_KVF), hk * HD, kv_row0);
      tma_load_2d(v_s + ATOM_K, &map_v, BAR(B_KVF), hk * HD + 64, kv_row0);
    }
    for (int it = 0; ok && it < n_it; ++it) {
      const int st = it % STAGES;
      const int g = it / n_qt, qt = it - g * n_qt;
      const int hq = hk * G + g;
      const int q_row0 = kv_row0 + qt * BQ;
      if (!mbar_wait(BAR(B_QE + st), ((it / STAGES) & 1) ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) {
        ok = false;
        break;
      }
      // the tile's softmax statistics (rows past the sequence read a clamped row and are masked by the consumers)
      float* sp = stats_g + st * 2 * BQ;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = min(q_row0 + h * 32 + lane, seq_end - 1);
        sp[h * 32 + lane] = p.lse2[static_cast<long long>(hq) * p.T + r];
        sp[BQ + h * 32 + lane] = p.dsum[static_cast<long long>(hq) * p.T + r];
      }
      __syncwarp();
      if (lane == 0) {
        mbar_expect_tx(BAR(B_QF + st), 2 * QTILE);
        const uint32_t qd = ring + st * 2 * QTILE, dd = qd + QTILE;
        tma_load_2d(qd, &map_q, BAR(B_QF + st), hq * HD, q_row0);
        tma_load_2d(qd + ATOM_Q, &map_q, BAR(B_QF + st), hq * HD + 64, q_row0);
        tma_load_2d(dd, &map_do, BAR(B_QF + st), hq * HD, q_row0);
        tma_load_2d(dd + ATOM_Q, &map_do, BAR(B_QF + st), hq * HD + 64, q_row0);
      }
    }
    if (!ok && lane == 0) {  // give copies in flight a bounded chance to land before shared memory is released
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) {
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t id_s = make_idesc_bf16(BK, BQ, false, false);    // S^T, dP^T
    constexpr uint32_t id_acc = make_idesc_bf16(BK, HD, false, true);   // dV, dK: A K-major (q), B d-contiguous
    constexpr uint32_t id_dq = make_idesc_bf16(HD, BQ, true, true);     // dQ^T: A d-contiguous, B q-contiguous
    bool ok = mbar_wait(BAR(B_KVF), 0, abort_flag, p.status, ERR_WAIT_FULL);
    auto issue_s = [&](int it) -> bool {
      const int st = it % STAGES;
      if (!mbar_wait(BAR(B_QF + st), (it / STAGES) & 1, abort_flag, p.status, ERR_WAIT_FULL)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t qd = ring + st * 2 * QTILE, dd = qd + QTILE;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t ka = (k >> 2) * ATOM_K + (k & 3) * 32, qa = (k >> 2) * ATOM_Q + (k & 3) * 32;
          umma_f16(t_S, make_smem_desc(k_s + ka, 16, 1024), make_smem_desc(qd + qa, 16, 1024), id_s, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t ka = (k >> 2) * ATOM_K + (k & 3) * 32, qa = (k >> 2) * ATOM_Q + (k & 3) * 32;
          umma_f16(t_dP, make_smem_desc(v_s + ka, 16, 1024), make_smem_desc(dd + qa, 16, 1024), id_s, k > 0 ? 1u : 0u);
        }
        umma_commit(BAR(B_SF));
      }
      __syncwarp();
      return true;
    };
    if (ok && n_it > 0) ok = issue_s(0);
    for (int it = 0; ok && it < n_it; ++it) {
      const int st = it % STAGES;
      if (!mbar_wait(BAR(B_PF), it & 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t qd = ring + st * 2 * QTILE, dd = qd + QTILE;
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k) {  // contraction over the 64 queries of the tile
          umma_f16(t_dV, make_smem_desc(pt_s + k * 32, 16, 1024), make_smem_desc(dd + k * 2048, ATOM_Q, 1024), id_acc,
                   (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k) {
          umma_f16(t_dK, make_smem_desc(ds_s + k * 32, 16, 1024), make_smem_desc(qd + k * 2048, ATOM_Q, 1024), id_acc,
                   (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(BAR(B_QE + st));  // the (Q, dO) stage is free once these have run
      }
      __syncwarp();
      if (it + 1 < n_it && !issue_s(it + 1)) {
        ok = false;
        break;
      }
      // dQ^T of this tile overwrites the read-out buffer of the previous one
      if (it > 0 && !mbar_wait(BAR(B_DQE), (it - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {  // contraction over the 128 keys
          umma_f16(t_dQ, make_smem_desc(k_s + k * 2048, ATOM_K, 1024), make_smem_desc(ds_s + k * 2048, ATOM_K, 1024), id_dq,
                   k > 0 ? 1u : 0u);
        }
        umma_commit(BAR(B_DQF));
      }
      __syncwarp();
    }
    if (ok && lane == 0) umma_commit(BAR(B_FIN));
    __syncwarp();
  } else if (warp < 10) {
    // ------------------------------------------------------------------ P^T / dS^T (two threads per key row)
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;                   // key row inside the block
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const bool key_ok = row < kv_rows;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int st = it % STAGES;
      const int g = it / n_qt, qt = it - g * n_qt;
      if (!mbar_wait(BAR(B_SF), it & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s[32], d[32];
      tmem_ld_32x32(t_S + lane_addr + half * 32, s);
      tmem_ld_32x32(t_dP + lane_addr + half * 32, d);
      tmem_ld_wait();
      const float* sp = stats_g + st * 2 * BQ + half * 32;
      // query j of this thread sits at sequence offset qt*64 + half*32 + j from the block's first key
      const int q_off0 = qt * BQ + half * 32;
      const int q_left = q_total - q_off0;              // queries of the tile half that exist
      uint32_t pp[16], dd[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float pv[2], dv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = 2 * j + e;
          const bool live = key_ok && c < q_left && row <= q_off0 + c;   // causal: key position <= query position
          const float pe = live ? ex2(__uint_as_float(s[c]) * p.scale_log2 - sp[c]) : 0.f;
          pv[e] = pe;
          dv[e] = pe * (__uint_as_float(d[c]) - sp[BQ + c]);
        }
        pp[j] = pack_bf16(pv[0], pv[1]);
        dd[j] = pack_bf16(dv[0], dv[1]);
      }
      // the P^T / dS^T tiles are still read by the MMAs of the previous tile until its dQ^T has run
      if (it > 0 && !mbar_wait(BAR(B_DQF), (it - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t o = swz_off(row, half * 4 + c);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(pt_s + o), "r"(pp[4 * c]), "r"(pp[4 * c + 1]),
                     "r"(pp[4 * c + 2]), "r"(pp[4 * c + 3])
                     : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ds_s + o), "r"(dd[4 * c]), "r"(dd[4 * c + 1]),
                     "r"(dd[4 * c + 2]), "r"(dd[4 * c + 3])
                     : "memory");
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(B_PF));
    }
    // ---- epilogue: dV, dK (scaled) -> bf16
    if (ok) ok = mbar_wait(BAR(B_FIN), 0, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      const long long orow = (static_cast<long long>(kv_row0 + row) * p.Hk + hk) * HD + half * 64;
      uint32_t o[32];
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = (which == 0 ? t_dV : t_dK) + lane_addr + half * 64;
        __nv_bfloat16* dst = (which == 0 ? p.dv : p.dk) + orow;
        const float sc = which == 0 ? 1.f : p.scale;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          tmem_ld_32x32(src + c * 32, o);
          tmem_ld_wait();
          if (key_ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(o[8 * i]) * sc, __uint_as_float(o[8 * i + 1]) * sc);
              v.y = pack_bf16(__uint_as_float(o[8 * i + 2]) * sc, __uint_as_float(o[8 * i + 3]) * sc);
              v.z = pack_bf16(__uint_as_float(o[8 * i + 4]) * sc, __uint_as_float(o[8 * i + 5]) * sc);
              v.w = pack_bf16(__uint_as_float(o[8 * i + 6]) * sc, __uint_as_float(o[8 * i + 7]) * sc);
              *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = v;
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ dQ^T read-out (one thread per d)
    const int quad = warp & 3;
    const int drow = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    for (int it = 0; it < n_it; ++it) {
      const int g = it / n_qt, qt = it - g * n_qt;
      const int hq = hk * G + g;
      if (!mbar_wait(BAR(B_DQF), it & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      uint32_t a[32], b[32];
      tmem_ld_32x32(t_dQ + lane_addr, a);
      tmem_ld_32x32(t_dQ + lane_addr + 32, b);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(B_DQE));
      const int q_row0 = kv_row0 + qt * BQ;
      const int q_left = seq_end - q_row0;
      float* dst = p.dq_acc + (static_cast<long long>(q_row0) * p.Hq + hq) * HD + drow;
      const long long pitch = static_cast<long long>(p.Hq) * HD;
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (c < q_left) red_add_f32(dst + c * pitch, __uint_as_float(a[c]) * p.scale);
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (32 + c < q_left) red_add_f32(dst + (32 + c) * pitch, __uint_as_float(b[c]) * p.scale);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// D[h, t] = sum_d dO[t, h, d] * O[t, h, d];  lse2[h, t] = lse[h, t] * log2(e). One warp per (t, h).
__global__ void fa_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                   const float* __restrict__ lse, float* __restrict__ dsum, float* __restrict__ lse2,
                                   long long T, int Hq) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= T * Hq) return;
  const long long t = w / Hq;
  const int h = static_cast<int>(w - t * Hq);
  const uint2 a = reinterpret_cast<const uint2*>(o + w * HD)[lane];
  const uint2 b = reinterpret_cast<const uint2*>(d_o + w * HD)[lane];
  const __nv_bfloat162* ab = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* bb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(ab[i]), y = __bfloat1622float2(bb[i]);
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    dsum[static_cast<long long>(h) * T + t] = s;
    lse2[static_cast<long long>(h) * T + t] = lse[static_cast<long long>(h) * T + t] * 1.4426950408889634f;
  }
}

__global__ void f32_to_bf16_kernel(const float4* __restrict__ in, uint2* __restrict__ out, long long n4) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = in[i];
    uint2 o;
    o.x = pack_bf16(v.x, v.y);
    o.y = pack_bf16(v.z, v.w);
    out[i] = o;
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::string g_err;
EncodeTiledFn g_encode = nullptr;
std::once_flag g_once;

int fail(const std::string& m) {
  g_err = m;
  return -1;
}

// bf16 [rows, heads*128] view with row pitch `ld` elements; box = 64 columns x `box_rows` rows, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld, unsigned box_rows) {
  std::call_once(g_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  if (!g_encode) return fail("cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return fail("attention operand base must be 16-byte aligned");
  if ((ld * 2) % 16 != 0) return fail("attention operand row pitch must be a multiple of 16 bytes");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64u, box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return 0;
}

}  // namespace

const char* flash_attn_bwd_last_error() { return g_err.c_str(); }

// q, d_o, o: [T, Hq, 128] (q and d_o with row pitches q_ld / do_ld elements, o contiguous); k, v: [T, Hk, 128] with
// pitches; lse [Hq, T]; blocks int32 [n, 4]; scratch fp32: dq_acc [T*Hq*128] (zeroed here) then dsum [Hq*T], lse2 [Hq*T].
int flash_attn_bwd(const void* q, long long q_ld, const void* k, long long k_ld, const void* v, long long v_ld, const void* o,
                   const void* d_o, long long do_ld, const float* lse, const int* blocks, int num_blocks, long long T, int Hq,
                   int Hk, int head_dim, float scale, float* scratch, void* dq, void* dk, void* dv, int* status,
                   cudaStream_t stream) {
  if (head_dim != HD) return fail("flash_attn_bwd supports head_dim 128 only");
  if (Hq % Hk != 0) return fail("query heads must be a multiple of kv heads");
  if (T <= 0 || num_blocks <= 0) return 0;
  float* dq_acc = scratch;
  float* dsum = scratch + T * Hq * HD;
  float* lse2 = dsum + T * Hq;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, sizeof(float) * T * Hq * HD, stream);
  if (e != cudaSuccess) return fail("cudaMemsetAsync failed for the dQ accumulator");
  {
    const long long warps = T * Hq;
    const long long blocks_n = (warps * 32 + 255) / 256;
    fa_bwd_prep_kernel<<<static_cast<unsigned>(blocks_n), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), lse, dsum, lse2, T, Hq);
  }
  CUtensorMap mq, mdo, mk, mv;
  if (make_map(&mq, q, T, static_cast<long long>(Hq) * HD, q_ld, BQ)) return -1;
  if (make_map(&mdo, d_o, T, static_cast<long long>(Hq) * HD, do_ld, BQ)) return -1;
  if (make_map(&mk, k, T, static_cast<long long>(Hk) * HD, k_ld, BK)) return -1;
  if (make_map(&mv, v, T, static_cast<long long>(Hk) * HD, v_ld, BK)) return -1;
  if (cudaFuncSetAttribute(fa_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess)
    return fail("cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed for the attention backward");
  FaBwdArgs a;
  a.blocks = reinterpret_cast<const int4*>(blocks);
  a.Hq = Hq;
  a.Hk = Hk;
  a.lse2 = lse2;
  a.dsum = dsum;
  a.dq_acc = dq_acc;
  a.dk = static_cast<__nv_bfloat16*>(dk);
  a.dv = static_cast<__nv_bfloat16*>(dv);
  a.T = T;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  fa_bwd_kernel<<<dim3(num_blocks, Hk), BWD_THREADS, BWD_SMEM, stream>>>(mq, mdo, mk, mv, a);
  if (cudaPeekAtLastError() != cudaSuccess) return fail("attention backward launch failed");
  const long long n4 = T * Hq * HD / 4;
  long long cb = (n4 + 255) / 256;
  if (cb > 148 * 8) cb = 148 * 8;
  f32_to_bf16_kernel<<<static_cast<unsigned>(cb), 256, 0, stream>>>(reinterpret_cast<const float4*>(dq_acc),
                                                                   reinterpret_cast<uint2*>(dq), n4);
  return 0;
}

}  // namespace mb
