// Paged-KV decode attention (one query token per sequence, GQA), split over the KV length.
//
// Cache layout: k_cache / v_cache are [num_slots, Hk, 128] bf16 where slot = page * page_size + offset
// and block_table[b, i] is the i-th page of sequence b. Grid = (B, Hk, splits); every CTA serves all
// G = Hq/Hk query heads of one KV head over its slice of the context so that each K/V row is read from
// HBM exactly once. Partial (max, sum, out) triples are merged by a second kernel.
//
// Reference counterpart: flashinfer's trtllm_mha decode backend selected by the B200 recipe
// (scripts/run_qwen3_30b_a3b.py:311-324).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "launchers.h"

namespace mb {
namespace {

using bf16 = __nv_bfloat16;
constexpr int D = 128;
constexpr int WARPS = 4;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, int num_splits) {
  const long long bh = blockIdx.x;  // b * Hq + head
  const int d = threadIdx.x;
  float gm = -FLT_MAX;
  for (int s = 0; s < num_splits; ++s) gm = fmaxf(gm, part_ml[(bh * num_splits + s) * 2]);
  float gl = 0.f, go = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float mm = part_ml[(bh * num_splits + s) * 2];
    const float c = mm == -FLT_MAX ? 0.f : __expf(mm - gm);
    gl += part_ml[(bh * num_splits + s) * 2 + 1] * c;
    go += part_o[(bh * num_splits + s) * D + d] * c;
  }
  out[bh * D + d] = __float2bfloat16(gl > 0.f ? go / gl : 0.f);
}


// ---------------------------------------------------------------------------------------------------
// Tensor-core variant: K/V pages are staged through shared memory with cp.async (double buffered, 64
// tokens per stage) and the G query heads of one KV head form the (zero padded) 16-row A operand of
// mma.sync m16n8k16, so the work per K/V byte is a handful of instructions and the kernel runs at the
// speed of the cache stream. Each of the 4 warps owns 16 tokens of a stage and keeps its own running
// (max, sum, out); warps are merged through shared memory at the end.
constexpr int TOK = 64;          // tokens per stage
constexpr int LDS = D + 8;       // padded row (272 B) -> conflict-free ldmatrix
constexpr int STAGE_ELEMS = TOK * LDS;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

template <int G>
__global__ void __launch_bounds__(WARPS * 32)
decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                  const int* __restrict__ block_table, const int* __restrict__ seq_lens, float* __restrict__ part_o,
                  float* __restrict__ part_ml, bf16* __restrict__ out, int Hq, int Hk, int page_size, int max_pages,
                  int num_splits, float scale, long long num_slots, int* __restrict__ status) {
  extern __shared__ __align__(16) unsigned char dsm[];
  bf16* Ks = reinterpret_cast<bf16*>(dsm);            // [2][TOK][LDS]
  bf16* Vs = Ks + 2 * STAGE_ELEMS;                    // [2][TOK][LDS]
  const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The length and the page ids come from device memory the caller filled: a length beyond the block-table row is
  // clamped, and a page outside the cache is read as zeros (status 9) instead of being dereferenced.
  int len = seq_lens[b];
  const long long row_cap = static_cast<long long>(max_pages) * page_size;
  if (len < 0 || len > row_cap) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, 8);
    len = len < 0 ? 0 : static_cast<int>(row_cap);
  }
  int per = (len + num_splits - 1) / num_splits;
  per = (per + TOK - 1) / TOK * TOK;
  const int t_lo = split * per;
  const int t_hi = min(len, t_lo + per);
  const int n_chunks = t_hi > t_lo ? (t_hi - t_lo + TOK - 1) / TOK : 0;
  const int* table = block_table + static_cast<long long>(b) * max_pages;

  // Q fragments: rows >= G are zero padding
  uint32_t qa[8][4];
  {
    const int r0 = lane >> 2, c = (lane & 3) * 2;
    const bf16* q0 = q + (static_cast<long long>(b) * Hq + h * G + r0) * D;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c) : 0u;
      qa[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c + 8) : 0u;
      qa[ks][1] = 0u;  // rows 8..15 exist only as padding (G <= 8)
      qa[ks][3] = 0u;
    }
  }
  float m_run = -FLT_MAX, l_run = 0.f;  // row lane/4
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  auto issue = [&](int chunk, int stage) {
    const int base = t_lo + chunk * TOK;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int piece = threadIdx.x + i * (WARPS * 32);
      const int r = piece >> 4, c16 = piece & 15;
      const int t = base + r;
      bool ok = t < t_hi;
      long long slot = 0;
      if (ok) {
        const long long page = table[t / page_size];
        if (page < 0 || (num_slots > 0 && (page + 1) * page_size > num_slots)) {
          ok = false;
          if (c16 == 0 && status) atomicCAS(status, 0, 9);
        } else {
          slot = page * page_size + (t % page_size);
        }
      }
      const long long off = (slot * Hk + h) * D + c16 * 8;
      const uint32_t dk = static_cast<uint32_t>(__cvta_generic_to_shared(Ks + stage * STAGE_ELEMS + r * LDS + c16 * 8));
      const uint32_t dv = static_cast<uint32_t>(__cvta_generic_to_shared(Vs + stage * STAGE_ELEMS + r * LDS + c16 * 8));
      cp_async16(dk, k_cache + off, ok ? 16 : 0);
      cp_async16(dv, v_cache + off, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  if (n_chunks > 0) issue(0, 0);
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int stage = ch & 1;
    if (ch + 1 < n_chunks) {
      issue(ch + 1, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const bf16* Kst = Ks + stage * STAGE_ELEMS + (warp * 16) * LDS;
    const bf16* Vst = Vs + stage * STAGE_ELEMS + (warp * 16) * LDS;
    // ---- S = Q K^T for this warp's 16 tokens (two 8-token n-tiles)
    float sacc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {  // 32 dims per ldmatrix.x4
        uint32_t b0, b1, b2, b3;
        const bf16* addr = Kst + (nt * 8 + (lane & 7)) * LDS + kp * 32 + (lane >> 3) * 8;
        ldsm_x4(static_cast<uint32_t>(__cvta_generic_to_shared(addr)), b0, b1, b2, b3);
        mma16816(sacc[nt], qa[2 * kp], b0, b1);
        mma16816(sacc[nt], qa[2 * kp + 1], b2, b3);
      }
    }
    // ---- online softmax on row lane/4 (values c0, c1 of both n-tiles)
    const int tok0 = t_lo + ch * TOK + warp * 16 + (lane & 3) * 2;
    float sv[4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int t = tok0 + nt * 8 + e;
        sv[nt * 2 + e] = t < t_hi ? sacc[nt][e] * scale : -FLT_MAX;
      }
    float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float corr = m_new == -FLT_MAX ? 1.f : __expf(m_run - m_new);
    float pv[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) pv[e] = sv[e] == -FLT_MAX ? 0.f : __expf(sv[e] - m_new);
    l_run = l_run * corr + (pv[0] + pv[1] + pv[2] + pv[3]);
    m_run = m_new;
    uint32_t pa[4];
    pa[0] = pack_bf16x2(pv[0], pv[1]);
    pa[1] = 0u;
    pa[2] = pack_bf16x2(pv[2], pv[3]);
    pa[3] = 0u;
    // ---- O = O * corr + P V
#pragma unroll
    for (int jp = 0; jp < 8; ++jp) {  // two 8-dim n-tiles per ldmatrix.x4.trans
      uint32_t b0, b1, b2, b3;
      const bf16* addr = Vst + (((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + (2 * jp + (lane >> 4)) * 8;
      ldsm_x4_t(static_cast<uint32_t>(__cvta_generic_to_shared(addr)), b0, b1, b2, b3);
      o[2 * jp][0] *= corr; o[2 * jp][1] *= corr;
      o[2 * jp + 1][0] *= corr; o[2 * jp + 1][1] *= corr;
      mma16816(o[2 * jp], pa, b0, b1);
      mma16816(o[2 * jp + 1], pa, b2, b3);
    }
    __syncthreads();  // everyone is done with this stage before it is refilled
  }
  // ---- merge the four warps (rows < G only) and write this split's partial
  float lsum = l_run;
  lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
  lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
  float* sm_o = reinterpret_cast<float*>(dsm);              // [WARPS][8][D]
  float* sm_m = sm_o + WARPS * 8 * D;                        // [WARPS][8]
  float* sm_l = sm_m + WARPS * 8;
  const int r0 = lane >> 2;
  if (r0 < G) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      sm_o[(warp * 8 + r0) * D + j * 8 + (lane & 3) * 2] = o[j][0];
      sm_o[(warp * 8 + r0) * D + j * 8 + (lane & 3) * 2 + 1] = o[j][1];
    }
    if ((lane & 3) == 0) {
      sm_m[warp * 8 + r0] = m_run;
      sm_l[warp * 8 + r0] = lsum;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += WARPS * 32) {
    const int g = idx / D, d = idx - g * D;
    float gm = -FLT_MAX;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) gm = fmaxf(gm, sm_m[w * 8 + g]);
    float gl = 0.f, go = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float mw = sm_m[w * 8 + g];
      const float c = mw == -FLT_MAX ? 0.f : __expf(mw - gm);
      gl += sm_l[w * 8 + g] * c;
      go += sm_o[(w * 8 + g) * D + d] * c;
    }
    if (num_splits == 1) {  // nothing to merge: write the normalised output directly
      out[(static_cast<long long>(b) * Hq + h * G + g) * D + d] = __float2bfloat16(gl > 0.f ? go / gl : 0.f);
      continue;
    }
    const long long base = ((static_cast<long long>(b) * Hq + h * G + g) * num_splits + split);
    part_o[base * D + d] = go;
    if (d == 0) {
      part_ml[base * 2] = gm;
      part_ml[base * 2 + 1] = gl;
    }
  }
}

}  // namespace

// scratch: fp32 [B*Hq*num_splits*(128+2)]. `num_slots` = rows of the cache (0: page ids are not range-checked);
// `status` (may be null) receives 8 for a length beyond the block-table row, 9 for a page outside the cache.
// Returns the error of this call's own launches (cudaSuccess = 0), not whatever an earlier call left behind.
int paged_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                           const int* seq_lens, void* out, float* scratch, int B, int Hq, int Hk, int page_size,
                           int max_pages, int num_splits, float scale, cudaStream_t s, long long num_slots, int* status) {
  if (B <= 0) return 0;
  float* part_o = scratch;
  float* part_ml = scratch + static_cast<long long>(B) * Hq * num_splits * D;
  const dim3 grid(B, Hk, num_splits);
  const int G = Hq / Hk;
  constexpr int SMEM = 4 * STAGE_ELEMS * 2;  // K and V, two stages each
  const bf16 *qp = static_cast<const bf16*>(q), *kp = static_cast<const bf16*>(k_cache), *vp = static_cast<const bf16*>(v_cache);
  bf16* op = static_cast<bf16*>(out);
  void* args[] = {&qp, &kp, &vp, &block_table, &seq_lens, &part_o, &part_ml, &op, &Hq, &Hk, &page_size, &max_pages,
                  &num_splits, &scale, &num_slots, &status};
  const void* fn = nullptr;
  switch (G) {
    case 1: fn = reinterpret_cast<const void*>(&decode_mma_kernel<1>); break;
    case 2: fn = reinterpret_cast<const void*>(&decode_mma_kernel<2>); break;
    case 4: fn = reinterpret_cast<const void*>(&decode_mma_kernel<4>); break;
    case 8: fn = reinterpret_cast<const void*>(&decode_mma_kernel<8>); break;
    default: return static_cast<int>(cudaErrorInvalidValue);
  }
  // The attribute belongs to the (function, device) pair; setting it costs a table lookup, so it is set on every
  // call rather than remembered per process (a second device would otherwise launch with the 48 KB default).
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaLaunchKernel(fn, grid, dim3(WARPS * 32), args, SMEM, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (num_splits > 1) {
    const float *po = part_o, *pm = part_ml;
    void* margs[] = {&po, &pm, &op, &num_splits};
    e = cudaLaunchKernel(reinterpret_cast<const void*>(&decode_merge_kernel), dim3(B * Hq), dim3(D), margs, 0, s);
  }
  return static_cast<int>(e);
}

}  // namespace mb

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant (declared in noalloc.h): same kernels, split-KV partials in a fixed array that
// is part of the library image instead of a caller-provided scratch tensor.
#include <stdio.h>

#include <mutex>

#include "noalloc.h"

namespace {

// Partial outputs [B*Hq*splits][128] followed by partial (max, sum) pairs [B*Hq*splits][2].
static __device__ __align__(256) float g_noalloc_scratch[MB_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};  // device address of the array, per device
std::mutex g_scratch_mutex;
thread_local char g_noalloc_err[256] = "";

int noalloc_fail(int code, const char* msg) {
  snprintf(g_noalloc_err, sizeof(g_noalloc_err), "%s", msg);
  return code;
}

// In host code `g_noalloc_scratch` is only a handle of the symbol; the address kernels may use has to
// be asked from the runtime, once per device, with that device current.
int noalloc_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return noalloc_fail(MB_NOALLOC_ERR_CUDA, "cudaGetDevice failed");
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_noalloc_err, sizeof(g_noalloc_err), "cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
      return MB_NOALLOC_ERR_CUDA;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return MB_NOALLOC_OK;
}

}  // namespace

extern "C" const char* mb_noalloc_last_error(void) { return g_noalloc_err; }

extern "C" int mb_paged_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                                 const int* block_table, const int* seq_lens, void* out, int B, int Hq,
                                                 int Hk, int page_size, int max_pages, int num_splits, float scale,
                                                 long long num_slots, int* status, cudaStream_t stream) {
  if (!q || !k_cache || !v_cache || !block_table || !seq_lens || !out)
    return noalloc_fail(MB_NOALLOC_ERR_BAD_ARG, "null pointer argument");
  if (B <= 0 || Hq <= 0 || Hk <= 0 || page_size <= 0 || max_pages <= 0 || num_splits <= 0 || num_slots <= 0)
    return noalloc_fail(MB_NOALLOC_ERR_BAD_ARG, "extents must be positive");
  if (Hq % Hk != 0) return noalloc_fail(MB_NOALLOC_ERR_BAD_ARG, "Hq must be a multiple of Hk");
  const int G = Hq / Hk;
  if (G != 1 && G != 2 && G != 4 && G != 8)
    return noalloc_fail(MB_NOALLOC_ERR_BAD_ARG, "Hq / Hk must be 1, 2, 4 or 8");
  const unsigned long long need = 130ull * static_cast<unsigned long long>(B) * Hq * num_splits;
  if (need > MB_NOALLOC_SCRATCH_FLOATS) {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err),
             "B*Hq*num_splits*130 = %llu floats exceed the built-in scratch of %u floats; lower num_splits or the batch",
             need, MB_NOALLOC_SCRATCH_FLOATS);
    return MB_NOALLOC_ERR_TOO_LARGE;
  }
  float* scratch = nullptr;
  const int rc = noalloc_scratch_for_current_device(&scratch);
  if (rc != MB_NOALLOC_OK) return rc;
  // the launcher reports the result of its own launches; an error some earlier, unrelated call left in the
  // runtime's "last error" slot is neither read nor cleared here
  const int e = mb::paged_decode_attention(q, k_cache, v_cache, block_table, seq_lens, out, scratch, B, Hq, Hk, page_size,
                                           max_pages, num_splits, scale, stream, num_slots, status);
  if (e != 0) {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err), "kernel launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(e)));
    return MB_NOALLOC_ERR_CUDA;
  }
  return MB_NOALLOC_OK;
}
