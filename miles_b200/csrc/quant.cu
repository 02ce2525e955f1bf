// Block-scaled quantisers used by the trainer -> rollout weight update and the offline converters.
//
//   MXFP8  : 1x32 blocks, E4M3 values, E8M0 scale = 2^ceil(log2(amax/448)) (OCP MX, scale rounded up
//            so that no element saturates).
//   NVFP4  : 1x16 blocks, E2M1 values packed two per byte (low nibble first), E4M3 block scale and one
//            fp32 per-tensor scale: S_enc = 448*6/global_amax, block scale = e4m3(block_amax/6 * S_enc),
//            q = e2m1(x * S_enc / block_scale); decode scale = 1/S_enc.
//   FP8 128x128 : one fp32 scale per block = max(amax, 1e-10)/448, optionally rounded up to a power of
//            two (UE8M0).
//   INT4   : fake-quant over [group_rows, group_cols] groups, symmetric (scale = max|x|/7) or asymmetric
//            (scale = (max-min)/15 with a zero point in [0, 15]); returns the integer-valued tensor,
//            the scales and the zero points.
//
// Reference counterparts: miles/utils/mxfp8.py:8-35, miles/utils/nvfp4.py:19-145,
// miles/utils/fp8_kernel.py:24-79 and
// miles/backends/megatron_utils/kernels/int4_qat/fake_int4_quant_cuda.cu:29-259.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "launchers.h"
#include "quant_math.cuh"

namespace mb {
namespace {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

using namespace qmath;

// ---------------------------------------------------------------- MXFP8: one warp per 32-block row strip
__global__ void mxfp8_quant_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sc,
                                   long long rows, long long cols) {
  const long long nblk = rows * (cols / 32);
  const int lane = threadIdx.x & 31;
  for (long long blk = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; blk < nblk;
       blk += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const float v = __bfloat162float(x[blk * 32 + lane]);
    const float amax = warp_max(fabsf(v));
    const uint8_t e = e8m0_ceil(amax / 448.f);
    const float inv = 1.f / e8m0_to_float(e);
    q[blk * 32 + lane] = to_e4m3(v * inv);
    if (lane == 0) sc[blk] = e;
  }
}
__global__ void mxfp8_dequant_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sc, bf16* __restrict__ x,
                                     long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    x[i] = __float2bfloat16(from_e4m3(q[i]) * e8m0_to_float(sc[i >> 5]));
}

// ---------------------------------------------------------------- NVFP4: 16 lanes per block
__global__ void nvfp4_quant_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sc,
                                   const float* __restrict__ global_amax, long long rows, long long cols) {
  const long long n = rows * cols;
  float genc = (448.f * 6.f) / *global_amax;
  if (!(genc < FLT_MAX)) genc = FLT_MAX;
  if (genc == 0.f || *global_amax == 0.f) genc = 1.f;
  const int lane = threadIdx.x & 31;
  for (long long base = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) - lane; base < n;
       base += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long i = base + lane;
    const bool valid = i < n;  // n is a multiple of 16, so a 16-lane half is entirely valid or not
    const float v = valid ? __bfloat162float(x[i]) : 0.f;
    float amax = fabsf(v);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const uint8_t sf8 = to_e4m3(amax / 6.f * genc);
    const float sf = from_e4m3(sf8);
    const float enc = sf > 0.f ? genc / sf : 0.f;
    const uint8_t code = to_e2m1(v * enc);
    const uint8_t hi = __shfl_down_sync(0xffffffffu, code, 1);
    if (!valid) continue;
    if ((i & 1) == 0) q[i >> 1] = static_cast<uint8_t>(code | (hi << 4));
    if ((i & 15) == 0) sc[i >> 4] = sf8;
  }
}
__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sc,
                                     const float* __restrict__ global_amax, bf16* __restrict__ x, long long n) {
  float genc = (448.f * 6.f) / *global_amax;
  if (genc == 0.f || *global_amax == 0.f) genc = 1.f;
  const float gdec = 1.f / genc;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint8_t b = q[i >> 1];
    const uint8_t c = (i & 1) ? (b >> 4) : (b & 15);
    x[i] = __float2bfloat16(from_e2m1(c) * from_e4m3(sc[i >> 4]) * gdec);
  }
}

__global__ void absmax_kernel(const bf16* __restrict__ x, long long n, float* __restrict__ out) {
  float m = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    m = fmaxf(m, fabsf(__bfloat162float(x[i])));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));  // valid for m >= 0
}

// ---------------------------------------------------------------- FP8 128x128 blocks: one CTA per block
__global__ void fp8_block_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ sc,
                                 long long rows, long long cols, int ue8m0) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const long long br = blockIdx.y, bc = blockIdx.x;
  const long long r0 = br * 128, c0 = bc * 128;
  float m = 0.f;
  for (int i = threadIdx.x; i < 128 * 128; i += blockDim.x) {
    const long long r = r0 + i / 128, c = c0 + i % 128;
    if (r < rows && c < cols) m = fmaxf(m, fabsf(__bfloat162float(x[r * cols + c])));
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = red[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) t = fmaxf(t, red[w]);
    float s = fmaxf(t, 1e-10f) / 448.f;
    if (ue8m0) s = e8m0_to_float(e8m0_ceil(s));
    s_scale = s;
    sc[br * gridDim.x + bc] = s;
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  for (int i = threadIdx.x; i < 128 * 128; i += blockDim.x) {
    const long long r = r0 + i / 128, c = c0 + i % 128;
    if (r < rows && c < cols) q[r * cols + c] = to_e4m3(__bfloat162float(x[r * cols + c]) * inv);
  }
}

// ---------------------------------------------------------------- INT4 fake quant: one warp per group
__global__ void int4_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, bf16* __restrict__ scale,
                            bf16* __restrict__ zero, long long rows, long long cols, int gr, int gc, int sym) {
  const long long groups_c = (cols + gc - 1) / gc, groups_r = (rows + gr - 1) / gr;
  const long long ngroups = groups_r * groups_c;
  const int lane = threadIdx.x & 31;
  const int gsize = gr * gc;
  for (long long g = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; g < ngroups;
       g += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const long long r0 = (g / groups_c) * gr, c0 = (g % groups_c) * gc;
    float mx = -FLT_MAX, mn = FLT_MAX, amax = 0.f;
    for (int i = lane; i < gsize; i += 32) {
      const long long r = r0 + i / gc, c = c0 + i % gc;
      const float v = (r < rows && c < cols) ? __bfloat162float(x[r * cols + c]) : 0.f;
      mx = fmaxf(mx, v);
      mn = fminf(mn, v);
      amax = fmaxf(amax, fabsf(v));
    }
    mx = warp_max(mx);
    mn = warp_min(mn);
    amax = warp_max(amax);
    float s, z = 0.f;
    if (sym) {
      s = fmaxf(amax * (1.f / 7.f), 1e-5f);
    } else {
      s = fmaxf((mx - mn) * (1.f / 15.f), 1e-5f);
      z = fminf(fmaxf(-rintf(mn / s), 0.f), 15.f);
    }
    for (int i = lane; i < gsize; i += 32) {
      const long long r = r0 + i / gc, c = c0 + i % gc;
      if (r < rows && c < cols) {
        const float v = __bfloat162float(x[r * cols + c]);
        y[r * cols + c] = __float2bfloat16(rintf(v / s) + z);
      }
    }
    if (lane == 0) {
      scale[g] = __float2bfloat16(s);
      if (!sym) zero[g] = __float2bfloat16(z);
    }
  }
}

int grid_for(long long items, int threads, int cap = 148 * 16) {
  long long b = (items + threads - 1) / threads;
  if (b < 1) b = 1;
  return static_cast<int>(b < cap ? b : cap);
}

}  // namespace

void quant_mxfp8(const void* x, uint8_t* q, uint8_t* scales, long long rows, long long cols, cudaStream_t s) {
  if (rows * cols <= 0) return;
  mxfp8_quant_kernel<<<grid_for(rows * cols, 256), 256, 0, s>>>(static_cast<const bf16*>(x), q, scales, rows, cols);
}
void dequant_mxfp8(const uint8_t* q, const uint8_t* scales, void* x, long long rows, long long cols, cudaStream_t s) {
  if (rows * cols <= 0) return;
  mxfp8_dequant_kernel<<<grid_for(rows * cols, 256), 256, 0, s>>>(q, scales, static_cast<bf16*>(x), rows * cols);
}
void quant_nvfp4(const void* x, uint8_t* q, uint8_t* block_scales, const float* global_amax, long long rows,
                 long long cols, cudaStream_t s) {
  if (rows * cols <= 0) return;
  nvfp4_quant_kernel<<<grid_for(rows * cols, 256), 256, 0, s>>>(static_cast<const bf16*>(x), q, block_scales, global_amax,
                                                               rows, cols);
}
void dequant_nvfp4(const uint8_t* q, const uint8_t* block_scales, const float* global_amax, void* x, long long rows,
                   long long cols, cudaStream_t s) {
  if (rows * cols <= 0) return;
  nvfp4_dequant_kernel<<<grid_for(rows * cols, 256), 256, 0, s>>>(q, block_scales, global_amax, static_cast<bf16*>(x),
                                                                 rows * cols);
}
void absmax(const void* x, long long n, float* out, cudaStream_t s) {
  if (n <= 0) return;
  absmax_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, s>>>(static_cast<const bf16*>(x), n, out);
}
void quant_fp8_block128(const void* x, uint8_t* q, float* scales, long long rows, long long cols, bool ue8m0,
                        cudaStream_t s) {
  if (rows * cols <= 0) return;
  dim3 grid(static_cast<unsigned>((cols + 127) / 128), static_cast<unsigned>((rows + 127) / 128));
  fp8_block_kernel<<<grid, 256, 0, s>>>(static_cast<const bf16*>(x), q, scales, rows, cols, ue8m0 ? 1 : 0);
}
void fake_int4_quant(const void* x, void* y, void* scale, void* zero, long long rows, long long cols, int group_rows,
                     int group_cols, bool symmetric, cudaStream_t s) {
  if (rows * cols <= 0) return;
  const long long groups = ((rows + group_rows - 1) / group_rows) * ((cols + group_cols - 1) / group_cols);
  int4_kernel<<<grid_for(groups * 32, 256), 256, 0, s>>>(static_cast<const bf16*>(x), static_cast<bf16*>(y),
                                                         static_cast<bf16*>(scale), static_cast<bf16*>(zero), rows, cols,
                                                         group_rows, group_cols, symmetric ? 1 : 0);
}

}  // namespace mb
