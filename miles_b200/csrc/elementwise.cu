// Bandwidth-bound fused kernels of the transformer block: RMSNorm (fwd/bwd), per-head QK-RMSNorm +
// rotary embedding (fwd/bwd, optionally scattering K/V into a paged cache), SwiGLU (fwd/bwd) and the
// fused Adam update. All rows are processed with 128-bit loads/stores and fp32 arithmetic.
//
// Reference counterparts: TransformerEngine RMSNorm / fused RoPE / bias-SwiGLU and FusedAdam as used
// by the Megatron trainer (miles/backends/megatron_utils/model.py:125-210, 560-570).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launchers.h"

namespace mb {
namespace {

using bf16 = __nv_bfloat16;

struct alignas(16) BF8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  const BF8 r = *reinterpret_cast<const BF8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  BF8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<BF8*>(p) = r;
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  const float r = red[0];
  __syncthreads();
  return r;
}

// ------------------------------------------------------------------ RMSNorm
// One CTA per row; H % 8 == 0. Optionally adds a residual first: h = x + res, writes h to res_out.
template <int THREADS>
__global__ void rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                                   const bf16* __restrict__ w, bf16* __restrict__ y, bf16* __restrict__ res_out,
                                   float* __restrict__ rstd, int H, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const bf16* xr = x + row * H;
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < H; c += THREADS * 8) {
    float f[8];
    load8(xr + c, f);
    if (res) {
      float g[8];
      load8(res + row * H + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      // round through bf16 so that the statistics match what is stored
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i]));
      store8(res_out + row * H + c, f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  const float tot = block_sum<THREADS>(ss, red);
  const float r = rsqrtf(tot / H + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  const bf16* src = res ? res_out + row * H : xr;
  for (int c = threadIdx.x * 8; c < H; c += THREADS * 8) {
    float f[8], g[8];
    load8(src + c, f);
    load8(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * r * g[i];
    store8(y + row * H + c, f);
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)); dw partials are accumulated per CTA over a strip of rows.
template <int THREADS>
__global__ void rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                   const bf16* __restrict__ w, const float* __restrict__ rstd,
                                   const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                   float* __restrict__ dw_partial, int T, int H) {
  __shared__ float red[32];
  extern __shared__ float dw_acc[];  // [H]
  for (int c = threadIdx.x; c < H; c += THREADS) dw_acc[c] = 0.f;
  __syncthreads();
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const float r = rstd[row];
    float dot = 0.f;
    for (int c = threadIdx.x * 8; c < H; c += THREADS * 8) {
      float a[8], b[8], g[8];
      load8(dy + row * H + c, a);
      load8(x + row * H + c, b);
      load8(w + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot += a[i] * g[i] * b[i] * r;
    }
    const float mean = block_sum<THREADS>(dot, red) / H;
    for (int c = threadIdx.x * 8; c < H; c += THREADS * 8) {
      float a[8], b[8], g[8], o[8];
      load8(dy + row * H + c, a);
      load8(x + row * H + c, b);
      load8(w + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xhat = b[i] * r;
        o[i] = r * (a[i] * g[i] - xhat * mean);
        dw_acc[c + i] += a[i] * xhat;
      }
      if (dres) {
        float e[8];
        load8(dres + row * H + c, e);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += e[i];
      }
      store8(dx + row * H + c, o);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += THREADS) dw_partial[static_cast<long long>(blockIdx.x) * H + c] = dw_acc[c];
}

__global__ void colsum_kernel(const float* __restrict__ part, float* __restrict__ out, int rows, int H, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int r = 0; r < rows; ++r) s += part[static_cast<long long>(r) * H + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ------------------------------------------------------------------ QK-norm + RoPE
// qkv: [T, (Hq + 2*Hk) * D] as produced by the fused QKV projection (q heads, then k heads, then v heads).
// One warp per (token, head); D == 128 (4 elements per lane: lane l holds d = l*4.. and the rotation
// partner d+64 lives in lane l+16, so pairs are exchanged with a shuffle).
// Outputs: q_out [T, Hq, D], k_out [T, Hk, D] (v is consumed in place by the attention kernels).
// When kv_cache pointers are given, K and V rows are also scattered to slot_mapping[t] of the paged cache.
// inv_freq_tab (64 floats, or null): inverse frequencies of a model with scaled rotary embeddings (Llama-3.1 style or
// linear scaling); null means theta^(-d/64).
__global__ void qk_norm_rope_fwd_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ qw,
                                        const bf16* __restrict__ kw, const int* __restrict__ pos,
                                        bf16* __restrict__ q_out, bf16* __restrict__ k_out,
                                        float* __restrict__ q_rstd, float* __restrict__ k_rstd,
                                        bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                        const int* __restrict__ slot_mapping, int T, int Hq, int Hk,
                                        float theta, float eps, int use_norm, const float* __restrict__ inv_freq_tab,
                                        int rot_half) {
  constexpr int D = 128;
  const int warps_per_block = blockDim.x >> 5;
  const long long gw = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hk;
  if (gw >= static_cast<long long>(T) * heads) return;
  const int t = gw / heads;
  const int h = gw - static_cast<long long>(t) * heads;
  const bf16* src = qkv + (static_cast<long long>(t) * heads + h) * D + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  if (h >= Hq + Hk) {  // V head: only the cache scatter
    if (v_cache) {
      const int slot = slot_mapping[t];
      if (slot >= 0)
        *reinterpret_cast<uint2*>(v_cache + (static_cast<long long>(slot) * Hk + (h - Hq - Hk)) * D + lane * 4) = raw;
    }
    return;
  }
  const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float f[4];
  {
    const float2 a = __bfloat1622float2(rb[0]), b = __bfloat1622float2(rb[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  const bool is_q = h < Hq;
  float r = 1.f;
  if (use_norm) {
    float ss = f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3];
    ss = warp_sum(ss);
    r = rsqrtf(ss / D + eps);
    const bf16* w = (is_q ? qw : kw) + lane * 4;
    const uint2 wr = *reinterpret_cast<const uint2*>(w);
    const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wr);
    const float2 a = __bfloat1622float2(wb[0]), b = __bfloat1622float2(wb[1]);
    // match the unfused path: normalised value is rounded to bf16 before the rotation
    f[0] = __bfloat162float(__float2bfloat16(f[0] * r * a.x));
    f[1] = __bfloat162float(__float2bfloat16(f[1] * r * a.y));
    f[2] = __bfloat162float(__float2bfloat16(f[2] * r * b.x));
    f[3] = __bfloat162float(__float2bfloat16(f[3] * r * b.y));
    if (lane == 0) {
      if (is_q && q_rstd) q_rstd[static_cast<long long>(t) * Hq + h] = r;
      if (!is_q && k_rstd) k_rstd[static_cast<long long>(t) * Hk + (h - Hq)] = r;
    }
  }
  // rotate-half RoPE: out[d] = x[d]*cos - x[d+64]*sin (d<64); out[d+64] = x[d+64]*cos + x[d]*sin
  const float p = static_cast<float>(pos[t]);
  float o[4];
#pragma unroll
  // rot_half = 64: the whole head rotates (dimension d pairs with d + 64). rot_half = 32: only the first 64 dimensions
  // do (d pairs with d + 32), the rest passes through (partial rotary embedding).
  const int hl = rot_half >> 2;  // lanes per half
  for (int i = 0; i < 4; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, f[i], hl);
    if (lane >= 2 * hl) {
      o[i] = f[i];
      continue;
    }
    const int d = (lane & (hl - 1)) * 4 + i;  // frequency index in [0, rot_half)
    const float inv_freq = inv_freq_tab ? inv_freq_tab[d] : powf(theta, -static_cast<float>(d) / static_cast<float>(rot_half));
    float s, c;
    sincosf(p * inv_freq, &s, &c);
    o[i] = (lane & hl) == 0 ? f[i] * c - partner * s : f[i] * c + partner * s;
  }
  uint2 outv;
  outv.x = pack2(o[0], o[1]);
  outv.y = pack2(o[2], o[3]);
  if (is_q) {
    *reinterpret_cast<uint2*>(q_out + (static_cast<long long>(t) * Hq + h) * D + lane * 4) = outv;
  } else {
    const int hk = h - Hq;
    if (k_out) *reinterpret_cast<uint2*>(k_out + (static_cast<long long>(t) * Hk + hk) * D + lane * 4) = outv;
    if (k_cache) {
      const int slot = slot_mapping[t];
      if (slot >= 0) *reinterpret_cast<uint2*>(k_cache + (static_cast<long long>(slot) * Hk + hk) * D + lane * 4) = outv;
    }
  }
}

// Backward of the kernel above. dq [T,Hq,D], dk [T,Hk,D], dv [T,Hk,D] -> dqkv [T, heads*D];
// weight gradients of the head norms are accumulated with atomics into fp32 [D] buffers.
__global__ void qk_norm_rope_bwd_kernel(const bf16* __restrict__ dq, const bf16* __restrict__ dk,
                                        const bf16* __restrict__ dv, const bf16* __restrict__ qkv,
                                        const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                                        const int* __restrict__ pos, const float* __restrict__ q_rstd,
                                        const float* __restrict__ k_rstd, bf16* __restrict__ dqkv,
                                        float* __restrict__ dqw, float* __restrict__ dkw, int T, int Hq, int Hk,
                                        float theta, int use_norm, const float* __restrict__ inv_freq_tab, int rot_half) {
  constexpr int D = 128;
  __shared__ float wacc[2][D];
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&wacc[0][0])[i] = 0.f;
  __syncthreads();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hk;
  const long long total = static_cast<long long>(T) * heads;
  for (long long gw = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); gw < total;
       gw += static_cast<long long>(gridDim.x) * warps_per_block) {
    const int t = gw / heads;
    const int h = gw - static_cast<long long>(t) * heads;
    bf16* dst = dqkv + (static_cast<long long>(t) * heads + h) * D + lane * 4;
    if (h >= Hq + Hk) {
      *reinterpret_cast<uint2*>(dst) =
          *reinterpret_cast<const uint2*>(dv + (static_cast<long long>(t) * Hk + (h - Hq - Hk)) * D + lane * 4);
      continue;
    }
    const bool is_q = h < Hq;
    const bf16* gsrc = is_q ? dq + (static_cast<long long>(t) * Hq + h) * D + lane * 4
                            : dk + (static_cast<long long>(t) * Hk + (h - Hq)) * D + lane * 4;
    const uint2 graw = *reinterpret_cast<const uint2*>(gsrc);
    const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&graw);
    float g[4];
    {
      const float2 a = __bfloat1622float2(gb[0]), b = __bfloat1622float2(gb[1]);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    }
    // inverse rotation: dx[d] = g[d]*cos + g[d+64]*sin ; dx[d+64] = g[d+64]*cos - g[d]*sin
    const float p = static_cast<float>(pos[t]);
    float dn[4];
#pragma unroll
    const int hl = rot_half >> 2;  // lanes per half (see the forward kernel)
    for (int i = 0; i < 4; ++i) {
      const float partner = __shfl_xor_sync(0xffffffffu, g[i], hl);
      if (lane >= 2 * hl) {
        dn[i] = g[i];
        continue;
      }
      const int d = (lane & (hl - 1)) * 4 + i;
      const float inv_freq = inv_freq_tab ? inv_freq_tab[d] : powf(theta, -static_cast<float>(d) / static_cast<float>(rot_half));
      float s, c;
      sincosf(p * inv_freq, &s, &c);
      dn[i] = (lane & hl) == 0 ? g[i] * c + partner * s : g[i] * c - partner * s;
    }
    float o[4];
    if (use_norm) {
      const uint2 xr = *reinterpret_cast<const uint2*>(qkv + (static_cast<long long>(t) * heads + h) * D + lane * 4);
      const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xr);
      const float2 xa = __bfloat1622float2(xb[0]), xc = __bfloat1622float2(xb[1]);
      const float x[4] = {xa.x, xa.y, xc.x, xc.y};
      const uint2 wr = *reinterpret_cast<const uint2*>((is_q ? qw : kw) + lane * 4);
      const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wr);
      const float2 wa = __bfloat1622float2(wb[0]), wc = __bfloat1622float2(wb[1]);
      const float w[4] = {wa.x, wa.y, wc.x, wc.y};
      const float r = is_q ? q_rstd[static_cast<long long>(t) * Hq + h] : k_rstd[static_cast<long long>(t) * Hk + (h - Hq)];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) dot += dn[i] * w[i] * x[i] * r;
      dot = warp_sum(dot) / D;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float xhat = x[i] * r;
        o[i] = r * (dn[i] * w[i] - xhat * dot);
        atomicAdd(&wacc[is_q ? 0 : 1][lane * 4 + i], dn[i] * xhat);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = dn[i];
    }
    uint2 outv;
    outv.x = pack2(o[0], o[1]);
    outv.y = pack2(o[2], o[3]);
    *reinterpret_cast<uint2*>(dst) = outv;
  }
  __syncthreads();
  if (use_norm) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      if (dqw) atomicAdd(dqw + i, wacc[0][i]);
      if (dkw) atomicAdd(dkw + i, wacc[1][i]);
    }
  }
}

// ------------------------------------------------------------------ SwiGLU
// in: [T, 2I] = [gate | up]; out: [T, I] = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, long long T, int I) {
  const long long n8 = T * (I / 8);
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n8;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / (I / 8);
    const int c = (idx - row * (I / 8)) * 8;
    float g[8], u[8], o[8];
    load8(in + row * 2 * I + c, g);
    load8(in + row * 2 * I + I + c, u);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    store8(out + row * I + c, o);
  }
}

__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ in,
                                  bf16* __restrict__ din, long long T, int I) {
  const long long n8 = T * (I / 8);
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n8;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / (I / 8);
    const int c = (idx - row * (I / 8)) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(in + row * 2 * I + c, g);
    load8(in + row * 2 * I + I + c, u);
    load8(dout + row * I + c, d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float s = 1.f / (1.f + __expf(-g[i]));
      const float silu = g[i] * s;
      du[i] = d[i] * silu;
      dg[i] = d[i] * u[i] * (s + silu * (1.f - s));
    }
    store8(din + row * 2 * I + c, dg);
    store8(din + row * 2 * I + I + c, du);
  }
}

// ------------------------------------------------------------------ fused Adam(W)
// One flat buffer per call. The parameter is bf16; its fp32 master copy is kept in one of two forms:
//   * `master` (fp32 array), or
//   * `lo` (16-bit array): the master is split over the bf16 weight itself and a signed 16-bit remainder,
//         master_bits = (weight_bits << 16) + lo,     weight_bits = (master_bits + 0x8000) >> 16,
//     so the weight the GEMMs read is the master rounded to nearest (ties away from zero) and the pair
//     reconstructs every fp32 bit. An update far below half a bf16 ulp therefore accumulates in `lo`
//     instead of being rounded away; memory per parameter is 4 bytes instead of 6.
// With neither, the update is applied to the bf16 value itself (only sensible for large learning rates).
// The gradient is bf16 or fp32; moments are fp32 or bf16. `skip_flag` / `grad_scale` are read from device
// memory so that the clip coefficient computed by a previous kernel never travels through the host.
// Eight elements per thread, 128-bit loads and stores; the host launcher handles a ragged tail.
template <typename T>
__device__ __forceinline__ void adam_load8(const T* p, float (&o)[8]);
template <>
__device__ __forceinline__ void adam_load8<bf16>(const bf16* p, float (&o)[8]) {
  load8(p, o);
}
template <>
__device__ __forceinline__ void adam_load8<float>(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
  o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void adam_store8(T* p, const float (&o)[8]);
template <>
__device__ __forceinline__ void adam_store8<bf16>(bf16* p, const float (&o)[8]) {
  store8(p, o);
}
template <>
__device__ __forceinline__ void adam_store8<float>(float* p, const float (&o)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(o[4], o[5], o[6], o[7]);
}

struct AdamScalars {
  float lr, b1, b2, eps, wd, bc1, bc2;
};

__device__ __forceinline__ float adam_update(float w, float grad, float& mi, float& vi, const AdamScalars& a) {
  mi = a.b1 * mi + (1.f - a.b1) * grad;
  vi = a.b2 * vi + (1.f - a.b2) * grad * grad;
  const float upd = (mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps);
  return w - a.lr * (upd + a.wd * w);
}

__device__ __forceinline__ float split_join(unsigned short hi, short lo) {
  return __uint_as_float((static_cast<unsigned>(hi) << 16) + static_cast<unsigned>(static_cast<int>(lo)));
}
__device__ __forceinline__ void split_cut(float w, unsigned short& hi, short& lo) {
  const unsigned bits = __float_as_uint(w);
  const unsigned h = (bits + 0x8000u) >> 16;
  hi = static_cast<unsigned short>(h);
  lo = static_cast<short>(static_cast<int>(bits - (h << 16)));
}

template <typename GT, typename MT>
__global__ void adam_kernel(bf16* __restrict__ p, float* __restrict__ master, short* __restrict__ lo,
                            const GT* __restrict__ g, MT* __restrict__ m, MT* __restrict__ v, long long n,
                            AdamScalars a, const float* __restrict__ grad_scale, const float* __restrict__ skip_flag) {
  if (skip_flag && *skip_flag != 0.f) return;
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long long n8 = n / 8;
  for (long long i8 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i8 < n8;
       i8 += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long i = i8 * 8;
    float gr[8], mi[8], vi[8], w[8];
    adam_load8<GT>(g + i, gr);
    adam_load8<MT>(m + i, mi);
    adam_load8<MT>(v + i, vi);
    uint4 pw = *reinterpret_cast<const uint4*>(p + i);
    unsigned short* ph = reinterpret_cast<unsigned short*>(&pw);
    uint4 lw;
    short* pl = reinterpret_cast<short*>(&lw);
    if (master) {
      adam_load8<float>(master + i, w);
    } else if (lo) {
      lw = *reinterpret_cast<const uint4*>(lo + i);
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = split_join(ph[j], pl[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = __uint_as_float(static_cast<unsigned>(ph[j]) << 16);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = adam_update(w[j], gr[j] * gs, mi[j], vi[j], a);
    adam_store8<MT>(m + i, mi);
    adam_store8<MT>(v + i, vi);
    if (master) {
      adam_store8<float>(master + i, w);
      store8(p + i, w);
    } else if (lo) {
#pragma unroll
      for (int j = 0; j < 8; ++j) split_cut(w[j], ph[j], pl[j]);
      *reinterpret_cast<uint4*>(p + i) = pw;
      *reinterpret_cast<uint4*>(lo + i) = lw;
    } else {
      store8(p + i, w);
    }
  }
  // ragged tail (fewer than eight elements): first threads of block 0
  if (blockIdx.x == 0 && threadIdx.x < n - n8 * 8) {
    const long long i = n8 * 8 + threadIdx.x;
    float mi = static_cast<float>(m[i]), vi = static_cast<float>(v[i]);
    unsigned short hi = reinterpret_cast<unsigned short*>(p)[i];
    float w = master ? master[i] : (lo ? split_join(hi, lo[i]) : __uint_as_float(static_cast<unsigned>(hi) << 16));
    w = adam_update(w, static_cast<float>(g[i]) * gs, mi, vi, a);
    m[i] = static_cast<MT>(mi);
    v[i] = static_cast<MT>(vi);
    if (master) {
      master[i] = w;
      p[i] = __float2bfloat16(w);
    } else if (lo) {
      short l;
      split_cut(w, hi, l);
      reinterpret_cast<unsigned short*>(p)[i] = hi;
      lo[i] = l;
    } else {
      p[i] = __float2bfloat16(w);
    }
  }
}

// master[i] = join(p[i], lo[i]) (fp32 view of a split master, for checkpoints and checks)
__global__ void split_master_join_kernel(const bf16* __restrict__ p, const short* __restrict__ lo, float* __restrict__ out,
                                         long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = split_join(reinterpret_cast<const unsigned short*>(p)[i], lo[i]);
}
// (p[i], lo[i]) = cut(master[i])
__global__ void split_master_cut_kernel(const float* __restrict__ master, bf16* __restrict__ p, short* __restrict__ lo,
                                        long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    unsigned short hi;
    short l;
    split_cut(master[i], hi, l);
    reinterpret_cast<unsigned short*>(p)[i] = hi;
    lo[i] = l;
  }
}

// ------------------------------------------------------------------ counter-based normal initialisation
// out[i] = std * N(key, first + i): Philox4x32-10 keyed by `key`, counter = element index / 4, Box-Muller on the four
// 32-bit outputs. The value of an element depends only on (key, its index in the logical tensor), so any sharding
// of the tensor (expert parallel, tensor parallel, pipeline stages) draws the same model, and a 30 B parameter
// model is filled at memory speed instead of through thousands of generator calls.
__device__ __forceinline__ void philox4x32_10(unsigned long long key, unsigned long long ctr, unsigned (&r)[4]) {
  unsigned c0 = static_cast<unsigned>(ctr), c1 = static_cast<unsigned>(ctr >> 32), c2 = 0x9E3779B9u, c3 = 0xBB67AE85u;
  unsigned k0 = static_cast<unsigned>(key), k1 = static_cast<unsigned>(key >> 32);
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const unsigned n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  r[0] = c0; r[1] = c1; r[2] = c2; r[3] = c3;
}
__device__ __forceinline__ void normal4(unsigned long long key, unsigned long long ctr, float std, float (&o)[4]) {
  unsigned r[4];
  philox4x32_10(key, ctr, r);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float u1 = (static_cast<float>(r[2 * j] >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
    const float u2 = static_cast<float>(r[2 * j + 1] >> 8) * (1.0f / 16777216.0f);       // [0, 1)
    const float rad = std * sqrtf(-2.0f * __logf(u1));
    float sn, cs;
    __sincosf(6.283185307179586f * u2, &sn, &cs);
    o[2 * j] = rad * cs;
    o[2 * j + 1] = rad * sn;
  }
}
template <typename T>
__global__ void init_normal_kernel(T* __restrict__ out, long long n, unsigned long long key, long long first, float std) {
  // one thread per group of four consecutive logical elements (aligned to four in the logical index space)
  const long long g0 = first / 4, g1 = (first + n + 3) / 4;
  for (long long g = g0 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; g < g1;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v[4];
    normal4(key, static_cast<unsigned long long>(g), std, v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = g * 4 + j - first;
      if (i >= 0 && i < n) out[i] = static_cast<T>(v[j]);
    }
  }
}

// Sum of squares of a flat buffer, added to a single fp32 accumulator (for the global grad norm), in two
// stages with a fixed summation order: every block writes its partial sum, one block adds the partials in index
// order. The same gradients therefore always give the same norm bits (an atomicAdd per block would not), which
// keeps the clip coefficient, and with it a whole training step, reproducible.
template <typename GT>
__global__ void sumsq_partial_kernel(const GT* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  const long long n8 = n / 8;
  for (long long i8 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i8 < n8;
       i8 += static_cast<long long>(gridDim.x) * blockDim.x) {
    float x[8];
    adam_load8<GT>(g + i8 * 8, x);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += x[j] * x[j];
  }
  if (blockIdx.x == 0 && threadIdx.x < n - n8 * 8) {
    const float x = static_cast<float>(g[n8 * 8 + threadIdx.x]);
    s += x * x;
  }
  s = block_sum<256>(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) s += partial[i];
  s = block_sum<256>(s, red);
  if (threadIdx.x == 0) *out += s;
}

int grid_for(long long work_items, int threads, int cap = 148 * 8) {
  long long b = (work_items + threads - 1) / threads;
  if (b < 1) b = 1;
  return static_cast<int>(b < cap ? b : cap);
}

}  // namespace

void rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, float* rstd, int T, int H,
                 float eps, cudaStream_t s) {
  if (T <= 0) return;
  rmsnorm_fwd_kernel<256><<<T, 256, 0, s>>>(static_cast<const bf16*>(x), static_cast<const bf16*>(res),
                                            static_cast<const bf16*>(w), static_cast<bf16*>(y),
                                            static_cast<bf16*>(res_out), rstd, H, eps);
}

int rmsnorm_bwd_num_partials(int T) { return T < 296 ? (T < 1 ? 1 : T) : 296; }

void rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                 float* dw_partial, float* dw, bool accumulate_dw, int T, int H, cudaStream_t s) {
  if (T <= 0) return;
  const int blocks = rmsnorm_bwd_num_partials(T);
  rmsnorm_bwd_kernel<256><<<blocks, 256, H * sizeof(float), s>>>(
      static_cast<const bf16*>(dy), static_cast<const bf16*>(x), static_cast<const bf16*>(w), rstd,
      static_cast<const bf16*>(dres), static_cast<bf16*>(dx), dw_partial, T, H);
  colsum_kernel<<<(H + 127) / 128, 128, 0, s>>>(dw_partial, dw, blocks, H, accumulate_dw ? 1 : 0);
}

void qk_norm_rope_fwd(const void* qkv, const void* qw, const void* kw, const int* pos, void* q_out, void* k_out,
                      float* q_rstd, float* k_rstd, void* k_cache, void* v_cache, const int* slot_mapping, int T,
                      int Hq, int Hk, float theta, float eps, bool use_norm, cudaStream_t s, const float* inv_freq,
                      int rotary_dim) {
  if (T <= 0) return;
  const long long warps = static_cast<long long>(T) * (Hq + 2 * Hk);
  const int wpb = 8;
  const long long blocks = (warps + wpb - 1) / wpb;
  qk_norm_rope_fwd_kernel<<<static_cast<unsigned>(blocks), wpb * 32, 0, s>>>(
      static_cast<const bf16*>(qkv), static_cast<const bf16*>(qw), static_cast<const bf16*>(kw), pos,
      static_cast<bf16*>(q_out), static_cast<bf16*>(k_out), q_rstd, k_rstd, static_cast<bf16*>(k_cache),
      static_cast<bf16*>(v_cache), slot_mapping, T, Hq, Hk, theta, eps, use_norm ? 1 : 0, inv_freq, rotary_dim / 2);
}

void qk_norm_rope_bwd(const void* dq, const void* dk, const void* dv, const void* qkv, const void* qw, const void* kw,
                      const int* pos, const float* q_rstd, const float* k_rstd, void* dqkv, float* dqw, float* dkw,
                      int T, int Hq, int Hk, float theta, bool use_norm, cudaStream_t s, const float* inv_freq,
                      int rotary_dim) {
  if (T <= 0) return;
  const long long warps = static_cast<long long>(T) * (Hq + 2 * Hk);
  const int wpb = 8;
  long long blocks = (warps + wpb - 1) / wpb;
  if (blocks > 148 * 8) blocks = 148 * 8;
  qk_norm_rope_bwd_kernel<<<static_cast<unsigned>(blocks), wpb * 32, 0, s>>>(
      static_cast<const bf16*>(dq), static_cast<const bf16*>(dk), static_cast<const bf16*>(dv),
      static_cast<const bf16*>(qkv), static_cast<const bf16*>(qw), static_cast<const bf16*>(kw), pos, q_rstd, k_rstd,
      static_cast<bf16*>(dqkv), dqw, dkw, T, Hq, Hk, theta, use_norm ? 1 : 0, inv_freq, rotary_dim / 2);
}

void swiglu_fwd(const void* in, void* out, long long T, int I, cudaStream_t s) {
  if (T <= 0) return;
  swiglu_fwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, s>>>(static_cast<const bf16*>(in), static_cast<bf16*>(out), T, I);
}

void swiglu_bwd(const void* dout, const void* in, void* din, long long T, int I, cudaStream_t s) {
  if (T <= 0) return;
  swiglu_bwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, s>>>(static_cast<const bf16*>(dout), static_cast<const bf16*>(in),
                                                               static_cast<bf16*>(din), T, I);
}

void adam_step(void* p, float* master, void* lo, const void* g, bool g_fp32, void* m, void* v, bool mv_bf16, long long n,
               float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, const float* grad_scale,
               const float* skip_flag, cudaStream_t s) {
  if (n <= 0) return;
  const int grid = grid_for((n + 7) / 8, 256, 148 * 8);
  bf16* pp = static_cast<bf16*>(p);
  const AdamScalars a{lr, b1, b2, eps, wd, bc1, bc2};
#define MB_ADAM(GT, MT)                                                                                            \
  adam_kernel<GT, MT><<<grid, 256, 0, s>>>(pp, master, static_cast<short*>(lo), static_cast<const GT*>(g),          \
                                           static_cast<MT*>(m), static_cast<MT*>(v), n, a, grad_scale, skip_flag)
  if (g_fp32 && !mv_bf16) MB_ADAM(float, float);
  else if (g_fp32 && mv_bf16) MB_ADAM(float, bf16);
  else if (!g_fp32 && !mv_bf16) MB_ADAM(bf16, float);
  else MB_ADAM(bf16, bf16);
#undef MB_ADAM
}

void split_master_join(const void* p, const void* lo, float* out, long long n, cudaStream_t s) {
  if (n <= 0) return;
  split_master_join_kernel<<<grid_for(n, 256), 256, 0, s>>>(static_cast<const bf16*>(p), static_cast<const short*>(lo), out, n);
}
void split_master_cut(const float* master, void* p, void* lo, long long n, cudaStream_t s) {
  if (n <= 0) return;
  split_master_cut_kernel<<<grid_for(n, 256), 256, 0, s>>>(master, static_cast<bf16*>(p), static_cast<short*>(lo), n);
}

void init_normal(void* out, bool fp32, long long n, unsigned long long key, long long first, float std, cudaStream_t s) {
  if (n <= 0) return;
  const int grid = grid_for((n + 3) / 4 + 1, 256, 148 * 16);
  if (fp32) init_normal_kernel<float><<<grid, 256, 0, s>>>(static_cast<float*>(out), n, key, first, std);
  else init_normal_kernel<bf16><<<grid, 256, 0, s>>>(static_cast<bf16*>(out), n, key, first, std);
}

int sumsq_num_partials(long long n) { return grid_for((n + 7) / 8, 256, 148 * 4); }

// `partial`: fp32 scratch of sumsq_num_partials(n) elements; g must be 16-byte aligned.
void sumsq(const void* g, bool g_fp32, long long n, float* partial, float* out, cudaStream_t s) {
  if (n <= 0) return;
  const int grid = sumsq_num_partials(n);
  if (g_fp32) sumsq_partial_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(g), n, partial);
  else sumsq_partial_kernel<bf16><<<grid, 256, 0, s>>>(static_cast<const bf16*>(g), n, partial);
  sumsq_final_kernel<<<1, 256, 0, s>>>(partial, grid, out);
}

}  // namespace mb
