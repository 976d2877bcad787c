// Bandwidth-bound model kernels for sm_100a: RMSNorm / LayerNorm, rotary embedding, SwiGLU / GEGLU / GELU,
// embedding gather and per-example compact embedding gradient, cross-entropy helpers.
// All activations are bf16 in memory with fp32 arithmetic; rows are processed with 16-byte vector accesses.
#include "opk_api.h"
#include "debug_bounds.cuh"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <limits.h>
#include <math.h>
#include <stdio.h>

namespace {

#define OPK_LAUNCH_CHECK()                                   \
  do {                                                       \
    cudaError_t e__ = cudaGetLastError();                    \
    if (e__ != cudaSuccess) return (int)e__;                 \
  } while (0)

struct alignas(16) bf16x8 {
  __nv_bfloat162 h[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& v, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(v.h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) v.h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

template <int NT>
__device__ __forceinline__ float block_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < NT / 32) ? sh[threadIdx.x] : 0.f;
  if (w == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    if (l == 0) sh[0] = r;
  }
  __syncthreads();
  return sh[0];
}

constexpr int NT = 256;

// ------------------------------------------------------------------------------------------- RMSNorm
template <bool ADD>
__global__ void __launch_bounds__(NT) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ r,
                                                         const __nv_bfloat16* __restrict__ w,
                                                         __nv_bfloat16* __restrict__ sum_out,
                                                         __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                         int D, float eps, float w_off, long long ldx, long long ldy) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * ldx);
  const bf16x8* rr = ADD ? reinterpret_cast<const bf16x8*>(r + row * D) : nullptr;
  bf16x8* sr = ADD ? reinterpret_cast<bf16x8*>(sum_out + row * D) : nullptr;
  const int nv = D >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += NT) {
    float f[8];
    unpack8(xr[i], f);
    if (ADD) {
      float g[8];
      unpack8(rr[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      bf16x8 s = pack8(f);
      sr[i] = s;
      unpack8(s, f);  // normalise the stored (rounded) residual stream
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  const float tot = block_sum<NT>(ss, sh);
  const float rs = rsqrtf(tot / (float)D + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = rs;
  const bf16x8* src = ADD ? reinterpret_cast<const bf16x8*>(sum_out + row * D) : xr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * ldy);
  for (int i = threadIdx.x; i < nv; i += NT) {
    float f[8], g[8];
    unpack8(src[i], f);
    unpack8(wr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * rs * (g[j] + w_off);
    yr[i] = pack8(f);
  }
}

// One warp per row, the row held in registers (VPL vectors of 8 per lane): one pass over memory, no block barrier.
// (Without the opaque barrier below the compiler keeps the row UNPACKED across the reduction, 255 registers per thread at
// 16 vectors per lane: one CTA per SM and 12 % of the warp slots in use. Packed, the row is 64 registers.)
template <int VPL>
__global__ void __launch_bounds__(256, VPL >= 16 ? 2 : 4) rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int T,
                                                               float eps, float w_off, long long ldx, long long ldy) {
  constexpr int D = VPL * 32 * 8;
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * 8ll + (threadIdx.x >> 5);
  if (row >= T) return;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * ldx);
  bf16x8 v[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) v[i] = xr[lane + 32 * i];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    float f[8];
    unpack8(v[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rs = rsqrtf(ss / (float)D + eps);
  if (lane == 0 && rstd) rstd[row] = rs;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * ldy);
  // the packed words pass through an empty asm: the floats computed for the reduction cannot be reused below
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
#pragma unroll
    for (int q = 0; q < 4; ++q) asm volatile("" : "+r"(*reinterpret_cast<uint32_t*>(&v[i].h[q])));
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    float f[8], g[8];
    unpack8(v[i], f);
    unpack8(wr[lane + 32 * i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * rs * (g[j] + w_off);
    yr[lane + 32 * i] = pack8(f);
  }
}

// RMSNorm backward. A CTA of 512 threads walks rows with a grid stride; every thread owns the same columns for
// all rows (ITERS vectors of 8), so the weight gradient accumulates in registers without atomics and is written once
// per CTA to partial[blockIdx][D]. A second kernel adds the column sums of `partial` into dw.
constexpr int MAX_COL_ITERS = 8;  // layernorm backward: D <= 8 * 2048
constexpr int RMS_BWD_NT = 512;
template <int ITERS>
__global__ void __launch_bounds__(RMS_BWD_NT) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                 const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ w,
                                                                 const float* __restrict__ rstd,
                                                                 const __nv_bfloat16* __restrict__ dres,
                                                                 __nv_bfloat16* __restrict__ dx,
                                                                 float* __restrict__ partial, int T, int D,
                                                                 float w_off, long long ld_dy, long long ldx,
                                                                 long long ld_dx) {
  __shared__ float sh[32];
  const int nv = D >> 3;
  float wv[ITERS][8], acc[ITERS][8];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int v = threadIdx.x + it * RMS_BWD_NT;
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc[it][j] = 0.f; wv[it][j] = 0.f; }
    if (v < nv) {
      unpack8(reinterpret_cast<const bf16x8*>(w)[v], wv[it]);
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[it][j] += w_off;
    }
  }
  int par = 0;
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + row * ld_dy);
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * ldx);
    const float rs = rstd[row];
    float g[ITERS][8], xv[ITERS][8];
    float dot = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int v = threadIdx.x + it * RMS_BWD_NT;
      if (v < nv) {
        unpack8(dyr[v], g[it]);
        unpack8(xr[v], xv[it]);
#pragma unroll
        for (int j = 0; j < 8; ++j) dot += g[it][j] * wv[it][j] * xv[it][j];
      }
    }
    // one barrier per row: warp sums go to one of two alternating sets of slots and every thread adds the sixteen
    // partials itself (a set is rewritten two rows later, after the barrier of the row in between)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    float* slots = sh + par * (RMS_BWD_NT / 32);
    par ^= 1;
    if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = dot;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int wq = 0; wq < RMS_BWD_NT / 32; ++wq) tot += slots[wq];
    const float mean_dot = tot * rs / (float)D;
    const bf16x8* drr = dres ? reinterpret_cast<const bf16x8*>(dres + row * ld_dx) : nullptr;
    bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + row * ld_dx);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int v = threadIdx.x + it * RMS_BWD_NT;
      if (v < nv) {
        float o[8];
        if (drr) unpack8(drr[v], o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = xv[it][j] * rs;
          const float d = rs * (g[it][j] * wv[it][j] - xh * mean_dot);
          o[j] = drr ? o[j] + d : d;
          acc[it][j] += g[it][j] * xh;
        }
        dxr[v] = pack8(o);
      }
    }
  }
  if (partial) {
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int v = threadIdx.x + it * RMS_BWD_NT;
      if (v < nv) {
        float4* dst = reinterpret_cast<float4*>(partial + (long long)blockIdx.x * D + v * 8);
        dst[0] = make_float4(acc[it][0], acc[it][1], acc[it][2], acc[it][3]);
        dst[1] = make_float4(acc[it][4], acc[it][5], acc[it][6], acc[it][7]);
      }
    }
  }
}

// dst[c] += sum_r partial[r][c]; CTA = 32 columns x 8 row groups.
__global__ void __launch_bounds__(256) colsum_add_kernel(const float* __restrict__ partial, float* __restrict__ dst,
                                                         int rows, int D) {
  __shared__ float sh[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < D)
    for (int r = ry; r < rows; r += 8) s += partial[(long long)r * D + c];
  sh[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c < D) {
#pragma unroll
    for (int k = 1; k < 8; ++k) s += sh[k][cx];
    dst[c] += s;
  }
}

// ------------------------------------------------------------------------------------------- LayerNorm
__global__ void __launch_bounds__(NT) layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           const __nv_bfloat16* __restrict__ b,
                                                           __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
                                                           float* __restrict__ rstd, int D, float eps) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
  const int nv = D >> 3;
  float s = 0.f;
  for (int i = threadIdx.x; i < nv; i += NT) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j];
  }
  const float mu = block_sum<NT>(s, sh) / (float)D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += NT) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += (f[j] - mu) * (f[j] - mu);
  }
  const float rs = rsqrtf(block_sum<NT>(ss, sh) / (float)D + eps);
  if (threadIdx.x == 0) {
    if (mean) mean[row] = mu;
    if (rstd) rstd[row] = rs;
  }
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  const bf16x8* br = b ? reinterpret_cast<const bf16x8*>(b) : nullptr;
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * D);
  for (int i = threadIdx.x; i < nv; i += NT) {
    float f[8], g[8], bb[8];
    unpack8(xr[i], f);
    unpack8(wr[i], g);
    if (br) unpack8(br[i], bb);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = (f[j] - mu) * rs * g[j] + (br ? bb[j] : 0.f);
    yr[i] = pack8(f);
  }
}

__global__ void __launch_bounds__(NT) layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                           const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           const float* __restrict__ mean,
                                                           const float* __restrict__ rstd,
                                                           const __nv_bfloat16* __restrict__ dres,
                                                           __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                                                           float* __restrict__ db, int T, int D) {
  __shared__ float sh[32];
  const int nv = D >> 3;
  float dwp[MAX_COL_ITERS][8], dbp[MAX_COL_ITERS][8];
#pragma unroll
  for (int c = 0; c < MAX_COL_ITERS; ++c)
#pragma unroll
    for (int j = 0; j < 8; ++j) { dwp[c][j] = 0.f; dbp[c][j] = 0.f; }
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + row * D);
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
    const float rs = rstd[row], mu = mean[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < MAX_COL_ITERS; ++c) {
      const int i = threadIdx.x + c * NT;
      if (i < nv) {
        float g[8], xv[8], wv[8];
        unpack8(dyr[i], g);
        unpack8(xr[i], xv);
        unpack8(wr[i], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mu) * rs;
          dwp[c][j] += g[j] * xh;
          dbp[c][j] += g[j];
          const float gw = g[j] * wv[j];
          s1 += gw;
          s2 += gw * xh;
        }
      }
    }
    const float m1 = block_sum<NT>(s1, sh) / (float)D;
    const float m2 = block_sum<NT>(s2, sh) / (float)D;
    const bf16x8* drr = dres ? reinterpret_cast<const bf16x8*>(dres + row * D) : nullptr;
    bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + row * D);
#pragma unroll
    for (int c = 0; c < MAX_COL_ITERS; ++c) {
      const int i = threadIdx.x + c * NT;
      if (i < nv) {
        float g[8], xv[8], wv[8], o[8];
        unpack8(dyr[i], g);
        unpack8(xr[i], xv);
        unpack8(wr[i], wv);
        if (drr) unpack8(drr[i], o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mu) * rs;
          const float d = rs * (g[j] * wv[j] - m1 - xh * m2);
          o[j] = drr ? o[j] + d : d;
        }
        dxr[i] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < MAX_COL_ITERS; ++c) {
    const int i = threadIdx.x + c * NT;
    if (i < nv) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (dw) atomicAdd(&dw[i * 8 + j], dwp[c][j]);
        if (db) atomicAdd(&db[i * 8 + j], dbp[c][j]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------- RoPE
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qk, const float* __restrict__ cs,
                            const int* __restrict__ pos, int T, int n_heads, int hd, long long ld, float sign) {
  const int half = hd >> 1;
  const long long total = (long long)T * n_heads * half;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int i = idx % half;
    const long long th = idx / half;
    const int h = th % n_heads;
    const long long t = th / n_heads;
    const long long p = pos ? pos[t] : t;
    const float c = cs[(p * half + i) * 2], s = cs[(p * half + i) * 2 + 1] * sign;
    __nv_bfloat16* base = qk + t * ld + (long long)h * hd;
    const float x1 = __bfloat162float(base[i]), x2 = __bfloat162float(base[i + half]);
    base[i] = __float2bfloat16(x1 * c - x2 * s);
    base[i + half] = __float2bfloat16(x2 * c + x1 * s);
  }
}

// Vector form: a thread rotates 8 consecutive pairs (x[i..i+7], x[i+half..i+half+7]) with 16-byte accesses.
__global__ void __launch_bounds__(256) rope_vec8_kernel(__nv_bfloat16* __restrict__ qk, const float* __restrict__ cs,
                                                        const int* __restrict__ pos, int T, int n_heads, int hd, long long ld,
                                                        float sign) {
  const int half = hd >> 1, hv = half >> 3;
  const long long total = (long long)T * n_heads * hv;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int iv = (int)(idx % hv);
    const long long th = idx / hv;
    const int h = (int)(th % n_heads);
    const long long t = th / n_heads;
    const long long p = pos ? pos[t] : t;
    const float4* c4 = reinterpret_cast<const float4*>(cs + (p * half + iv * 8) * 2);
    bf16x8* lo = reinterpret_cast<bf16x8*>(qk + t * ld + (long long)h * hd + iv * 8);
    bf16x8* hi = reinterpret_cast<bf16x8*>(qk + t * ld + (long long)h * hd + half + iv * 8);
    float a[8], b[8];
    unpack8(*lo, a);
    unpack8(*hi, b);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 v = c4[q];            // (cos, sin) of pairs 2q and 2q + 1
      const float s0 = v.y * sign, s1 = v.w * sign;
      const float x1 = a[2 * q], x2 = b[2 * q], y1 = a[2 * q + 1], y2 = b[2 * q + 1];
      a[2 * q] = x1 * v.x - x2 * s0;
      b[2 * q] = x2 * v.x + x1 * s0;
      a[2 * q + 1] = y1 * v.z - y2 * s1;
      b[2 * q + 1] = y2 * v.z + y1 * s1;
    }
    *lo = pack8(a);
    *hi = pack8(b);
  }
}

// ------------------------------------------------------------------------------------------- gated activations
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k = 0.7978845608028654f;
  const float u = k * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
}
__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.7071067811865476f)); }
__device__ __forceinline__ float gelu_erf_grad(float x) {
  return 0.5f * (1.f + erff(x * 0.7071067811865476f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}

// MODE 0 = SwiGLU, 1 = GEGLU exact, 2 = GEGLU tanh
template <int MODE>
__device__ __forceinline__ float gate_fn(float g) {
  return MODE == 0 ? g * sigmoidf_(g) : (MODE == 1 ? gelu_erf(g) : gelu_tanh(g));
}
template <int MODE>
__device__ __forceinline__ float gate_grad(float g) {
  if (MODE == 0) {
    const float s = sigmoidf_(g);
    return s * (1.f + g * (1.f - s));
  }
  return MODE == 1 ? gelu_erf_grad(g) : gelu_tanh_grad(g);
}

template <int MODE>
__global__ void glu_fwd_kernel(const __nv_bfloat162* __restrict__ gu, __nv_bfloat16* __restrict__ act, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float2 p = __bfloat1622float2(gu[i]);
    act[i] = __float2bfloat16(gate_fn<MODE>(p.x) * p.y);
  }
}
template <int MODE>
__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ dact, const __nv_bfloat162* __restrict__ gu,
                               __nv_bfloat162* __restrict__ dgu, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float2 p = __bfloat1622float2(gu[i]);
    const float d = __bfloat162float(dact[i]);
    dgu[i] = __floats2bfloat162_rn(d * p.y * gate_grad<MODE>(p.x), d * gate_fn<MODE>(p.x));
  }
}
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16(gelu_tanh(__bfloat162float(x[i])));
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                __nv_bfloat16* __restrict__ dx, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dx[i] = __float2bfloat16(__bfloat162float(dy[i]) * gelu_tanh_grad(__bfloat162float(x[i])));
}

// ------------------------------------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const int* __restrict__ tok, const __nv_bfloat16* __restrict__ table,
                                     const __nv_bfloat16* __restrict__ pos_table, __nv_bfloat16* __restrict__ out,
                                     int D, int vocab) {
  const long long t = blockIdx.x;
  // an id outside the table yields a zero embedding row: never an address outside the table
  const bool in_table = tok[t] >= 0 && tok[t] < vocab;
  (void)OPK_IDX_OK(tok[t], vocab);
  const bf16x8* src = reinterpret_cast<const bf16x8*>(table + (long long)(in_table ? tok[t] : 0) * D);
  const bf16x8* ps = pos_table ? reinterpret_cast<const bf16x8*>(pos_table + t * D) : nullptr;
  bf16x8* dst = reinterpret_cast<bf16x8*>(out + t * D);
  for (int i = threadIdx.x; i < (D >> 3); i += blockDim.x) {
    if (ps || !in_table) {
      float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (in_table) unpack8(src[i], a);
      if (ps) unpack8(ps[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
      dst[i] = pack8(a);
    } else {
      dst[i] = src[i];
    }
  }
}
// Token ids outside [0, vocab) are skipped by all three table kernels (their rep[] entry becomes -1, which the
// accumulate / add-rows kernels treat as "not a representative row"), so a bad id can never index past the table.
__device__ __forceinline__ bool emb_tok_ok(int tok, int vocab) {
  (void)OPK_IDX_OK(tok, vocab);
  return (unsigned)tok < (unsigned)vocab;
}
OPK_DEBUG_BOUNDS_UNIT();
__global__ void emb_first_pos_kernel(const int* __restrict__ tok, int* __restrict__ first_pos, int T, int vocab) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < T && emb_tok_ok(tok[t], vocab)) atomicMin(&first_pos[tok[t]], t);
}
__global__ void emb_scatter_kernel(const int* __restrict__ tok, const __nv_bfloat16* __restrict__ dx,
                                   const int* __restrict__ first_pos, int* __restrict__ rep, float* __restrict__ gc,
                                   int D, int vocab) {
  const long long t = blockIdx.x;
  if (!emb_tok_ok(tok[t], vocab)) {
    if (threadIdx.x == 0) rep[t] = -1;
    return;
  }
  const int r = first_pos[tok[t]];
  if (threadIdx.x == 0) rep[t] = r;
  const __nv_bfloat16* src = dx + t * D;
  float* dst = gc + (long long)r * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) atomicAdd(&dst[d], __bfloat162float(src[d]));
}
__global__ void emb_reset_kernel(const int* __restrict__ tok, int* __restrict__ first_pos, int T, int vocab) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < T && emb_tok_ok(tok[t], vocab)) first_pos[tok[t]] = INT_MAX;
}
// ATOMIC: the rows of acc are shared with other GPUs' kernels (sharded sums, acc may be peer-mapped), so the add is a
// reduction instead of a read-modify-write.
template <bool ATOMIC>
__global__ void emb_accumulate_kernel(const int* __restrict__ tok, const int* __restrict__ rep,
                                      const float* __restrict__ gc, const float* __restrict__ scale,
                                      float* __restrict__ acc, int D) {
  const long long t = blockIdx.x;
  if (rep[t] != (int)t) return;
  const float s = *scale;
  const float* src = gc + t * D;
  float* dst = acc + (long long)tok[t] * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float g = __bfloat162float(__float2bfloat16(src[d]));            // the stored per-example gradient
    const float c = __bfloat162float(__float2bfloat16(g * s));             // clipped in storage precision
    if (ATOMIC) atomicAdd(&dst[d], c);
    else dst[d] += c;
  }
}

// ------------------------------------------------------------------------------------------- reductions
template <bool FP32, bool ROUND>
__global__ void __launch_bounds__(NT) sumsq_kernel(const void* __restrict__ x, long long n, double* out) {
  __shared__ float sh[32];
  double acc = 0.0;
  float part = 0.f;
  int cnt = 0;
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    float v = FP32 ? reinterpret_cast<const float*>(x)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
    if (ROUND) v = __bfloat162float(__float2bfloat16(v));
    part += v * v;
    if (++cnt == 64) { acc += (double)part; part = 0.f; cnt = 0; }
  }
  acc += (double)part;
  // fp64 block reduction through two fp32 words would lose bits; reduce doubles with shuffles directly
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ double shd[NT / 32];
  if ((threadIdx.x & 31) == 0) shd[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < NT / 32; ++w) t += shd[w];
    atomicAdd(out, t);
  }
  (void)sh;
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(in[i]);
}

// ------------------------------------------------------------------------------------------- cross entropy
__global__ void lce_finalize_kernel(const float* __restrict__ pmax, const float* __restrict__ psum,
                                    const float* __restrict__ tgt, const int* __restrict__ labels,
                                    float* __restrict__ lse, float* __restrict__ nll, int T, int tiles) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const float* pm = pmax + (long long)row * tiles;
  const float* ps = psum + (long long)row * tiles;
  float m = -INFINITY;
  for (int i = lane; i < tiles; i += 32) m = fmaxf(m, pm[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float s = 0.f;
  for (int i = lane; i < tiles; i += 32) s += ps[i] * __expf(pm[i] - m);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    const float l = m + logf(s);
    lse[row] = l;
    if (nll) nll[row] = labels[row] >= 0 ? l - tgt[row] : 0.f;
  }
}

// Per-example RMSNorm weight gradient: dw[b][c] += sum over the rows of example b of dy * x * rstd (the normalised
// input). One thread per column, grid.y = example, grid.z = row chunk; fp32 atomics combine the row chunks.
__global__ void __launch_bounds__(256) rmsnorm_dw_per_example_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                     const __nv_bfloat16* __restrict__ x,
                                                                     const float* __restrict__ rstd, float* __restrict__ dw,
                                                                     int rows, int D) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= D) return;
  const long long b = blockIdx.y;
  const int chunk = (rows + gridDim.z - 1) / gridDim.z;
  const int r0 = blockIdx.z * chunk, r1 = min(rows, r0 + chunk);
  float acc = 0.f;
  for (int r = r0; r < r1; ++r) {
    const long long row = b * rows + r;
    acc += __bfloat162float(dy[row * D + c]) * __bfloat162float(x[row * D + c]) * rstd[row];
  }
  if (r1 > r0) atomicAdd(&dw[b * D + c], acc);
}

// Per-example loss bookkeeping in one CTA: ntok = max(1, #labels >= 0); coef[t] = [label >= 0] / ntok (* *weight);
// loss = sum_t nll[t] * coef[t]. Two block reductions; T is a sequence length.
__global__ void __launch_bounds__(1024) loss_coef_kernel(const int* __restrict__ labels, const float* __restrict__ nll,
                                                         const float* __restrict__ weight, float* __restrict__ coef,
                                                         float* __restrict__ loss, float* __restrict__ ntok, int T) {
  __shared__ float red[32];
  __shared__ float bcast;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float cnt = 0.f;
  for (int t = threadIdx.x; t < T; t += blockDim.x) cnt += labels[t] >= 0 ? 1.f : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0) red[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[w];
    bcast = fmaxf(s, 1.f);
  }
  __syncthreads();
  const float n = bcast;
  const float w = weight ? *weight : 1.f;
  float acc = 0.f;
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    const float c = labels[t] >= 0 ? w / n : 0.f;
    coef[t] = c;
    acc += nll[t] * c;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __syncthreads();
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int wi = 0; wi < (int)(blockDim.x >> 5); ++wi) s += red[wi];
    *loss = s;
    if (ntok) *ntok = n;
  }
}

template <bool FP32>
__device__ __forceinline__ float load_logit(const void* p, long long i) {
  return FP32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ float cap(float z, float scale, float softcap) {
  z *= scale;
  return softcap > 0.f ? softcap * tanhf(z / softcap) : z;
}

template <bool FP32>
__global__ void __launch_bounds__(NT) ce_fwd_kernel(const void* __restrict__ logits, const int* __restrict__ labels,
                                                    float* __restrict__ nll, float* __restrict__ lse, int V,
                                                    long long ld, float scale, float softcap) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const long long base = row * ld;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < V; i += NT) {
    const float z = cap(load_logit<FP32>(logits, base + i), scale, softcap);
    const float nm = fmaxf(m, z);
    s = s * __expf(m - nm) + __expf(z - nm);
    m = nm;
  }
  // combine (m, s) pairs: first the max, then rescaled sums
  float gm = m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = gm;
  __syncthreads();
  float bm = sh[0];
  for (int w = 1; w < NT / 32; ++w) bm = fmaxf(bm, sh[w]);
  const float tot = block_sum<NT>(m == -INFINITY ? 0.f : s * __expf(m - bm), sh);
  if (threadIdx.x == 0) {
    const float l = bm + logf(tot);
    if (lse) lse[row] = l;
    const int lab = labels[row];
    if (lab >= 0) (void)OPK_IDX_OK(lab, V);
    nll[row] = (lab >= 0 && lab < V) ? l - cap(load_logit<FP32>(logits, base + lab), scale, softcap) : 0.f;
  }
}

template <bool FP32>
__global__ void __launch_bounds__(NT) ce_bwd_kernel(const void* __restrict__ logits, const int* __restrict__ labels,
                                                    const float* __restrict__ lse, const float* __restrict__ coef,
                                                    void* __restrict__ dlogits, int V, long long ld, float scale,
                                                    float softcap) {
  const long long row = blockIdx.x;
  const long long base = row * ld;
  const float l = lse[row], c = coef[row];
  const int lab = labels[row];
  for (int i = threadIdx.x; i < V; i += NT) {
    const float raw = load_logit<FP32>(logits, base + i) * scale;
    float z = raw, dz = scale;
    if (softcap > 0.f) {
      const float th = tanhf(raw / softcap);
      z = softcap * th;
      dz = scale * (1.f - th * th);
    }
    const float g = (__expf(z - l) - (i == lab ? 1.f : 0.f)) * c * dz;
    if (FP32) reinterpret_cast<float*>(dlogits)[base + i] = g;
    else reinterpret_cast<__nv_bfloat16*>(dlogits)[base + i] = __float2bfloat16(g);
  }
}

// rows of an fp32 [R][D] matrix -> bf16 at dst_base + offsets[r]; sumsq += sum(bf16(v)^2)
__global__ void __launch_bounds__(NT) scatter_rows_cast_sumsq_kernel(const float* __restrict__ src,
                                                                     __nv_bfloat16* __restrict__ dst_base,
                                                                     const long long* __restrict__ offsets, int D,
                                                                     double* sumsq) {
  __shared__ float sh[32];
  const long long r = blockIdx.x;
  const float* s = src + r * D;
  __nv_bfloat16* d = dst_base + offsets[r];
  float part = 0.f;
  for (int i = threadIdx.x; i < D; i += NT) {
    const __nv_bfloat16 b = __float2bfloat16(s[i]);
    d[i] = b;
    const float f = __bfloat162float(b);
    part += f * f;
  }
  const float tot = block_sum<NT>(part, sh);
  if (threadIdx.x == 0 && sumsq) atomicAdd(sumsq, (double)tot);
}

// out[n] (+)= sum_t dy[t][n]  (bias gradient)
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ out, int T, int N, long long ld) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float a = 0.f;
  for (int t = blockIdx.y; t < T; t += gridDim.y) a += __bfloat162float(dy[(long long)t * ld + n]);
  atomicAdd(&out[n], a);
}

// tied embeddings: dense[tok[t]] += gc[t] for representative rows (no two representatives share a row)
__global__ void emb_add_rows_kernel(const int* __restrict__ tok, const int* __restrict__ rep,
                                    const float* __restrict__ gc, __nv_bfloat16* __restrict__ dense, int D) {
  const long long t = blockIdx.x;
  if (rep[t] != (int)t) return;
  const float* src = gc + t * D;
  __nv_bfloat16* dst = dense + (long long)tok[t] * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = __float2bfloat16(__bfloat162float(dst[d]) + src[d]);
}

inline int grid_for(long long n, int block, int cap_blocks = 148 * 16) {
  long long g = (n + block - 1) / block;
  if (g > cap_blocks) g = cap_blocks;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFM(p) reinterpret_cast<__nv_bfloat16*>(p)

extern "C" int opk_rmsnorm_fwd_ld(const void* x, int64_t ldx, const void* w, void* y, int64_t ldy, float* rstd, int T, int D,
                                  float eps, float w_offset, void* stream) {
  if (T <= 0) return 0;
  if (D % 8 || ldx % 8 || ldy % 8 || ldx < D || ldy < D) return -1;
  const int warp_grid = (T + 7) / 8;
  if (D == 4096)
    rmsnorm_fwd_warp_kernel<16><<<warp_grid, 256, 0, ST(stream)>>>(BF(x), BF(w), BFM(y), rstd, T, eps, w_offset, ldx, ldy);
  else if (D == 2048)
    rmsnorm_fwd_warp_kernel<8><<<warp_grid, 256, 0, ST(stream)>>>(BF(x), BF(w), BFM(y), rstd, T, eps, w_offset, ldx, ldy);
  else if (D == 1024)
    rmsnorm_fwd_warp_kernel<4><<<warp_grid, 256, 0, ST(stream)>>>(BF(x), BF(w), BFM(y), rstd, T, eps, w_offset, ldx, ldy);
  else
    rmsnorm_fwd_kernel<false><<<T, NT, 0, ST(stream)>>>(BF(x), nullptr, BF(w), nullptr, BFM(y), rstd, D, eps, w_offset, ldx, ldy);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int T, int D, float eps,
                               float w_offset, void* stream) {
  return opk_rmsnorm_fwd_ld(x, D, w, y, D, rstd, T, D, eps, w_offset, stream);
}
extern "C" int opk_add_rmsnorm_fwd(const void* x, const void* r, const void* w, void* sum_out, void* y, float* rstd,
                                   int T, int D, float eps, float w_offset, void* stream) {
  if (T <= 0) return 0;
  if (D % 8) return -1;
  rmsnorm_fwd_kernel<true><<<T, NT, 0, ST(stream)>>>(BF(x), BF(r), BF(w), BFM(sum_out), BFM(y), rstd, D, eps, w_offset, D, D);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_rmsnorm_bwd_ld(const void* dy, int64_t ld_dy, const void* x, int64_t ldx, const void* w, const float* rstd,
                                  const void* dres, void* dx_out, int64_t ld_dx, float* dw, float* workspace, int ws_rows,
                                  int T, int D, float w_offset, void* stream) {
  if (T <= 0) return 0;
  if (D % 8 || D > 3 * RMS_BWD_NT * 8) return -1;
  if (ld_dy % 8 || ldx % 8 || ld_dx % 8 || ld_dy < D || ldx < D || ld_dx < D) return -1;
  if (dw && (!workspace || ws_rows < 1)) return -1;
  int grid = T < 148 * 2 ? T : 148 * 2;
  if (dw && grid > ws_rows) grid = ws_rows;
  float* part = dw ? workspace : nullptr;
  const int iters = (D / 8 + RMS_BWD_NT - 1) / RMS_BWD_NT;
  if (iters == 1)
    rmsnorm_bwd_kernel<1><<<grid, RMS_BWD_NT, 0, ST(stream)>>>(BF(dy), BF(x), BF(w), rstd, BF(dres), BFM(dx_out), part, T, D, w_offset, ld_dy, ldx, ld_dx);
  else if (iters == 2)
    rmsnorm_bwd_kernel<2><<<grid, RMS_BWD_NT, 0, ST(stream)>>>(BF(dy), BF(x), BF(w), rstd, BF(dres), BFM(dx_out), part, T, D, w_offset, ld_dy, ldx, ld_dx);
  else
    rmsnorm_bwd_kernel<3><<<grid, RMS_BWD_NT, 0, ST(stream)>>>(BF(dy), BF(x), BF(w), rstd, BF(dres), BFM(dx_out), part, T, D, w_offset, ld_dy, ldx, ld_dx);
  OPK_LAUNCH_CHECK();
  if (dw) {
    colsum_add_kernel<<<(D + 31) / 32, 256, 0, ST(stream)>>>(part, dw, grid, D);
    OPK_LAUNCH_CHECK();
  }
  return 0;
}
extern "C" int opk_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                               void* dx_out, float* dw, float* workspace, int ws_rows, int T, int D, float w_offset,
                               void* stream) {
  return opk_rmsnorm_bwd_ld(dy, D, x, D, w, rstd, dres, dx_out, D, dw, workspace, ws_rows, T, D, w_offset, stream);
}
extern "C" int opk_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int T,
                                 int D, float eps, void* stream) {
  if (T <= 0) return 0;
  if (D % 8) return -1;
  layernorm_fwd_kernel<<<T, NT, 0, ST(stream)>>>(BF(x), BF(w), BF(b), BFM(y), mean, rstd, D, eps);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                 const void* dres, void* dx_out, float* dw, float* db, int T, int D, void* stream) {
  if (T <= 0) return 0;
  if (D % 8 || D > MAX_COL_ITERS * NT * 8) return -1;
  const int grid = T < 148 * 2 ? T : 148 * 2;
  layernorm_bwd_kernel<<<grid, NT, 0, ST(stream)>>>(BF(dy), BF(x), BF(w), mean, rstd, BF(dres), BFM(dx_out), dw, db, T, D);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_rope(void* qk, const float* cs, const int32_t* pos, int T, int n_rot_heads, int head_dim, int64_t ld,
                        float sign, void* stream) {
  const long long n = (long long)T * n_rot_heads * (head_dim / 2);
  if (n <= 0) return 0;
  if ((head_dim % 16) == 0 && (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(qk) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(cs) & 15) == 0)
    rope_vec8_kernel<<<grid_for(n / 8, 256), 256, 0, ST(stream)>>>(BFM(qk), cs, pos, T, n_rot_heads, head_dim, ld, sign);
  else
    rope_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(BFM(qk), cs, pos, T, n_rot_heads, head_dim, ld, sign);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_swiglu_fwd(const void* gu, void* act, int T, int F, void* stream) {
  const long long n = (long long)T * F;
  if (n <= 0) return 0;
  glu_fwd_kernel<0><<<grid_for(n, 256), 256, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat162*>(gu), BFM(act), n);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_swiglu_bwd(const void* dact, const void* gu, void* dgu, int T, int F, void* stream) {
  const long long n = (long long)T * F;
  if (n <= 0) return 0;
  glu_bwd_kernel<0><<<grid_for(n, 256), 256, 0, ST(stream)>>>(BF(dact), reinterpret_cast<const __nv_bfloat162*>(gu),
                                                             reinterpret_cast<__nv_bfloat162*>(dgu), n);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_geglu_fwd(const void* gu, void* act, int T, int F, int approx, void* stream) {
  const long long n = (long long)T * F;
  if (n <= 0) return 0;
  if (approx) glu_fwd_kernel<2><<<grid_for(n, 256), 256, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat162*>(gu), BFM(act), n);
  else glu_fwd_kernel<1><<<grid_for(n, 256), 256, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat162*>(gu), BFM(act), n);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_geglu_bwd(const void* dact, const void* gu, void* dgu, int T, int F, int approx, void* stream) {
  const long long n = (long long)T * F;
  if (n <= 0) return 0;
  if (approx)
    glu_bwd_kernel<2><<<grid_for(n, 256), 256, 0, ST(stream)>>>(BF(dact), reinterpret_cast<const __nv_bfloat162*>(gu),
                                                               reinterpret_cast<__nv_bfloat162*>(dgu), n);
  else
    glu_bwd_kernel<1><<<grid_for(n, 256), 256, 0, ST(stream)>>>(BF(dact), reinterpret_cast<const __nv_bfloat162*>(gu),
                                                               reinterpret_cast<__nv_bfloat162*>(dgu), n);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_gelu_fwd(const void* x, void* y, int64_t n, void* stream) {
  if (n <= 0) return 0;
  gelu_fwd_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(BF(x), BFM(y), n);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_gelu_bwd(const void* dy, const void* x, void* dx, int64_t n, void* stream) {
  if (n <= 0) return 0;
  gelu_bwd_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(BF(dy), BF(x), BFM(dx), n);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_embedding_fwd(const int32_t* tok, const void* table, const void* pos_table, void* out, int T, int D,
                                 int vocab, void* stream) {
  if (T <= 0) return 0;
  if (D % 8 || vocab <= 0) return -1;
  embedding_fwd_kernel<<<T, 128, 0, ST(stream)>>>(tok, BF(table), BF(pos_table), BFM(out), D, vocab);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_embedding_bwd_compact(const int32_t* tok, const void* dx, int32_t* first_pos, int32_t* rep,
                                         float* gc, double* sumsq, int T, int D, int vocab, void* stream) {
  if (T <= 0) return 0;
  if (vocab <= 0) return -1;
  cudaStream_t st = ST(stream);
  cudaError_t e = cudaMemsetAsync(gc, 0, sizeof(float) * (size_t)T * D, st);
  if (e != cudaSuccess) return (int)e;
  emb_first_pos_kernel<<<(T + 255) / 256, 256, 0, st>>>(tok, first_pos, T, vocab);
  emb_scatter_kernel<<<T, 256, 0, st>>>(tok, BF(dx), first_pos, rep, gc, D, vocab);
  emb_reset_kernel<<<(T + 255) / 256, 256, 0, st>>>(tok, first_pos, T, vocab);
  if (sumsq) sumsq_kernel<true, true><<<grid_for((long long)T * D, NT, 148 * 4), NT, 0, st>>>(gc, (long long)T * D, sumsq);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_embedding_accumulate(const int32_t* tok, const int32_t* rep, const float* gc, const float* scale,
                                        float* acc, int T, int D, void* stream) {
  if (T <= 0) return 0;
  emb_accumulate_kernel<false><<<T, 256, 0, ST(stream)>>>(tok, rep, gc, scale, acc, D);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_embedding_accumulate_shared(const int32_t* tok, const int32_t* rep, const float* gc, const float* scale,
                                               float* acc, int T, int D, void* stream) {
  if (T <= 0) return 0;
  emb_accumulate_kernel<true><<<T, 256, 0, ST(stream)>>>(tok, rep, gc, scale, acc, D);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_lce_finalize(const float* pmax, const float* psum, const float* tgt, const int32_t* labels,
                                float* lse, float* nll, int T, int tiles, void* stream) {
  if (T <= 0) return 0;
  lce_finalize_kernel<<<(T + 7) / 8, 256, 0, ST(stream)>>>(pmax, psum, tgt, labels, lse, nll, T, tiles);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_rmsnorm_dw_per_example(const void* dy, const void* x, const float* rstd, float* dw, int B, int rows, int D,
                                          void* stream) {
  if (B <= 0 || rows <= 0 || D <= 0) return 0;
  if (B > 65535) return -1;
  int z = (rows + 63) / 64;
  if (z > 32) z = 32;
  dim3 grid((D + 255) / 256, B, z);
  rmsnorm_dw_per_example_kernel<<<grid, 256, 0, ST(stream)>>>(BF(dy), BF(x), rstd, dw, rows, D);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_loss_coef(const int32_t* labels, const float* nll, const float* weight, float* coef, float* loss, float* ntok,
                             int T, void* stream) {
  if (T <= 0 || !labels || !nll || !coef || !loss) return -1;
  loss_coef_kernel<<<1, 1024, 0, ST(stream)>>>(labels, nll, weight, coef, loss, ntok, T);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_cross_entropy_fwd(const void* logits, int is_fp32, const int32_t* labels, float* nll, float* lse,
                                     int T, int V, int64_t ld, float scale, float softcap, void* stream) {
  if (T <= 0) return 0;
  if (is_fp32) ce_fwd_kernel<true><<<T, NT, 0, ST(stream)>>>(logits, labels, nll, lse, V, ld, scale, softcap);
  else ce_fwd_kernel<false><<<T, NT, 0, ST(stream)>>>(logits, labels, nll, lse, V, ld, scale, softcap);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_cross_entropy_bwd(const void* logits, int is_fp32, const int32_t* labels, const float* lse,
                                     const float* coef, void* dlogits, int T, int V, int64_t ld, float scale,
                                     float softcap, void* stream) {
  if (T <= 0) return 0;
  if (is_fp32) ce_bwd_kernel<true><<<T, NT, 0, ST(stream)>>>(logits, labels, lse, coef, dlogits, V, ld, scale, softcap);
  else ce_bwd_kernel<false><<<T, NT, 0, ST(stream)>>>(logits, labels, lse, coef, dlogits, V, ld, scale, softcap);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_sumsq(const void* x, int is_fp32, int round_bf16, int64_t n, double* sumsq, void* stream) {
  if (n <= 0) return 0;
  const int g = grid_for(n, NT, 148 * 8);
  if (is_fp32) {
    if (round_bf16) sumsq_kernel<true, true><<<g, NT, 0, ST(stream)>>>(x, n, sumsq);
    else sumsq_kernel<true, false><<<g, NT, 0, ST(stream)>>>(x, n, sumsq);
  } else {
    sumsq_kernel<false, false><<<g, NT, 0, ST(stream)>>>(x, n, sumsq);
  }
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_cast_f32_bf16(const float* in, void* out, int64_t n, void* stream) {
  if (n <= 0) return 0;
  cast_f32_bf16_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(in, BFM(out), n);
  OPK_LAUNCH_CHECK();
  return 0;
}

extern "C" int opk_scatter_rows_cast_sumsq(const float* src, void* dst_base, const int64_t* offsets, int R, int D,
                                           double* sumsq, void* stream) {
  if (R <= 0) return 0;
  scatter_rows_cast_sumsq_kernel<<<R, NT, 0, ST(stream)>>>(src, BFM(dst_base), reinterpret_cast<const long long*>(offsets), D, sumsq);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_colsum(const void* dy, float* out, int T, int N, int64_t ld, void* stream) {
  if (T <= 0 || N <= 0) return 0;
  dim3 grid((N + 127) / 128, T < 32 ? T : 32);
  colsum_kernel<<<grid, 128, 0, ST(stream)>>>(BF(dy), out, T, N, ld);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_embedding_add_rows(const int32_t* tok, const int32_t* rep, const float* gc, void* dense, int T, int D,
                                      void* stream) {
  if (T <= 0) return 0;
  emb_add_rows_kernel<<<T, 256, 0, ST(stream)>>>(tok, rep, gc, BFM(dense), D);
  OPK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Allocation-free variant of the compact embedding gradient (declared in opk_noalloc.h).
// The scratch table is a file-scope device array; host code must not pass its name to a kernel (on the host the name
// is only a stand-in), so the device address is resolved once per device with cudaGetSymbolAddress.
#include "opk_noalloc.h"

namespace {
static __device__ __align__(256) int g_noalloc_first_pos[OPK_NOALLOC_MAX_VOCAB];

__global__ void noalloc_fill_kernel(int* __restrict__ p, int n, int value) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) p[i] = value;
}

constexpr int kMaxDevices = 64;
int* g_noalloc_ptr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" int opk_embedding_bwd_compact_noalloc(const int32_t* tok, const void* dx, int32_t* rep, float* gc,
                                                 double* sumsq, int T, int D, int vocab, void* stream) {
  if (T < 0 || D <= 0 || vocab <= 0 || !tok || !dx || !rep || !gc) return -1;
  if (vocab > OPK_NOALLOC_MAX_VOCAB) return -2;
  if (T == 0) return 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return -1;
  cudaStream_t st = ST(stream);
  if (g_noalloc_ptr[dev] == nullptr) {
    // one-time set-up for this device: resolve the device address and put every entry into the idle state
    int* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_first_pos);
    if (e != cudaSuccess) return (int)e;
    noalloc_fill_kernel<<<256, 256, 0, st>>>(p, OPK_NOALLOC_MAX_VOCAB, INT_MAX);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    g_noalloc_ptr[dev] = p;
  }
  int* first_pos = g_noalloc_ptr[dev];
  e = cudaMemsetAsync(gc, 0, sizeof(float) * (size_t)T * D, st);
  if (e != cudaSuccess) return (int)e;
  // entries touched by this call are forced to the idle value first: the table keeps whatever the previous call
  // (possibly one that was interrupted) left behind
  emb_reset_kernel<<<(T + 255) / 256, 256, 0, st>>>(tok, first_pos, T, vocab);
  emb_first_pos_kernel<<<(T + 255) / 256, 256, 0, st>>>(tok, first_pos, T, vocab);
  emb_scatter_kernel<<<T, 256, 0, st>>>(tok, BF(dx), first_pos, rep, gc, D, vocab);
  emb_reset_kernel<<<(T + 255) / 256, 256, 0, st>>>(tok, first_pos, T, vocab);
  if (sumsq) sumsq_kernel<true, true><<<grid_for((long long)T * D, NT, 148 * 4), NT, 0, st>>>(gc, (long long)T * D, sumsq);
  OPK_LAUNCH_CHECK();
  return 0;
}
