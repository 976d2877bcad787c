// Multi-tensor clip-and-sum for materialised per-example gradients (the generic vmap path).
//
// Input: L leaves, leaf l holding B examples of n_l elements each (bf16 or fp32, example-major). Three steps:
//   1. sumsq_partial: grid (tiles, B). Every CTA squares up to TILE elements of one example of one leaf in fp32 and
//      sums the squares in fp64; partial[b][tile] is written once (no atomics, so the later sum has a fixed order).
//   2. (host side, on the [B] vector) norm -> guarded clip factor per storage dtype.
//   3. apply_sum: grid (tiles). out[i] = sum_b stored(g_b[i] * f_b) accumulated in fp32, where stored() rounds the
//      fp32 product to the leaf's storage dtype and flushes results that rounded UP into the subnormal range to zero
//      (so a clipped example can never exceed its bound in storage precision). Optionally the squared norm of every
//      example after clipping (again per tile, fp64).
// The reference does the same with three Triton programs driven by pointer tables
// (packages/opake-patches/src/opake/api/patches/kernels/_clip_sum.py:74-152, driver :270-379); here one table of tile
// descriptors serves both kernels and the per-example loop of step 3 keeps the running sum in registers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "opk_api.h"

namespace {

constexpr int CS_THREADS = 256;
constexpr int CS_TILE = 4096;          // elements per CTA
constexpr int CS_PER_THREAD = CS_TILE / CS_THREADS;

struct TileDesc {
  const void* base;       // leaf base pointer
  float* out;             // leaf output (fp32 sums)
  long long n;            // elements per example in this leaf
  long long off;          // first element of the tile inside an example
  int is_bf16;
  int pad;
};

__device__ __forceinline__ float load_elem(const TileDesc& t, long long idx) {
  return t.is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(t.base)[idx])
                   : reinterpret_cast<const float*>(t.base)[idx];
}

// Eight consecutive elements starting at idx (`valid` of them exist). Vector loads when the address allows it.
__device__ __forceinline__ void load8(const TileDesc& t, long long idx, long long valid, bool vec, float (&x)[8]) {
  if (vec && valid >= 8) {
    if (t.is_bf16) {
      const uint4 v = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(t.base) + idx));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); x[2 * j] = f.x; x[2 * j + 1] = f.y; }
    } else {
      const float4 a = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(t.base) + idx));
      const float4 b = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(t.base) + idx + 4));
      x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = j < valid ? load_elem(t, idx + j) : 0.f;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (!isfinite(x[j])) x[j] = 0.f;           // NaN / Inf are sanitised to zero before clipping
}

__device__ __forceinline__ double block_sum_f64(double v, double* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  double s = 0.0;
  if (threadIdx.x == 0)
    for (int i = 0; i < CS_THREADS / 32; ++i) s += sh[i];
  return s;   // valid in thread 0
}

__global__ void __launch_bounds__(CS_THREADS) sumsq_partial_kernel(const TileDesc* __restrict__ tiles, int n_tiles,
                                                                   double* __restrict__ partial) {
  __shared__ double sh[CS_THREADS / 32];
  const TileDesc t = tiles[blockIdx.x];
  const int b = blockIdx.y;
  const long long base = (long long)b * t.n + t.off;
  const long long lim = t.n - t.off;
  // vector loads need 16-byte aligned rows: the leaf base is, so the example stride must be a multiple of 8 elements
  const bool vec = (t.n & 7) == 0 && (reinterpret_cast<uintptr_t>(t.base) & 15) == 0;
  double acc = 0.0;
#pragma unroll
  for (int k = 0; k < CS_PER_THREAD / 8; ++k) {
    const long long i = ((long long)k * CS_THREADS + threadIdx.x) * 8;
    if (i < lim) {
      float x[8];
      load8(t, base + i, lim - i, vec, x);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += (double)(x[j] * x[j]);
    }
  }
  const double s = block_sum_f64(acc, sh);
  if (threadIdx.x == 0) partial[(long long)b * n_tiles + blockIdx.x] = s;
}

__device__ __forceinline__ float store_round(float scaled, int is_bf16) {
  if (!is_bf16) return scaled;
  const float back = __bfloat162float(__float2bfloat16_rn(scaled));
  const float tiny = 1.1754943508222875e-38f;   // smallest normal of bf16 (= fp32)
  return (fabsf(back) <= tiny && fabsf(back) > fabsf(scaled)) ? 0.f : back;
}

template <bool POSTSQ>
__global__ void __launch_bounds__(CS_THREADS) apply_sum_kernel(const TileDesc* __restrict__ tiles, int n_tiles, int B,
                                                               const float* __restrict__ f_bf16,
                                                               const float* __restrict__ f_fp32,
                                                               double* __restrict__ post_partial) {
  __shared__ double sh[CS_THREADS / 32];
  const TileDesc t = tiles[blockIdx.x];
  const long long lim = t.n - t.off;
  const float* fac = t.is_bf16 ? f_bf16 : f_fp32;
  const bool vec = (t.n & 7) == 0 && (reinterpret_cast<uintptr_t>(t.base) & 15) == 0;
  float acc[CS_PER_THREAD];
#pragma unroll
  for (int k = 0; k < CS_PER_THREAD; ++k) acc[k] = 0.f;
  for (int b = 0; b < B; ++b) {
    const float f = fac[b];
    const long long base = (long long)b * t.n + t.off;
    double post = 0.0;
#pragma unroll
    for (int k = 0; k < CS_PER_THREAD / 8; ++k) {
      const long long i = ((long long)k * CS_THREADS + threadIdx.x) * 8;
      if (i < lim) {
        float x[8];
        load8(t, base + i, lim - i, vec, x);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float st = store_round(x[j] * f, t.is_bf16);
          acc[k * 8 + j] += st;
          if (POSTSQ) post += (double)(st * st);
        }
      }
    }
    if (POSTSQ) {
      const double s = block_sum_f64(post, sh);
      if (threadIdx.x == 0) post_partial[(long long)b * n_tiles + blockIdx.x] = s;
    }
  }
#pragma unroll
  for (int k = 0; k < CS_PER_THREAD / 8; ++k) {
    const long long i = ((long long)k * CS_THREADS + threadIdx.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i + j < lim) t.out[t.off + i + j] = acc[k * 8 + j];
  }
}

}  // namespace

extern "C" int opk_clip_sum_tile() { return CS_TILE; }
extern "C" int opk_clip_sum_desc_bytes() { return (int)sizeof(TileDesc); }

extern "C" int opk_clip_sumsq_partial(const void* tiles, int n_tiles, int B, double* partial, void* stream) {
  if (n_tiles <= 0 || B <= 0) return 0;
  if (B > 65535) return -1;
  dim3 grid(n_tiles, B);
  sumsq_partial_kernel<<<grid, CS_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const TileDesc*>(tiles), n_tiles, partial);
  return (int)cudaGetLastError();
}

extern "C" int opk_clip_apply_sum(const void* tiles, int n_tiles, int B, const float* f_bf16, const float* f_fp32,
                                  double* post_partial, void* stream) {
  if (n_tiles <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (post_partial)
    apply_sum_kernel<true><<<n_tiles, CS_THREADS, 0, st>>>(reinterpret_cast<const TileDesc*>(tiles), n_tiles, B, f_bf16,
                                                          f_fp32, post_partial);
  else
    apply_sum_kernel<false><<<n_tiles, CS_THREADS, 0, st>>>(reinterpret_cast<const TileDesc*>(tiles), n_tiles, B, f_bf16,
                                                           f_fp32, nullptr);
  return (int)cudaGetLastError();
}
