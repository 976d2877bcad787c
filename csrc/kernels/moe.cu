// Mixture-of-experts routing, permutation and combination kernels for the native decoder runtime.
//
// A MoE layer of one example runs as: router GEMM -> route (softmax, top-k) -> plan (stable counting sort of the
// T*k (token, slot) entries by expert into 128-row aligned segments, plus the tile / reduction-range tables that the
// grouped GEMM modes consume) -> gather rows -> grouped GEMM (gate/up, SwiGLU epilogue) -> grouped GEMM (down) ->
// combine (weighted sum over the k slots + residual). Everything data-dependent stays on the device: segment sizes
// are only ever read by kernels, so the whole layer is capturable in a CUDA graph with static launch shapes
// (buffers are sized for the worst case R = T*k + E*128 rows).
// The reference routes with eager PyTorch ops and calls torch._grouped_mm
// (packages/opake-patches/src/opake/api/patches/kernels/fused_moe.py:159-335, moe.py:570-627).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "opk_api.h"
#include "debug_bounds.cuh"

namespace {

constexpr int MAX_E = 256;

// ------------------------------------------------------------------------------------------------ route
// One warp per token. probs = softmax(logits); top-k by k rounds of warp arg-max (ties: lowest expert index).
__global__ void __launch_bounds__(256) moe_route_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int T, int E,
                                                        int k, int norm_topk, int* __restrict__ idx,
                                                        float* __restrict__ wts, float* __restrict__ probs) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= T) return;
  float v[MAX_E / 32];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAX_E / 32; ++j) {
    const int e = j * 32 + lane;
    v[j] = e < E ? __bfloat162float(logits[(long long)t * ld + e]) : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < MAX_E / 32; ++j) {
    v[j] = (j * 32 + lane < E) ? __expf(v[j] - mx) : 0.f;
    sum += v[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
#pragma unroll
  for (int j = 0; j < MAX_E / 32; ++j) {
    v[j] *= inv;
    if (j * 32 + lane < E) probs[(long long)t * E + j * 32 + lane] = v[j];
  }
  float sel_sum = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int r = 0; r < k; ++r) {
    float best = -1.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAX_E / 32; ++j) {
      const int e = j * 32 + lane;
      if (v[j] > best) { best = v[j]; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
#pragma unroll
    for (int j = 0; j < MAX_E / 32; ++j)
      if (j * 32 + lane == be) v[j] = -2.f;     // remove the winner
    if (lane == r) { my_w = best; my_e = be; }
    sel_sum += best;
  }
  if (lane < k) {
    idx[(long long)t * k + lane] = my_e;
    wts[(long long)t * k + lane] = norm_topk ? my_w / sel_sum : my_w;
  }
}

// d logits from d weights: p_e * (g_e - sum_j p_j g_j) with g = dL/dp restricted to the selected experts.
__global__ void __launch_bounds__(256) moe_route_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ idx,
                                                            const float* __restrict__ dwts, int T, int E, int k,
                                                            int norm_topk, __nv_bfloat16* __restrict__ dlogits,
                                                            long long ld) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= T) return;
  float p[MAX_E / 32], g[MAX_E / 32];
#pragma unroll
  for (int j = 0; j < MAX_E / 32; ++j) {
    const int e = j * 32 + lane;
    p[j] = e < E ? probs[(long long)t * E + e] : 0.f;
    g[j] = 0.f;
  }
  // selected experts and their upstream gradients
  float S = 0.f, dot_w = 0.f;   // S = sum of selected probabilities, dot_w = sum_i dw_i * w_i (normalised case)
  for (int r = 0; r < k; ++r) {
    const int e = idx[(long long)t * k + r];
    const float pe = probs[(long long)t * E + e];
    S += pe;
  }
  if (norm_topk) {
    for (int r = 0; r < k; ++r) {
      const int e = idx[(long long)t * k + r];
      dot_w += dwts[(long long)t * k + r] * probs[(long long)t * E + e] / S;
    }
  }
  for (int r = 0; r < k; ++r) {
    const int e = idx[(long long)t * k + r];
    const float dw = dwts[(long long)t * k + r];
    const float gv = norm_topk ? (dw - dot_w) / S : dw;
#pragma unroll
    for (int j = 0; j < MAX_E / 32; ++j)
      if (j * 32 + lane == e) g[j] = gv;
  }
  float pg = 0.f;
#pragma unroll
  for (int j = 0; j < MAX_E / 32; ++j) pg += p[j] * g[j];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) pg += __shfl_xor_sync(0xffffffffu, pg, o);
#pragma unroll
  for (int j = 0; j < MAX_E / 32; ++j) {
    const int e = j * 32 + lane;
    if (e < E) dlogits[(long long)t * ld + e] = __float2bfloat16(p[j] * (g[j] - pg));
  }
}

// ------------------------------------------------------------------------------------------------ plan
// Single CTA, one pass over the entries. Stable counting sort by expert: entry n = t*k + slot goes to row off[e] +
// (number of earlier entries with the same expert). Warp w owns the contiguous chunk w of the entry list: per-warp
// histograms in shared memory, per expert an exclusive prefix over the warps (the rank of the warp's first entry of
// that expert), then every warp walks its chunk in order, 32 entries at a time, lanes with the same expert finding
// each other with match.any. Segments are padded to multiples of 128 rows and are at least 128 rows long (an expert
// without tokens still owns one all-zero tile, so its weight gradient is produced as exact zeros by the GEMM).
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ idx, int n_entries, int E, int r_cap,
                                                        int* __restrict__ dest, int* __restrict__ src_entry,
                                                        int* __restrict__ tile_group, int* __restrict__ group_k,
                                                        int* __restrict__ counts_out) {
  __shared__ int hist[32][MAX_E];     // [warp][expert]; becomes the next free row of (warp, expert)
  __shared__ int counts[MAX_E];
  __shared__ int offs[MAX_E + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * MAX_E; i += blockDim.x) (&hist[0][0])[i] = 0;
  __syncthreads();
  const int chunk = ((n_entries + 31) / 32 + 31) / 32 * 32;   // entries per warp, a multiple of 32
  const int c0 = warp * chunk, c1 = min(c0 + chunk, n_entries);
  // an expert id outside [0, E) is dropped from the plan (its dest stays -1): never an index past the histograms
  for (int n = c0 + lane; n < c1; n += 32)
    if (OPK_IDX_OK(idx[n], E) && (unsigned)idx[n] < (unsigned)E) atomicAdd(&hist[warp][idx[n]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = hist[w][e];
      hist[w][e] = run;
      run += c;
    }
    counts[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = off;
      const int padded = counts[e] == 0 ? 128 : (counts[e] + 127) / 128 * 128;
      group_k[2 * e] = off;
      group_k[2 * e + 1] = padded / 64;
      off += padded;
      if (counts_out) counts_out[e] = counts[e];
    }
    offs[E] = off;
  }
  __syncthreads();
  const int total = offs[E];
  // tile -> expert table, padding rows of every segment, everything past the last segment
  for (int e = warp; e < E; e += 32) {
    for (int tl = offs[e] / 128 + lane; tl < offs[e + 1] / 128; tl += 32) tile_group[tl] = e;
    for (int r = offs[e] + counts[e] + lane; r < offs[e + 1]; r += 32) src_entry[r] = -1;
  }
  for (int tl = total / 128 + threadIdx.x; tl < r_cap / 128; tl += blockDim.x) tile_group[tl] = -1;
  for (int r = total + threadIdx.x; r < r_cap; r += blockDim.x) src_entry[r] = -1;
  for (int base = c0; base < c1; base += 32) {
    const int n = base + lane;
    const bool valid = n < c1 && (unsigned)idx[n < c1 ? n : c0] < (unsigned)E;
    if (n < c1 && !valid) dest[n] = -1;
    const int e = valid ? idx[n] : -1 - lane;                 // invalid lanes match nobody
    const unsigned m = __match_any_sync(0xffffffffu, e);
    if (valid) {
      const int row = offs[e] + hist[warp][e] + __popc(m & ((1u << lane) - 1u));
      dest[n] = row;
      src_entry[row] = n;
    }
    __syncwarp();
    if (valid && (m >> lane) == 1u) hist[warp][e] += __popc(m);   // highest lane of each match group
    __syncwarp();
  }
}

// ------------------------------------------------------------------------------------------------ gather / combine
// out[row] = scale * x[src_entry[row] / k] (zeros for padding rows); scale = row_scale[src_entry[row]] when given.
__global__ void __launch_bounds__(256) moe_gather_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                         const int* __restrict__ src_entry, int k,
                                                         const float* __restrict__ entry_scale, int R, int D,
                                                         __nv_bfloat16* __restrict__ out) {
  const int nv = D >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)R * nv; i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / nv), c = (int)(i % nv);
    const int n = src_entry[row];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (n >= 0) {
      v = *reinterpret_cast<const uint4*>(x + (long long)(n / k) * ldx + c * 8);
      if (entry_scale) {
        const float s = entry_scale[n];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(h[j]);
          h[j] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
      }
    }
    *reinterpret_cast<uint4*>(out + (long long)row * D + c * 8) = v;
  }
}

// out[t] = residual[t] + sum_slot w[t][slot] * y[dest[t][slot]] (fp32 accumulation, slots in order: deterministic).
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ dest,
                                                          const float* __restrict__ wts, int k,
                                                          const __nv_bfloat16* __restrict__ residual, int T, int D,
                                                          __nv_bfloat16* __restrict__ out) {
  const int nv = D >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)T * nv; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / nv), c = (int)(i % nv);
    float acc[8];
    if (residual) {
      const uint4 r = *reinterpret_cast<const uint4*>(residual + (long long)t * D + c * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    for (int s = 0; s < k; ++s) {
      const int row = dest[(long long)t * k + s];
      if (row < 0) continue;                                   // entry dropped by the plan (expert id out of range)
      const float w = wts ? wts[(long long)t * k + s] : 1.f;
      const uint4 v = *reinterpret_cast<const uint4*>(y + (long long)row * D + c * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); acc[2 * j] += w * f.x; acc[2 * j + 1] += w * f.y; }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + (long long)t * D + c * 8) = o;
  }
}

// dw[t][slot] = <dy[t], y[dest[t][slot]]>; one warp per entry.
__global__ void __launch_bounds__(256) moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                              const __nv_bfloat16* __restrict__ y,
                                                              const int* __restrict__ dest, int n_entries, int k, int D,
                                                              float* __restrict__ dwts) {
  const int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (n >= n_entries) return;
  if (dest[n] < 0) {
    if (lane == 0) dwts[n] = 0.f;
    return;
  }
  const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(dy + (long long)(n / k) * D);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(y + (long long)dest[n] * D);
  float s = 0.f;
  for (int i = lane; i < D / 2; i += 32) {
    const float2 p = __bfloat1622float2(a[i]), q = __bfloat1622float2(b[i]);
    s += p.x * q.x + p.y * q.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) dwts[n] = s;
}

inline int grid_for(long long n, int block, int cap = 148 * 8) {
  long long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

OPK_DEBUG_BOUNDS_UNIT();

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFM(p) reinterpret_cast<__nv_bfloat16*>(p)

extern "C" int opk_moe_route(const void* logits, int64_t ld, int T, int E, int k, int norm_topk, int32_t* idx, float* wts,
                             float* probs, void* stream) {
  if (T <= 0) return 0;
  if (E > MAX_E || k > 32 || k > E || k < 1) return -1;
  moe_route_kernel<<<(T * 32 + 255) / 256, 256, 0, ST(stream)>>>(BF(logits), ld, T, E, k, norm_topk, idx, wts, probs);
  return (int)cudaGetLastError();
}

extern "C" int opk_moe_route_bwd(const float* probs, const int32_t* idx, const float* dwts, int T, int E, int k, int norm_topk,
                                 void* dlogits, int64_t ld, void* stream) {
  if (T <= 0) return 0;
  if (E > MAX_E || k > 32) return -1;
  moe_route_bwd_kernel<<<(T * 32 + 255) / 256, 256, 0, ST(stream)>>>(probs, idx, dwts, T, E, k, norm_topk, BFM(dlogits), ld);
  return (int)cudaGetLastError();
}

extern "C" int opk_moe_rows_capacity(int n_entries, int E) { return (n_entries + 127) / 128 * 128 + E * 128; }

extern "C" int opk_moe_plan(const int32_t* idx, int n_entries, int E, int r_cap, int32_t* dest, int32_t* src_entry,
                            int32_t* tile_group, int32_t* group_k, int32_t* counts, void* stream) {
  if (E > MAX_E || r_cap % 128 || r_cap < opk_moe_rows_capacity(n_entries, E)) return -1;
  moe_plan_kernel<<<1, 1024, 0, ST(stream)>>>(idx, n_entries, E, r_cap, dest, src_entry, tile_group, group_k, counts);
  return (int)cudaGetLastError();
}

extern "C" int opk_moe_gather(const void* x, int64_t ldx, const int32_t* src_entry, int k, const float* entry_scale, int R,
                              int D, void* out, void* stream) {
  if (R <= 0) return 0;
  if (D % 8) return -1;
  moe_gather_kernel<<<grid_for((long long)R * (D / 8), 256), 256, 0, ST(stream)>>>(BF(x), ldx, src_entry, k, entry_scale, R, D, BFM(out));
  return (int)cudaGetLastError();
}

extern "C" int opk_moe_combine(const void* y, const int32_t* dest, const float* wts, int k, const void* residual, int T, int D,
                               void* out, void* stream) {
  if (T <= 0) return 0;
  if (D % 8) return -1;
  moe_combine_kernel<<<grid_for((long long)T * (D / 8), 256), 256, 0, ST(stream)>>>(BF(y), dest, wts, k, BF(residual), T, D, BFM(out));
  return (int)cudaGetLastError();
}

extern "C" int opk_moe_combine_bwd(const void* dy, const void* y, const int32_t* dest, int n_entries, int k, int D, float* dwts,
                                   void* stream) {
  if (n_entries <= 0) return 0;
  if (D % 2) return -1;
  moe_combine_bwd_kernel<<<(int)(((long long)n_entries * 32 + 255) / 256), 256, 0, ST(stream)>>>(BF(dy), BF(y), dest, n_entries, k, D, dwts);
  return (int)cudaGetLastError();
}
