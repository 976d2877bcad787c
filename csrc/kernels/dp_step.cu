// Differential-privacy step kernels for sm_100a:
//   * guarded clip scale from a per-example squared norm (conservative rounding: the stored clipped
//     gradient never exceeds the clipping norm),
//   * clipped accumulation  acc += bf16(g * scale),
//   * counter-based Philox4x32-10 Gaussian noise indexed by the global element offset, so every
//     sharding of the parameter vector draws the same global noise tensor exactly once,
//   * the fused step: reduce-scatter of the clipped-gradient sums over peer memory (plain P2P loads),
//     normalisation, noise (optionally correlated through a buffered-linear-Toeplitz state), DP-AdamW with
//     noise bias correction, and the all-gather of the updated bf16 parameters as P2P stores.
#include "opk_api.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

namespace {

#define OPK_LAUNCH_CHECK()                                   \
  do {                                                       \
    cudaError_t e__ = cudaGetLastError();                    \
    if (e__ != cudaSuccess) return (int)e__;                 \
  } while (0)

// ------------------------------------------------------------------------------------------- Philox4x32-10
struct U4 { uint32_t x, y, z, w; };
__host__ __device__ __forceinline__ U4 philox4x32_10(U4 c, uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)M0 * c.x, p1 = (uint64_t)M1 * c.z;
    U4 n;
    n.x = (uint32_t)(p1 >> 32) ^ c.y ^ k0;
    n.y = (uint32_t)p1;
    n.z = (uint32_t)(p0 >> 32) ^ c.w ^ k1;
    n.w = (uint32_t)p0;
    c = n;
    k0 += W0;
    k1 += W1;
  }
  return c;
}
// Four standard normals for the aligned group of four elements with index q = element / 4.
__device__ __forceinline__ void normal4(uint64_t q, uint64_t seed, uint32_t stream_id, uint32_t step, float (&z)[4]) {
  U4 c{(uint32_t)q, (uint32_t)(q >> 32), step, stream_id};
  const U4 r = philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
  const float k = 2.3283064365386963e-10f;  // 2^-32
  const float u1 = ((float)r.x + 1.0f) * k, u2 = (float)r.y * k;
  const float u3 = ((float)r.z + 1.0f) * k, u4 = (float)r.w * k;
  // hardware lg2 / sin / cos (absolute error about 1e-6 here); the angle is taken in [-pi, pi), where the fast
  // sine and cosine are most accurate, and the half-turn is undone by the sign: sin(t + pi) = -sin t, cos likewise
  const float ra = sqrtf(-2.0f * __logf(fminf(u1, 1.0f))), rb = sqrtf(-2.0f * __logf(fminf(u3, 1.0f)));
  const float two_pi = 6.283185307179586f;
  const float ta = two_pi * (u2 - 0.5f), tb = two_pi * (u4 - 0.5f);
  z[0] = -ra * __cosf(ta);
  z[1] = -ra * __sinf(ta);
  z[2] = -rb * __cosf(tb);
  z[3] = -rb * __sinf(tb);
}

__global__ void philox_normal_kernel(float* __restrict__ out, long long n, uint64_t seed, uint32_t stream_id,
                                     uint32_t step, uint64_t offset, float sigma, int accumulate) {
  // thread handles one aligned quad of the GLOBAL index space; elements outside [offset, offset+n) are skipped
  const uint64_t q0 = offset >> 2;
  const uint64_t q1 = (offset + (uint64_t)n + 3) >> 2;
  for (uint64_t q = q0 + blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; q < q1; q += (uint64_t)gridDim.x * blockDim.x) {
    float z[4];
    normal4(q, seed, stream_id, step, z);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint64_t e = q * 4 + j;
      if (e >= offset && e < offset + (uint64_t)n) {
        const long long i = (long long)(e - offset);
        out[i] = accumulate ? out[i] + sigma * z[j] : sigma * z[j];
      }
    }
  }
}

// ------------------------------------------------------------------------------------------- clip scale
// Conservative clip factor (fixed clipping): the factor is shrunk by the worst-case rounding of the norm
// accumulation, of the fp32 multiply and of the bf16 store, so that the norm of the *stored* clipped gradient
// is <= clip. AUTO-S (mode_auto): R / (norm + gamma) with the same guard and no clamp to one.
__global__ void clip_scale_kernel(double* sumsq, float clip, int mode_auto, float gamma, int n_leaves,
                                  long long widest_leaf, float* scale_out, float* norm_out, int* counters, int reset) {
  const double sq = *sumsq;
  if (reset) *sumsq = 0.0;
  const double norm = sqrt(sq > 0.0 ? sq : 0.0);
  if (norm_out) *norm_out = (float)norm;
  const double c = clip > 0.f ? (double)clip : 0.0;
  double ratio;
  if (mode_auto) ratio = c / (norm + (double)gamma);
  else ratio = norm > 0.0 ? c / norm : INFINITY;
  if (counters && !mode_auto && norm > c) atomicAdd(counters, 1);
  // unit roundoffs
  const double u_acc = 1.1920928955078125e-07 / 2.0;   // fp32
  const double u_sq = 2.220446049250313e-16 / 2.0;     // fp64
  const double n_red = widest_leaf > 4096 ? 2048.0 + ceil((double)widest_leaf / 2048.0) : (double)widest_leaf;
  // the tile epilogues add 256 squares per thread in fp32 plus a 5-level shuffle tree before going to fp64
  const double tile_slack = 264.0 * u_acc;
  const double roundoff = (u_acc + ((double)(n_leaves > 1 ? n_leaves : 1) + n_red) * u_sq + tile_slack) / 2.0;
  const double store_eps = 0.0078125, mult_eps = 1.1920928955078125e-07;  // bf16 store, fp32 multiply
  const double rounding = store_eps / 2.0 + mult_eps;
  double s = ratio * (1.0 - rounding - 2.0 * roundoff) - 1.1754943508222875e-38 * store_eps;
  if (!mode_auto && s > 1.0) s = 1.0;
  if (!isfinite(s)) s = (!mode_auto && ratio > 0) ? 1.0 : 0.0;
  if (s < 0.0) s = 0.0;
  if (clip <= 0.f) s = 0.0;
  // round the fp32 factor toward zero so the cast itself cannot enlarge it
  float sf = (float)s;
  if ((double)sf > s) sf = nextafterf(sf, 0.0f);
  *scale_out = sf;
}

struct alignas(16) bf16x8 { __nv_bfloat162 h[4]; };

__device__ __forceinline__ float clip_store(float g, float s) {
  const float scaled = g * s;
  float stored = __bfloat162float(__float2bfloat16(scaled));
  // a value that rounded *up* into (or within) the subnormal range would break the bound: flush it
  if (fabsf(stored) <= 1.1754943508222875e-38f && fabsf(stored) > fabsf(scaled)) stored = 0.f;
  return stored;
}

__global__ void __launch_bounds__(256) clip_accumulate_kernel(const bf16x8* __restrict__ g, const float* __restrict__ scale,
                                                              float4* __restrict__ acc, long long nvec, int overwrite) {
  const float s = *scale;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < nvec; i += (long long)gridDim.x * 256) {
    // streaming accesses: this kernel runs next to tensor-core GEMMs whose operand tiles live in L2
    const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(g) + i);
    const bf16x8 v = *reinterpret_cast<const bf16x8*>(&raw);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(v.h[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
    float4 a0, a1;
    if (overwrite) {
      a0 = make_float4(0.f, 0.f, 0.f, 0.f);
      a1 = a0;
    } else {
      a0 = __ldcs(acc + 2 * i);
      a1 = __ldcs(acc + 2 * i + 1);
    }
    a0.x += clip_store(f[0], s); a0.y += clip_store(f[1], s); a0.z += clip_store(f[2], s); a0.w += clip_store(f[3], s);
    a1.x += clip_store(f[4], s); a1.y += clip_store(f[5], s); a1.z += clip_store(f[6], s); a1.w += clip_store(f[7], s);
    __stcs(acc + 2 * i, a0);
    __stcs(acc + 2 * i + 1, a1);
  }
}
// N examples in one pass over the fp32 sums: acc += sum_j stored(g_j * s_j). Per example this moves 2 + 8 / N bytes per
// parameter; N is bounded by how many whole-model gradient buffers fit next to the optimizer state.
struct AccGroup {
  const bf16x8* g[OPK_ACC_GROUP_MAX];
  const float* scale[OPK_ACC_GROUP_MAX];
};
template <int N>
__global__ void __launch_bounds__(256) clip_accumulate_group_kernel(const AccGroup grp, float4* __restrict__ acc, long long nvec,
                                                                    int overwrite) {
  float s[N];
#pragma unroll
  for (int j = 0; j < N; ++j) s[j] = *grp.scale[j];
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < nvec; i += (long long)gridDim.x * 256) {
    uint4 r[N];
#pragma unroll
    for (int j = 0; j < N; ++j) r[j] = __ldcs(reinterpret_cast<const uint4*>(grp.g[j]) + i);
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    if (!overwrite) {
      a0 = __ldcs(acc + 2 * i);
      a1 = __ldcs(acc + 2 * i + 1);
    }
    float f[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) f[q] = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) {       // examples in slot order: the sum does not depend on the launch shape
      const bf16x8 v = *reinterpret_cast<const bf16x8*>(&r[j]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 t = __bfloat1622float2(v.h[q]);
        f[2 * q] += clip_store(t.x, s[j]);
        f[2 * q + 1] += clip_store(t.y, s[j]);
      }
    }
    a0.x += f[0]; a0.y += f[1]; a0.z += f[2]; a0.w += f[3];
    a1.x += f[4]; a1.y += f[5]; a1.z += f[6]; a1.w += f[7];
    __stcs(acc + 2 * i, a0);
    __stcs(acc + 2 * i + 1, a1);
  }
}
__global__ void clip_accumulate_tail_kernel(const __nv_bfloat16* __restrict__ g, const float* __restrict__ scale,
                                            float* __restrict__ acc, long long begin, long long n, int overwrite) {
  const float s = *scale;
  const long long i = begin + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < n) acc[i] = (overwrite ? 0.f : acc[i]) + clip_store(__bfloat162float(g[i]), s);
}

// ------------------------------------------------------------------------------------------- fused DP step
struct StepParams {
  OpkDpStepArgs a;
};

constexpr int MAX_PEERS = 16;
struct PeerTable {
  const float* grad[MAX_PEERS];
  __nv_bfloat16* param[MAX_PEERS];
};

// One parameter update given the averaged, noised gradient. Returns the new parameter value.
template <bool ADAM>
__device__ __forceinline__ float dp_update(const OpkDpStepArgs& a, float inv_bc1, float inv_bc2, float grad, float p_old,
                                           float& m, float& v) {
  float upd;
  if (!ADAM) {
    upd = grad + a.weight_decay * p_old;
  } else {
    m = a.beta1 * m + (1.f - a.beta1) * grad;
    v = a.beta2 * v + (1.f - a.beta2) * grad * grad;
    const float mh = m * inv_bc1, vh = v * inv_bc2;
    const float d = vh - a.phi_hat;            // noise bias correction: subtract the noise's share of v-hat
    const float den = sqrtf(d > 0.f ? d : vh) + a.eps;
    upd = __fdividef(mh, den) + a.weight_decay * p_old;
  }
  return p_old - a.lr * upd;
}

// Correlated-noise transforms of the iid draw z (DP-FTRL), applied element-wise on the shard:
//   CORR_BLT       buffered linear Toeplitz C^{-1}: zhat = z - <scale, state>; state_k = decay_k * state_k + zhat
//   CORR_TOEPLITZ  banded Toeplitz C^{-1} (band-MF, banded square root): zhat = (z - sum_{k>=1} c_k zhat_{t-k}) / c_0
//                  with the last nlag outputs kept in a ring; lag k lives in ring slot (pos + k - 1) mod nlag and the
//                  new output overwrites the oldest slot, (pos + nlag - 1) mod nlag, which the host makes the next pos
enum { CORR_NONE = 0, CORR_BLT = 1, CORR_TOEPLITZ = 2 };

template <int CORR>
__device__ __forceinline__ void correlate_quad(const OpkDpStepArgs& a, long long i0, float (&z)[4]) {
  if (CORR == CORR_BLT) {
    float rd[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < a.blt_nbuf; ++k) {
      const float4 st = *reinterpret_cast<const float4*>(a.blt_state + (long long)k * a.shard_len + i0);
      const float sc = a.blt_scale[k];
      rd[0] += sc * st.x; rd[1] += sc * st.y; rd[2] += sc * st.z; rd[3] += sc * st.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) z[j] -= rd[j];
    for (int k = 0; k < a.blt_nbuf; ++k) {
      float4* sp = reinterpret_cast<float4*>(a.blt_state + (long long)k * a.shard_len + i0);
      float4 st = *sp;
      const float dc = a.blt_decay[k];
      st.x = dc * st.x + z[0]; st.y = dc * st.y + z[1]; st.z = dc * st.z + z[2]; st.w = dc * st.w + z[3];
      *sp = st;
    }
  } else if (CORR == CORR_TOEPLITZ) {
    float rd[4] = {0.f, 0.f, 0.f, 0.f};
    int slot = a.toep_pos;
    for (int k = 1; k <= a.toep_nlag; ++k) {
      const float4 st = __ldcs(reinterpret_cast<const float4*>(a.toep_state + (long long)slot * a.shard_len + i0));
      const float c = a.toep_coef[k];
      rd[0] += c * st.x; rd[1] += c * st.y; rd[2] += c * st.z; rd[3] += c * st.w;
      if (++slot == a.toep_nlag) slot = 0;
    }
    const float inv_c0 = 1.f / a.toep_coef[0];
#pragma unroll
    for (int j = 0; j < 4; ++j) z[j] = (z[j] - rd[j]) * inv_c0;
    if (a.toep_nlag > 0) {
      const int oldest = a.toep_pos == 0 ? a.toep_nlag - 1 : a.toep_pos - 1;
      __stcs(reinterpret_cast<float4*>(a.toep_state + (long long)oldest * a.shard_len + i0), make_float4(z[0], z[1], z[2], z[3]));
    }
  }
}
template <int CORR>
__device__ __forceinline__ float correlate_one(const OpkDpStepArgs& a, long long i, float z) {
  if (CORR == CORR_BLT) {
    float rd = 0.f;
    for (int k = 0; k < a.blt_nbuf; ++k) rd += a.blt_scale[k] * a.blt_state[(long long)k * a.shard_len + i];
    z -= rd;
    for (int k = 0; k < a.blt_nbuf; ++k) {
      float* sp = &a.blt_state[(long long)k * a.shard_len + i];
      *sp = a.blt_decay[k] * (*sp) + z;
    }
  } else if (CORR == CORR_TOEPLITZ) {
    float rd = 0.f;
    int slot = a.toep_pos;
    for (int k = 1; k <= a.toep_nlag; ++k) {
      rd += a.toep_coef[k] * a.toep_state[(long long)slot * a.shard_len + i];
      if (++slot == a.toep_nlag) slot = 0;
    }
    z = (z - rd) / a.toep_coef[0];
    if (a.toep_nlag > 0) a.toep_state[(long long)(a.toep_pos == 0 ? a.toep_nlag - 1 : a.toep_pos - 1) * a.shard_len + i] = z;
  }
  return z;
}

// Everything a full quad needs from memory, fetched before any arithmetic so that two quads per thread keep eight to
// ten 16-byte loads in flight.
struct QuadIn {
  float4 g, m, v, mw;
  uint2 pw;
};
template <bool ADAM, bool MASTER>
__device__ __forceinline__ void load_quad(const OpkDpStepArgs& a, const PeerTable& pt, long long i0, long long e0, QuadIn& q) {
  // reduce-scatter: sum the owned quad over every rank's buffer (peer reads travel over NVLink)
  q.g = __ldcs(reinterpret_cast<const float4*>(pt.grad[0] + e0));
  for (int r = 1; r < a.n_src; ++r) {
    const float4 t = __ldcs(reinterpret_cast<const float4*>(pt.grad[r] + e0));
    q.g.x += t.x; q.g.y += t.y; q.g.z += t.z; q.g.w += t.w;
  }
  if (MASTER) q.mw = __ldcs(reinterpret_cast<const float4*>(a.master + i0));
  else q.pw = __ldcs(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.param_src) + e0));
  if (ADAM) {
    q.m = __ldcs(reinterpret_cast<const float4*>(a.m + i0));
    q.v = __ldcs(reinterpret_cast<const float4*>(a.v + i0));
  }
}
template <bool ADAM, bool MASTER, int CORR>
__device__ __forceinline__ void finish_quad(const OpkDpStepArgs& a, const PeerTable& pt, float inv_bc1, float inv_bc2,
                                            long long i0, long long e0, const QuadIn& q) {
  float z[4] = {0.f, 0.f, 0.f, 0.f};
  if (a.sigma != 0.f) normal4((uint64_t)e0 >> 2, a.seed, a.stream_id, a.step, z);
  correlate_quad<CORR>(a, i0, z);
  float po[4];
  if (MASTER) {
    po[0] = q.mw.x; po[1] = q.mw.y; po[2] = q.mw.z; po[3] = q.mw.w;
  } else {
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.pw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.pw.y));
    po[0] = lo.x; po[1] = lo.y; po[2] = hi.x; po[3] = hi.y;
  }
  const float gr[4] = {q.g.x, q.g.y, q.g.z, q.g.w};
  float mm[4] = {q.m.x, q.m.y, q.m.z, q.m.w}, vv[4] = {q.v.x, q.v.y, q.v.z, q.v.w};
  float pn[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    pn[j] = dp_update<ADAM>(a, inv_bc1, inv_bc2, gr[j] * a.inv_batch + a.sigma * z[j], po[j], mm[j], vv[j]);
  if (ADAM) {
    __stcs(reinterpret_cast<float4*>(a.m + i0), make_float4(mm[0], mm[1], mm[2], mm[3]));
    __stcs(reinterpret_cast<float4*>(a.v + i0), make_float4(vv[0], vv[1], vv[2], vv[3]));
  }
  if (MASTER) __stcs(reinterpret_cast<float4*>(a.master + i0), make_float4(pn[0], pn[1], pn[2], pn[3]));
  // all-gather: write the updated bf16 quad into every destination parameter buffer
  uint2 o;
  __nv_bfloat162 lo = __floats2bfloat162_rn(pn[0], pn[1]), hi = __floats2bfloat162_rn(pn[2], pn[3]);
  o.x = *reinterpret_cast<uint32_t*>(&lo);
  o.y = *reinterpret_cast<uint32_t*>(&hi);
  for (int r = 0; r < a.n_dst; ++r) *reinterpret_cast<uint2*>(pt.param[r] + e0) = o;
  if (a.zero_grad) *reinterpret_cast<float4*>(const_cast<float*>(pt.grad[0]) + e0) = make_float4(0.f, 0.f, 0.f, 0.f);
}

template <bool ADAM, bool MASTER, int CORR>
__global__ void __launch_bounds__(256) dp_step_kernel(const OpkDpStepArgs a, const PeerTable pt) {
  // Each thread owns aligned quads of the shard, two per iteration; shard_begin is a multiple of 4 and a ragged last
  // quad takes the scalar path. Everything is touched exactly once: streaming loads and stores.
  const long long nfull = a.shard_len >> 2;                // whole quads
  const float inv_bc1 = 1.f / a.bc1, inv_bc2 = 1.f / a.bc2;
  const long long stride = (long long)gridDim.x * 256;
  long long q = blockIdx.x * 256ll + threadIdx.x;
  for (; q + stride < nfull; q += 2 * stride) {
    const long long ia = q << 2, ib = (q + stride) << 2;
    QuadIn qa, qb;
    qa.m = qa.v = qb.m = qb.v = make_float4(0.f, 0.f, 0.f, 0.f);
    load_quad<ADAM, MASTER>(a, pt, ia, a.shard_begin + ia, qa);
    load_quad<ADAM, MASTER>(a, pt, ib, a.shard_begin + ib, qb);
    finish_quad<ADAM, MASTER, CORR>(a, pt, inv_bc1, inv_bc2, ia, a.shard_begin + ia, qa);
    finish_quad<ADAM, MASTER, CORR>(a, pt, inv_bc1, inv_bc2, ib, a.shard_begin + ib, qb);
  }
  if (q < nfull) {
    const long long ia = q << 2;
    QuadIn qa;
    qa.m = qa.v = make_float4(0.f, 0.f, 0.f, 0.f);
    load_quad<ADAM, MASTER>(a, pt, ia, a.shard_begin + ia, qa);
    finish_quad<ADAM, MASTER, CORR>(a, pt, inv_bc1, inv_bc2, ia, a.shard_begin + ia, qa);
  }
  // ragged tail (fewer than 4 elements): one thread
  const int cnt = (int)(a.shard_len & 3);
  if (cnt && blockIdx.x == 0 && threadIdx.x == 0) {
    const long long i0 = nfull << 2, e0 = a.shard_begin + i0;
    float z[4] = {0.f, 0.f, 0.f, 0.f};
    if (a.sigma != 0.f) normal4((uint64_t)e0 >> 2, a.seed, a.stream_id, a.step, z);
    for (int j = 0; j < cnt; ++j) {
      const long long i = i0 + j;
      float g = 0.f;
      for (int r = 0; r < a.n_src; ++r) g += pt.grad[r][e0 + j];
      const float noise = correlate_one<CORR>(a, i, z[j]);
      const float p_old = MASTER ? a.master[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.param_src)[e0 + j]);
      float m = ADAM ? a.m[i] : 0.f, v = ADAM ? a.v[i] : 0.f;
      const float p_new = dp_update<ADAM>(a, inv_bc1, inv_bc2, g * a.inv_batch + a.sigma * noise, p_old, m, v);
      if (ADAM) { a.m[i] = m; a.v[i] = v; }
      if (MASTER) a.master[i] = p_new;
      for (int r = 0; r < a.n_dst; ++r) pt.param[r][e0 + j] = __float2bfloat16(p_new);
      if (a.zero_grad) const_cast<float*>(pt.grad[0])[e0 + j] = 0.f;
    }
  }
}

// ------------------------------------------------------------------------------------------- sharded sums (push)
// The fp32 sums are sharded: rank o owns elements [begin[o], begin[o+1]) of the flat parameter vector and keeps them in
// a peer-addressable buffer. A group of clipped per-example gradients is added with reductions sent to the owner
// (red.add over NVLink for remote owners), so no rank ever holds a full-size fp32 sum. Peers add into the same shard
// concurrently, hence reductions for the local part as well.
struct ShardTable {
  float* acc[MAX_PEERS];
  long long begin[MAX_PEERS + 1];
  int n;
};
__device__ __forceinline__ void red_add_f32x4(float* dst, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
template <int N>
__global__ void __launch_bounds__(256) clip_accumulate_group_push_kernel(const AccGroup grp, const ShardTable sh, long long nvec,
                                                                         long long rot) {
  float s[N];
#pragma unroll
  for (int j = 0; j < N; ++j) s[j] = *grp.scale[j];
  for (long long t = blockIdx.x * 256ll + threadIdx.x; t < nvec; t += (long long)gridDim.x * 256) {
    // every rank starts at its own shard and walks the owners in rank order: at any moment the ranks push to
    // different owners
    long long i = t + rot;
    if (i >= nvec) i -= nvec;
    uint4 r[N];
#pragma unroll
    for (int j = 0; j < N; ++j) r[j] = __ldcs(reinterpret_cast<const uint4*>(grp.g[j]) + i);
    float f[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) f[q] = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const bf16x8 v = *reinterpret_cast<const bf16x8*>(&r[j]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 u = __bfloat1622float2(v.h[q]);
        f[2 * q] += clip_store(u.x, s[j]);
        f[2 * q + 1] += clip_store(u.y, s[j]);
      }
    }
    const long long e = i << 3;
    int o = 0;
    while (o + 1 < sh.n && e >= sh.begin[o + 1]) ++o;
    float* dst = sh.acc[o] + (e - sh.begin[o]);
    red_add_f32x4(dst, f[0], f[1], f[2], f[3]);
    red_add_f32x4(dst + 4, f[4], f[5], f[6], f[7]);
  }
}
template <int N>
void launch_acc_group_push(const AccGroup& grp, const ShardTable& sh, long long nvec, long long rot, cudaStream_t st) {
  long long g = (nvec + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  clip_accumulate_group_push_kernel<N><<<(int)g, 256, 0, st>>>(grp, sh, nvec, rot);
}

// Plain copy between two device buffers that may live on different GPUs (peer-mapped memory): 16-byte vectors, eight
// loads in flight per thread. Used to refresh the parts of a parameter replica that no GEMM stages for itself.
__global__ void __launch_bounds__(256) copy_vec_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long nvec) {
  constexpr int U = 8;
  const long long stride = (long long)gridDim.x * 256;
  for (long long i0 = blockIdx.x * 256ll + threadIdx.x; i0 < nvec; i0 += U * stride) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) v[u] = __ldcg(src + i);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) dst[i] = v[u];
    }
  }
}

inline int grid_for(long long n, int block, int cap_blocks) {
  long long g = (n + block - 1) / block;
  if (g > cap_blocks) g = cap_blocks;
  if (g < 1) g = 1;
  return (int)g;
}

// ragged tail (fewer than 8 elements) of the group pass, same association as the vector body
__global__ void clip_accumulate_group_tail_kernel(const AccGroup grp, int n_group, float* __restrict__ acc, long long begin,
                                                  long long n, int overwrite) {
  const long long i = begin + threadIdx.x;
  if (i >= n) return;
  float f = 0.f;
  for (int j = 0; j < n_group; ++j)
    f += clip_store(__bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grp.g[j])[i]), *grp.scale[j]);
  acc[i] = (overwrite ? 0.f : acc[i]) + f;
}
template <int N>
void launch_acc_group(const AccGroup& grp, float* acc, long long nvec, int overwrite, cudaStream_t st) {
  clip_accumulate_group_kernel<N><<<grid_for(nvec, 256, 148 * 16), 256, 0, st>>>(grp, reinterpret_cast<float4*>(acc), nvec, overwrite);
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int opk_philox_normal(float* out, int64_t n, uint64_t seed, uint32_t stream_id, uint32_t step,
                                 uint64_t offset, float sigma, int accumulate, void* stream) {
  if (n <= 0) return 0;
  philox_normal_kernel<<<grid_for((n + 3) / 4 + 1, 256, 148 * 8), 256, 0, ST(stream)>>>(out, n, seed, stream_id, step,
                                                                                      offset, sigma, accumulate);
  OPK_LAUNCH_CHECK();
  return 0;
}

extern "C" int opk_clip_scale(double* sumsq, float clip, int mode_auto, float gamma, int n_leaves, int64_t widest_leaf,
                              float* scale_out, float* norm_out, int32_t* counters, int reset, void* stream) {
  clip_scale_kernel<<<1, 1, 0, ST(stream)>>>(sumsq, clip, mode_auto, gamma, n_leaves, widest_leaf, scale_out, norm_out,
                                            counters, reset);
  OPK_LAUNCH_CHECK();
  return 0;
}

extern "C" int opk_clip_accumulate(const void* g, const float* scale, float* acc, int64_t n, void* stream);
extern "C" int opk_clip_accumulate2(const void* g, const float* scale, float* acc, int64_t n, int overwrite,
                                    void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(g) & 15) || (reinterpret_cast<uintptr_t>(acc) & 15)) return -1;
  const long long nvec = n >> 3;
  static int cap_ctas = -1;
  if (cap_ctas < 0) {
    // Same shared-memory carve-out as the GEMM kernels, so that CTAs of this kernel can be co-resident with them
    // on an SM (an SM does not mix carve-out configurations).
    cudaFuncSetAttribute(clip_accumulate_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    cap_ctas = 148 * 16;
  }
  if (nvec > 0)
    clip_accumulate_kernel<<<grid_for(nvec, 256, cap_ctas), 256, 0, ST(stream)>>>(
        reinterpret_cast<const bf16x8*>(g), scale, reinterpret_cast<float4*>(acc), nvec, overwrite);
  const long long tail = n - (nvec << 3);
  if (tail > 0)
    clip_accumulate_tail_kernel<<<1, 32, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(g), scale, acc,
                                                         nvec << 3, n, overwrite);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_clip_accumulate_group(const void* const* g, const float* const* scale, int n_group, float* acc, int64_t n,
                                         int overwrite, void* stream) {
  if (n <= 0 || n_group <= 0) return 0;
  if (n_group > OPK_ACC_GROUP_MAX || (reinterpret_cast<uintptr_t>(acc) & 15)) return -1;
  AccGroup grp;
  for (int j = 0; j < OPK_ACC_GROUP_MAX; ++j) {
    grp.g[j] = j < n_group ? reinterpret_cast<const bf16x8*>(g[j]) : nullptr;
    grp.scale[j] = j < n_group ? scale[j] : nullptr;
    if (j < n_group && (reinterpret_cast<uintptr_t>(g[j]) & 15)) return -1;
  }
  const long long nvec = n >> 3;
  cudaStream_t st = ST(stream);
  if (nvec > 0) {
    switch (n_group) {
      case 1: launch_acc_group<1>(grp, acc, nvec, overwrite, st); break;
      case 2: launch_acc_group<2>(grp, acc, nvec, overwrite, st); break;
      case 3: launch_acc_group<3>(grp, acc, nvec, overwrite, st); break;
      case 4: launch_acc_group<4>(grp, acc, nvec, overwrite, st); break;
      case 5: launch_acc_group<5>(grp, acc, nvec, overwrite, st); break;
      case 6: launch_acc_group<6>(grp, acc, nvec, overwrite, st); break;
      case 7: launch_acc_group<7>(grp, acc, nvec, overwrite, st); break;
      default: launch_acc_group<8>(grp, acc, nvec, overwrite, st); break;
    }
  }
  const long long tail = n - (nvec << 3);
  if (tail > 0) clip_accumulate_group_tail_kernel<<<1, 32, 0, st>>>(grp, n_group, acc, nvec << 3, n, overwrite);
  OPK_LAUNCH_CHECK();
  return 0;
}
extern "C" int opk_clip_accumulate(const void* g, const float* scale, float* acc, int64_t n, void* stream) {
  return opk_clip_accumulate2(g, scale, acc, n, 0, stream);
}

// grad_src / param_dst are HOST arrays of device pointers here (copied into the kernel's parameter space).
extern "C" int opk_dp_step(const OpkDpStepArgs* args, void* stream) {
  if (!args || args->shard_len <= 0) return 0;
  if (args->n_src < 1 || args->n_src > MAX_PEERS || args->n_dst < 0 || args->n_dst > MAX_PEERS) return -1;
  if (args->shard_begin & 3) return -2;
  PeerTable pt;
  for (int r = 0; r < MAX_PEERS; ++r) {
    pt.grad[r] = r < args->n_src ? args->grad_src[r] : nullptr;
    pt.param[r] = r < args->n_dst ? reinterpret_cast<__nv_bfloat16*>(args->param_dst[r]) : nullptr;
  }
  if (args->blt_nbuf > 0 && args->toep_nlag > 0) return -3;       // one correlation transform per step
  // rows of the [buffers][shard_len] state are read as 16-byte vectors: every row must start on a 16-byte boundary
  if ((args->blt_nbuf > 1 || args->toep_nlag > 1) && (args->shard_len & 3)) return -2;
  if ((args->blt_nbuf > 0 && (reinterpret_cast<uintptr_t>(args->blt_state) & 15)) ||
      (args->toep_nlag > 0 && (reinterpret_cast<uintptr_t>(args->toep_state) & 15)) ||
      (reinterpret_cast<uintptr_t>(args->m) & 15) || (reinterpret_cast<uintptr_t>(args->v) & 15) ||
      (reinterpret_cast<uintptr_t>(args->master) & 15))
    return -2;
  if (args->toep_nlag > 0 && (!args->toep_state || !args->toep_coef || args->toep_pos < 0 || args->toep_pos >= args->toep_nlag)) return -3;
  const long long nq = (args->shard_len + 3) >> 2;
  const int grid = grid_for((nq + 1) / 2, 256, 148 * 8);
  cudaStream_t st = ST(stream);
  const int corr = args->blt_nbuf > 0 ? CORR_BLT : (args->toep_coef ? CORR_TOEPLITZ : CORR_NONE);
  const bool adam = !args->sgd_mode, master = args->master != nullptr;
#define OPK_DP_STEP_LAUNCH(A, M, C) dp_step_kernel<A, M, C><<<grid, 256, 0, st>>>(*args, pt)
#define OPK_DP_STEP_CORR(A, M)                                      \
  do {                                                              \
    if (corr == CORR_BLT) OPK_DP_STEP_LAUNCH(A, M, CORR_BLT);       \
    else if (corr == CORR_TOEPLITZ) OPK_DP_STEP_LAUNCH(A, M, CORR_TOEPLITZ); \
    else OPK_DP_STEP_LAUNCH(A, M, CORR_NONE);                       \
  } while (0)
  if (adam && master) OPK_DP_STEP_CORR(true, true);
  else if (adam) OPK_DP_STEP_CORR(true, false);
  else if (master) OPK_DP_STEP_CORR(false, true);
  else OPK_DP_STEP_CORR(false, false);
#undef OPK_DP_STEP_CORR
#undef OPK_DP_STEP_LAUNCH
  OPK_LAUNCH_CHECK();
  return 0;
}

// Sharded fp32 sums: acc_shards[o] is the base of owner o's shard (a peer-mapped address for o != this rank), which
// holds the elements [bounds[o], bounds[o+1]) of the flat vector; bounds are multiples of 8. rank selects where this
// rank starts walking (its own shard first).
extern "C" int opk_clip_accumulate_group_push(const void* const* g, const float* const* scale, int n_group,
                                              float* const* acc_shards, const int64_t* bounds, int n_shards, int rank,
                                              int64_t n, void* stream) {
  if (n <= 0 || n_group <= 0) return 0;
  if (n_group > OPK_ACC_GROUP_MAX || n_shards < 1 || n_shards > MAX_PEERS || rank < 0 || rank >= n_shards || (n & 7)) return -1;
  AccGroup grp;
  for (int j = 0; j < OPK_ACC_GROUP_MAX; ++j) {
    grp.g[j] = j < n_group ? reinterpret_cast<const bf16x8*>(g[j]) : nullptr;
    grp.scale[j] = j < n_group ? scale[j] : nullptr;
    if (j < n_group && (reinterpret_cast<uintptr_t>(g[j]) & 15)) return -1;
  }
  ShardTable sh;
  sh.n = n_shards;
  for (int o = 0; o < MAX_PEERS; ++o) sh.acc[o] = o < n_shards ? acc_shards[o] : nullptr;
  for (int o = 0; o <= MAX_PEERS; ++o) sh.begin[o] = o <= n_shards ? bounds[o] : bounds[n_shards];
  for (int o = 0; o < n_shards; ++o) {
    if ((bounds[o] & 7) || bounds[o + 1] < bounds[o] || (reinterpret_cast<uintptr_t>(acc_shards[o]) & 15)) return -1;
  }
  if (bounds[0] != 0 || bounds[n_shards] < n) return -1;
  const long long nvec = n >> 3;
  long long rot = bounds[rank] >> 3;
  if (rot >= nvec) rot = 0;
  cudaStream_t st = ST(stream);
  switch (n_group) {
    case 1: launch_acc_group_push<1>(grp, sh, nvec, rot, st); break;
    case 2: launch_acc_group_push<2>(grp, sh, nvec, rot, st); break;
    case 3: launch_acc_group_push<3>(grp, sh, nvec, rot, st); break;
    case 4: launch_acc_group_push<4>(grp, sh, nvec, rot, st); break;
    case 5: launch_acc_group_push<5>(grp, sh, nvec, rot, st); break;
    case 6: launch_acc_group_push<6>(grp, sh, nvec, rot, st); break;
    case 7: launch_acc_group_push<7>(grp, sh, nvec, rot, st); break;
    default: launch_acc_group_push<8>(grp, sh, nvec, rot, st); break;
  }
  OPK_LAUNCH_CHECK();
  return 0;
}

extern "C" int opk_copy_bytes(void* dst, const void* src, int64_t nbytes, void* stream) {
  if (nbytes <= 0) return 0;
  if ((nbytes & 15) || (reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return -1;
  const long long nvec = nbytes >> 4;
  copy_vec_kernel<<<grid_for((nvec + 7) / 8, 256, 148 * 8), 256, 0, ST(stream)>>>(reinterpret_cast<uint4*>(dst),
                                                                                  reinterpret_cast<const uint4*>(src), nvec);
  OPK_LAUNCH_CHECK();
  return 0;
}
