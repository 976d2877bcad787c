// Causal grouped-query flash attention for sm_100a on tcgen05 / TMEM, operating in place on the fused projection
// buffer qkv[T][(H + 2*KV) * hd] (bf16, row pitch ld): Q head h at column h*hd, K head g at (H+g)*hd, V head g at
// (H+KV+g)*hd. head_dim is 64 or 128. One example (sequence) per launch; heads are the parallel dimension.
//
// Shared design of the three kernels (forward, dK/dV, dQ):
//   * 192 threads: warp 0 = TMA producer, warp 1 = TMEM owner + UMMA issuer, warps 2..5 = softmax / epilogue with
//     thread <-> TMEM lane (= row of the 128-row tile),
//   * operand tiles are TMA boxes of 64 columns x R rows with 128-byte swizzle; a tile of hd columns is hd/64 such
//     boxes. The same bytes serve as a K-major operand (rows = M/N index) or as an MN-major operand (rows = reduction
//     index), which is what lets P^T / dS^T / K / Q / dO be reused across the five products without transposes,
//   * probabilities and score gradients are written by the softmax threads into shared memory in the same swizzled
//     layout and consumed as the A operand of the following UMMA,
//   * all mbarrier waits are bounded (ptx_sm100.cuh): on expiry the CTA unwinds, frees TMEM and sets *err.
#pragma once
#include "ptx_sm100.cuh"

namespace opk {

struct AttnParams {
  int T, H, KV, hd;
  long long ld;            // row pitch of qkv / dqkv (elements)
  long long ldo;           // row pitch of out / dout (elements)
  void* out;               // fwd: bf16 [T][H*hd]
  float* lse;              // [H][T] natural-log-sum-exp of scaled scores
  const void* dout;        // bwd: bf16 [T][H*hd]
  const float* dsum;       // bwd: [H][T64] rowsum(dO * O), T64 = T rounded up to a multiple of 64
  const float* nlse2;      // bwd: [H][T64] -lse * log2(e), -inf in the padding
  int T64;
  float* part;             // bwd, optional: fp32 [2][H/KV][T][KV*hd] partial dK / dV (one CTA per query head)
  void* dqkv;              // bwd: bf16, same layout as qkv
  float scale;             // 1/sqrt(hd)
  int* err;
};

// Byte offset of element (row r, column c) inside a [rows][64]-column, 128-byte-swizzled tile chunk.
__device__ __forceinline__ uint32_t swz_off(int r, int c) {
  return (uint32_t)(r * 128 + ((((c >> 3) ^ (r & 7)) << 4) | ((c & 7) << 1)));
}

// 2-D TMA load of a {64 cols, rows} box (the tensor map fixes the box shape).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// Issue the UMMAs of one product D[128 x N] (+)= A[128 x Kred] * B[N x Kred]^T.
//   A_MN / B_MN select the operand interpretation; a_rows / b_rows = rows of one 64-column chunk of that operand
//   (chunk stride in bytes = rows * 128).
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void issue_product(uint32_t d_tmem, uint32_t a_base, int a_rows, uint32_t b_base, int b_rows,
                                              int n, int kred, bool accumulate) {
  const uint32_t idesc = make_idesc_bf16(128, n, A_MN, B_MN);
  for (int k = 0; k < kred; k += 16) {
    uint64_t ad, bd;
    if (A_MN) ad = make_smem_desc(a_base + (uint32_t)k * 128, (uint32_t)a_rows * 128, 1024);
    else ad = make_smem_desc(a_base + (uint32_t)(k >> 6) * (uint32_t)a_rows * 128 + (uint32_t)(k & 63) * 2, 16, 1024);
    if (B_MN) bd = make_smem_desc(b_base + (uint32_t)k * 128, (uint32_t)b_rows * 128, 1024);
    else bd = make_smem_desc(b_base + (uint32_t)(k >> 6) * (uint32_t)b_rows * 128 + (uint32_t)(k & 63) * 2, 16, 1024);
    umma_bf16(d_tmem, ad, bd, idesc, (accumulate || k > 0) ? 1u : 0u);
  }
}

// One warp-collective bounded wait: lane 0 polls (acquire), __syncwarp orders the other lanes' later memory reads
// after it (a shuffle alone is no memory barrier: without the __syncwarp the compiler may hoist a shared-memory
// load of lanes 1..31 above the wait), then the result is broadcast.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane) {
  int w = 1;
  if (lane == 0) w = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
  __syncwarp();
  return __shfl_sync(0xffffffffu, w, 0) != 0;
}

// ------------------------------------------------------------------------------------------------ forward
// CTA = (query tile of 128 rows, head). KV tiles of 128 keys, double-buffered K and V stages, S double-buffered in
// TMEM. O accumulates in TMEM across KV tiles; the running maximum is updated lazily: rows are rescaled (TMEM
// load-multiply-store by the softmax warps) only when their maximum grew by more than 2^8, otherwise the stale
// maximum stays in use (probabilities may then exceed 1 by at most 2^8, harmless in bf16 / fp32). The softmax of a
// tile is a single pass over registers: 128 fmax, 128 ffma + ex2.approx, 64 packs, 16 shared stores per thread.
#ifdef OPK_ATTN_TRACE
// Debug-only timeline of CTA 0 (clock64 stamps per role / tile / event); never compiled into the library.
__device__ long long g_attn_trace[3 * 1024];
#define OPK_TRACE(role, j, e) do { if (blockIdx.x == 0) g_attn_trace[(role) * 1024 + (j) * 8 + (e)] = clock64(); } while (0)
#else
#define OPK_TRACE(role, j, e) do { } while (0)
#endif

constexpr int kSoftmaxWarps = 8;                       // warps 2..9; warps 0 / 1 drive TMA / MMA
constexpr int kAttnThreads = (2 + kSoftmaxWarps) * 32;

template <int HD>
struct FwdSmem {
  static constexpr int TILE = 128 * HD * 2;           // bytes of one [128][HD] tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE;                  // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * TILE;      // 2 stages
  static constexpr int P_OFF = V_OFF + 2 * TILE;      // 2 x [128][128] bf16 = 64 KB
  static constexpr int P_BYTES = 128 * 128 * 2;
  static constexpr int BAR_OFF = P_OFF + 2 * P_BYTES;      // 256 B of barriers, then 2 KB of row exchange space
  static constexpr int USED = BAR_OFF + 256 + 2048;
  // The tiles need a 1024-byte-aligned base. The launch asks for the per-CTA maximum, which leaves less than 1 KB
  // of slack; the kernel checks that the alignment padding fits and reports an error otherwise.
  static constexpr int BYTES = (USED + 1024 <= 232448) ? USED + 1024 : 232448;
};

// Maximum of 64 scores (columns col0 .. col0+63 of the tile) with four independent chains; MASKED drops columns > r.
template <bool MASKED>
__device__ __forceinline__ float row_max64(const uint32_t (&a)[32], const uint32_t (&b)[32], int col0, int r) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    if (!MASKED || col0 + i <= r) m0 = fmaxf(m0, __uint_as_float(a[i]));
    if (!MASKED || col0 + i + 1 <= r) m1 = fmaxf(m1, __uint_as_float(a[i + 1]));
    if (!MASKED || col0 + 32 + i <= r) m2 = fmaxf(m2, __uint_as_float(b[i]));
    if (!MASKED || col0 + 33 + i <= r) m3 = fmaxf(m3, __uint_as_float(b[i + 1]));
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// Rendezvous of the two warps that share a TMEM lane quarter, on an mbarrier of count 2 (bounded like every wait
// here; a named bar.sync would hang the partner if one side had given up). Shared-memory writes made before the
// call are visible to the partner after it.
__device__ __forceinline__ bool pair_sync(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
  return warp_wait(bar, parity, abort_flag, lane);
}

// exp2(x * c2 - mc) for 32 columns starting at col0, packed to bf16 and stored swizzled; returns the partial row sum.
template <bool MASKED>
__device__ __forceinline__ float softmax_chunk(const uint32_t (&x)[32], int col0, int r, float c2, float mc,
                                               uint8_t* p_smem) {
  float sum0 = 0.f, sum1 = 0.f;
  uint32_t packed[16];
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float e0 = ex2_approx(fmaf(__uint_as_float(x[i]), c2, -mc));
    float e1 = ex2_approx(fmaf(__uint_as_float(x[i + 1]), c2, -mc));
    if (MASKED) {
      if (col0 + i > r) e0 = 0.f;
      if (col0 + i + 1 > r) e1 = 0.f;
    }
    sum0 += e0;
    sum1 += e1;
    packed[i >> 1] = pack_bf16x2(e0, e1);
  }
  const float sum = sum0 + sum1;
  uint8_t* chunk = p_smem + (col0 >> 6) * 16384;
#pragma unroll
  for (int q = 0; q < 4; ++q)
    *reinterpret_cast<uint4*>(chunk + swz_off(r, (col0 & 63) + q * 8)) =
        make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
  return sum;
}

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm, const AttnParams p) {
  using SM = FwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if ((int)(smem - smem_raw) + SM::USED > SM::BYTES) {   // uniform over the CTA; nothing has been set up yet
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 2);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_free = bars + 11;   // [2]
  uint64_t* p_full = bars + 13;   // [2]
  uint64_t* o_done = bars + 15;   // [2] P*V of a tile has completed (its P buffer is reusable, O is consistent)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* x_bar = bars + 20;    // [2 tiles][4 quads] pair rendezvous for the row maxima; [8..11]: final row sums
  float* xchg = reinterpret_cast<float*>(bars + 32);   // [2 tiles][2 halves][128 rows] partial maxima (row sums at the end)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.T + 127) / 128;
  const int h = blockIdx.x % p.H;
  const int qt = n_qt - 1 - (int)(blockIdx.x / p.H);   // heavy (late) query tiles first
  const int g = h / (p.H / p.KV);
  const int n_kv = qt + 1;
  const int q_col = h * HD, k_col = (p.H + g) * HD, v_col = (p.H + p.KV + g) * HD;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_free[i], kSoftmaxWarps);
      mbar_init(&p_full[i], kSoftmaxWarps); mbar_init(&o_done[i], 1);
    }
    for (int i = 0; i < 12; ++i) mbar_init(&x_bar[i], 2);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t S_COL = 0, O_COL = 256;   // S buffers at 0 / 128, O accumulator at 256

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm);
      mbar_expect_tx(q_full, SM::TILE);
      for (int c = 0; c < HD / 64; ++c) tma_load_2d(smem + SM::Q_OFF + c * 16384, &tm, q_full, q_col + c * 64, qt * 128);
      // K(j) is issued one tile ahead of V(j-1): the K stage frees when S(j-2) has completed, well before the V
      // stage (which waits for P*V of tile j-3), so neither wait holds the other load back.
      for (int j = 0; j <= n_kv; ++j) {
        if (j < n_kv) {
          const int s = j & 1;
          const uint32_t ph = (j >> 1) & 1;
          if (!mbar_wait(&k_empty[s], ph ^ 1u, abort_flag)) break;
          OPK_TRACE(0, j, 0);
          mbar_expect_tx(&k_full[s], SM::TILE);
          for (int c = 0; c < HD / 64; ++c)
            tma_load_2d(smem + SM::K_OFF + s * SM::TILE + c * 16384, &tm, &k_full[s], k_col + c * 64, j * 128);
        }
        if (j >= 1) {
          const int jv = j - 1, s = jv & 1;
          const uint32_t ph = (jv >> 1) & 1;
          if (!mbar_wait(&v_empty[s], ph ^ 1u, abort_flag)) break;
          OPK_TRACE(0, jv, 1);
          mbar_expect_tx(&v_full[s], SM::TILE);
          for (int c = 0; c < HD / 64; ++c)
            tma_load_2d(smem + SM::V_OFF + s * SM::TILE + c * 16384, &tm, &v_full[s], v_col + c * 64, jv * 128);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t q_s = smem_u32(smem + SM::Q_OFF), p_s = smem_u32(smem + SM::P_OFF);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[s], ph, abort_flag)) return false;
        OPK_TRACE(1, j, 0);
        if (!mbar_wait(&s_free[s], ph ^ 1u, abort_flag)) return false;
        OPK_TRACE(1, j, 1);
        tc_fence_after();
        issue_product<false, false>(tmem + S_COL + s * 128, q_s, 128, smem_u32(smem + SM::K_OFF + s * SM::TILE), 128, 128,
                                    HD, false);
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        OPK_TRACE(1, j, 2);
        if (!mbar_wait(&v_full[s], ph, abort_flag)) break;
        OPK_TRACE(1, j, 3);
        if (!mbar_wait(&p_full[s], ph, abort_flag)) break;
        OPK_TRACE(1, j, 4);
        tc_fence_after();
        // O[128 x HD] += P[128 x 128 keys] * V[keys x HD]: B is MN-major (rows = keys)
        issue_product<false, true>(tmem + O_COL, p_s + s * SM::P_BYTES, 128, smem_u32(smem + SM::V_OFF + s * SM::TILE), 128, HD, 128, j > 0);
        umma_commit(&v_empty[s]);
        umma_commit(&o_done[s]);
        OPK_TRACE(1, j, 5);
      }
    }
    __syncwarp();
  } else {
    // 8 softmax warps: warps with the same (warp & 3) share 32 TMEM lanes (rows); `half` selects 64 of the 128 keys.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;            // row inside the query tile
    const int row = qt * 128 + r;
    const int col0 = half * 64;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;      // m_run: maximum in use (possibly stale); l_run: this half's row sum
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      uint8_t* p_smem = smem + SM::P_OFF + s * SM::P_BYTES;
      if (warp == 2 && lane == 0) OPK_TRACE(2, j, 0);
      if (!warp_wait(&s_full[s], ph, abort_flag, lane)) { ok = false; break; }
      if (warp == 2 && lane == 0) OPK_TRACE(2, j, 1);
      tc_fence_after();
      uint32_t x0[32], x1[32];
      __syncwarp();
      const uint32_t sa = tmem + lane_base + S_COL + s * 128 + col0;
      tmem_ld32(sa, x0); tmem_ld32(sa + 32, x1);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[s]);   // S lives in registers now
      if (warp == 2 && lane == 0) OPK_TRACE(2, j, 2);
      const bool diag = (j == qt);
      float mx = diag ? row_max64<true>(x0, x1, col0, r) : row_max64<false>(x0, x1, col0, r);
      // combine with the other half of the row (through shared memory, 64-thread named barrier)
      float* xm = xchg + s * 256;
      xm[half * 128 + r] = mx;
      if (!pair_sync(&x_bar[s * 4 + quad], ph, abort_flag, lane)) { ok = false; break; }
      mx = fmaxf(fmaxf(mx, xm[(half ^ 1) * 128 + r]), m_run);
      if (warp == 2 && lane == 0) OPK_TRACE(2, j, 3);
      // lazy rescale: adopt the new maximum only if it grew by more than 8 in the exponent domain
      const bool grow = (mx - m_run) * c2 > 8.f;   // true on the first tile (m_run = -inf)
      const unsigned any_grow = __ballot_sync(0xffffffffu, grow);
      // P buffer s was last read by the P*V of tile j-2
      if (j > 1 && !warp_wait(&o_done[s], ph ^ 1u, abort_flag, lane)) { ok = false; break; }
      float alpha = 1.f;
      if (grow) {
        alpha = ex2_approx((m_run - mx) * c2);     // 0 when m_run = -inf
        l_run *= alpha;
        m_run = mx;
      }
      if (any_grow && j > 0) {
        // O may only be touched once the P*V of tile j-1 has completed; the next one waits for this warp's P
        if (!warp_wait(&o_done[s ^ 1], ((j - 1) >> 1) & 1, abort_flag, lane)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < HD / 2; c0 += 32) {
          uint32_t o[32];
          __syncwarp();
          tmem_ld32(tmem + lane_base + O_COL + half * (HD / 2) + c0, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tmem + lane_base + O_COL + half * (HD / 2) + c0, o);
        }
        tc_wait_st();
      }
      if (warp == 2 && lane == 0) OPK_TRACE(2, j, 4);
      const float mc = m_run * c2;
      if (diag) l_run += softmax_chunk<true>(x0, col0, r, c2, mc, p_smem) + softmax_chunk<true>(x1, col0 + 32, r, c2, mc, p_smem);
      else l_run += softmax_chunk<false>(x0, col0, r, c2, mc, p_smem) + softmax_chunk<false>(x1, col0 + 32, r, c2, mc, p_smem);
      if (warp == 2 && lane == 0) OPK_TRACE(2, j, 5);
      tc_fence_before();
      fence_proxy_async();           // make the generic-proxy writes of P visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[s]);
      if (warp == 2 && lane == 0) OPK_TRACE(2, j, 6);
    }
    if (ok && warp_wait(&o_done[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort_flag, lane)) {
      tc_fence_after();
      // total row sum = both halves (same running maximum on both sides)
      float* xl = xchg + (n_kv & 1) * 256;      // the buffer the last tile did not use
      xl[half * 128 + r] = l_run;
      const bool both = pair_sync(&x_bar[8 + quad], 0, abort_flag, lane);
      const float l_tot = l_run + xl[(half ^ 1) * 128 + r];
      const float inv = both ? 1.f / l_tot : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)row * p.ldo + h * HD + half * (HD / 2);
#pragma unroll
      for (int c0 = 0; c0 < HD / 2; c0 += 32) {
        uint32_t raw[32];
        __syncwarp();
        tmem_ld32(tmem + lane_base + O_COL + half * (HD / 2) + c0, raw);
        tc_wait_ld();
        if (row < p.T) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(raw[8 * q + 0]) * inv, __uint_as_float(raw[8 * q + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(raw[8 * q + 2]) * inv, __uint_as_float(raw[8 * q + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(raw[8 * q + 4]) * inv, __uint_as_float(raw[8 * q + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(raw[8 * q + 6]) * inv, __uint_as_float(raw[8 * q + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c0 + q * 8) = o;
          }
        }
      }
      if (half == 0 && row < p.T) p.lse[(long long)h * p.T + row] = m_run * p.scale + logf(l_tot);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

// ------------------------------------------------------------------------------------------------ backward helpers
// Backward preprocessing, one warp per (t, h) with t < T64 (T rounded up to a multiple of 64):
//   dsum[h][t] = sum_d dO[t][h*hd + d] * O[t][h*hd + d]        nlse2[h][t] = -lse[h][t] * log2(e)
// Rows t >= T get dsum = 0 and nlse2 = -inf, so that exp2(s * c + nlse2) is exactly 0 for padded queries.
__global__ void attn_dsum_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                 const float* __restrict__ lse, float* __restrict__ dsum, float* __restrict__ nlse2,
                                 int T, int T64, int H, int hd, long long ldo) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T64 * H) return;
  const int t = w / H, h = w % H;
  if (t >= T) {
    if (lane == 0) { dsum[(long long)h * T64 + t] = 0.f; nlse2[(long long)h * T64 + t] = -INFINITY; }
    return;
  }
  const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(o + (long long)t * ldo + h * hd);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(dout + (long long)t * ldo + h * hd);
  float s = 0.f;
  for (int i = lane; i < hd / 2; i += 32) {
    const float2 x = __bfloat1622float2(a[i]), y = __bfloat1622float2(b[i]);
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    dsum[(long long)h * T64 + t] = s;
    nlse2[(long long)h * T64 + t] = -lse[(long long)h * T + t] * 1.4426950408889634f;
  }
}

// Write 32 packed bf16 values (16 words) of row r, columns col0 .. col0+31, into a [128 rows][64 cols] swizzled chunk.
__device__ __forceinline__ void store_row32(uint8_t* chunk, int r, int col0, const uint32_t (&w)[16]) {
#pragma unroll
  for (int q = 0; q < 4; ++q)
    *reinterpret_cast<uint4*>(chunk + swz_off(r, col0 + q * 8)) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
}

// Store NCOLS fp32 accumulator columns of this thread's TMEM lane (starting at tmem_addr) as bf16 to dst.
template <int NCOLS>
__device__ __forceinline__ void store_acc_rows(uint32_t tmem_addr, __nv_bfloat16* dst, bool valid, float mul) {
#pragma unroll
  for (int c0 = 0; c0 < NCOLS; c0 += 32) {
    uint32_t raw[32];
    __syncwarp();
    tmem_ld32(tmem_addr + c0, raw);
    tc_wait_ld();
    if (valid) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack_bf16x2(__uint_as_float(raw[8 * q + 0]) * mul, __uint_as_float(raw[8 * q + 1]) * mul);
        o.y = pack_bf16x2(__uint_as_float(raw[8 * q + 2]) * mul, __uint_as_float(raw[8 * q + 3]) * mul);
        o.z = pack_bf16x2(__uint_as_float(raw[8 * q + 4]) * mul, __uint_as_float(raw[8 * q + 5]) * mul);
        o.w = pack_bf16x2(__uint_as_float(raw[8 * q + 6]) * mul, __uint_as_float(raw[8 * q + 7]) * mul);
        *reinterpret_cast<uint4*>(dst + c0 + q * 8) = o;
      }
    }
  }
}

// Same, keeping fp32 (partial results that a later kernel sums).
template <int NCOLS>
__device__ __forceinline__ void store_acc_rows_f32(uint32_t tmem_addr, float* dst, bool valid, float mul) {
#pragma unroll
  for (int c0 = 0; c0 < NCOLS; c0 += 32) {
    uint32_t raw[32];
    __syncwarp();
    tmem_ld32(tmem_addr + c0, raw);
    tc_wait_ld();
    if (valid) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<float4*>(dst + c0 + q * 4) =
            make_float4(__uint_as_float(raw[4 * q]) * mul, __uint_as_float(raw[4 * q + 1]) * mul,
                        __uint_as_float(raw[4 * q + 2]) * mul, __uint_as_float(raw[4 * q + 3]) * mul);
    }
  }
}

// dqkv[t][K | V columns] = bf16(sum over the G partials), summed in index order (deterministic).
__global__ void attn_dkv_reduce_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ dqkv, int T, int G,
                                       int kvw, long long ld, int k_col0) {
  const long long n4 = (long long)T * (kvw / 4) * 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const int which = (int)(i / ((long long)T * (kvw / 4)));          // 0 = dK, 1 = dV
    const long long rem = i - (long long)which * T * (kvw / 4);
    const int t = (int)(rem / (kvw / 4)), c = (int)(rem % (kvw / 4)) * 4;
    const float* src = part + ((long long)which * G * T + t) * kvw + c;
    float4 a = *reinterpret_cast<const float4*>(src);
    for (int gq = 1; gq < G; ++gq) {
      const float4 b = *reinterpret_cast<const float4*>(src + (long long)gq * T * kvw);
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    uint2 o;
    o.x = pack_bf16x2(a.x, a.y);
    o.y = pack_bf16x2(a.z, a.w);
    *reinterpret_cast<uint2*>(dqkv + (long long)t * ld + k_col0 + (long long)which * kvw + c) = o;
  }
}

// ------------------------------------------------------------------------------------------------ dK / dV
// CTA = (key tile of 128 keys, KV head). Iterates over the query heads of the group and over 64-row query sub-tiles
// at or after the key tile; dK and dV accumulate in TMEM over all iterations (no atomics, no partial buffers).
//   St  = K Q^T        [keys x 64 q]      dPt = V dO^T     [keys x 64 q]
//   Pt  = exp(St*scale - lse[q]),  dSt = Pt * (dPt - D[q]) * scale       (thread = key row)
//   dV += Pt dO        dK += dSt Q
template <int HD>
struct DkvSmem {
  // The Q / dO ring is deeper than the two score buffers in TMEM: a stage stays occupied from the score products of
  // its sub-tile until the dK product of the same sub-tile has completed (about two iterations), and the refill needs
  // a full TMA round trip on top, so two stages leave that round trip exposed in every iteration.
  static constexpr int NS = 4;
  static constexpr int KV_TILE = 128 * HD * 2;
  static constexpr int Q_TILE = 64 * HD * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = KV_TILE;
  static constexpr int Q_OFF = 2 * KV_TILE;               // NS stages
  static constexpr int DO_OFF = Q_OFF + NS * Q_TILE;      // NS stages
  static constexpr int PT_OFF = DO_OFF + NS * Q_TILE;     // [128][64] bf16
  static constexpr int DST_OFF = PT_OFF + 16384;
  static constexpr int ROW_OFF = DST_OFF + 16384;         // NS stages x (64 nlse2 + 64 dsum) floats
  static constexpr int BAR_OFF = ROW_OFF + NS * 512;
  static constexpr int USED = BAR_OFF + 256;
  // up to 1 KB of alignment padding in front; at HD = 128 the layout only fits when the padding is below 768 bytes,
  // which the kernel checks before it touches anything
  static constexpr int BYTES = (USED + 1024 <= 232448) ? USED + 1024 : 232448;
  static_assert(USED <= 232448, "dK/dV shared-memory layout does not fit");
};

// One 32-query chunk of the transposed backward softmax for a key row: Pt = exp2(St*c2 + nlse2[q]) and
// dSt = Pt * (dPt - D[q]) (the softmax scale is applied when dK is stored). `kd` = key - first query of the chunk.
template <bool MASKED>
__device__ __forceinline__ void dkv_chunk(const uint32_t (&sraw)[32], const uint32_t (&draw)[32], const float4* nl4,
                                          const float4* d4, float c2, int kd, uint32_t* pw, uint32_t* dw) {
#pragma unroll
  for (int e = 0; e < 32; e += 4) {
    const float4 L = nl4[e >> 2], D = d4[e >> 2];
    float p0 = ex2_approx(fmaf(__uint_as_float(sraw[e + 0]), c2, L.x));
    float p1 = ex2_approx(fmaf(__uint_as_float(sraw[e + 1]), c2, L.y));
    float p2 = ex2_approx(fmaf(__uint_as_float(sraw[e + 2]), c2, L.z));
    float p3 = ex2_approx(fmaf(__uint_as_float(sraw[e + 3]), c2, L.w));
    if (MASKED) {
      if (e + 0 < kd) p0 = 0.f;
      if (e + 1 < kd) p1 = 0.f;
      if (e + 2 < kd) p2 = 0.f;
      if (e + 3 < kd) p3 = 0.f;
    }
    pw[(e >> 1) + 0] = pack_bf16x2(p0, p1);
    pw[(e >> 1) + 1] = pack_bf16x2(p2, p3);
    dw[(e >> 1) + 0] = pack_bf16x2(p0 * (__uint_as_float(draw[e + 0]) - D.x), p1 * (__uint_as_float(draw[e + 1]) - D.y));
    dw[(e >> 1) + 1] = pack_bf16x2(p2 * (__uint_as_float(draw[e + 2]) - D.z), p3 * (__uint_as_float(draw[e + 3]) - D.w));
  }
}

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_dkv_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
                const __grid_constant__ CUtensorMap tm_do, const AttnParams p) {
  using SM = DkvSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if ((int)(smem - smem_raw) + SM::USED > SM::BYTES) {   // uniform over the CTA; nothing has been set up yet
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 2);
    return;
  }
  constexpr int NS = SM::NS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;             // [NS]
  uint64_t* q_empty = q_full + NS;         // [NS]
  uint64_t* st_full = q_empty + NS;        // [2]
  uint64_t* st_free = st_full + 2;         // [2]
  uint64_t* pd_full = st_free + 2;
  uint64_t* pd_free = pd_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pd_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.H / p.KV;
  // Two work splits: one CTA per (key tile, KV head) that loops over the G query heads of the group and stores
  // bf16 results directly; or, with a partial buffer, one CTA per (key tile, query head) that stores fp32 partials
  // which a second kernel sums in a fixed order (4x more CTAs: the causal triangle balances far better).
  const bool split = p.part != nullptr;
  const int per_kt = split ? p.H : p.KV;
  const int kt = blockIdx.x / per_kt;                    // low key tiles (most work) first
  const int g = split ? (int)(blockIdx.x % per_kt) / G : (int)(blockIdx.x % per_kt);
  const int h_first = split ? (int)(blockIdx.x % per_kt) : g * G;
  const int n_q64 = (p.T + 63) / 64;
  const int q_first = 2 * kt;
  const int per_head = n_q64 - q_first;
  const int n_it = per_head * (split ? 1 : G);
  const int k_col = (p.H + g) * HD, v_col = (p.H + p.KV + g) * HD;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < NS; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&st_full[i], 1); mbar_init(&st_free[i], kSoftmaxWarps); }
    mbar_init(pd_full, kSoftmaxWarps);
    mbar_init(pd_free, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // columns: St buffers 0 / 64, dPt buffers 128 / 192, dV at 256, dK at 256 + HD
  const uint32_t ST_COL = 0, DPT_COL = 128, DV_COL = 256, DK_COL = 256 + HD;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_kv); tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_do);
      mbar_expect_tx(kv_full, 2 * SM::KV_TILE);
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_2d(smem + SM::K_OFF + c * 16384, &tm_kv, kv_full, k_col + c * 64, kt * 128);
        tma_load_2d(smem + SM::V_OFF + c * 16384, &tm_kv, kv_full, v_col + c * 64, kt * 128);
      }
      for (int i = 0; i < n_it; ++i) {
        const int s = i % NS;
        const uint32_t ph = (i / NS) & 1;
        const int h = h_first + i / per_head, q64 = q_first + i % per_head;
        if (!mbar_wait(&q_empty[s], ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(&q_full[s], 2 * SM::Q_TILE + 512);
        bulk_load_1d(smem + SM::ROW_OFF + s * 512, p.nlse2 + (long long)h * p.T64 + q64 * 64, 256, &q_full[s]);
        bulk_load_1d(smem + SM::ROW_OFF + s * 512 + 256, p.dsum + (long long)h * p.T64 + q64 * 64, 256, &q_full[s]);
        for (int c = 0; c < HD / 64; ++c) {
          tma_load_2d(smem + SM::Q_OFF + s * SM::Q_TILE + c * 8192, &tm_q, &q_full[s], h * HD + c * 64, q64 * 64);
          tma_load_2d(smem + SM::DO_OFF + s * SM::Q_TILE + c * 8192, &tm_do, &q_full[s], h * HD + c * 64, q64 * 64);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t k_s = smem_u32(smem + SM::K_OFF), v_s = smem_u32(smem + SM::V_OFF);
      const uint32_t pt_s = smem_u32(smem + SM::PT_OFF), dst_s = smem_u32(smem + SM::DST_OFF);
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      auto scores = [&](int i) -> bool {
        const int s = i & 1, sq = i % NS;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&q_full[sq], (i / NS) & 1, abort_flag)) return false;
        if (!mbar_wait(&st_free[s], ph ^ 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t q_s = smem_u32(smem + SM::Q_OFF + sq * SM::Q_TILE), do_s = smem_u32(smem + SM::DO_OFF + sq * SM::Q_TILE);
        issue_product<false, false>(tmem + ST_COL + s * 64, k_s, 128, q_s, 64, 64, HD, false);
        issue_product<false, false>(tmem + DPT_COL + s * 64, v_s, 128, do_s, 64, 64, HD, false);
        umma_commit(&st_full[s]);
        return true;
      };
      if (ok) ok = scores(0);
      for (int i = 0; i < n_it && ok; ++i) {
        if (i + 1 < n_it) ok = scores(i + 1);
        if (!ok) break;
        const int sq = i % NS;
        if (!mbar_wait(pd_full, i & 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t q_s = smem_u32(smem + SM::Q_OFF + sq * SM::Q_TILE), do_s = smem_u32(smem + SM::DO_OFF + sq * SM::Q_TILE);
        // dV[keys x HD] += Pt[keys x 64 q] * dO[64 q x HD]   (B rows = queries: MN-major)
        issue_product<false, true>(tmem + DV_COL, pt_s, 128, do_s, 64, HD, 64, i > 0);
        issue_product<false, true>(tmem + DK_COL, dst_s, 128, q_s, 64, HD, 64, i > 0);
        umma_commit(&q_empty[sq]);
        umma_commit(pd_free);
      }
    }
    __syncwarp();
  } else {
    // 8 softmax warps: (warp & 3) picks the 32 key rows (TMEM lanes), `half` 32 of the 64 queries of the sub-tile
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int key = kt * 128 + r;
    const int c0 = half * 32;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;
    bool ok = true;
    for (int i = 0; i < n_it && ok; ++i) {
      const int s = i & 1, sq = i % NS;
      const uint32_t ph = (i >> 1) & 1;
      const int q64 = q_first + i % per_head;
      if (!warp_wait(&st_full[s], ph, abort_flag, lane)) { ok = false; break; }
      tc_fence_after();
      // the row vectors of this stage arrived with Q / dO; the phase has completed already (the scores needed it),
      // the wait only orders this warp's shared-memory reads after the bulk copy
      if (!warp_wait(&q_full[sq], (i / NS) & 1, abort_flag, lane)) { ok = false; break; }
      const float4* nl4 = reinterpret_cast<const float4*>(smem + SM::ROW_OFF + sq * 512) + (c0 >> 2);
      const float4* d4 = nl4 + 16;
      const bool masked = (q64 - q_first) < 2;
      uint32_t pw[16], dw[16];
      {
        uint32_t sraw[32], draw[32];
        __syncwarp();
        tmem_ld32(tmem + lane_base + ST_COL + s * 64 + c0, sraw);
        tmem_ld32(tmem + lane_base + DPT_COL + s * 64 + c0, draw);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&st_free[s]);     // scores are in registers
        if (masked) dkv_chunk<true>(sraw, draw, nl4, d4, c2, key - (q64 * 64 + c0), pw, dw);
        else dkv_chunk<false>(sraw, draw, nl4, d4, c2, 0, pw, dw);
      }
      if (i > 0 && !warp_wait(pd_free, (i - 1) & 1, abort_flag, lane)) { ok = false; break; }
      store_row32(smem + SM::PT_OFF, r, c0, pw);
      store_row32(smem + SM::DST_OFF, r, c0, dw);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(pd_full);
    }
    if (ok && warp_wait(pd_free, (n_it - 1) & 1, abort_flag, lane)) {
      tc_fence_after();
      if (split) {
        const long long kvw = (long long)p.KV * HD;
        float* pk = p.part + ((long long)(h_first % G) * p.T + key) * kvw + g * HD + half * (HD / 2);
        float* pv = pk + (long long)G * p.T * kvw;
        store_acc_rows_f32<HD / 2>(tmem + lane_base + DK_COL + half * (HD / 2), pk, key < p.T, p.scale);
        store_acc_rows_f32<HD / 2>(tmem + lane_base + DV_COL + half * (HD / 2), pv, key < p.T, 1.f);
      } else {
        __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.dqkv) + (long long)key * p.ld + half * (HD / 2);
        store_acc_rows<HD / 2>(tmem + lane_base + DV_COL + half * (HD / 2), base + v_col, key < p.T, 1.f);
        store_acc_rows<HD / 2>(tmem + lane_base + DK_COL + half * (HD / 2), base + k_col, key < p.T, p.scale);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

// ------------------------------------------------------------------------------------------------ dQ
// CTA = (query tile of 128 rows, head). Iterates over 64-key sub-tiles up to the diagonal; dQ accumulates in TMEM.
//   S = Q K^T [q x 64 keys]   dP = dO V^T [q x 64 keys]   dS = P * (dP - D) * scale   dQ += dS K
template <int HD>
struct DqSmem {
  static constexpr int NS = 4;                            // K / V ring depth (see DkvSmem)
  static constexpr int Q_TILE = 128 * HD * 2;
  static constexpr int KV_TILE = 64 * HD * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int DO_OFF = Q_TILE;
  static constexpr int K_OFF = 2 * Q_TILE;                // NS stages
  static constexpr int V_OFF = K_OFF + NS * KV_TILE;      // NS stages
  static constexpr int DS_OFF = V_OFF + NS * KV_TILE;     // [128][64] bf16
  static constexpr int BAR_OFF = DS_OFF + 16384;
  static constexpr int BYTES = BAR_OFF + 256 + 1024;
  static_assert(BYTES <= 232448, "dQ shared-memory layout does not fit");
};

// One 32-key chunk of the backward softmax for a query row: dS = exp2(S*c2 + nlse2) * (dP - D); keys with local
// index above `lim` are masked (causal diagonal).
template <bool MASKED>
__device__ __forceinline__ void dq_chunk(const uint32_t (&sraw)[32], const uint32_t (&draw)[32], float c2, float nl,
                                         float d, int lim, uint32_t* dw) {
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    float p0 = ex2_approx(fmaf(__uint_as_float(sraw[e]), c2, nl));
    float p1 = ex2_approx(fmaf(__uint_as_float(sraw[e + 1]), c2, nl));
    if (MASKED) {
      if (e > lim) p0 = 0.f;
      if (e + 1 > lim) p1 = 0.f;
    }
    dw[e >> 1] = pack_bf16x2(p0 * (__uint_as_float(draw[e]) - d), p1 * (__uint_as_float(draw[e + 1]) - d));
  }
}

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
               const __grid_constant__ CUtensorMap tm_do, const AttnParams p) {
  using SM = DqSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  constexpr int NS = SM::NS;
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;            // [NS]
  uint64_t* kv_empty = kv_full + NS;       // [NS]
  uint64_t* s_full = kv_empty + NS;        // [2]
  uint64_t* s_free = s_full + 2;           // [2]
  uint64_t* ds_full = s_free + 2;
  uint64_t* ds_free = ds_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ds_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.T + 127) / 128;
  const int h = blockIdx.x % p.H;
  const int qt = n_qt - 1 - (int)(blockIdx.x / p.H);
  const int g = h / (p.H / p.KV);
  const int n_it = min(2 * qt + 2, (p.T + 63) / 64);
  const int q_col = h * HD, k_col = (p.H + g) * HD, v_col = (p.H + p.KV + g) * HD;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < NS; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_free[i], kSoftmaxWarps); }
    mbar_init(ds_full, kSoftmaxWarps);
    mbar_init(ds_free, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t S_COL = 0, DP_COL = 128, DQ_COL = 256;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_kv); tma_prefetch_desc(&tm_do);
      mbar_expect_tx(q_full, 2 * SM::Q_TILE);
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_2d(smem + SM::Q_OFF + c * 16384, &tm_q, q_full, q_col + c * 64, qt * 128);
        tma_load_2d(smem + SM::DO_OFF + c * 16384, &tm_do, q_full, q_col + c * 64, qt * 128);
      }
      for (int i = 0; i < n_it; ++i) {
        const int s = i % NS;
        const uint32_t ph = (i / NS) & 1;
        if (!mbar_wait(&kv_empty[s], ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(&kv_full[s], 2 * SM::KV_TILE);
        for (int c = 0; c < HD / 64; ++c) {
          tma_load_2d(smem + SM::K_OFF + s * SM::KV_TILE + c * 8192, &tm_kv, &kv_full[s], k_col + c * 64, i * 64);
          tma_load_2d(smem + SM::V_OFF + s * SM::KV_TILE + c * 8192, &tm_kv, &kv_full[s], v_col + c * 64, i * 64);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t q_s = smem_u32(smem + SM::Q_OFF), do_s = smem_u32(smem + SM::DO_OFF);
      const uint32_t ds_s = smem_u32(smem + SM::DS_OFF);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto scores = [&](int i) -> bool {
        const int s = i & 1, sk = i % NS;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&kv_full[sk], (i / NS) & 1, abort_flag)) return false;
        if (!mbar_wait(&s_free[s], ph ^ 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_s = smem_u32(smem + SM::K_OFF + sk * SM::KV_TILE), v_s = smem_u32(smem + SM::V_OFF + sk * SM::KV_TILE);
        issue_product<false, false>(tmem + S_COL + s * 64, q_s, 128, k_s, 64, 64, HD, false);
        issue_product<false, false>(tmem + DP_COL + s * 64, do_s, 128, v_s, 64, 64, HD, false);
        umma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = scores(0);
      for (int i = 0; i < n_it && ok; ++i) {
        if (i + 1 < n_it) ok = scores(i + 1);
        if (!ok) break;
        const int sk = i % NS;
        if (!mbar_wait(ds_full, i & 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t k_s = smem_u32(smem + SM::K_OFF + sk * SM::KV_TILE);
        // dQ[q x HD] += dS[q x 64 keys] * K[64 keys x HD]   (B rows = keys: MN-major)
        issue_product<false, true>(tmem + DQ_COL, ds_s, 128, k_s, 64, HD, 64, i > 0);
        umma_commit(&kv_empty[sk]);
        umma_commit(ds_free);
      }
    }
    __syncwarp();
  } else {
    // 8 softmax warps: (warp & 3) picks the 32 query rows (TMEM lanes), `half` 32 of the 64 keys of the sub-tile
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int qrow = qt * 128 + r;
    const int c0 = half * 32;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;
    const bool qvalid = qrow < p.T;
    const float nl_r = qvalid ? p.nlse2[(long long)h * p.T64 + qrow] : -INFINITY;   // invalid rows give P = 0
    const float d_r = qvalid ? p.dsum[(long long)h * p.T64 + qrow] : 0.f;
    bool ok = true;
    for (int i = 0; i < n_it && ok; ++i) {
      const int s = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      if (!warp_wait(&s_full[s], ph, abort_flag, lane)) { ok = false; break; }
      tc_fence_after();
      uint32_t dw[16];
      const bool masked = i >= 2 * qt;          // the two sub-tiles on the causal diagonal
      {
        uint32_t sraw[32], draw[32];
        __syncwarp();
        tmem_ld32(tmem + lane_base + S_COL + s * 64 + c0, sraw);
        tmem_ld32(tmem + lane_base + DP_COL + s * 64 + c0, draw);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[s]);      // scores are in registers
        if (masked) dq_chunk<true>(sraw, draw, c2, nl_r, d_r, qrow - (i * 64 + c0), dw);
        else dq_chunk<false>(sraw, draw, c2, nl_r, d_r, 0, dw);
      }
      if (i > 0 && !warp_wait(ds_free, (i - 1) & 1, abort_flag, lane)) { ok = false; break; }
      store_row32(smem + SM::DS_OFF, r, c0, dw);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok && warp_wait(ds_free, (n_it - 1) & 1, abort_flag, lane)) {
      tc_fence_after();
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.dqkv) + (long long)qrow * p.ld + q_col + half * (HD / 2);
      store_acc_rows<HD / 2>(tmem + lane_base + DQ_COL + half * (HD / 2), dst, qvalid, p.scale);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

// ------------------------------------------------------------------------------------------------ dQ, 128-key tiles
// Same contract as attn_dq_kernel with key tiles of 128 instead of sub-tiles of 64: per tile the three products are
// 8 + 8 + 8 `tcgen05.mma` of 128x128x16 instead of 2 x (8 + 8 + 4) of 128x64x16 / 128x128x16, and every instruction
// with M = 128 costs about 45 cycles on top of its arithmetic whatever its width, so the wider tile nearly halves the
// tensor-pipe time per key. S and dP are single-buffered in TMEM (128 + 128 columns, dQ in another 128): the softmax
// warps release them as soon as the second half of their columns is in registers, i.e. after about half of their
// work on the tile, and the score products of the next tile run under the rest.
// Shared memory (head_dim 128: 224 KB): K(i) stays resident until dQ(i) has completed, i.e. across the score products of
// tile i+1, and its refill needs a TMA round trip on top, so K has THREE stages; V(i) is dead as soon as dP(i) has
// completed and has ONE stage: V(i+1) is requested then and is first needed a whole tile later (S(i+1) goes first).
template <int HD>
struct Dq128Smem {
  static constexpr int NS = 3;                            // K ring depth (V: one stage)
  static constexpr int Q_TILE = 128 * HD * 2;
  static constexpr int KV_TILE = 128 * HD * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int DO_OFF = Q_TILE;
  static constexpr int K_OFF = 2 * Q_TILE;                // NS stages
  static constexpr int V_OFF = K_OFF + NS * KV_TILE;      // one stage
  static constexpr int DS_OFF = V_OFF + KV_TILE;          // [128 q][128 keys] bf16 as two 64-key chunks of 16 KB
  static constexpr int BAR_OFF = DS_OFF + 32768;
  static constexpr int USED = BAR_OFF + 256;
  static constexpr int BYTES = USED + 1024;
  static_assert(BYTES <= 232448, "dQ (128-key tiles) shared-memory layout does not fit");
};

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_dq128_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                  const __grid_constant__ CUtensorMap tm_do, const AttnParams p) {
  using SM = Dq128Smem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if ((int)(smem - smem_raw) + SM::USED > SM::BYTES) {   // uniform over the CTA; nothing has been set up yet
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 2);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  constexpr int NS = SM::NS;
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;             // [NS]
  uint64_t* k_empty = k_full + NS;         // [NS]
  uint64_t* v_full = k_empty + NS;
  uint64_t* v_empty = v_full + 1;
  uint64_t* s_full = v_empty + 1;
  uint64_t* s_free = s_full + 1;
  uint64_t* ds_full = s_free + 1;
  uint64_t* ds_free = ds_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ds_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.T + 127) / 128;
  const int h = blockIdx.x % p.H;
  const int qt = n_qt - 1 - (int)(blockIdx.x / p.H);     // heavy (late) query tiles first
  const int g = h / (p.H / p.KV);
  const int n_it = qt + 1;                               // key tiles 0 .. qt; the last one is the causal diagonal
  const int q_col = h * HD, k_col = (p.H + g) * HD, v_col = (p.H + p.KV + g) * HD;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < NS; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(s_free, kSoftmaxWarps);
    mbar_init(ds_full, kSoftmaxWarps);
    mbar_init(ds_free, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t S_COL = 0, DP_COL = 128, DQ_COL = 256;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_kv); tma_prefetch_desc(&tm_do);
      mbar_expect_tx(q_full, 2 * SM::Q_TILE);
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_2d(smem + SM::Q_OFF + c * 16384, &tm_q, q_full, q_col + c * 64, qt * 128);
        tma_load_2d(smem + SM::DO_OFF + c * 16384, &tm_do, q_full, q_col + c * 64, qt * 128);
      }
      for (int i = 0; i < n_it; ++i) {
        const int s = i % NS;
        if (!mbar_wait(&k_empty[s], (uint32_t)((i / NS) & 1) ^ 1u, abort_flag)) break;
        mbar_expect_tx(&k_full[s], SM::KV_TILE);
        for (int c = 0; c < HD / 64; ++c)
          tma_load_2d(smem + SM::K_OFF + s * SM::KV_TILE + c * 16384, &tm_kv, &k_full[s], k_col + c * 64, i * 128);
        if (!mbar_wait(v_empty, (uint32_t)(i & 1) ^ 1u, abort_flag)) break;
        mbar_expect_tx(v_full, SM::KV_TILE);
        for (int c = 0; c < HD / 64; ++c)
          tma_load_2d(smem + SM::V_OFF + c * 16384, &tm_kv, v_full, v_col + c * 64, i * 128);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t q_s = smem_u32(smem + SM::Q_OFF), do_s = smem_u32(smem + SM::DO_OFF);
      const uint32_t ds_s = smem_u32(smem + SM::DS_OFF);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto scores = [&](int i) -> bool {
        const int sk = i % NS;
        if (!mbar_wait(&k_full[sk], (i / NS) & 1, abort_flag)) return false;
        if (!mbar_wait(s_free, (uint32_t)(i & 1) ^ 1u, abort_flag)) return false;   // tile i-1's scores are in registers
        tc_fence_after();
        issue_product<false, false>(tmem + S_COL, q_s, 128, smem_u32(smem + SM::K_OFF + sk * SM::KV_TILE), 128, 128, HD, false);
        if (!mbar_wait(v_full, i & 1, abort_flag)) return false;
        tc_fence_after();
        issue_product<false, false>(tmem + DP_COL, do_s, 128, smem_u32(smem + SM::V_OFF), 128, 128, HD, false);
        umma_commit(v_empty);        // V(i) is dead once dP(i) has completed
        umma_commit(s_full);
        return true;
      };
      if (ok) ok = scores(0);
      for (int i = 0; i < n_it && ok; ++i) {
        if (i + 1 < n_it) ok = scores(i + 1);
        if (!ok) break;
        const int sk = i % NS;
        if (!mbar_wait(ds_full, i & 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t k_s = smem_u32(smem + SM::K_OFF + sk * SM::KV_TILE);
        // dQ[q x HD] += dS[q x 128 keys] * K[128 keys x HD]   (B rows = keys: MN-major)
        issue_product<false, true>(tmem + DQ_COL, ds_s, 128, k_s, 128, HD, 128, i > 0);
        umma_commit(&k_empty[sk]);
        umma_commit(ds_free);
      }
    }
    __syncwarp();
  } else {
    // 8 softmax warps: (warp & 3) picks the 32 query rows (TMEM lanes), `half` 64 of the 128 keys of the tile
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int qrow = qt * 128 + r;
    const int c0 = half * 64;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;
    const bool qvalid = qrow < p.T;
    const float nl_r = qvalid ? p.nlse2[(long long)h * p.T64 + qrow] : -INFINITY;   // invalid rows give P = 0
    const float d_r = qvalid ? p.dsum[(long long)h * p.T64 + qrow] : 0.f;
    uint8_t* ds_chunk = smem + SM::DS_OFF + half * 16384;       // this warp's 64 keys are one 64-column chunk
    bool ok = true;
    for (int i = 0; i < n_it && ok; ++i) {
      if (!warp_wait(s_full, i & 1, abort_flag, lane)) { ok = false; break; }
      tc_fence_after();
      uint32_t dw0[16], dw1[16];
      const bool masked = (i == qt);              // the tile on the causal diagonal
      {
        uint32_t sraw[32], draw[32];
        __syncwarp();
        tmem_ld32(tmem + lane_base + S_COL + c0, sraw);
        tmem_ld32(tmem + lane_base + DP_COL + c0, draw);
        tc_wait_ld();
        if (masked) dq_chunk<true>(sraw, draw, c2, nl_r, d_r, r - c0, dw0);
        else dq_chunk<false>(sraw, draw, c2, nl_r, d_r, 0, dw0);
        __syncwarp();
        tmem_ld32(tmem + lane_base + S_COL + c0 + 32, sraw);
        tmem_ld32(tmem + lane_base + DP_COL + c0 + 32, draw);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);        // all of this warp's scores are in registers
        if (masked) dq_chunk<true>(sraw, draw, c2, nl_r, d_r, r - (c0 + 32), dw1);
        else dq_chunk<false>(sraw, draw, c2, nl_r, d_r, 0, dw1);
      }
      if (i > 0 && !warp_wait(ds_free, (i - 1) & 1, abort_flag, lane)) { ok = false; break; }
      store_row32(ds_chunk, r, 0, dw0);
      store_row32(ds_chunk, r, 32, dw1);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok && warp_wait(ds_free, (n_it - 1) & 1, abort_flag, lane)) {
      tc_fence_after();
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.dqkv) + (long long)qrow * p.ld + q_col + half * (HD / 2);
      store_acc_rows<HD / 2>(tmem + lane_base + DQ_COL + half * (HD / 2), dst, qvalid, p.scale);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

}  // namespace opk
