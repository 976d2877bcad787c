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
  const float* dsum;       // bwd: [H][T] rowsum(dO * O)
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

// ------------------------------------------------------------------------------------------------ forward
// CTA = (query tile of 128 rows, head). KV tiles of 128 keys, double-buffered K and V stages, S double-buffered in
// TMEM, O partials double-buffered in TMEM and folded into register accumulators one iteration late so that the
// P*V product of tile j overlaps the softmax of tile j+1.
template <int HD>
struct FwdSmem {
  static constexpr int TILE = 128 * HD * 2;           // bytes of one [128][HD] tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE;                  // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * TILE;      // 2 stages
  static constexpr int P_OFF = V_OFF + 2 * TILE;      // [128][128] bf16 = 32 KB
  static constexpr int BAR_OFF = P_OFF + 128 * 128 * 2;
  static constexpr int BYTES = BAR_OFF + 256 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(192, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm, const AttnParams p) {
  using SM = FwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_free = bars + 11;   // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* o_full = bars + 14;   // [2]
  uint64_t* o_free = bars + 16;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

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
      mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 4);
      mbar_init(&o_full[i], 1); mbar_init(&o_free[i], 4);
    }
    mbar_init(p_full, 4);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t S_COL = 0, O_COL = 256;   // S buffers at 0 / 128, O buffers at 256 / 256 + HD

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm);
      mbar_expect_tx(q_full, SM::TILE);
      for (int c = 0; c < HD / 64; ++c) tma_load_2d(smem + SM::Q_OFF + c * 16384, &tm, q_full, q_col + c * 64, qt * 128);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[s], ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(&k_full[s], SM::TILE);
        for (int c = 0; c < HD / 64; ++c)
          tma_load_2d(smem + SM::K_OFF + s * SM::TILE + c * 16384, &tm, &k_full[s], k_col + c * 64, j * 128);
        if (!mbar_wait(&v_empty[s], ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(&v_full[s], SM::TILE);
        for (int c = 0; c < HD / 64; ++c)
          tma_load_2d(smem + SM::V_OFF + s * SM::TILE + c * 16384, &tm, &v_full[s], v_col + c * 64, j * 128);
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
        if (!mbar_wait(&s_free[s], ph ^ 1u, abort_flag)) return false;
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
        if (!mbar_wait(&v_full[s], ph, abort_flag)) break;
        if (!mbar_wait(&o_free[s], ph ^ 1u, abort_flag)) break;
        if (!mbar_wait(p_full, j & 1, abort_flag)) break;
        tc_fence_after();
        // O_j[128 x HD] = P[128 x 128 keys] * V[keys x HD]: B is MN-major (rows = keys)
        issue_product<false, true>(tmem + O_COL + s * HD, p_s, 128, smem_u32(smem + SM::V_OFF + s * SM::TILE), 128, HD,
                                   128, false);
        umma_commit(&v_empty[s]);
        umma_commit(&o_full[s]);
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;            // row inside the query tile
    const int row = qt * 128 + r;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;
    float acc[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    uint8_t* p_smem = smem + SM::P_OFF;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      int w = 1;
      if (lane == 0) w = mbar_wait(&s_full[s], ph, abort_flag) ? 1 : 0;
      w = __shfl_sync(0xffffffffu, w, 0);
      if (!w) { ok = false; break; }
      tc_fence_after();
      const bool diag = (j == qt);
      // pass 1: row maximum
      float mx = m_run;
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t raw[32];
        __syncwarp();
        tmem_ld32(tmem + lane_base + S_COL + s * 128 + c0, raw);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float v = __uint_as_float(raw[i]);
          if (!diag || (c0 + i) <= r) mx = fmaxf(mx, v);
        }
      }
      const float alpha = exp2f((m_run - mx) * c2);     // 0 on the first tile (m_run = -inf), 1 if unchanged
      // P of the previous tile must have been consumed (its P*V finished) before the buffer is overwritten
      if (j > 0) {
        int w2 = 1;
        if (lane == 0) w2 = mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag) ? 1 : 0;
        w2 = __shfl_sync(0xffffffffu, w2, 0);
        if (!w2) { ok = false; break; }
      }
      // pass 2: probabilities -> shared memory (bf16, swizzled), row sum
      float lsum = 0.f;
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t raw[32];
        __syncwarp();
        tmem_ld32(tmem + lane_base + S_COL + s * 128 + c0, raw);
        tc_wait_ld();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float e0 = (!diag || (c0 + i) <= r) ? exp2f((__uint_as_float(raw[i]) - mx) * c2) : 0.f;
          float e1 = (!diag || (c0 + i + 1) <= r) ? exp2f((__uint_as_float(raw[i + 1]) - mx) * c2) : 0.f;
          // the row sum uses the rounded values that the P*V product will see
          __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
          float2 f = __bfloat1622float2(b);
          lsum += f.x + f.y;
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&b);
        }
        uint8_t* chunk = p_smem + (c0 >> 6) * 16384;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c = (c0 & 63) + q * 8;
          *reinterpret_cast<uint4*>(chunk + swz_off(r, c)) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[s]);
      fence_proxy_async();           // make the generic-proxy writes of P visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      l_run = l_run * alpha + lsum;
      m_run = mx;
      // fold in O of the previous tile (already waited for above): acc = acc * alpha_prev + O_{j-1}
      if (j > 0) {
        const int so = (j - 1) & 1;
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t raw[32];
          __syncwarp();
          tmem_ld32(tmem + lane_base + O_COL + so * HD + c0, raw);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c0 + i] = acc[c0 + i] * alpha_prev + __uint_as_float(raw[i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_free[so]);
      }
      alpha_prev = alpha;
    }
    if (ok) {
      const int so = (n_kv - 1) & 1;
      int w = 1;
      if (lane == 0) w = mbar_wait(&o_full[so], ((n_kv - 1) >> 1) & 1, abort_flag) ? 1 : 0;
      w = __shfl_sync(0xffffffffu, w, 0);
      if (w) {
        tc_fence_after();
        const float inv = 1.f / l_run;
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)row * p.ldo + h * HD;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t raw[32];
          __syncwarp();
          tmem_ld32(tmem + lane_base + O_COL + so * HD + c0, raw);
          tc_wait_ld();
          if (row < p.T) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = q * 8 + e * 2;
                const float a0 = (acc[c0 + i] * alpha_prev + __uint_as_float(raw[i])) * inv;
                const float a1 = (acc[c0 + i + 1] * alpha_prev + __uint_as_float(raw[i + 1])) * inv;
                ow[e] = pack_bf16x2(a0, a1);
              }
              *reinterpret_cast<uint4*>(orow + c0 + q * 8) = o;
            }
          }
        }
        if (row < p.T) p.lse[(long long)h * p.T + row] = m_run * p.scale + logf(l_run);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}


// ------------------------------------------------------------------------------------------------ backward helpers
// D[h][t] = sum_d dO[t][h*hd + d] * O[t][h*hd + d]
__global__ void attn_dsum_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                 float* __restrict__ dsum, int T, int H, int hd, long long ldo) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T * H) return;
  const int t = w / H, h = w % H;
  const __nv_bfloat16* a = o + (long long)t * ldo + h * hd;
  const __nv_bfloat16* b = dout + (long long)t * ldo + h * hd;
  float s = 0.f;
  for (int i = lane; i < hd; i += 32) s += __bfloat162float(a[i]) * __bfloat162float(b[i]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) dsum[(long long)h * T + t] = s;
}

// One warp-collective bounded wait: lane 0 polls, the result is broadcast.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane) {
  int w = 1;
  if (lane == 0) w = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
  return __shfl_sync(0xffffffffu, w, 0) != 0;
}

// Write 64 packed bf16 values (32 words) of row r into a [128 rows][64 cols] swizzled chunk.
__device__ __forceinline__ void store_row64(uint8_t* chunk, int r, const uint32_t (&w)[32]) {
#pragma unroll
  for (int q = 0; q < 8; ++q)
    *reinterpret_cast<uint4*>(chunk + swz_off(r, q * 8)) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
}

// Store one TMEM accumulator row block (HD fp32 columns starting at tmem column `col`) as bf16.
template <int HD>
__device__ __forceinline__ void store_acc_rows(uint32_t tmem_addr, __nv_bfloat16* dst, bool valid) {
#pragma unroll
  for (int c0 = 0; c0 < HD; c0 += 32) {
    uint32_t raw[32];
    __syncwarp();
    tmem_ld32(tmem_addr + c0, raw);
    tc_wait_ld();
    if (valid) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack_bf16x2(__uint_as_float(raw[8 * q + 0]), __uint_as_float(raw[8 * q + 1]));
        o.y = pack_bf16x2(__uint_as_float(raw[8 * q + 2]), __uint_as_float(raw[8 * q + 3]));
        o.z = pack_bf16x2(__uint_as_float(raw[8 * q + 4]), __uint_as_float(raw[8 * q + 5]));
        o.w = pack_bf16x2(__uint_as_float(raw[8 * q + 6]), __uint_as_float(raw[8 * q + 7]));
        *reinterpret_cast<uint4*>(dst + c0 + q * 8) = o;
      }
    }
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
  static constexpr int KV_TILE = 128 * HD * 2;
  static constexpr int Q_TILE = 64 * HD * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = KV_TILE;
  static constexpr int Q_OFF = 2 * KV_TILE;               // 2 stages
  static constexpr int DO_OFF = Q_OFF + 2 * Q_TILE;       // 2 stages
  static constexpr int PT_OFF = DO_OFF + 2 * Q_TILE;      // [128][64] bf16
  static constexpr int DST_OFF = PT_OFF + 16384;
  static constexpr int BAR_OFF = DST_OFF + 16384;
  static constexpr int BYTES = BAR_OFF + 256 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(192, 1)
attn_dkv_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
                const __grid_constant__ CUtensorMap tm_do, const AttnParams p) {
  using SM = DkvSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;    // [2]
  uint64_t* q_empty = bars + 3;   // [2]
  uint64_t* st_full = bars + 5;   // [2]
  uint64_t* st_free = bars + 7;   // [2]
  uint64_t* pd_full = bars + 9;
  uint64_t* pd_free = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.H / p.KV;
  const int g = blockIdx.x % p.KV;
  const int kt = blockIdx.x / p.KV;                      // low key tiles (most work) first
  const int n_q64 = (p.T + 63) / 64;
  const int q_first = 2 * kt;
  const int per_head = n_q64 - q_first;
  const int n_it = per_head * G;
  const int k_col = (p.H + g) * HD, v_col = (p.H + p.KV + g) * HD;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1);
      mbar_init(&st_full[i], 1); mbar_init(&st_free[i], 4);
    }
    mbar_init(pd_full, 4);
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
        const int s = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        const int h = g * G + i / per_head, q64 = q_first + i % per_head;
        if (!mbar_wait(&q_empty[s], ph ^ 1u, abort_flag)) break;
        mbar_expect_tx(&q_full[s], 2 * SM::Q_TILE);
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
        const int s = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&q_full[s], ph, abort_flag)) return false;
        if (!mbar_wait(&st_free[s], ph ^ 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t q_s = smem_u32(smem + SM::Q_OFF + s * SM::Q_TILE), do_s = smem_u32(smem + SM::DO_OFF + s * SM::Q_TILE);
        issue_product<false, false>(tmem + ST_COL + s * 64, k_s, 128, q_s, 64, 64, HD, false);
        issue_product<false, false>(tmem + DPT_COL + s * 64, v_s, 128, do_s, 64, 64, HD, false);
        umma_commit(&st_full[s]);
        return true;
      };
      if (ok) ok = scores(0);
      for (int i = 0; i < n_it && ok; ++i) {
        if (i + 1 < n_it) ok = scores(i + 1);
        if (!ok) break;
        const int s = i & 1;
        if (!mbar_wait(pd_full, i & 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t q_s = smem_u32(smem + SM::Q_OFF + s * SM::Q_TILE), do_s = smem_u32(smem + SM::DO_OFF + s * SM::Q_TILE);
        // dV[keys x HD] += Pt[keys x 64 q] * dO[64 q x HD]   (B rows = queries: MN-major)
        issue_product<false, true>(tmem + DV_COL, pt_s, 128, do_s, 64, HD, 64, i > 0);
        issue_product<false, true>(tmem + DK_COL, dst_s, 128, q_s, 64, HD, 64, i > 0);
        umma_commit(&q_empty[s]);
        umma_commit(pd_free);
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int key = kt * 128 + r;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;
    bool ok = true;
    for (int i = 0; i < n_it && ok; ++i) {
      const int s = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      const int h = g * G + i / per_head, q64 = q_first + i % per_head;
      if (!warp_wait(&st_full[s], ph, abort_flag, lane)) { ok = false; break; }
      tc_fence_after();
      const float* lse_h = p.lse + (long long)h * p.T;
      const float* ds_h = p.dsum + (long long)h * p.T;
      uint32_t pw[32], dw[32];
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t sraw[32], draw[32];
        __syncwarp();
        tmem_ld32(tmem + lane_base + ST_COL + s * 64 + c0, sraw);
        tmem_ld32(tmem + lane_base + DPT_COL + s * 64 + c0, draw);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int q = q64 * 64 + c0 + e + u;
            const bool live = (q < p.T) && (q >= key) && (key < p.T);
            const float l = live ? __ldg(lse_h + q) : 0.f;
            const float dd = live ? __ldg(ds_h + q) : 0.f;
            const float pr = live ? exp2f(__uint_as_float(sraw[e + u]) * c2 - l * 1.4426950408889634f) : 0.f;
            pv[u] = pr;
            dv[u] = pr * (__uint_as_float(draw[e + u]) - dd) * p.scale;
          }
          pw[(c0 + e) >> 1] = pack_bf16x2(pv[0], pv[1]);
          dw[(c0 + e) >> 1] = pack_bf16x2(dv[0], dv[1]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&st_free[s]);
      if (i > 0 && !warp_wait(pd_free, (i - 1) & 1, abort_flag, lane)) { ok = false; break; }
      store_row64(smem + SM::PT_OFF, r, pw);
      store_row64(smem + SM::DST_OFF, r, dw);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(pd_full);
    }
    if (ok && warp_wait(pd_free, (n_it - 1) & 1, abort_flag, lane)) {
      tc_fence_after();
      __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.dqkv) + (long long)key * p.ld;
      store_acc_rows<HD>(tmem + lane_base + DV_COL, base + v_col, key < p.T);
      store_acc_rows<HD>(tmem + lane_base + DK_COL, base + k_col, key < p.T);
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
  static constexpr int Q_TILE = 128 * HD * 2;
  static constexpr int KV_TILE = 64 * HD * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int DO_OFF = Q_TILE;
  static constexpr int K_OFF = 2 * Q_TILE;                // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * KV_TILE;       // 2 stages
  static constexpr int DS_OFF = V_OFF + 2 * KV_TILE;      // [128][64] bf16
  static constexpr int BAR_OFF = DS_OFF + 16384;
  static constexpr int BYTES = BAR_OFF + 256 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(192, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
               const __grid_constant__ CUtensorMap tm_do, const AttnParams p) {
  using SM = DqSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;    // [2]
  uint64_t* s_free = bars + 7;    // [2]
  uint64_t* ds_full = bars + 9;
  uint64_t* ds_free = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 4);
    }
    mbar_init(ds_full, 4);
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
        const int s = i & 1;
        const uint32_t ph = (i >> 1) & 1;
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
        const int s = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&kv_full[s], ph, abort_flag)) return false;
        if (!mbar_wait(&s_free[s], ph ^ 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_s = smem_u32(smem + SM::K_OFF + s * SM::KV_TILE), v_s = smem_u32(smem + SM::V_OFF + s * SM::KV_TILE);
        issue_product<false, false>(tmem + S_COL + s * 64, q_s, 128, k_s, 64, 64, HD, false);
        issue_product<false, false>(tmem + DP_COL + s * 64, do_s, 128, v_s, 64, 64, HD, false);
        umma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = scores(0);
      for (int i = 0; i < n_it && ok; ++i) {
        if (i + 1 < n_it) ok = scores(i + 1);
        if (!ok) break;
        const int s = i & 1;
        if (!mbar_wait(ds_full, i & 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t k_s = smem_u32(smem + SM::K_OFF + s * SM::KV_TILE);
        // dQ[q x HD] += dS[q x 64 keys] * K[64 keys x HD]   (B rows = keys: MN-major)
        issue_product<false, true>(tmem + DQ_COL, ds_s, 128, k_s, 64, HD, 64, i > 0);
        umma_commit(&kv_empty[s]);
        umma_commit(ds_free);
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int qrow = qt * 128 + r;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;
    const bool qvalid = qrow < p.T;
    const float lse_r = qvalid ? p.lse[(long long)h * p.T + qrow] * 1.4426950408889634f : 0.f;
    const float d_r = qvalid ? p.dsum[(long long)h * p.T + qrow] : 0.f;
    bool ok = true;
    for (int i = 0; i < n_it && ok; ++i) {
      const int s = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      if (!warp_wait(&s_full[s], ph, abort_flag, lane)) { ok = false; break; }
      tc_fence_after();
      uint32_t dw[32];
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t sraw[32], draw[32];
        __syncwarp();
        tmem_ld32(tmem + lane_base + S_COL + s * 64 + c0, sraw);
        tmem_ld32(tmem + lane_base + DP_COL + s * 64 + c0, draw);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float dv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int key = i * 64 + c0 + e + u;
            const bool live = qvalid && key <= qrow;
            const float pr = live ? exp2f(__uint_as_float(sraw[e + u]) * c2 - lse_r) : 0.f;
            dv[u] = pr * (__uint_as_float(draw[e + u]) - d_r) * p.scale;
          }
          dw[(c0 + e) >> 1] = pack_bf16x2(dv[0], dv[1]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[s]);
      if (i > 0 && !warp_wait(ds_free, (i - 1) & 1, abort_flag, lane)) { ok = false; break; }
      store_row64(smem + SM::DS_OFF, r, dw);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok && warp_wait(ds_free, (n_it - 1) & 1, abort_flag, lane)) {
      tc_fence_after();
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.dqkv) + (long long)qrow * p.ld + q_col;
      store_acc_rows<HD>(tmem + lane_base + DQ_COL, dst, qvalid);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

}  // namespace opk
