// Causal grouped-query flash attention for sm_100a on tcgen05 / TMEM, operating in place on the fused projection
// buffer qkv[T][(H + 2*KV) * hd] (bf16, row pitch ld): Q head h at column h*hd, K head g at (H+g)*hd, V head g at
// (H+KV+g)*hd. head_dim is 64 or 128. One example (sequence) per launch; heads are the parallel dimension.
//
// Shared design of the three kernels (forward, dK/dV, dQ):
//   * 384 threads: warp 0 = TMA producer (Q, K), warp 1 = TMEM owner + issuer of the score products, warps 2..9 =
//     softmax / epilogue with thread <-> TMEM lane (= row of the 128-row tile; warps w and w+4 share a lane quarter),
//     warps 10 and 11 = issuer of the second kind of products (P*V; dV and dK; dQ) and V producer (forward, dQ).
//     Two issuing threads because a thread's barrier probes queue up behind the tensor-core instructions it has
//     issued itself: one issuer alternating between the two kinds leaves the tensor core idle during its waits,
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

// 2-D TMA store of a {64 cols, rows} box from shared memory (rows outside the tensor are clipped), as one bulk group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// 3-D TMA store of one box (the tensor map fixes its shape), joined to the calling thread's current bulk group by
// the next commit.
__device__ __forceinline__ void tma_store_3d_nocommit(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// The calling thread's bulk stores have finished reading shared memory.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

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
// Work item = (query tile of 128 rows, head). One persistent CTA per SM walks a balanced share of the items, heavy
// ones first; the key tiles of its items form one stream, so the loads and score products of an item start under the
// tail of the one before. KV tiles of 128 keys, double-buffered K and V stages. The key tiles are split
// between two softmax groups of four warps: even tiles of the stream go to group 0, odd tiles to group 1, and each group has its own
// score buffer and its own output accumulator in TMEM (4 x 128 columns), its own probability buffer in shared memory
// and its own running maximum and row sum, as if the keys had been split in two; the two partial results are merged
// once, in the epilogue. One group's exponentials therefore run under the other group's waits and under the tensor
// core's work on the other buffers. The running maximum is updated lazily: rows are rescaled (TMEM
// load-multiply-store) only when their maximum grew by more than 2^8, otherwise the stale maximum stays in use
// (probabilities may then exceed 1 by at most 2^8, harmless in bf16 / fp32). A thread owns one row and all 128 keys of
// a tile: pass 1 reads the scores from TMEM for the maximum, pass 2 reads them again 32 at a time for ffma +
// ex2.approx, pack and the swizzled store.
#ifdef OPK_ATTN_TRACE
// Debug-only timeline of CTA 0 (clock64 stamps per role / tile / event); never compiled into the library.
__device__ long long g_attn_trace[3 * 1024];
#ifndef OPK_TRACE_K
#define OPK_TRACE_K 0
#endif
#define OPK_TRACE(role, j, e) do { if (blockIdx.x == 0) g_attn_trace[(role) * 1024 + (j) * 8 + (e)] = clock64(); } while (0)
// Per-item record (SM id, start and end in globaltimer nanoseconds) of up to 1024 work items.
__device__ long long g_attn_cta[1024 * 4];
__device__ __forceinline__ long long opk_globaltimer() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ int opk_smid() {
  int v;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
  return v;
}
#define OPK_TRACE_ITEM(w, e) do { if ((w) < 1024) { g_attn_cta[(w) * 4 + (e)] = opk_globaltimer(); g_attn_cta[(w) * 4 + 3] = opk_smid(); } } while (0)
#else
#define OPK_TRACE_K 0
#define OPK_TRACE(role, j, e) do { } while (0)
#define OPK_TRACE_ITEM(w, e) do { } while (0)
#endif

constexpr int kSoftmaxWarps = 8;                       // warps 2..9; warps 0 / 1 drive TMA / MMA
constexpr int kAttnThreads = (2 + kSoftmaxWarps) * 32;
constexpr int kFwdThreads = kAttnThreads + 64;          // forward: two more warps, the V producer and the P*V issuer
constexpr int kBwdThreads = kAttnThreads + 64;          // backward: two more warps, the second issuer and (dQ) the V producer

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

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Maximum of 64 scores with four independent chains of three-input maxima (two columns per instruction). The causal
// mask needs no variant here: the forward kernel writes -inf over the masked scores of a diagonal tile beforehand.
__device__ __forceinline__ float row_max64(const uint32_t (&a)[32], const uint32_t (&b)[32]) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    m0 = fmax3(m0, __uint_as_float(a[i]), __uint_as_float(a[i + 1]));
    m1 = fmax3(m1, __uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
    m2 = fmax3(m2, __uint_as_float(b[i]), __uint_as_float(b[i + 1]));
    m3 = fmax3(m3, __uint_as_float(b[i + 2]), __uint_as_float(b[i + 3]));
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// exp2(x * c2 - mc) for 32 columns starting at col0, packed to bf16 and stored swizzled; returns the partial row sum.
// Masked scores arrive as -inf and come out as exact zeros.
__device__ __forceinline__ float softmax_chunk(const uint32_t (&x)[32], int col0, int r, float c2, float mc,
                                               uint8_t* p_smem) {
  float sum0 = 0.f, sum1 = 0.f;
  uint32_t packed[16];
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float e0 = ex2_approx(fmaf(__uint_as_float(x[i]), c2, -mc));
    float e1 = ex2_approx(fmaf(__uint_as_float(x[i + 1]), c2, -mc));
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

// One work item of the forward kernel: (query tile, head), decoded from its rank in the heavy-first order.
struct FwdItem {
  int qt, h, g, n_kv;
};
__device__ __forceinline__ FwdItem fwd_item(int w, int n_qt, int H, int KV) {
  FwdItem it;
  it.qt = n_qt - 1 - w / H;
  it.h = w % H;
  it.g = it.h / (H / KV);
  it.n_kv = it.qt + 1;
  return it;
}
// Rank of the k-th item of CTA c out of G: boustrophedon over the heavy-first list, so that every CTA gets nearly the
// same number of key tiles. Monotone in k; the CTA is done at the first rank >= the number of items.
__device__ __forceinline__ int fwd_rank(int k, int c, int G) { return (k & 1) ? (k + 1) * G - 1 - c : k * G + c; }

template <int HD>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm, const __grid_constant__ CUtensorMap tm_out, const AttnParams p) {
  using SM = FwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if ((int)(smem - smem_raw) + SM::USED > SM::BYTES) {   // uniform over the CTA; nothing has been set up yet
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 2);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* q_full = bars + 0;
  uint64_t* q_empty = bars + 1;   // every score product of the item has completed: Q may be replaced
  uint64_t* k_full = bars + 2;    // [2]
  uint64_t* k_empty = bars + 4;   // [2]
  uint64_t* v_full = bars + 6;    // [2]
  uint64_t* v_empty = bars + 8;   // [2]
  uint64_t* s_full = bars + 10;   // [2]
  uint64_t* s_free = bars + 12;   // [2]
  uint64_t* p_full = bars + 14;   // [2]
  uint64_t* o_done = bars + 16;   // [2] P*V of a tile has completed (its P buffer is reusable, its accumulator consistent)
  uint64_t* o_free = bars + 18;   // all eight softmax warps have read the item's accumulators (and the exchange area)
  uint64_t* xr = bars + 19;       // [2 groups][4 quads] the warp's (maximum, row sum) of the item are in the exchange
                                  // area and, if its group owns the item's last tile, that tile's P*V has completed
  uint64_t* stage_free = bars + 27;   // [2] the other group has read its staged output out of group b's buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 29);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xchg = reinterpret_cast<float*>(bars + 32);   // [2 groups][128 rows] running maxima, then [2][128] row sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.T + 127) / 128;
  const int n_items = n_qt * p.H;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int k_col0 = p.H * HD, v_col0 = (p.H + p.KV) * HD;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_free[i], kSoftmaxWarps / 2);
      mbar_init(&p_full[i], kSoftmaxWarps / 2); mbar_init(&o_done[i], 1);
    }
    mbar_init(o_free, kSoftmaxWarps);
    for (int i = 0; i < 8; ++i) mbar_init(&xr[i], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&stage_free[i], kSoftmaxWarps / 2);
    *abort_flag = 0;
    fence_barrier_init();
    // The producer thread starts the loads of Q and of the first K tile of its first item before the CTA-wide setup
    // barrier: their latency then runs under the TMEM allocation.
    const FwdItem it = fwd_item(fwd_rank(0, cta, G), n_qt, p.H, p.KV);
    tma_prefetch_desc(&tm);
    mbar_expect_tx(q_full, SM::TILE);
    for (int c = 0; c < HD / 64; ++c) tma_load_2d(smem + SM::Q_OFF + c * 16384, &tm, q_full, it.h * HD + c * 64, it.qt * 128);
    mbar_expect_tx(&k_full[0], SM::TILE);
    for (int c = 0; c < HD / 64; ++c) tma_load_2d(smem + SM::K_OFF + c * 16384, &tm, &k_full[0], k_col0 + it.g * HD + c * 64, 0);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t S_COL = 0, O_COL = 256;   // score buffers at 0 / 128, the two output accumulators at 256 / 384

  // All roles walk the same stream of key tiles: the items of this CTA one after the other, tile t of the stream
  // using K / V stage, score buffer, probability buffer, accumulator and softmax group t & 1 with barrier phase
  // (t >> 1) & 1. Nothing but the item-level hand-offs (Q, accumulators) separates one item from the next, so the
  // loads and score products of an item start under the last tiles and the epilogue of the one before.
  if (warp == 0) {
    // Q and K producer. K(t+2) is requested as soon as the score product of tile t has completed.
    if (lane == 0) {
      tma_prefetch_desc(&tm_out);
      int t_base = 0;
      bool alive = true;
      for (int k = 0; alive; ++k) {
        const int w = fwd_rank(k, cta, G);
        if (w >= n_items) break;
        const FwdItem it = fwd_item(w, n_qt, p.H, p.KV);
        const int q_col = it.h * HD, k_col = k_col0 + it.g * HD;
        if (k > 0) {
          if (!mbar_wait(q_empty, (uint32_t)((k - 1) & 1), abort_flag)) break;
          mbar_expect_tx(q_full, SM::TILE);
          for (int c = 0; c < HD / 64; ++c) tma_load_2d(smem + SM::Q_OFF + c * 16384, &tm, q_full, q_col + c * 64, it.qt * 128);
        }
        for (int j = (k == 0 ? 1 : 0); j < it.n_kv; ++j) {   // K(0) of the first item was requested during the setup
          const int t = t_base + j, s = t & 1;
          const uint32_t ph = (t >> 1) & 1;
          if (!mbar_wait(&k_empty[s], ph ^ 1u, abort_flag)) { alive = false; break; }
          if (k == OPK_TRACE_K) OPK_TRACE(0, j, 0);
          mbar_expect_tx(&k_full[s], SM::TILE);
          for (int c = 0; c < HD / 64; ++c)
            tma_load_2d(smem + SM::K_OFF + s * SM::TILE + c * 16384, &tm, &k_full[s], k_col + c * 64, j * 128);
        }
        t_base += it.n_kv;
      }
    }
    __syncwarp();
  } else if (warp == 2 + kSoftmaxWarps) {
    // V producer, on a warp of its own so that a wait for a V stage (freed by a P*V) never delays a K request.
    if (lane == 0) {
      int t_base = 0;
      bool alive = true;
      for (int k = 0; alive; ++k) {
        const int w = fwd_rank(k, cta, G);
        if (w >= n_items) break;
        const FwdItem it = fwd_item(w, n_qt, p.H, p.KV);
        const int v_col = v_col0 + it.g * HD;
        for (int j = 0; j < it.n_kv; ++j) {
          const int t = t_base + j, s = t & 1;
          const uint32_t ph = (t >> 1) & 1;
          if (!mbar_wait(&v_empty[s], ph ^ 1u, abort_flag)) { alive = false; break; }
          if (k == OPK_TRACE_K) OPK_TRACE(0, j, 1);
          mbar_expect_tx(&v_full[s], SM::TILE);
          for (int c = 0; c < HD / 64; ++c)
            tma_load_2d(smem + SM::V_OFF + s * SM::TILE + c * 16384, &tm, &v_full[s], v_col + c * 64, j * 128);
        }
        t_base += it.n_kv;
      }
    }
#ifdef OPK_ATTN_TRACE
    // observers: arrival times of the K and V tiles of the first item
    if (lane == 1 || lane == 2) {
      int tb = 0;
      for (int kk = 0; kk < OPK_TRACE_K; ++kk) tb += fwd_item(fwd_rank(kk, cta, G), n_qt, p.H, p.KV).n_kv;
      const int n0 = fwd_item(fwd_rank(OPK_TRACE_K, cta, G), n_qt, p.H, p.KV).n_kv;
      for (int jj = 0; jj < tb + n0; ++jj) {
        const int j = jj - tb;
        if (!mbar_wait(lane == 1 ? &k_full[jj & 1] : &v_full[jj & 1], (uint32_t)((jj >> 1) & 1), abort_flag)) break;
        if (j >= 0) OPK_TRACE(0, j, 1 + lane);
      }
    }
#endif
    __syncwarp();
  } else if (warp == 1) {
    // Score-product issuer. The two kinds of products are issued by two threads of different warps: a thread's
    // barrier probes queue up behind the tensor-core instructions it has issued itself, so a single issuer that
    // alternates "wait, 8 x mma, commit" for both kinds leaves the tensor core idle during its waits, whereas
    // two issuers fill each other's gaps. S(t) only needs K(t) and score buffer t & 1 (free once softmax t-2 has read it).
    if (lane == 0) {
      const uint32_t q_s = smem_u32(smem + SM::Q_OFF);
      int t = 0;
      bool ok = true;
      for (int k = 0; ok; ++k) {
        const int w = fwd_rank(k, cta, G);
        if (w >= n_items) break;
        const int n_kv = n_qt - w / p.H;
        if (!mbar_wait(q_full, (uint32_t)(k & 1), abort_flag)) break;
        for (int j = 0; j < n_kv; ++j, ++t) {
          const int s = t & 1;
          const uint32_t ph = (t >> 1) & 1;
          if (k == OPK_TRACE_K) OPK_TRACE(1, j, 6);
          if (!mbar_wait(&k_full[s], ph, abort_flag)) { ok = false; break; }
          if (k == OPK_TRACE_K) OPK_TRACE(1, j, 0);
          if (!mbar_wait(&s_free[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          if (k == OPK_TRACE_K) OPK_TRACE(1, j, 1);
          tc_fence_after();
          issue_product<false, false>(tmem + S_COL + s * 128, q_s, 128, smem_u32(smem + SM::K_OFF + s * SM::TILE), 128, 128,
                                      HD, false);
          umma_commit(&k_empty[s]);
          umma_commit(&s_full[s]);
          if (j == n_kv - 1) umma_commit(q_empty);
          if (k == OPK_TRACE_K) OPK_TRACE(1, j, 7);
        }
      }
    }
    __syncwarp();
  } else if (warp == 3 + kSoftmaxWarps) {
    // P*V issuer: O_s[128 x HD] (+)= P[128 x 128 keys] * V[keys x HD], B MN-major (rows = keys); the first tile of
    // each group in an item (j = 0, 1) starts its accumulator afresh.
    if (lane == 0) {
      const uint32_t p_s = smem_u32(smem + SM::P_OFF);
      int t = 0;
      bool ok = true;
      for (int k = 0; ok; ++k) {
        const int w = fwd_rank(k, cta, G);
        if (w >= n_items) break;
        const int n_kv = n_qt - w / p.H;
        // the accumulators of the previous item must have been read before this item's first P*V overwrites one
        if (k > 0 && !mbar_wait(o_free, (uint32_t)((k - 1) & 1), abort_flag)) break;
        for (int j = 0; j < n_kv; ++j, ++t) {
          const int s = t & 1;
          const uint32_t ph = (t >> 1) & 1;
          if (k == OPK_TRACE_K) OPK_TRACE(1, j, 2);
          if (!mbar_wait(&v_full[s], ph, abort_flag)) { ok = false; break; }
          if (k == OPK_TRACE_K) OPK_TRACE(1, j, 3);
          if (!mbar_wait(&p_full[s], ph, abort_flag)) { ok = false; break; }
          if (k == OPK_TRACE_K) OPK_TRACE(1, j, 4);
          tc_fence_after();
          issue_product<false, true>(tmem + O_COL + s * 128, p_s + s * SM::P_BYTES, 128, smem_u32(smem + SM::V_OFF + s * SM::TILE), 128, HD, 128, j > 1);
          umma_commit(&v_empty[s]);
          umma_commit(&o_done[s]);
          if (k == OPK_TRACE_K) OPK_TRACE(1, j, 5);
        }
      }
    }
    __syncwarp();
  } else {
    // Two softmax groups of four warps. Group g owns the stream tiles with t & 1 == g together with score buffer g,
    // probability buffer g and output accumulator g, and keeps its own running maximum and row sum, so the groups
    // never synchronise inside an item: while one waits for its next score tile the other one computes.
    // Thread <-> row of the query tile; warps with the same (warp & 3) share a TMEM lane quarter.
    const int quad = warp & 3;
    const int grp = (warp - 2) >> 2;
    const int r = quad * 32 + lane;            // row inside the query tile
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const uint32_t s_addr = tmem + lane_base + S_COL + grp * 128;
    const uint32_t o_addr = tmem + lane_base + O_COL + grp * 128;
    uint8_t* p_smem = smem + SM::P_OFF + grp * SM::P_BYTES;
    const float c2 = p.scale * 1.4426950408889634f;
    int t_base = 0;
    bool ok = true;
    // An item ends with an epilogue that merges the two groups' accumulators. The group that owns the item's last key
    // tile runs it as soon as that tile's P*V has completed. The other group is done a tile earlier: instead of
    // waiting it publishes its (maximum, row sum), goes on with the first tile of the next item (whose P*V the issuer
    // holds back until both groups have read the accumulators) and runs the deferred epilogue right after it.
    bool pend = false;              // a deferred epilogue: item rank, index, first stream tile, tiles, this group's state
    int pend_w = 0, pend_k = 0, pend_tb = 0, pend_n = 0;
    float pend_m = 0.f, pend_l = 0.f;
    bool stage_wait = false;        // the other group staged its output in this group's buffer: wait before writing P
    int own_cnt = 0;                // items so far whose last tile this group owned (phase of stage_free[grp])
    uint32_t stage_par = 0;
    // Merge and store the output rows of item (e_w, e_k) whose stream started at tile e_tb with e_n tiles; e_m / e_l are
    // this group's maximum and row sum. O = (a * O_0 + b * O_1) / (a * l_0 + b * l_1), a, b = 2^(c2 * (m_g - max)).
    // Group g writes output columns [g * HD/2, (g+1) * HD/2).
    auto epilogue = [&](int e_w, int e_k, int e_tb, int e_n, float e_m, float e_l) -> bool {
      const FwdItem eit = fwd_item(e_w, n_qt, p.H, p.KV);
      const int qt = eit.qt, h = eit.h;
      const int row = qt * 128 + r;
      const bool owner = ((e_tb + e_n - 1) & 1) == grp;
      // the other group's values; from the owner they also tell that every P*V of the item has completed
      if (!warp_wait(&xr[(grp ^ 1) * 4 + quad], (uint32_t)(e_k & 1), abort_flag, lane)) return false;
      if (e_k == OPK_TRACE_K && quad == 2 && lane == 0) OPK_TRACE(2, 100 + grp, 0);
      tc_fence_after();
      const float m_o = xchg[(grp ^ 1) * 128 + r], l_o = xchg[256 + (grp ^ 1) * 128 + r];
      const float m_tot = fmaxf(e_m, m_o);
      const float w_me = ex2_approx((e_m - m_tot) * c2), w_o = ex2_approx((m_o - m_tot) * c2);
      const float l_tot = w_me * e_l + w_o * l_o;
      const float inv = 1.f / l_tot;
      const float w0 = (grp == 0 ? w_me : w_o) * inv, w1 = (grp == 0 ? w_o : w_me) * inv;
      // with a single key tile only the accumulator of the group that owned it was written
      const bool has0 = e_n > 1 || (e_tb & 1) == 0, has1 = e_n > 1 || (e_tb & 1) == 1;
      const uint32_t o0 = tmem + lane_base + O_COL + grp * (HD / 2), o1 = o0 + 128;
      // HD = 128: the group's 64 output columns are staged in the swizzled row layout and each warp stores its 32
      // rows with one TMA store, which clips the rows past T. The owner stages in the first half of its own
      // probability buffer (free: its last P*V is complete); the other group's own buffer already holds the
      // probabilities of the next item, so it borrows the second half of the owner's. HD = 64: written directly.
      uint8_t* stage = owner ? p_smem : smem + SM::P_OFF + (grp ^ 1) * SM::P_BYTES + 16384;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)row * p.ldo + h * HD + grp * (HD / 2);
#pragma unroll
      for (int c0 = 0; c0 < HD / 2; c0 += 32) {
        uint32_t ra[32], rb[32];
        __syncwarp();
        tmem_ld32(o0 + c0, ra);                 // an accumulator without a tile holds stale bits: dropped below
        tmem_ld32(o1 + c0, rb);
        tc_wait_ld();
        if (c0 + 32 >= HD / 2) {                  // last accumulator read of the item by this warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(o_free);
        }
        if (HD == 128 || row < p.T) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              v[i] = __uint_as_float(has0 ? ra[8 * q + i] : 0u) * w0;
              v[i] = fmaf(__uint_as_float(has1 ? rb[8 * q + i] : 0u), w1, v[i]);
            }
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]);
            o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]);
            o.w = pack_bf16x2(v[6], v[7]);
            if (HD == 128) *reinterpret_cast<uint4*>(stage + swz_off(r, c0 + q * 8)) = o;
            else *reinterpret_cast<uint4*>(orow + c0 + q * 8) = o;
          }
        }
      }
      if (HD == 128) {
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && qt * 128 + quad * 32 < p.T)
          tma_store_2d(&tm_out, stage + quad * 32 * 128, h * HD + grp * 64, qt * 128 + quad * 32);
      }
      if (!owner) {                               // hand the borrowed half back once the store has read it
        if (lane == 0) {
          if (HD == 128) tma_store_wait_read();
          mbar_arrive(&stage_free[grp ^ 1]);
        }
      }
      __syncwarp();
      if (grp == 0 && row < p.T) p.lse[(long long)h * p.T + row] = m_tot * p.scale + logf(l_tot);
      if (e_k == OPK_TRACE_K && quad == 2 && lane == 0) OPK_TRACE(2, 100 + grp, 1);
      if (quad == 2 && lane == 0 && grp == 0) OPK_TRACE_ITEM(e_w, 1);
      return true;
    };
    for (int k = 0; ok; ++k) {
      const int w = fwd_rank(k, cta, G);
      if (w >= n_items) break;
      const FwdItem it = fwd_item(w, n_qt, p.H, p.KV);
      const int qt = it.qt, n_kv = it.n_kv;
      if (quad == 2 && lane == 0 && grp == 0) OPK_TRACE_ITEM(w, 0);
      if (HD == 128) {                         // this warp's output slab of the previous item has left shared memory
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
      }
      float m_run = -INFINITY, l_run = 0.f;    // m_run: maximum in use (possibly stale); l_run: this group's row sum
      const int j0 = ((t_base & 1) == grp) ? 0 : 1;   // first tile of the item that belongs to this group
      bool first_tile = true;
      for (int j = j0; j < n_kv && ok; j += 2) {
        const int t = t_base + j;
        const uint32_t ph = (t >> 1) & 1;
        if (k == OPK_TRACE_K && quad == 2 && lane == 0) OPK_TRACE(2, j, 0);
        if (!warp_wait(&s_full[grp], ph, abort_flag, lane)) { ok = false; break; }
        if (k == OPK_TRACE_K && quad == 2 && lane == 0) OPK_TRACE(2, j, 1);
        tc_fence_after();
#ifdef OPK_FWD_SKIP_SOFTMAX
        if (t > 1 && !warp_wait(&o_done[grp], ph ^ 1u, abort_flag, lane)) { ok = false; break; }
        first_tile = false;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[grp]);
#else
        uint32_t x0[32], x1[32];
        if (j == qt) {
          // causal diagonal: the scores right of the diagonal are replaced by -inf in TMEM once, so that the two
          // passes below need no masked variant (exp2 of -inf is 0 and the maximum ignores it)
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 32) {
            if (c0 + 31 <= (quad * 32)) continue;          // whole chunk left of the diagonal for every row of this warp
            __syncwarp();
            tmem_ld32(s_addr + c0, x0);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c0 + i > r) x0[i] = 0xff800000u;
            tmem_st32(s_addr + c0, x0);
          }
          tc_wait_st();
        }
        // pass 1: row maximum over the 128 keys (the scores stay in TMEM and are read again in pass 2)
        float mx = m_run;
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 64) {
          __syncwarp();
          tmem_ld32(s_addr + c0, x0); tmem_ld32(s_addr + c0 + 32, x1);
          tc_wait_ld();
          mx = fmaxf(mx, row_max64(x0, x1));
        }
        __syncwarp();
        tmem_ld32(s_addr, x0);                     // first chunk of pass 2, in flight during the bookkeeping below
        if (k == OPK_TRACE_K && quad == 2 && lane == 0) OPK_TRACE(2, j, 2);
        // lazy rescale: adopt the new maximum only if it grew by more than 8 in the exponent domain
        const bool grow = (mx - m_run) * c2 > 8.f;   // true on the group's first tile of the item (m_run = -inf)
        const unsigned any_grow = __ballot_sync(0xffffffffu, grow);
        // P buffer and accumulator of this group were last used by the P*V of stream tile t-2
        if (t > 1 && !warp_wait(&o_done[grp], ph ^ 1u, abort_flag, lane)) { tc_wait_ld(); ok = false; break; }
        if (stage_wait) {          // ... and its second half by the other group's staged output of an earlier item
          if (!warp_wait(&stage_free[grp], stage_par, abort_flag, lane)) { tc_wait_ld(); ok = false; break; }
          stage_wait = false;
        }
        float alpha = 1.f;
        if (grow) {
          alpha = ex2_approx((m_run - mx) * c2);     // 0 when m_run = -inf
          l_run *= alpha;
          m_run = mx;
        }
        if (any_grow && !first_tile) {
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < HD; c0 += 32) {
            __syncwarp();
            tmem_ld32(o_addr + c0, x1);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) x1[i] = __float_as_uint(__uint_as_float(x1[i]) * alpha);
            tmem_st32(o_addr + c0, x1);
          }
          tc_wait_st();
        }
        first_tile = false;
        if (k == OPK_TRACE_K && quad == 2 && lane == 0) OPK_TRACE(2, j, 3);
        const float mc = m_run * c2;
        // pass 2: exp2, pack, store; the load of the next chunk is in flight while a chunk is computed
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 64) {
          tc_wait_ld();
          __syncwarp();
          tmem_ld32(s_addr + c0 + 32, x1);
          l_run += softmax_chunk(x0, c0, r, c2, mc, p_smem);
          tc_wait_ld();
          __syncwarp();
          if (c0 == 0) {
            tmem_ld32(s_addr + 64, x0);
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[grp]);   // the whole score tile has been read
          }
          l_run += softmax_chunk(x1, c0 + 32, r, c2, mc, p_smem);
        }
#endif
        if (k == OPK_TRACE_K && quad == 2 && lane == 0) OPK_TRACE(2, j, 5);
        fence_proxy_async();           // make the generic-proxy writes of P visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[grp]);
        if (k == OPK_TRACE_K && quad == 2 && lane == 0) OPK_TRACE(2, j, 6);
        if (pend) {                // the previous item's epilogue, deferred past this group's first tile of this item
          pend = false;
          if (!epilogue(pend_w, pend_k, pend_tb, pend_n, pend_m, pend_l)) { ok = false; break; }
        }
      }
      if (!ok) break;
      // This group's tiles of the item are done: publish (maximum, row sum), then run the epilogue now or defer it.
      const int n_mine = (n_kv - j0 + 1) / 2;      // tiles of this item that this group processed
      const bool owner = ((t_base + n_kv - 1) & 1) == grp;
      if (owner) {                                 // the owner's publication also vouches for the last P*V
        const int t_last = t_base + j0 + 2 * (n_mine - 1);
        if (!warp_wait(&o_done[grp], (uint32_t)((t_last >> 1) & 1), abort_flag, lane)) { ok = false; break; }
      }
      // the exchange area is rewritten only after every warp has read the previous item's values
      if (k > 0 && !warp_wait(o_free, (uint32_t)((k - 1) & 1), abort_flag, lane)) { ok = false; break; }
      xchg[grp * 128 + r] = m_run;
      xchg[256 + grp * 128 + r] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(&xr[grp * 4 + quad]);
      if (owner) {
        // before this group writes probabilities again, the other group's staged rows must have left its buffer
        stage_wait = true;
        stage_par = (uint32_t)(own_cnt & 1);
        ++own_cnt;
        if (!epilogue(w, k, t_base, n_kv, m_run, l_run)) { ok = false; break; }
      } else if (fwd_rank(k + 1, cta, G) < n_items) {
        pend = true;
        pend_w = w; pend_k = k; pend_tb = t_base; pend_n = n_kv; pend_m = m_run; pend_l = l_run;
      } else {
        if (!epilogue(w, k, t_base, n_kv, m_run, l_run)) { ok = false; break; }
      }
      t_base += n_kv;
    }
    if (HD == 128 && lane == 0) tma_store_wait_read();   // shared memory must outlive the stores' reads
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

// ------------------------------------------------------------------------------------------------ backward helpers
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

// dqkv[t][K | V columns] = bf16(sum over the G partials), summed in index order (deterministic).
__global__ void attn_dkv_reduce_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ dqkv, int T, int G,
                                       int kvw, long long ld, int k_col0) {
  // eight columns per thread and step: 2 * G independent 16-byte loads in flight, one 16-byte store
  const long long n8 = (long long)T * (kvw / 8) * 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const int which = (int)(i / ((long long)T * (kvw / 8)));          // 0 = dK, 1 = dV
    const long long rem = i - (long long)which * T * (kvw / 8);
    const int t = (int)(rem / (kvw / 8)), c = (int)(rem % (kvw / 8)) * 8;
    const float* src = part + ((long long)which * G * T + t) * kvw + c;
    float4 a = __ldcs(reinterpret_cast<const float4*>(src));
    float4 b = __ldcs(reinterpret_cast<const float4*>(src) + 1);
    for (int gq = 1; gq < G; ++gq) {
      const float4 x = __ldcs(reinterpret_cast<const float4*>(src + (long long)gq * T * kvw));
      const float4 y = __ldcs(reinterpret_cast<const float4*>(src + (long long)gq * T * kvw) + 1);
      a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
      b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
    }
    uint4 o;
    o.x = pack_bf16x2(a.x, a.y);
    o.y = pack_bf16x2(a.z, a.w);
    o.z = pack_bf16x2(b.x, b.y);
    o.w = pack_bf16x2(b.z, b.w);
    *reinterpret_cast<uint4*>(dqkv + (long long)t * ld + k_col0 + (long long)which * kvw + c) = o;
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
  // a full TMA round trip on top, so two stages leave that round trip exposed in every iteration. Pt and dSt are
  // double-buffered: the softmax warps store sub-tile i+1 while the gradient products of sub-tile i run.
  static constexpr int NS = 3;
  static constexpr int KV_TILE = 128 * HD * 2;
  static constexpr int Q_TILE = 64 * HD * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = KV_TILE;
  static constexpr int Q_OFF = 2 * KV_TILE;               // NS stages
  static constexpr int DO_OFF = Q_OFF + NS * Q_TILE;      // NS stages
  static constexpr int PT_OFF = DO_OFF + NS * Q_TILE;     // 2 x [128][64] bf16
  static constexpr int DST_OFF = PT_OFF + 2 * 16384;      // 2 x [128][64] bf16
  static constexpr int ROW_OFF = DST_OFF + 2 * 16384;     // NS stages x (64 nlse2 + 64 dsum) floats
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
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_dkv_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
                const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_part,
                const AttnParams p) {
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
  uint64_t* pd_full = st_free + 2;         // [2]
  uint64_t* pd_free = pd_full + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pd_free + 2);
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&st_full[i], 1); mbar_init(&st_free[i], kSoftmaxWarps);
      mbar_init(&pd_full[i], kSoftmaxWarps); mbar_init(&pd_free[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    // K, V and the first Q / dO sub-tile are requested before the CTA-wide set-up barrier: their latency runs under
    // the TMEM allocation.
    tma_prefetch_desc(&tm_kv); tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_do);
    mbar_expect_tx(kv_full, 2 * SM::KV_TILE);
    for (int c = 0; c < HD / 64; ++c) {
      tma_load_2d(smem + SM::K_OFF + c * 16384, &tm_kv, kv_full, k_col + c * 64, kt * 128);
      tma_load_2d(smem + SM::V_OFF + c * 16384, &tm_kv, kv_full, v_col + c * 64, kt * 128);
    }
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
      tma_prefetch_desc(&tm_part);
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
      // The score products and the gradient products are issued by two threads of different warps: a thread's
      // barrier probes queue up behind the tensor-core instructions it has issued itself, so one issuer that
      // alternates between the two kinds leaves the tensor core idle during its waits.
      for (int i = 0; i < n_it && ok; ++i) ok = scores(i);
    }
    __syncwarp();
  } else if (warp == 2 + kSoftmaxWarps) {
    if (lane == 0) {
      const uint32_t pt_s = smem_u32(smem + SM::PT_OFF), dst_s = smem_u32(smem + SM::DST_OFF);
      for (int i = 0; i < n_it; ++i) {
        const int sq = i % NS, b = i & 1;
        if (!mbar_wait(&pd_full[b], (uint32_t)((i >> 1) & 1), abort_flag)) break;
        tc_fence_after();
        const uint32_t q_s = smem_u32(smem + SM::Q_OFF + sq * SM::Q_TILE), do_s = smem_u32(smem + SM::DO_OFF + sq * SM::Q_TILE);
        // dV[keys x HD] += Pt[keys x 64 q] * dO[64 q x HD]   (B rows = queries: MN-major)
        issue_product<false, true>(tmem + DV_COL, pt_s + b * 16384, 128, do_s, 64, HD, 64, i > 0);
        issue_product<false, true>(tmem + DK_COL, dst_s + b * 16384, 128, q_s, 64, HD, 64, i > 0);
        umma_commit(&q_empty[sq]);
        umma_commit(&pd_free[b]);
      }
    }
    __syncwarp();
  } else if (warp > 2 + kSoftmaxWarps) {
    // spare warp of the common backward launch shape
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
      // buffer s of Pt / dSt was last read by the gradient products of sub-tile i-2
      if (i > 1 && !warp_wait(&pd_free[s], ph ^ 1u, abort_flag, lane)) { ok = false; break; }
      store_row32(smem + SM::PT_OFF + s * 16384, r, c0, pw);
      store_row32(smem + SM::DST_OFF + s * 16384, r, c0, dw);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pd_full[s]);
    }
    // the gradient products complete in issue order: the last one done means all done
    if (ok && warp_wait(&pd_free[(n_it - 1) & 1], (uint32_t)(((n_it - 1) >> 1) & 1), abort_flag, lane)) {
      tc_fence_after();
      if (split) {
        // fp32 partials part[dK | dV][query head of the group][t][KV * HD]: each warp stages its 32 key rows x HD/2
        // columns of both matrices in the (now dead) Q / dO ring as {32 floats, 32 rows} boxes with 128-byte swizzle
        // and stores them with TMA, which also clips the rows past T.
        constexpr int NB = HD / 64;                                  // boxes per matrix and warp
        uint8_t* stage = smem + SM::Q_OFF + (warp - 2) * (2 * NB * 4096);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const float mul = m == 0 ? p.scale : 1.f;
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            uint32_t raw[32];
            __syncwarp();
            tmem_ld32(tmem + lane_base + (m == 0 ? DK_COL : DV_COL) + half * (HD / 2) + b * 32, raw);
            tc_wait_ld();
            uint8_t* box = stage + (m * NB + b) * 4096 + lane * 128;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<float4*>(box + ((q ^ (lane & 7)) << 4)) =
                  make_float4(__uint_as_float(raw[4 * q]) * mul, __uint_as_float(raw[4 * q + 1]) * mul,
                              __uint_as_float(raw[4 * q + 2]) * mul, __uint_as_float(raw[4 * q + 3]) * mul);
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && kt * 128 + quad * 32 < p.T) {
#pragma unroll
          for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int b = 0; b < NB; ++b)
              tma_store_3d_nocommit(&tm_part, stage + (m * NB + b) * 4096, g * HD + half * (HD / 2) + b * 32,
                                    kt * 128 + quad * 32, m * G + (h_first % G));
          tma_store_commit();
          tma_store_wait_read();
        }
        __syncwarp();
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
// CTA = (query tile of 128 rows, head). Iterates over key tiles of 128 up to the diagonal; dQ accumulates in TMEM.
//   S = Q K^T [q x 128 keys]   dP = dO V^T [q x 128 keys]   dS = P * (dP - D) * scale   dQ += dS K
// per tile 8 + 8 + 8 `tcgen05.mma` of 128x128x16. TMEM: S double-buffered (2 x 128 columns), dP single (128), dQ 128.
// The softmax warps take their 64 dP columns into registers first and release the dP buffer at once, so dP of the
// next tile is computed under their work on this one; S of the next tile was issued even earlier.
// Shared memory (head_dim 128: 224 KB): K(i) stays resident until dQ(i) has completed, i.e. across the score products of
// tile i+1, and its refill needs a TMA round trip on top, so K has THREE stages; V(i) is dead as soon as dP(i) has
// completed and has ONE stage: V(i+1) is requested then and is first needed a whole tile later (S(i+1) goes first).
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
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_dq128_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                  const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_dq,
                  const __grid_constant__ CUtensorMap tm_o, const AttnParams p) {
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
  uint64_t* s_full = v_empty + 1;          // [2]
  uint64_t* s_free = s_full + 2;           // [2]
  uint64_t* dp_full = s_free + 2;
  uint64_t* dp_free = dp_full + 1;
  uint64_t* ds_full = dp_free + 1;
  uint64_t* ds_free = ds_full + 1;
  uint64_t* o_full = ds_free + 1;          // the O tile (parked in the dS buffer) has arrived
  uint64_t* o_read = o_full + 1;           // all softmax warps have taken their row sums of dO * O from it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_read + 1);
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
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_free[i], kSoftmaxWarps); }
    mbar_init(dp_full, 1);
    mbar_init(dp_free, kSoftmaxWarps);
    mbar_init(ds_full, kSoftmaxWarps);
    mbar_init(ds_free, 1);
    mbar_init(o_full, 1);
    mbar_init(o_read, kSoftmaxWarps);
    *abort_flag = 0;
    fence_barrier_init();
    // Q, dO and the first K tile are requested before the CTA-wide set-up barrier: their latency runs under the
    // TMEM allocation.
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_kv); tma_prefetch_desc(&tm_do);
    mbar_expect_tx(q_full, 2 * SM::Q_TILE);
    for (int c = 0; c < HD / 64; ++c) {
      tma_load_2d(smem + SM::Q_OFF + c * 16384, &tm_q, q_full, q_col + c * 64, qt * 128);
      tma_load_2d(smem + SM::DO_OFF + c * 16384, &tm_do, q_full, q_col + c * 64, qt * 128);
    }
    mbar_expect_tx(&k_full[0], SM::KV_TILE);
    for (int c = 0; c < HD / 64; ++c) tma_load_2d(smem + SM::K_OFF + c * 16384, &tm_kv, &k_full[0], k_col + c * 64, 0);
    // the O tile of these rows goes into the dS buffer, which is idle until the first score gradients are stored
    mbar_expect_tx(o_full, SM::Q_TILE);
    for (int c = 0; c < HD / 64; ++c) tma_load_2d(smem + SM::DS_OFF + c * 16384, &tm_o, o_full, q_col + c * 64, qt * 128);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t S_COL = 0, DP_COL = 256, DQ_COL = 384;   // two S buffers at 0 / 128

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_dq);
      for (int i = 1; i < n_it; ++i) {          // K(0) was requested during the set-up
        const int s = i % NS;
        if (!mbar_wait(&k_empty[s], (uint32_t)((i / NS) & 1) ^ 1u, abort_flag)) break;
        mbar_expect_tx(&k_full[s], SM::KV_TILE);
        for (int c = 0; c < HD / 64; ++c)
          tma_load_2d(smem + SM::K_OFF + s * SM::KV_TILE + c * 16384, &tm_kv, &k_full[s], k_col + c * 64, i * 128);
      }
    }
    __syncwarp();
  } else if (warp == 3 + kSoftmaxWarps) {
    // V producer, on a warp of its own: the wait for the single V stage never delays a K request
    if (lane == 0) {
      for (int i = 0; i < n_it; ++i) {
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
      bool ok = mbar_wait(q_full, 0, abort_flag);
      // S is double-buffered, dP single: S(i+1) is issued right behind dP(i) and is long complete when the softmax
      // warps get to it; dP(i+1) waits until they have taken dP(i) into registers, which is the first thing they do.
      auto scores = [&](int i) -> bool {
        const int sk = i % NS, b = i & 1;
        if (!mbar_wait(&k_full[sk], (i / NS) & 1, abort_flag)) return false;
        OPK_TRACE(1, i, 0);
        if (!mbar_wait(&s_free[b], (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag)) return false;   // tile i-2's scores were read
        OPK_TRACE(1, i, 1);
        tc_fence_after();
        issue_product<false, false>(tmem + S_COL + b * 128, q_s, 128, smem_u32(smem + SM::K_OFF + sk * SM::KV_TILE), 128, 128, HD, false);
        umma_commit(&s_full[b]);
        OPK_TRACE(1, i, 2);
        if (!mbar_wait(v_full, i & 1, abort_flag)) return false;
        if (!mbar_wait(dp_free, (uint32_t)(i & 1) ^ 1u, abort_flag)) return false;           // tile i-1's dP is in registers
        OPK_TRACE(1, i, 3);
        tc_fence_after();
        issue_product<false, false>(tmem + DP_COL, do_s, 128, smem_u32(smem + SM::V_OFF), 128, 128, HD, false);
        umma_commit(v_empty);        // V(i) is dead once dP(i) has completed
        umma_commit(dp_full);
        OPK_TRACE(1, i, 4);
        return true;
      };
      // The score products and the dQ products are issued by two threads of different warps (a thread's barrier
      // probes queue up behind the tensor-core instructions it has issued itself).
      for (int i = 0; i < n_it && ok; ++i) ok = scores(i);
    }
    __syncwarp();
  } else if (warp == 2 + kSoftmaxWarps) {
    if (lane == 0) {
      const uint32_t ds_s = smem_u32(smem + SM::DS_OFF);
      for (int i = 0; i < n_it; ++i) {
        const int sk = i % NS;
        if (!mbar_wait(ds_full, i & 1, abort_flag)) break;
        OPK_TRACE(0, i, 0);
        tc_fence_after();
        const uint32_t k_s = smem_u32(smem + SM::K_OFF + sk * SM::KV_TILE);
        // dQ[q x HD] += dS[q x 128 keys] * K[128 keys x HD]   (B rows = keys: MN-major)
        issue_product<false, true>(tmem + DQ_COL, ds_s, 128, k_s, 128, HD, 128, i > 0);
        umma_commit(&k_empty[sk]);
        umma_commit(ds_free);
        OPK_TRACE(0, i, 1);
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
    uint8_t* ds_chunk = smem + SM::DS_OFF + half * 16384;       // this warp's 64 keys are one 64-column chunk
    bool ok = true;
    // Row statistics of the backward pass, computed here and published for the dK/dV kernel that follows:
    //   dsum[h][t] = sum_d dO[t][d] * O[t][d]      nlse2[h][t] = -lse[h][t] * log2(e)
    // Rows t >= T (up to the padded length T64) get dsum = 0 and nlse2 = -inf, so that exp2(s * c + nlse2) is exactly
    // 0 for padded queries. Every thread sums its whole row (the two warps of a lane quarter do the same work).
    float d_r = 0.f;
    if (!warp_wait(q_full, 0, abort_flag, lane) || !warp_wait(o_full, 0, abort_flag, lane)) ok = false;
    if (ok) {
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 a = *reinterpret_cast<const uint4*>(smem + SM::DO_OFF + c * 16384 + swz_off(r, 8 * j));
          const uint4 o = *reinterpret_cast<const uint4*>(smem + SM::DS_OFF + c * 16384 + swz_off(r, 8 * j));
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[e]));
            const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ow[e]));
            d_r = fmaf(x.x, y.x, fmaf(x.y, y.y, d_r));
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(o_read);
    const float nl_r = qvalid ? -p.lse[(long long)h * p.T + qrow] * 1.4426950408889634f : -INFINITY;   // invalid rows give P = 0
    if (!qvalid) d_r = 0.f;
    if (half == 0 && qrow < p.T64) {
      const_cast<float*>(p.dsum)[(long long)h * p.T64 + qrow] = d_r;
      const_cast<float*>(p.nlse2)[(long long)h * p.T64 + qrow] = nl_r;
    }
    for (int i = 0; i < n_it && ok; ++i) {
      const int b = i & 1;
      if (warp == 2 && lane == 0) OPK_TRACE(2, i, 0);
      if (!warp_wait(dp_full, i & 1, abort_flag, lane)) { ok = false; break; }
      if (warp == 2 && lane == 0) OPK_TRACE(2, i, 1);
      tc_fence_after();
      uint32_t dw0[16], dw1[16];
      const bool masked = (i == qt);              // the tile on the causal diagonal
      {
        // dP first, all 64 columns of this warp at once: the single dP buffer is free for tile i+1 right away
        uint32_t draw0[32], draw1[32], sraw[32];
        __syncwarp();
        tmem_ld32(tmem + lane_base + DP_COL + c0, draw0);
        tmem_ld32(tmem + lane_base + DP_COL + c0 + 32, draw1);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dp_free);
        if (warp == 2 && lane == 0) OPK_TRACE(2, i, 2);
        if (!warp_wait(&s_full[b], (uint32_t)((i >> 1) & 1), abort_flag, lane)) { ok = false; break; }
        tc_fence_after();
        __syncwarp();
        tmem_ld32(tmem + lane_base + S_COL + b * 128 + c0, sraw);
        tc_wait_ld();
        if (masked) dq_chunk<true>(sraw, draw0, c2, nl_r, d_r, r - c0, dw0);
        else dq_chunk<false>(sraw, draw0, c2, nl_r, d_r, 0, dw0);
        __syncwarp();
        tmem_ld32(tmem + lane_base + S_COL + b * 128 + c0 + 32, sraw);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[b]);    // all of this warp's scores are in registers
        if (warp == 2 && lane == 0) OPK_TRACE(2, i, 3);
        if (masked) dq_chunk<true>(sraw, draw1, c2, nl_r, d_r, r - (c0 + 32), dw1);
        else dq_chunk<false>(sraw, draw1, c2, nl_r, d_r, 0, dw1);
      }
      if (warp == 2 && lane == 0) OPK_TRACE(2, i, 4);
      if (i > 0 && !warp_wait(ds_free, (i - 1) & 1, abort_flag, lane)) { ok = false; break; }
      if (i == 0 && !warp_wait(o_read, 0, abort_flag, lane)) { ok = false; break; }   // the O tile is no longer needed
      if (warp == 2 && lane == 0) OPK_TRACE(2, i, 5);
      store_row32(ds_chunk, r, 0, dw0);
      store_row32(ds_chunk, r, 32, dw1);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
      if (warp == 2 && lane == 0) OPK_TRACE(2, i, 6);
    }
    if (ok && warp_wait(ds_free, (n_it - 1) & 1, abort_flag, lane)) {
      tc_fence_after();
      if (HD == 128) {
        // this warp's 32 rows x 64 columns are staged in the (now dead) dS buffer in the swizzled row layout and
        // leave with one TMA store, which clips the rows past T
        uint8_t* chunk = smem + SM::DS_OFF + half * 16384;
#pragma unroll
        for (int cc = 0; cc < 64; cc += 32) {
          uint32_t raw[32];
          __syncwarp();
          tmem_ld32(tmem + lane_base + DQ_COL + half * 64 + cc, raw);
          tc_wait_ld();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(raw[8 * q + 0]) * p.scale, __uint_as_float(raw[8 * q + 1]) * p.scale);
            o.y = pack_bf16x2(__uint_as_float(raw[8 * q + 2]) * p.scale, __uint_as_float(raw[8 * q + 3]) * p.scale);
            o.z = pack_bf16x2(__uint_as_float(raw[8 * q + 4]) * p.scale, __uint_as_float(raw[8 * q + 5]) * p.scale);
            o.w = pack_bf16x2(__uint_as_float(raw[8 * q + 6]) * p.scale, __uint_as_float(raw[8 * q + 7]) * p.scale);
            *reinterpret_cast<uint4*>(chunk + swz_off(r, cc + q * 8)) = o;
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && qt * 128 + quad * 32 < p.T) {
          tma_store_2d(&tm_dq, chunk + quad * 32 * 128, q_col + half * 64, qt * 128 + quad * 32);
          tma_store_wait_read();
        }
        __syncwarp();
      } else {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.dqkv) + (long long)qrow * p.ld + q_col + half * (HD / 2);
        store_acc_rows<HD / 2>(tmem + lane_base + DQ_COL + half * (HD / 2), dst, qvalid, p.scale);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

}  // namespace opk
