// Persistent, warp-specialised bf16 GEMM for sm_100a built on tcgen05.mma with TMEM accumulators.
//
//   D[b][M][N] = sum_k A[b][m][k] * B[b'][n][k]           (fp32 accumulate in TMEM)
//
// * operands arrive through TMA into 128-byte-swizzled shared-memory tiles (4-6 stage mbarrier ring),
// * one elected thread issues 128 x BN x 16 UMMAs, the accumulator is double-buffered in TMEM so the
//   epilogue of tile i overlaps the main loop of tile i+1,
// * each operand may be K-major (reduction index contiguous in memory) or MN-major (row/column index
//   contiguous), which covers forward (X W^T), data-gradient (dY W) and weight-gradient (dY^T X)
//   products without any transposed copies,
// * the epilogue is a template hook: plain store (+bias, +residual), store + sum of squares (per-example
//   gradient norm), SwiGLU, and the two halves of a fused linear-cross-entropy.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue
// (warp w may touch TMEM lanes 32*(w%4) .. +31).
#pragma once
#include "ptx_sm100.cuh"

namespace opk {

enum GemmEpilogue : int {
  EPI_STORE = 0,    // C = alpha*acc (+bias[n]) (+R[m][n])
  EPI_SUMSQ = 1,    // C = bf16(alpha*acc); *sumsq += sum(C^2); with C == nullptr only the sum is produced
  EPI_SWIGLU = 2,   // columns interleaved (gate, up): C = raw, act[m][n/2] = silu(gate)*up
  EPI_LCE_FWD = 3,  // per-(row, column-tile) max / sum-exp partials and the target logit; no logits stored
  EPI_LCE_BWD = 4,  // C = (exp(z - lse[m]) - [n == label[m]]) * coef[m]
  EPI_SWIGLU_BWD = 5,  // acc = d(act); act = saved (gate, up) pairs [M][2N]; C[m][2n], C[m][2n+1] = d(gate), d(up)
};

struct GemmParams {
  int M, N, K, batch;
  int b_batch_div;       // B uses batch index b / b_batch_div (shared K/V heads, shared weights)
  long long ldc;         // elements
  long long strideC;     // elements between batches of C / R
  void* C;               // bf16
  const void* R;         // optional residual, same layout as C (may alias C)
  const void* bias;      // optional bf16 [N]
  float alpha;
  double* sumsq;         // EPI_SUMSQ: one accumulator per batch entry (sumsq[b])
  void* act;             // EPI_SWIGLU: bf16 [M][ld_act] (written); EPI_SWIGLU_BWD: saved pre-activations (read)
  long long ld_act;
  const int* labels;     // EPI_LCE_*: [M], negative = ignored
  float* pmax;           // EPI_LCE_FWD: [M][tiles_n]
  float* psum;           // EPI_LCE_FWD: [M][tiles_n]
  float* tgt;            // EPI_LCE_FWD: [M] target logit (written by the tile that owns the label)
  const float* lse;      // EPI_LCE_BWD: [M]
  const float* coef;     // EPI_LCE_BWD: [M] per-row scale (mask / divisor * upstream grad)
  float softcap;         // EPI_LCE_*: 0 = off, else z = cap * tanh(z / cap)
  int* err;              // set to 1 when a bounded wait expired
  // Grouped modes (mixture-of-experts), both driven by small device-side tables so that data-dependent group sizes
  // need no host synchronisation and the launch stays capturable in a CUDA graph:
  //  * tile_group[m_tile] (forward / dgrad): A and C are ONE row-grouped matrix, every 128-row tile belongs to one
  //    group; B is batched and the tile uses B[tile_group[m_tile]]; tiles marked -1 are skipped.
  //  * group_k[2*b] / group_k[2*b+1] (wgrad): first reduction element and number of 64-element blocks of batch entry
  //    b inside the un-batched operands, i.e. C[b] = A[:, k0:k0+len]^T-style reduction over that group's rows.
  const int* tile_group;
  const int* group_k;
  int sumsq_stride;      // EPI_SUMSQ accumulator index = b * sumsq_stride (0: all batch entries share sumsq[0])
  // Staged B operand (two-CTA kernel only): B lives in ANOTHER GPU's memory. Extra warps of every CTA copy it, one
  // band of column tiles at a time, into a local scratch matrix [N][K]; the TMA producers read the scratch and wait
  // per band for stage_ready[band] to reach the number of CTAs. Each remote byte crosses NVLink exactly once.
  const void* stage_src;   // remote [N][stage_ld] bf16
  long long stage_ld;
  void* stage_dst;         // local [N][K] bf16
  int* stage_ready;        // [ceil(N / (kRasterBand * BN))] counters, zero at launch
};

// Epilogue warps per CTA: four (one per TMEM lane quadrant) for the epilogues that only store; eight (two per
// quadrant, each taking half of the tile's columns) for the SwiGLU-backward epilogue, which reads and writes four
// times the bytes of a plain store per accumulator column and needs the extra loads in flight to stay hidden under
// the next tile's main loop. (With eight warps the store-only kernels measured 3-5 % slower.)
__host__ __device__ constexpr int gemm_epi_warps(int epi) { return epi == EPI_SWIGLU_BWD ? 8 : 4; }
// The single-CTA kernel serves the grouped (mixture-of-experts) modes, whose per-expert reductions are only a few
// k-blocks long while every tile is still written in full: there the epilogue, not the main loop, sets the pace.
__host__ __device__ constexpr int gemm1_epi_warps(int epi) { return epi == EPI_LCE_FWD ? 4 : 8; }

template <int BN>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int BK = 64;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = 2 * BN;
};

__device__ __forceinline__ void store_row_chunk(__nv_bfloat16* dst, const float (&v)[32], int ncols, bool vec_ok) {
  if (ncols >= 32 && vec_ok) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 o;
      o.x = pack_bf16x2(v[8 * q + 0], v[8 * q + 1]);
      o.y = pack_bf16x2(v[8 * q + 2], v[8 * q + 3]);
      o.z = pack_bf16x2(v[8 * q + 4], v[8 * q + 5]);
      o.w = pack_bf16x2(v[8 * q + 6], v[8 * q + 7]);
      d4[q] = o;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) dst[j] = __float2bfloat16(v[j]);
  }
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

// L2 prefetch of the 2 * BN saved pre-activation values (gate / up pairs) that the SwiGLU-backward epilogue of this
// thread's row will read: issued before the wait for the accumulator, so the loads later hit L2 instead of DRAM.
template <int BN>
__device__ __forceinline__ void prefetch_swiglu_row(const GemmParams& p, int row, int tn) {
  if (row < p.M) {
    const char* g = reinterpret_cast<const char*>(reinterpret_cast<const __nv_bfloat16*>(p.act) + (long long)row * p.ld_act +
                                                  2LL * tn * BN);
    const int cols = min(2 * BN, 2 * (p.N - tn * BN));
#pragma unroll
    for (int b = 0; b < 2 * BN * 2; b += 128)
      if (b < cols * 2) asm volatile("prefetch.global.L2 [%0];" ::"l"(g + b));
  }
}

// Epilogue of one accumulator tile for one thread's row: reads BN fp32 columns from TMEM (tmem_tile = lane-adjusted
// address of the tile) and applies the epilogue EPI. Returns the thread's partial sum of squares (EPI_SUMSQ).
// The tile's columns [c_begin, c_end) are handled by the calling warp (the column range is split over the epilogue
// warps that share a TMEM lane quadrant).
template <int BN, int EPI>
__device__ __forceinline__ float epilogue_tile(const GemmParams& p, uint32_t tmem_tile, int row, int tn, int tiles_n, int b,
                                               int c_begin = 0, int c_end = BN) {
  const bool row_ok = row < p.M;
  const int n0 = tn * BN;
  __nv_bfloat16* Crow = reinterpret_cast<__nv_bfloat16*>(p.C) + b * p.strideC + (long long)row * p.ldc;
  const __nv_bfloat16* Rrow =
      p.R ? reinterpret_cast<const __nv_bfloat16*>(p.R) + b * p.strideC + (long long)row * p.ldc : nullptr;
  const bool vec_ok = ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                      (((b * p.strideC) & 7) == 0);

  float sq_acc = 0.f;  // per-tile fp32 partial (256 squares per thread), flushed to fp64 below

  // LCE forward running statistics for this (row, column tile)
  float run_max = -INFINITY, run_sum = 0.f;
  int label = -1;
  float lse_row = 0.f, coef_row = 0.f;
  if (EPI == EPI_LCE_FWD || EPI == EPI_LCE_BWD) {
    if (row_ok) label = p.labels[row];
    if (EPI == EPI_LCE_BWD && row_ok) { lse_row = p.lse[row]; coef_row = p.coef[row]; }
  }

#pragma unroll 1
  for (int c0 = c_begin; c0 < c_end; c0 += 32) {
    uint32_t raw[32];
    __syncwarp();  // tcgen05.ld is warp-collective: reconverge after the predicated body below
    tmem_ld32(tmem_tile + c0, raw);
    tc_wait_ld();
    const int col0 = n0 + c0;
    const int ncols = min(32, p.N - col0);
    if (row_ok && ncols > 0) {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]) * p.alpha;

    if (EPI == EPI_STORE || EPI == EPI_SUMSQ || EPI == EPI_SWIGLU) {
      if (p.bias) {
        const __nv_bfloat16* bs = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
        for (int j = 0; j < 32; ++j) if (j < ncols) v[j] += __bfloat162float(bs[j]);
      }
      if (Rrow) {
        if (ncols >= 32 && vec_ok) {
          const uint4* r4 = reinterpret_cast<const uint4*>(Rrow + col0);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 rr = r4[q];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float2 f = __bfloat1622float2(h[e]);
              v[8 * q + 2 * e] += f.x;
              v[8 * q + 2 * e + 1] += f.y;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) if (j < ncols) v[j] += __bfloat162float(Rrow[col0 + j]);
        }
      }
      if (EPI == EPI_SUMSQ) {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (j < ncols) { float q = bf16_round(v[j]); sq_acc += q * q; }
      }
      if (EPI != EPI_SUMSQ || p.C) store_row_chunk(Crow + col0, v, ncols, vec_ok);   // EPI_SUMSQ without C: norm only
      if (EPI == EPI_SWIGLU) {
        __nv_bfloat16* arow = reinterpret_cast<__nv_bfloat16*>(p.act) + (long long)row * p.ld_act + (col0 >> 1);
        float a[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          // match the stored (bf16-rounded) pre-activations so backward recomputes the same values
          const float g = bf16_round(v[2 * j]), u = bf16_round(v[2 * j + 1]);
          a[j] = g / (1.f + __expf(-g)) * u;
        }
        const int na = ncols >> 1;
        if (na == 16 && ((p.ld_act & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.act) & 15) == 0)) {
          uint4* d4 = reinterpret_cast<uint4*>(arow);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            uint4 o;
            o.x = pack_bf16x2(a[8 * q + 0], a[8 * q + 1]);
            o.y = pack_bf16x2(a[8 * q + 2], a[8 * q + 3]);
            o.z = pack_bf16x2(a[8 * q + 4], a[8 * q + 5]);
            o.w = pack_bf16x2(a[8 * q + 6], a[8 * q + 7]);
            d4[q] = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) if (j < na) arow[j] = __float2bfloat16(a[j]);
        }
      }
    } else if (EPI == EPI_SWIGLU_BWD) {
      // 32 accumulator columns = 32 (gate, up) pairs = 64 stored columns, read and written as 8 x 16 bytes
      const __nv_bfloat16* grow = reinterpret_cast<const __nv_bfloat16*>(p.act) + (long long)row * p.ld_act + 2 * col0;
      __nv_bfloat16* drow = Crow + 2 * col0;
      const bool v2 = ncols >= 32 && vec_ok && ((p.ld_act & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.act) & 15) == 0);
      if (v2) {
        const uint4* g4 = reinterpret_cast<const uint4*>(grow);
        uint4* d4 = reinterpret_cast<uint4*>(drow);
        uint4 gin[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) gin[q] = g4[q];       // all eight loads in flight before the first use
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint4 in = gin[q];
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&in);
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 gu = __bfloat1622float2(h[e]);
            const float d = bf16_round(v[4 * q + e]);
            const float sg = 1.f / (1.f + __expf(-gu.x));
            o[e] = pack_bf16x2(d * gu.y * (sg * (1.f + gu.x * (1.f - sg))), d * (gu.x * sg));
          }
          d4[q] = make_uint4(o[0], o[1], o[2], o[3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncols) {
            const float g = __bfloat162float(grow[2 * j]), u = __bfloat162float(grow[2 * j + 1]);
            const float d = bf16_round(v[j]);
            const float sg = 1.f / (1.f + __expf(-g));
            drow[2 * j] = __float2bfloat16(d * u * (sg * (1.f + g * (1.f - sg))));
            drow[2 * j + 1] = __float2bfloat16(d * (g * sg));
          }
      }
    } else {
      if (p.softcap > 0.f) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = p.softcap * tanhf(v[j] / p.softcap);
      }
      if (EPI == EPI_LCE_FWD) {
        float cmax = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) if (j < ncols) cmax = fmaxf(cmax, v[j]);
        const float nmax = fmaxf(run_max, cmax);
        float add = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) if (j < ncols) add += __expf(v[j] - nmax);
        run_sum = run_sum * __expf(run_max - nmax) + add;
        run_max = nmax;
        if (label >= col0 && label < col0 + ncols) {
          float t = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) if (col0 + j == label) t = v[j];
          p.tgt[row] = t;
        }
      } else {  // EPI_LCE_BWD
        float d[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float pr = __expf(v[j] - lse_row);
          float g = (pr - ((col0 + j == label) ? 1.f : 0.f)) * coef_row;
          if (p.softcap > 0.f) { const float th = v[j] / p.softcap; g *= (1.f - th * th); }
          d[j] = g;
        }
        store_row_chunk(Crow + col0, d, ncols, vec_ok);
      }
    }
    }  // row_ok && ncols > 0
  }
  if (EPI == EPI_LCE_FWD && row_ok) {
    p.pmax[(long long)row * tiles_n + tn] = run_max;
    p.psum[(long long)row * tiles_n + tn] = run_sum;
  }
  return sq_acc;
}

// Tile order of the persistent schedule. Column tiles are walked in bands of kRasterBand; inside a band the column
// index runs fastest, then the row index. The CTAs that run at the same time therefore cover a roughly square patch
// of the output (8 column tiles x as many row tiles as there are CTAs / 8): the band's B tiles and the patch's A tiles
// stay in L2 and each operand is fetched from DRAM about once per band instead of once per column tile.
constexpr int kRasterBand = 8;
__device__ __forceinline__ void tile_coords(int r, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int band_tiles = kRasterBand * tiles_m;
  const int band = r / band_tiles;
  const int rr = r - band * band_tiles;
  const int w = min(kRasterBand, tiles_n - band * kRasterBand);
  tm = rr / w;
  tn = band * kRasterBand + (rr - tm * w);
}

template <bool A_MN, bool B_MN, int BN, int EPI>
__global__ void __launch_bounds__(64 + 32 * gemm1_epi_warps(EPI), 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int BM = Cfg::BM, BK = Cfg::BK, STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], gemm1_epi_warps(EPI));
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int per_batch = tiles_m * tiles_n;
  const int total = per_batch * p.batch;
  const int kblocks = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int b = tile / per_batch;
        const int r = tile - b * per_batch;
        int tm, tn;
        tile_coords(r, tiles_m, tiles_n, tm, tn);
        int bb = b / p.b_batch_div, ba = b;
        int kb0 = 0, nkb = kblocks;
        if (p.tile_group) {
          bb = p.tile_group[tm];
          if (bb < 0) continue;
        }
        if (p.group_k) { kb0 = p.group_k[2 * b] / BK; nkb = p.group_k[2 * b + 1]; ba = 0; bb = 0; }
        for (int kq = 0; kq < nkb; ++kq) {
          const int kb = kb0 + kq;
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d(sa + j * (BK * 128), &tmA, &full[s], tm * BM + j * 64, kb * BK, ba);
          } else {
            tma_load_3d(sa, &tmA, &full[s], kb * BK, tm * BM, ba);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(sb + j * (BK * 128), &tmB, &full[s], tn * BN + j * 64, kb * BK, bb);
          } else {
            tma_load_3d(sb, &tmB, &full[s], kb * BK, tn * BN, bb);
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        int nkb = kblocks;
        if (p.tile_group || p.group_k) {
          const int b = tile / per_batch;
          const int r = tile - b * per_batch;
          int tm, tn;
          tile_coords(r, tiles_m, tiles_n, tm, tn);
          if (p.tile_group && p.tile_group[tm] < 0) continue;
          if (p.group_k) nkb = p.group_k[2 * b + 1];
        }
        const int buf = it & 1;
        const uint32_t tph = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tempty[buf], tph ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            const uint64_t ad = A_MN ? make_smem_desc(sa + k4 * 2048, BK * 128, 1024)
                                     : make_smem_desc(sa + k4 * 32, 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(sb + k4 * 2048, BK * 128, 1024)
                                     : make_smem_desc(sb + k4 * 32, 16, 1024);
            umma_bf16(d_tmem, ad, bd, idesc, (kb | k4) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // frees the smem stage once these UMMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok) umma_commit(&tfull[buf]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (one TMEM lane quadrant per warp & 3)
    const int quad = warp & 3;
    constexpr int CSPLIT = gemm1_epi_warps(EPI) / 4;
    const int c_begin = ((warp - 2) >> 2) * (BN / CSPLIT), c_end = c_begin + BN / CSPLIT;
    int it = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      const int b = tile / per_batch;
      const int r = tile - b * per_batch;
      int tm, tn;
      tile_coords(r, tiles_m, tiles_n, tm, tn);
      if (p.tile_group && p.tile_group[tm] < 0) continue;
      const int buf = it & 1;
      const uint32_t tph = (it >> 1) & 1;
      ++it;
      if (EPI == EPI_SWIGLU_BWD) prefetch_swiglu_row<BN>(p, tm * BM + quad * 32 + lane, tn);
      int ok = 1;
      if (lane == 0) ok = mbar_wait(&tfull[buf], tph, abort_flag) ? 1 : 0;
      __syncwarp();   // orders the other lanes' accesses after lane 0's acquire (a shuffle is no memory barrier)
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();

      const int row = tm * BM + quad * 32 + lane;
      const float sq_acc = epilogue_tile<BN, EPI>(p, tmem_base + (uint32_t(quad * 32) << 16) + buf * BN, row, tn, tiles_n, b,
                                                  c_begin, c_end);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
      if (EPI == EPI_SUMSQ) {
        float w = sq_acc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
        if (lane == 0) atomicAdd(&p.sumsq[b * p.sumsq_stride], (double)w);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

}  // namespace opk
