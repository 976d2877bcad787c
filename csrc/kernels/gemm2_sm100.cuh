// Two-CTA (cta_group::2) variant of the bf16 GEMM: a cluster of two CTAs on a pair of SMs computes one 256 x 256
// output tile per step. Each CTA stages its own 128 rows of A and its own 128 columns of B (32 KB per pipeline stage
// instead of 48 KB for a 128 x 256 tile), the even CTA of the pair issues tcgen05.mma.cta_group::2 instructions that
// read both CTAs' shared memory, and each CTA ends up with the accumulator of its own 128 rows (all 256 columns) in
// its own TMEM. Per tensor-core cycle this halves the shared-memory and TMA traffic of the B operand, which is what
// limits the single-CTA kernel.
//
// Roles per CTA: warp 0 = TMA producer (both CTAs; every load reports its bytes to the EVEN CTA's `full`
// barrier), warp 1 = TMEM allocation (both) and MMA issue (even CTA only), warps 2.. = epilogue (both; they
// release the accumulator buffer by arriving on the even CTA's `tempty` barrier). tcgen05.commit with a CTA mask
// signals the barriers at the same offset in both CTAs. All mbarrier waits are bounded as in the single-CTA kernel;
// the loads are ordinary tile loads that each CTA issues for its own shared memory.
#pragma once
#include "gemm_sm100.cuh"

namespace opk {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_out, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Tile load into this CTA's shared memory whose completion bytes are counted on the barrier at `bar_cluster_addr`
// (a shared::cluster address: the even CTA's barrier).
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}
// Arrives (once all earlier MMAs of this thread have completed) on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}

struct Gemm2Cfg {
  static constexpr int BM = 128;            // rows per CTA (256 per pair)
  static constexpr int BN = 256;            // columns per pair; each CTA stages BN / 2 of them
  static constexpr int BK = 64;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;          // 32 KB
  static constexpr int STAGES = 7;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 2 * BN;                        // two accumulator buffers
};

constexpr int kStageWarps = 8;     // copier warps per CTA of the staged variant

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <bool A_MN, bool B_MN, int EPI, bool STAGE = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(64 + 32 * gemm_epi_warps(EPI) + (STAGE ? 32 * kStageWarps : 0), 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  using Cfg = Gemm2Cfg;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);   // used in the even CTA
  uint64_t* empty = full + STAGES;                                                  // one set per CTA
  uint64_t* tfull = empty + STAGES;                                                 // one set per CTA
  uint64_t* tempty = tfull + 2;                                                     // used in the even CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);      // one arm (expect_tx) by the even CTA's producer, bytes from both CTAs
      mbar_init(&empty[s], 1);     // one commit per use
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 2 * gemm_epi_warps(EPI));    // the epilogue warps of both CTAs
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  cluster_sync_all();              // barriers of both CTAs are initialised before anyone signals a peer
  if (warp == 1) {
    tmem_alloc2(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + BN - 1) / BN;
  const int per_batch = tiles_m * tiles_n;
  const int total = per_batch * p.batch;
  const int kblocks = (p.K + BK - 1) / BK;
  const int n_clusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int have_band = -1;
      for (int tile = cluster_id; tile < total && ok; tile += n_clusters) {
        const int b = tile / per_batch;
        const int r = tile - b * per_batch;
        int tm, tn;
        tile_coords(r, tiles_m, tiles_n, tm, tn);
        if (STAGE && tn / kRasterBand > have_band) {
          // the band's rows of B must have been copied into the local scratch by the copier warps of every CTA
          const int band = tn / kRasterBand;
          const int* ready = p.stage_ready + band;
          const long long t0 = clock64();
          while (ld_acquire_gpu(ready) < (int)gridDim.x) {
            if (*abort_flag || clock64() - t0 > kWaitBudgetCycles) { *abort_flag = 1; ok = false; break; }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy stores -> TMA (async proxy) loads
          have_band = band;
        }
        const int bb = b / p.b_batch_div;
        const int row0 = tm * 2 * BM + (int)rank * BM;          // this CTA's rows of A
        const int col0 = tn * BN + (int)rank * (BN / 2);        // this CTA's columns of B
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          const uint32_t full_leader = mapa_u32(smem_u32(&full[s]), 0);
          if (leader) mbar_expect_tx(&full[s], 2 * Cfg::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d_pair(sa + j * (BK * 128), &tmA, full_leader, row0 + j * 64, kb * BK, b);
          } else {
            tma_load_3d_pair(sa, &tmA, full_leader, kb * BK, row0, b);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 2 / 64; ++j) tma_load_3d_pair(sb + j * (BK * 128), &tmB, full_leader, col0 + j * 64, kb * BK, bb);
          } else {
            tma_load_3d_pair(sb, &tmB, full_leader, kb * BK, col0, bb);
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      for (int tile = cluster_id; tile < total && ok; tile += n_clusters, ++it) {
        const int buf = it & 1;
        const uint32_t tph = (it >> 1) & 1;
        if (!mbar_wait(&tempty[buf], tph ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            const uint64_t ad = A_MN ? make_smem_desc(sa + k4 * 2048, BK * 128, 1024) : make_smem_desc(sa + k4 * 32, 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(sb + k4 * 2048, BK * 128, 1024) : make_smem_desc(sb + k4 * 32, 16, 1024);
            umma2_bf16(d_tmem, ad, bd, idesc, (kb | k4) != 0 ? 1u : 0u);
          }
          umma2_commit_both(&empty[s]);       // frees this stage in both CTAs
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok) umma2_commit_both(&tfull[buf]);
      }
    }
    __syncwarp();
  } else if (STAGE && warp >= 2 + gemm_epi_warps(EPI)) {
    // ------------------------------------------------------------ copiers: remote B -> local scratch, band by band
    const int ctid = (warp - 2 - gemm_epi_warps(EPI)) * 32 + lane;
    const long long nthreads = (long long)gridDim.x * (32 * kStageWarps);
    const long long gtid = (long long)blockIdx.x * (32 * kStageWarps) + ctid;
    // K-major B ([N][K], a band = 2048 whole rows) or MN-major B ([K][N], a band = 2048 columns of every row)
    const int band_span = kRasterBand * BN;
    const int n_bands = (p.N + band_span - 1) / band_span;
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(p.stage_src);
    uint4* dst = reinterpret_cast<uint4*>(p.stage_dst);
    for (int band = 0; band < n_bands; ++band) {
      const int n0 = band * band_span, n1 = min(p.N, n0 + band_span);
      const int vec_per_row = B_MN ? (n1 - n0) >> 3 : p.K >> 3;     // 16-byte vectors per copied row segment
      const int n_rows = B_MN ? p.K : n1 - n0;
      const long long dst_ld = B_MN ? p.N >> 3 : p.K >> 3;           // scratch row pitch in vectors
      const long long nvec = (long long)n_rows * vec_per_row;
      constexpr int U = 8;                                     // remote loads in flight per thread
      for (long long i0 = gtid; i0 < nvec; i0 += U * nthreads) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * nthreads;
          if (i < nvec) {
            const long long rr = i / vec_per_row, cv = i % vec_per_row;
            const long long row = B_MN ? rr : n0 + rr;
            const long long col = B_MN ? n0 + cv * 8 : cv * 8;
            v[u] = __ldcg(reinterpret_cast<const uint4*>(src + row * p.stage_ld + col));
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * nthreads;
          if (i < nvec) {
            const long long rr = i / vec_per_row, cv = i % vec_per_row;
            const long long row = B_MN ? rr : n0 + rr;
            dst[row * dst_ld + (B_MN ? (n0 >> 3) + cv : cv)] = v[u];
          }
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kStageWarps) : "memory");
      if (ctid == 0) atomicAdd(p.stage_ready + band, 1);
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows each)
    const int quad = warp & 3;
    constexpr int CSPLIT = gemm_epi_warps(EPI) / 4;
    const int c_begin = ((warp - 2) >> 2) * (BN / CSPLIT), c_end = c_begin + BN / CSPLIT;
    int it = 0;
    for (int tile = cluster_id; tile < total; tile += n_clusters, ++it) {
      const int b = tile / per_batch;
      const int r = tile - b * per_batch;
      int tm, tn;
      tile_coords(r, tiles_m, tiles_n, tm, tn);
      const int buf = it & 1;
      const uint32_t tph = (it >> 1) & 1;
      if (EPI == EPI_SWIGLU_BWD) prefetch_swiglu_row<BN>(p, tm * 2 * BM + (int)rank * BM + quad * 32 + lane, tn);
      int ok = 1;
      if (lane == 0) ok = mbar_wait(&tfull[buf], tph, abort_flag) ? 1 : 0;
      __syncwarp();
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const int row = tm * 2 * BM + (int)rank * BM + quad * 32 + lane;
      const float sq_acc = epilogue_tile<BN, EPI>(p, tmem_base + (uint32_t(quad * 32) << 16) + buf * BN, row, tn, tiles_n, b,
                                                  c_begin, c_end);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[buf]), 0));
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
  cluster_sync_all();              // neither CTA frees TMEM or exits while its partner may still use its memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, 1);
}

}  // namespace opk
