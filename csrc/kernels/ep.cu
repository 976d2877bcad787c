// Expert-parallel dispatch and combine over peer memory (NVLink loads / stores), one process per GPU.
//
// The experts of a mixture-of-experts layer are sharded over W ranks (E / W each). Every rank routes its own tokens;
// entry n = (token, slot) must reach the rank that owns its expert, be processed there by the grouped tcgen05 GEMMs,
// and come back weighted. A library all-to-all needs the split sizes on the host (a device-to-host copy and a
// synchronisation per layer), a second all-to-all for the rows and separate permutation kernels on both sides. Here
// each of the two exchanges is ONE kernel that does the permutation and the transfer together:
//
//   count     histogram of this rank's routing + stable rank of every entry inside its expert; the histogram is stored
//             into every peer's control block, then a flag is raised there.
//   dispatch  waits (bounded) for all histograms, derives the global row layout that every rank computes identically,
//             and STORES each entry's row straight into its slot of the owner's receive buffer over NVLink (the
//             gather by expert and the all-to-all are the same store). Raises a flag on every peer when done.
//   prepare   owner side: waits (bounded) for every source's flag, builds the tile -> expert table and the reduction
//             ranges of the grouped GEMM modes, and the row -> source table used for per-example clipping.
//   combine   waits (bounded) for the owners' "outputs ready" flags and LOADS each entry's output row from the owner's
//             buffer over NVLink while forming the weighted sum over the k slots (+ residual) in registers.
//
// Row layout on the owner of local expert el: experts in order, inside an expert the groups of the source ranks in
// rank order; a group holds count rows padded to a multiple of 64 (at least 64), an expert segment is padded to a
// multiple of 128. So every 128-row tile belongs to one expert, every (expert, source) group is a whole number of
// 64-row reduction blocks (the weight gradient of ONE source example restricted to one expert is one batch entry of
// the grouped weight-gradient GEMM, which is what per-example clipping needs), and padding rows are zero.
//
// Nothing data-dependent reaches the host, launch shapes are static (buffers sized for the worst case), and every
// wait gives up after a cycle budget and reports through the error word instead of spinning forever.
// The reference has no expert parallelism (single-device MoE: packages/opake-patches/src/opake/api/patches/kernels/
// fused_moe.py); the protocol and its per-example clipping are specified by parallel/expert_parallel.py.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "opk_api.h"
#include "debug_bounds.cuh"

namespace {

constexpr int MAX_E = 256;
constexpr int MAX_W = OPK_EP_MAX_RANKS;
constexpr int N_PHASES = OPK_EP_PHASES;
constexpr long long kWaitBudget = 4000000000LL;   // about 2 s

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// control block of one rank (int32): counts[W][E], flags[N_PHASES][MAX_W], done counter
__device__ __forceinline__ int* ctrl_counts(void* ctrl) { return reinterpret_cast<int*>(ctrl); }
__device__ __forceinline__ int* ctrl_flags(void* ctrl, int W, int E, int phase) {
  return reinterpret_cast<int*>(ctrl) + W * E + phase * MAX_W;
}
__device__ __forceinline__ int* ctrl_done(void* ctrl, int W, int E) {
  return reinterpret_cast<int*>(ctrl) + W * E + N_PHASES * MAX_W;
}

__device__ __forceinline__ int gpad(int c) { return c <= 64 ? 64 : (c + 63) / 64 * 64; }

// Threads 0..W-1 of the CTA each wait for one source's flag; returns (to every thread) whether all arrived.
__device__ __forceinline__ int abs_epoch(const OpkEpGroup& g, int phase, int epoch) {
  return g.epoch_base ? epoch + __ldcg(g.epoch_base + (phase == OPK_EP_PHASE_BARRIER ? 1 : 0)) : epoch;
}

__device__ bool wait_phase_all(const OpkEpGroup& g, int phase, int epoch) {
  int ok = 1;
  if (phase >= 0) epoch = abs_epoch(g, phase, epoch);
  if (phase >= 0 && (int)threadIdx.x < g.world) {
    const int* f = ctrl_flags(g.ctrl[g.rank], g.world, g.n_experts, phase) + threadIdx.x;
    if (ld_acquire_sys(f) < epoch) {
      const long long t0 = clock64();
      while (ld_acquire_sys(f) < epoch) {
        if (clock64() - t0 > kWaitBudget) { ok = 0; break; }
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

// Raises flag[phase][my rank] = epoch on every rank. Called by one thread after a system-scope fence.
__device__ void signal_all(const OpkEpGroup& g, int phase, int epoch) {
  epoch = abs_epoch(g, phase, epoch);
  for (int r = 0; r < g.world; ++r) st_release_sys(ctrl_flags(g.ctrl[r], g.world, g.n_experts, phase) + g.rank, epoch);
}

// ------------------------------------------------------------------------------------------------ count
// One CTA, one pass over the entries. Warp w owns the contiguous chunk w of the entry list: (1) per-warp histograms
// in shared memory, (2) per expert an exclusive prefix over the warps, which is the rank of the warp's first entry of
// that expert, (3) every warp walks its chunk in order, 32 entries at a time; lanes with the same expert find each
// other with match.any, their rank is the warp's running count plus the number of lower lanes in the match group.
__global__ void __launch_bounds__(1024) ep_count_kernel(const OpkEpGroup g, const int* __restrict__ idx, int n_entries,
                                                        int* __restrict__ entry_rank, int epoch) {
  __shared__ int hist[32][MAX_E];     // [warp][expert]; becomes the running rank base of the warp
  __shared__ int counts[MAX_E];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int E = g.n_experts;
  for (int i = threadIdx.x; i < 32 * MAX_E; i += blockDim.x) (&hist[0][0])[i] = 0;
  __syncthreads();
  const int chunk = ((n_entries + 31) / 32 + 31) / 32 * 32;   // entries per warp, a multiple of 32
  const int c0 = warp * chunk, c1 = min(c0 + chunk, n_entries);
  // an expert id outside [0, E) is dropped (no row is sent for it, its position becomes -1 in dispatch)
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
  for (int base = c0; base < c1; base += 32) {
    const int n = base + lane;
    const bool valid = n < c1 && (unsigned)idx[n < c1 ? n : c0] < (unsigned)E;
    if (n < c1 && !valid) entry_rank[n] = 0;
    const int e = valid ? idx[n] : -1 - lane;                 // invalid lanes match nobody
    const unsigned m = __match_any_sync(0xffffffffu, e);
    if (valid) {
      const int before = __popc(m & ((1u << lane) - 1u));
      entry_rank[n] = hist[warp][e] + before;
    }
    __syncwarp();
    if (valid && (m >> lane) == 1u) hist[warp][e] += __popc(m);   // highest lane of each match group
    __syncwarp();
  }
  for (int i = threadIdx.x; i < E * g.world; i += blockDim.x) {
    const int r = i / E, e = i - r * E;
    ctrl_counts(g.ctrl[r])[g.rank * E + e] = counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) signal_all(g, OPK_EP_PHASE_COUNTS, epoch);
}

// ------------------------------------------------------------------------------------------------ dispatch
// Row offset, on its owner, of the group (expert e, source `src`) for every expert: base[e].
__device__ void layout_bases(const OpkEpGroup& g, const int* counts /*[W][E] local*/, int src, int* base, int* seg_scratch) {
  const int E = g.n_experts, W = g.world, El = E / W;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int before = 0, all = 0;
    for (int s = 0; s < W; ++s) {
      const int p = gpad(__ldcg(&counts[s * E + e]));
      if (s < src) before += p;
      all += p;
    }
    base[e] = before;
    seg_scratch[e] = (all + 127) / 128 * 128;
  }
  __syncthreads();
  if ((int)threadIdx.x < W) {
    int off = 0;
    for (int el = 0; el < El; ++el) {
      const int e = threadIdx.x * El + el;
      const int len = seg_scratch[e];
      seg_scratch[e] = off;
      off += len;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) base[e] += seg_scratch[e];
  __syncthreads();
}

__global__ void __launch_bounds__(256) ep_dispatch_kernel(const OpkEpGroup g, const OpkEpPeers rows,
                                                          const __nv_bfloat16* __restrict__ x, long long ldx, int k,
                                                          const float* __restrict__ entry_scale,
                                                          const int* __restrict__ idx, const int* __restrict__ entry_rank,
                                                          int* __restrict__ entry_pos, int replay, int n_entries, int D,
                                                          int wait_phase, int signal_phase, int epoch, int* err) {
  __shared__ int base[MAX_E];
  __shared__ int scratch[MAX_E];
  const int E = g.n_experts, El = E / g.world;
  bool ok = wait_phase_all(g, wait_phase, epoch);
  if (ok && !replay) {
    layout_bases(g, ctrl_counts(g.ctrl[g.rank]), g.rank, base, scratch);
    // a layout that does not fit the receive buffers is reported, never written
    if (threadIdx.x == 0) {
      int bad = 0;
      for (int e = 0; e < E; ++e) {
        const int c = __ldcg(&ctrl_counts(g.ctrl[g.rank])[g.rank * E + e]);
        if (base[e] + gpad(c) > g.r_cap) bad = 1;
      }
      scratch[0] = bad;
    }
    __syncthreads();
    if (scratch[0]) {
      if (threadIdx.x == 0 && err) atomicExch(err, 4);
      ok = false;
    }
  }
  if (ok) {
    // four (entry, 16-byte chunk) items per thread and step: their index, rank and row loads form four independent
    // dependency chains, so the latency of one chain is not what paces the stores
    const int nv = D >> 3;
    constexpr int U = 4;
    const long long total = (long long)n_entries * nv, stride = (long long)gridDim.x * blockDim.x;
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < total; i0 += U * stride) {
      uint4 v[U];
      int pos[U], cc[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        pos[u] = -1;
        if (i < total) {
          const int n = (int)(i / nv), c = (int)(i - (long long)n * nv);
          cc[u] = c;
          if (replay) {
            pos[u] = entry_pos[n];
          } else {
            const int e = idx[n];
            pos[u] = (unsigned)e < (unsigned)E ? (((e / El) << 26) | (base[e] + entry_rank[n])) : -1;
            if (c == 0) entry_pos[n] = pos[u];
          }
          v[u] = *reinterpret_cast<const uint4*>(x + (long long)(n / k) * ldx + c * 8);
          if (entry_scale) {
            const float sc = entry_scale[n];
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v[u]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(h[j]);
              h[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (pos[u] >= 0) {
          __nv_bfloat16* dst =
              reinterpret_cast<__nv_bfloat16*>(rows.p[pos[u] >> 26]) + (long long)(pos[u] & 0x3FFFFFF) * D + cc[u] * 8;
          *reinterpret_cast<uint4*>(dst) = v[u];
        }
      }
    }
  } else if (threadIdx.x == 0 && err) {
    atomicCAS(err, 0, 1);
  }
  // completion: the last CTA to finish raises this rank's flag everywhere (also after a failed wait, so that the
  // peers' own bounded waits are the only thing that decides how long they wait)
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* done = ctrl_done(g.ctrl[g.rank], g.world, E);
    if (atomicAdd(done, 1) == (int)gridDim.x - 1) {
      *done = 0;
      __threadfence_system();
      if (ok) signal_all(g, signal_phase, epoch);
    }
  }
}

// ------------------------------------------------------------------------------------------------ prepare (owner side)
__global__ void __launch_bounds__(1024) ep_prepare_kernel(const OpkEpGroup g, int wait_phase, int epoch,
                                                          int* __restrict__ tile_group, int* __restrict__ group_k_expert,
                                                          int* __restrict__ group_k_src, int* __restrict__ row_src,
                                                          int* __restrict__ rows_total, int* err) {
  __shared__ int seg_start[MAX_E + 1];
  const int E = g.n_experts, W = g.world, El = E / W;
  const int* counts = ctrl_counts(g.ctrl[g.rank]);
  if (!wait_phase_all(g, wait_phase, epoch)) {
    if (threadIdx.x == 0 && err) atomicCAS(err, 0, 1);
    return;
  }
  if (threadIdx.x == 0) {
    int off = 0;
    for (int el = 0; el < El; ++el) {
      const int e = g.rank * El + el;
      int all = 0;
      for (int s = 0; s < W; ++s) all += gpad(__ldcg(&counts[s * E + e]));
      seg_start[el] = off;
      off += (all + 127) / 128 * 128;
    }
    seg_start[El] = off;
    rows_total[0] = off;
  }
  __syncthreads();
  const int total = min(seg_start[El], g.r_cap);
  for (int r = total + threadIdx.x; r < g.r_cap; r += blockDim.x) row_src[r] = -1;
  for (int tl = total / 128 + threadIdx.x; tl < g.r_cap / 128; tl += blockDim.x) tile_group[tl] = -1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int el = warp; el < El; el += nwarps) {
    const int e = g.rank * El + el;
    const int s0 = seg_start[el], s1 = min(seg_start[el + 1], g.r_cap);
    if (lane == 0) { group_k_expert[2 * el] = s0; group_k_expert[2 * el + 1] = (s1 - s0) / 64; }
    for (int tl = s0 / 128 + lane; tl < s1 / 128; tl += 32) tile_group[tl] = el;
    int off = s0;
    for (int s = 0; s < W; ++s) {
      const int c = __ldcg(&counts[s * E + e]), p = gpad(c);
      if (lane == 0) { group_k_src[2 * (el * W + s)] = min(off, g.r_cap - 64); group_k_src[2 * (el * W + s) + 1] = p / 64; }
      for (int r = off + lane; r < min(off + p, s1); r += 32) row_src[r] = (r - off) < c ? s : -1;
      off += p;
    }
    for (int r = off + lane; r < s1; r += 32) row_src[r] = -1;
  }
}

// Zeroes the padding rows (row_src < 0) below rows_total of a row buffer.
__global__ void __launch_bounds__(256) ep_zero_pad_kernel(__nv_bfloat16* __restrict__ rows, const int* __restrict__ row_src,
                                                          const int* __restrict__ rows_total, int r_cap, int D) {
  const int nv = D >> 3;
  const int total = min(rows_total[0], r_cap);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)total * nv;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / nv), c = (int)(i - (long long)r * nv);
    if (row_src[r] < 0) *reinterpret_cast<uint4*>(rows + (long long)r * D + c * 8) = make_uint4(0, 0, 0, 0);
  }
}

// out[r] = rows[r] * scale[row_src[r]] (zeros for padding rows): clip factors folded into the weight-gradient operand.
__global__ void __launch_bounds__(256) ep_scale_rows_kernel(const __nv_bfloat16* __restrict__ rows,
                                                            const int* __restrict__ row_src, const float* __restrict__ scale,
                                                            int r_cap, int D, __nv_bfloat16* __restrict__ out) {
  const int nv = D >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)r_cap * nv;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / nv), c = (int)(i - (long long)r * nv);
    const int s = row_src[r];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (s >= 0) {
      v = *reinterpret_cast<const uint4*>(rows + (long long)r * D + c * 8);
      const float f = scale[s];
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(h[j]);
        h[j] = __floats2bfloat162_rn(a.x * f, a.y * f);
      }
    }
    *reinterpret_cast<uint4*>(out + (long long)r * D + c * 8) = v;
  }
}

__global__ void ep_signal_kernel(const OpkEpGroup g, int phase, int epoch) {
  __threadfence_system();
  if (threadIdx.x == 0) signal_all(g, phase, epoch);
}

__global__ void ep_advance_kernel(int* base, int d_epoch, int d_barrier) {
  if (threadIdx.x == 0) { base[0] += d_epoch; base[1] += d_barrier; }
}

// One CTA of 512 threads: store, fence, signal, bounded wait, ordered sum.
__global__ void __launch_bounds__(512) ep_allreduce_f64_kernel(const OpkEpGroup g, const OpkEpPeers slots,
                                                               const double* __restrict__ local, int n, int epoch,
                                                               double* __restrict__ out, int* err) {
  for (int t = threadIdx.x; t < g.world * n; t += blockDim.x) {
    const int r = t / n, i = t - r * n;
    reinterpret_cast<double*>(slots.p[r])[g.rank * 64 + i] = local[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) signal_all(g, OPK_EP_PHASE_SUMS, epoch);
  if (!wait_phase_all(g, OPK_EP_PHASE_SUMS, epoch)) {
    if (threadIdx.x == 0 && err) atomicCAS(err, 0, 1);
    return;
  }
  const volatile double* mine = reinterpret_cast<const volatile double*>(slots.p[g.rank]);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    double s = 0.0;
    for (int r = 0; r < g.world; ++r) s += mine[r * 64 + i];
    out[i] = s;
  }
}

__global__ void __launch_bounds__(32) ep_wait_kernel(const OpkEpGroup g, int phase, int epoch, int* err) {
  if (!wait_phase_all(g, phase, epoch) && threadIdx.x == 0 && err) atomicCAS(err, 0, 1);
}

// ------------------------------------------------------------------------------------------------ combine
// out[t] = residual[t] + sum_slot w[t][slot] * Y_owner[row(t, slot)], rows loaded from the owners' buffers.
__global__ void __launch_bounds__(256) ep_combine_kernel(const OpkEpGroup g, const OpkEpPeers y,
                                                         const int* __restrict__ entry_pos, const float* __restrict__ wts,
                                                         int k, const __nv_bfloat16* __restrict__ residual, int T, int D,
                                                         __nv_bfloat16* __restrict__ out, int wait_phase, int epoch, int* err) {
  if (!wait_phase_all(g, wait_phase, epoch)) {
    if (threadIdx.x == 0 && err) atomicCAS(err, 0, 1);
    return;
  }
  const int nv = D >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)T * nv;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / nv), c = (int)(i - (long long)t * nv);
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
    // the remote loads of eight slots are issued together, then summed in slot order (deterministic)
    constexpr int B = 8;
    for (int s0 = 0; s0 < k; s0 += B) {
      uint4 v[B];
      float w[B];
#pragma unroll
      for (int q = 0; q < B; ++q) {
        v[q] = make_uint4(0, 0, 0, 0);
        w[q] = 0.f;
        if (s0 + q < k) {
          const int pos = entry_pos[(long long)t * k + s0 + q];
          if (pos < 0) continue;                               // dropped entry: contributes nothing
          w[q] = wts ? wts[(long long)t * k + s0 + q] : 1.f;
          const __nv_bfloat16* src =
              reinterpret_cast<const __nv_bfloat16*>(y.p[pos >> 26]) + (long long)(pos & 0x3FFFFFF) * D + c * 8;
          v[q] = __ldcg(reinterpret_cast<const uint4*>(src));
        }
      }
#pragma unroll
      for (int q = 0; q < B; ++q) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[q]);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); acc[2 * j] += w[q] * f.x; acc[2 * j + 1] += w[q] * f.y; }
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + (long long)t * D + c * 8) = o;
  }
}

// dw[t][slot] = <dy[t], Y_owner[row(t, slot)]>; one warp per entry, rows loaded from the owners' buffers.
__global__ void __launch_bounds__(256) ep_combine_bwd_kernel(const OpkEpPeers y, const __nv_bfloat16* __restrict__ dy,
                                                             const int* __restrict__ entry_pos, int n_entries, int k, int D,
                                                             float* __restrict__ dwts) {
  const int n = (int)((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (n >= n_entries) return;
  const int pos = entry_pos[n];
  if (pos < 0) {
    if (lane == 0) dwts[n] = 0.f;
    return;
  }
  const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(dy + (long long)(n / k) * D);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const __nv_bfloat16*>(y.p[pos >> 26]) +
                                                                  (long long)(pos & 0x3FFFFFF) * D);
  float s = 0.f;
  for (int j = lane; j < (D >> 1); j += 32) {
    const float2 fa = __bfloat1622float2(a[j]);
    const unsigned raw = __ldcg(reinterpret_cast<const unsigned*>(b + j));
    const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
    s += fa.x * fb.x + fa.y * fb.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) dwts[n] = s;
}

int grid_for(long long n, int block) {
  long long b = (n + block - 1) / block;
  if (b > 148 * 8) b = 148 * 8;
  if (b < 1) b = 1;
  return (int)b;
}

bool group_ok(const OpkEpGroup* g) {
  return g && g->world >= 1 && g->world <= MAX_W && g->rank >= 0 && g->rank < g->world && g->n_experts >= g->world &&
         g->n_experts <= MAX_E && g->n_experts % g->world == 0 && g->r_cap > 0 && g->r_cap % 128 == 0 && g->r_cap < (1 << 26);
}

OPK_DEBUG_BOUNDS_UNIT();

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFM(p) reinterpret_cast<__nv_bfloat16*>(p)

extern "C" int opk_ep_ctrl_ints(int world, int n_experts) { return world * n_experts + N_PHASES * MAX_W + 8; }

extern "C" int opk_ep_rows_capacity(int world, int n_entries, int n_experts) {
  const int el = n_experts / (world > 0 ? world : 1);
  const long long r = (long long)world * n_entries + 64LL * world * el + 128LL * el;
  return (int)((r + 127) / 128 * 128);
}

extern "C" int opk_ep_count(const OpkEpGroup* g, const int32_t* idx, int n_entries, int32_t* entry_rank, int epoch, void* stream) {
  if (!group_ok(g) || n_entries < 0) return -1;
  ep_count_kernel<<<1, 1024, 0, ST(stream)>>>(*g, idx, n_entries, entry_rank, epoch);
  return (int)cudaGetLastError();
}

extern "C" int opk_ep_dispatch(const OpkEpGroup* g, const OpkEpPeers* rows, const void* x, int64_t ldx, int k,
                               const float* entry_scale, const int32_t* idx, const int32_t* entry_rank, int32_t* entry_pos,
                               int replay, int n_entries, int D, int wait_phase, int signal_phase, int epoch, int32_t* err,
                               void* stream) {
  if (!group_ok(g) || !rows || D % 8 || k < 1 || n_entries < 0 || signal_phase < 0 || signal_phase >= N_PHASES ||
      wait_phase >= N_PHASES)
    return -1;
  ep_dispatch_kernel<<<grid_for((long long)n_entries * (D / 8), 256), 256, 0, ST(stream)>>>(
      *g, *rows, BF(x), ldx, k, entry_scale, idx, entry_rank, entry_pos, replay, n_entries, D, wait_phase, signal_phase, epoch, err);
  return (int)cudaGetLastError();
}

extern "C" int opk_ep_prepare(const OpkEpGroup* g, int wait_phase, int epoch, int32_t* tile_group, int32_t* group_k_expert,
                              int32_t* group_k_src, int32_t* row_src, int32_t* rows_total, int32_t* err, void* stream) {
  if (!group_ok(g) || wait_phase >= N_PHASES) return -1;
  ep_prepare_kernel<<<1, 1024, 0, ST(stream)>>>(*g, wait_phase, epoch, tile_group, group_k_expert, group_k_src, row_src,
                                                rows_total, err);
  return (int)cudaGetLastError();
}

extern "C" int opk_ep_zero_pad(void* rows, const int32_t* row_src, const int32_t* rows_total, int r_cap, int D, void* stream) {
  if (D % 8 || r_cap <= 0) return -1;
  ep_zero_pad_kernel<<<grid_for((long long)r_cap * (D / 8), 256), 256, 0, ST(stream)>>>(BFM(rows), row_src, rows_total, r_cap, D);
  return (int)cudaGetLastError();
}

extern "C" int opk_ep_scale_rows(const void* rows, const int32_t* row_src, const float* scale, int r_cap, int D, void* out,
                                 void* stream) {
  if (D % 8 || r_cap <= 0) return -1;
  ep_scale_rows_kernel<<<grid_for((long long)r_cap * (D / 8), 256), 256, 0, ST(stream)>>>(BF(rows), row_src, scale, r_cap, D, BFM(out));
  return (int)cudaGetLastError();
}

extern "C" int opk_ep_signal(const OpkEpGroup* g, int phase, int epoch, void* stream) {
  if (!group_ok(g) || phase < 0 || phase >= N_PHASES) return -1;
  ep_signal_kernel<<<1, 32, 0, ST(stream)>>>(*g, phase, epoch);
  return (int)cudaGetLastError();
}

extern "C" int opk_ep_advance(int32_t* epoch_base, int d_epoch, int d_barrier, void* stream) {
  if (!epoch_base || d_epoch < 0 || d_barrier < 0) return -1;
  ep_advance_kernel<<<1, 32, 0, ST(stream)>>>(epoch_base, d_epoch, d_barrier);
  return (int)cudaGetLastError();
}

extern "C" int opk_ep_allreduce_f64(const OpkEpGroup* g, const OpkEpPeers* slots, const double* local, int n, int epoch, double* out,
                                    int32_t* err, void* stream) {
  if (!group_ok(g) || !slots || !local || !out || n < 1 || n > 64) return -1;
  ep_allreduce_f64_kernel<<<1, 512, 0, ST(stream)>>>(*g, *slots, local, n, epoch, out, err);
  return (int)cudaGetLastError();
}

extern "C" int opk_ep_wait(const OpkEpGroup* g, int phase, int epoch, int32_t* err, void* stream) {
  if (!group_ok(g) || phase < 0 || phase >= N_PHASES) return -1;
  ep_wait_kernel<<<1, 32, 0, ST(stream)>>>(*g, phase, epoch, err);
  return (int)cudaGetLastError();
}

extern "C" int opk_ep_combine(const OpkEpGroup* g, const OpkEpPeers* y, const int32_t* entry_pos, const float* wts, int k,
                              const void* residual, int T, int D, void* out, int wait_phase, int epoch, int32_t* err,
                              void* stream) {
  if (!group_ok(g) || !y || D % 8 || k < 1 || wait_phase >= N_PHASES) return -1;
  if (T <= 0) return 0;
  ep_combine_kernel<<<grid_for((long long)T * (D / 8), 256), 256, 0, ST(stream)>>>(*g, *y, entry_pos, wts, k, BF(residual), T, D,
                                                                                  BFM(out), wait_phase, epoch, err);
  return (int)cudaGetLastError();
}

extern "C" int opk_ep_combine_bwd(const OpkEpPeers* y, const void* dy, const int32_t* entry_pos, int n_entries, int k, int D,
                                  float* dwts, void* stream) {
  if (!y || D % 2 || k < 1) return -1;
  if (n_entries <= 0) return 0;
  ep_combine_bwd_kernel<<<(int)(((long long)n_entries * 32 + 255) / 256), 256, 0, ST(stream)>>>(*y, BF(dy), entry_pos, n_entries, k, D, dwts);
  return (int)cudaGetLastError();
}
