// Host side of the tcgen05 GEMM: builds the TMA tensor maps and launches the persistent kernel.
#include "gemm2_sm100.cuh"
#include "opk_api.h"
#include "debug_bounds.cuh"

#include <cudaTypedefs.h>
#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace {

thread_local char g_err[512] = "";
void set_err(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

// 3-D bf16 map {inner, rows, batch} with a {64, box_rows, 1} box and 128-byte swizzle.
bool make_map(CUtensorMap* m, const void* base, uint64_t inner, uint64_t rows, uint64_t batch, uint64_t ld,
              uint64_t batch_stride, uint32_t box_rows) {
  EncodeFn enc = get_encode();
  if (!enc) { set_err("cuTensorMapEncodeTiled not available"); return false; }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) { set_err("TMA operand base must be 16-byte aligned"); return false; }
  if ((ld * 2) % 16 != 0) { set_err("TMA operand row pitch must be a multiple of 8 elements"); return false; }
  if (batch > 1 && (batch_stride * 2) % 16 != 0) { set_err("TMA batch stride must be a multiple of 8 elements"); return false; }
  cuuint64_t dims[3] = {inner, rows, batch};
  cuuint64_t bs = batch > 1 ? batch_stride * 2 : rows * ld * 2;
  cuuint64_t strides[2] = {ld * 2, bs};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed (%d): inner=%llu rows=%llu batch=%llu ld=%llu", (int)r,
             (unsigned long long)inner, (unsigned long long)rows, (unsigned long long)batch, (unsigned long long)ld);
    set_err(buf);
    return false;
  }
  return true;
}

int g_num_sms = 0;
int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <bool A_MN, bool B_MN, int BN, int EPI>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const opk::GemmParams& p, int max_ctas, cudaStream_t st) {
  using Cfg = opk::GemmCfg<BN>;
  auto kern = opk::gemm_bf16_kernel<A_MN, B_MN, BN, EPI>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) { set_err(cudaGetErrorString(e)); return (int)e; }
    attr_done = true;
  }
  const int tiles = ((p.M + 127) / 128) * ((p.N + BN - 1) / BN) * p.batch;
  int grid = max_ctas > 0 ? max_ctas : num_sms();
  if (grid > tiles) grid = tiles;
  kern<<<grid, 64 + 32 * opk::gemm1_epi_warps(EPI), Cfg::SMEM_BYTES, st>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_err(cudaGetErrorString(e)); return (int)e; }
  return 0;
}

// Pair mode: eligible products (256-wide column tiles, no grouped tables, at least 256 rows) run on the two-CTA
// kernel. On by default; opk_gemm_set_pair_mode selects the single-CTA kernel (the tests run both).
int g_pair_mode = 1;
bool pair_mode() { return g_pair_mode == 1; }

template <bool A_MN, bool B_MN, int EPI, bool STAGE = false>
int launch2(const CUtensorMap& ta, const CUtensorMap& tb, const opk::GemmParams& p, int max_ctas, cudaStream_t st) {
  using Cfg = opk::Gemm2Cfg;
  auto kern = opk::gemm2_bf16_kernel<A_MN, B_MN, EPI, STAGE>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) { set_err(cudaGetErrorString(e)); return (int)e; }
    attr_done = true;
  }
  const int tiles = ((p.M + 255) / 256) * ((p.N + Cfg::BN - 1) / Cfg::BN) * p.batch;
  int grid = (max_ctas > 0 ? max_ctas : num_sms()) & ~1;   // whole CTA pairs
  if (grid < 2) grid = 2;
  if (grid > 2 * tiles) grid = 2 * tiles;
  kern<<<grid, 64 + 32 * opk::gemm_epi_warps(EPI) + (STAGE ? 32 * opk::kStageWarps : 0), Cfg::SMEM_BYTES, st>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_err(cudaGetErrorString(e)); return (int)e; }
  return 0;
}

int pick_bn(int N, int epilogue) {
  if (epilogue == opk::EPI_LCE_FWD || epilogue == opk::EPI_LCE_BWD || epilogue == opk::EPI_SWIGLU ||
      epilogue == opk::EPI_SWIGLU_BWD)
    return 256;
  return N <= 128 ? 128 : 256;
}

}  // namespace

extern "C" const char* opk_last_error(void) { return g_err; }

// ---- debug-build index checks: registry of the translation units' records (see debug_bounds.cuh)
#ifdef OPK_DEBUG_BOUNDS
namespace opk { namespace dbg {
struct Unit { ReadFn fn; const char* file; };
static Unit* units() { static Unit u[16]; return u; }       // function-local: usable from other units' static initialisers
static int& n_units() { static int n = 0; return n; }
void register_unit(ReadFn fn, const char* file) {
  if (n_units() < 16) units()[n_units()++] = Unit{fn, file};
}
}}  // namespace opk::dbg
#endif

extern "C" int opk_debug_bounds_read(int64_t* out4, char* file_out, int file_cap, int reset) {
#ifdef OPK_DEBUG_BOUNDS
  using namespace opk::dbg;
  out4[0] = out4[1] = out4[2] = out4[3] = 0;
  if (file_out && file_cap > 0) file_out[0] = 0;
  for (int i = 0; i < n_units(); ++i) {
    unsigned long long rec[4] = {0, 0, 0, 0};
    const int e = units()[i].fn(rec, reset);
    if (e != 0) { set_err(cudaGetErrorString((cudaError_t)e)); return e; }
    if (rec[0] && !out4[0]) {
      out4[1] = (int64_t)rec[1]; out4[2] = (int64_t)rec[2]; out4[3] = (int64_t)rec[3];
      if (file_out && file_cap > 0) snprintf(file_out, (size_t)file_cap, "%s", units()[i].file);
    }
    out4[0] += (int64_t)rec[0];
  }
  return 0;
#else
  (void)out4; (void)file_out; (void)file_cap; (void)reset;
  set_err("this library was built without OPK_DEBUG_BOUNDS");
  return -3;
#endif
}
extern "C" int opk_num_sms(void) { return num_sms(); }
extern "C" void opk_gemm_set_pair_mode(int on) { g_pair_mode = on ? 1 : 0; }
extern "C" int opk_gemm_get_pair_mode(void) { return pair_mode() ? 1 : 0; }
extern "C" int opk_gemm_tiles_n(int N, int epilogue) {
  const int bn = pick_bn(N, epilogue);
  return (N + bn - 1) / bn;
}

extern "C" int opk_gemm(const OpkGemmArgs* a, void* stream) {
  if (!a || a->M <= 0 || a->N <= 0 || a->K <= 0 || a->batch <= 0) { set_err("opk_gemm: bad sizes"); return -1; }
  const int bn = pick_bn(a->N, a->epilogue);
  const bool pair = bn == 256 && !a->tile_group && !a->group_k && a->M >= 256 && pair_mode();
  CUtensorMap ta, tb;
  // A: K-major -> {K, M, batch} box {64, 128}; MN-major -> {M, K, batch} box {64, 64}
  if (a->tile_group && (a->batch != 1 || a->n_groups <= 0)) { set_err("opk_gemm: tile_group needs batch == 1 and n_groups"); return -1; }
  if (a->tile_group && a->group_k) { set_err("opk_gemm: tile_group and group_k are exclusive"); return -1; }
  const int abatch = a->group_k ? 1 : a->batch;
  if (a->a_mn) {
    if (!make_map(&ta, a->A, a->M, a->K, abatch, a->lda, a->strideA, 64)) return -2;
  } else {
    if (!make_map(&ta, a->A, a->K, a->M, abatch, a->lda, a->strideA, 128)) return -2;
  }
  const int bdiv = a->b_batch_div > 0 ? a->b_batch_div : 1;
  const int bbatch = a->tile_group ? a->n_groups : (a->group_k ? 1 : (a->batch + bdiv - 1) / bdiv);
  const bool stage = a->stage_dst != nullptr;
  if (stage) {
    // B is read once over NVLink by the kernel's copier warps into stage_dst; the tensor map covers the scratch
    if (!pair || a->a_mn || (a->epilogue != opk::EPI_STORE && !(a->epilogue == opk::EPI_SWIGLU && !a->b_mn && a->act && !(a->N & 1))) ||
        a->batch != 1 || !a->stage_ready || (a->K % 8) || (a->N % 8) ||
        (a->ldb % 8) || (reinterpret_cast<uintptr_t>(a->B) & 15) || (reinterpret_cast<uintptr_t>(a->stage_dst) & 15)) {
      set_err("opk_gemm: staged B needs a plain or SwiGLU product with at least 256 rows, 256-wide tiles and 16-byte aligned rows");
      return -1;
    }
    if (a->b_mn) {
      if (!make_map(&tb, a->stage_dst, a->N, a->K, 1, a->N, 0, 64)) return -2;
    } else {
      if (!make_map(&tb, a->stage_dst, a->K, a->N, 1, a->K, 0, 128)) return -2;
    }
  } else if (a->b_mn) {
    if (!make_map(&tb, a->B, a->N, a->K, bbatch, a->ldb, a->strideB, 64)) return -2;
  } else {
    if (!make_map(&tb, a->B, a->K, a->N, bbatch, a->ldb, a->strideB, pair ? 128 : bn)) return -2;
  }
  opk::GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = a->M; p.N = a->N; p.K = a->K; p.batch = a->batch; p.b_batch_div = bdiv;
  p.ldc = a->ldc; p.strideC = a->strideC; p.C = a->C; p.R = a->R; p.bias = a->bias;
  p.alpha = a->alpha; p.sumsq = a->sumsq; p.act = a->act; p.ld_act = a->ld_act; p.labels = a->labels;
  p.pmax = a->pmax; p.psum = a->psum; p.tgt = a->tgt; p.lse = a->lse; p.coef = a->coef; p.softcap = a->softcap;
  p.err = a->err;
  p.tile_group = a->tile_group; p.group_k = a->group_k; p.sumsq_stride = a->sumsq_shared ? 0 : 1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int key = (a->a_mn ? 1 : 0) | (a->b_mn ? 2 : 0);
  const int mc = a->max_ctas;
  if (stage) {
    const int n_bands = (a->N + opk::kRasterBand * 256 - 1) / (opk::kRasterBand * 256);
    cudaError_t e = cudaMemsetAsync(a->stage_ready, 0, sizeof(int32_t) * n_bands, st);
    if (e != cudaSuccess) { set_err(cudaGetErrorString(e)); return (int)e; }
    p.stage_src = a->B; p.stage_ld = a->ldb; p.stage_dst = a->stage_dst; p.stage_ready = a->stage_ready;
    if (a->epilogue == opk::EPI_SWIGLU) return launch2<false, false, opk::EPI_SWIGLU, true>(ta, tb, p, mc, st);
    return a->b_mn ? launch2<false, true, opk::EPI_STORE, true>(ta, tb, p, mc, st)
                   : launch2<false, false, opk::EPI_STORE, true>(ta, tb, p, mc, st);
  }
  if (pair) {
    switch (a->epilogue) {
      case opk::EPI_STORE:
        if (key == 0) return launch2<false, false, opk::EPI_STORE>(ta, tb, p, mc, st);
        if (key == 2) return launch2<false, true, opk::EPI_STORE>(ta, tb, p, mc, st);
        if (key == 3) return launch2<true, true, opk::EPI_STORE>(ta, tb, p, mc, st);
        break;
      case opk::EPI_SUMSQ:
        if (!a->sumsq) { set_err("opk_gemm: sumsq pointer required"); return -1; }
        if (key == 3) return launch2<true, true, opk::EPI_SUMSQ>(ta, tb, p, mc, st);
        break;
      case opk::EPI_SWIGLU:
        if (!a->act || (a->N & 1)) { set_err("opk_gemm: swiglu needs act and even N"); return -1; }
        if (key == 0) return launch2<false, false, opk::EPI_SWIGLU>(ta, tb, p, mc, st);
        break;
      case opk::EPI_SWIGLU_BWD:
        if (!a->act || a->R || a->bias) { set_err("opk_gemm: swiglu backward needs the saved pre-activations and takes no bias / residual"); return -1; }
        if (key == 2) return launch2<false, true, opk::EPI_SWIGLU_BWD>(ta, tb, p, mc, st);
        break;
      case opk::EPI_LCE_FWD:
        if (!a->labels || !a->pmax || !a->psum || !a->tgt) { set_err("opk_gemm: lce fwd buffers required"); return -1; }
        if (key == 0) return launch2<false, false, opk::EPI_LCE_FWD>(ta, tb, p, mc, st);
        break;
      case opk::EPI_LCE_BWD:
        if (!a->labels || !a->lse || !a->coef) { set_err("opk_gemm: lce bwd buffers required"); return -1; }
        if (key == 0) return launch2<false, false, opk::EPI_LCE_BWD>(ta, tb, p, mc, st);
        break;
      default: break;
    }
    set_err("opk_gemm: unsupported (layout, epilogue) combination");
    return -3;
  }
  switch (a->epilogue) {
    case opk::EPI_STORE:
      if (key == 0) return bn == 256 ? launch<false, false, 256, opk::EPI_STORE>(ta, tb, p, mc, st)
                                     : launch<false, false, 128, opk::EPI_STORE>(ta, tb, p, mc, st);
      if (key == 2) return bn == 256 ? launch<false, true, 256, opk::EPI_STORE>(ta, tb, p, mc, st)
                                     : launch<false, true, 128, opk::EPI_STORE>(ta, tb, p, mc, st);
      if (key == 3) return bn == 256 ? launch<true, true, 256, opk::EPI_STORE>(ta, tb, p, mc, st)
                                     : launch<true, true, 128, opk::EPI_STORE>(ta, tb, p, mc, st);
      break;
    case opk::EPI_SUMSQ:
      if (!a->sumsq) { set_err("opk_gemm: sumsq pointer required"); return -1; }
      if (key == 3) return bn == 256 ? launch<true, true, 256, opk::EPI_SUMSQ>(ta, tb, p, mc, st)
                                     : launch<true, true, 128, opk::EPI_SUMSQ>(ta, tb, p, mc, st);
      break;
    case opk::EPI_SWIGLU:
      if (!a->act || (a->N & 1)) { set_err("opk_gemm: swiglu needs act and even N"); return -1; }
      if (key == 0) return launch<false, false, 256, opk::EPI_SWIGLU>(ta, tb, p, mc, st);
      break;
    case opk::EPI_SWIGLU_BWD:
      if (!a->act || a->R || a->bias) { set_err("opk_gemm: swiglu backward needs the saved pre-activations and takes no bias / residual"); return -1; }
      if (key == 2) return launch<false, true, 256, opk::EPI_SWIGLU_BWD>(ta, tb, p, mc, st);
      break;
    case opk::EPI_LCE_FWD:
      if (!a->labels || !a->pmax || !a->psum || !a->tgt) { set_err("opk_gemm: lce fwd buffers required"); return -1; }
      if (key == 0) return launch<false, false, 256, opk::EPI_LCE_FWD>(ta, tb, p, mc, st);
      break;
    case opk::EPI_LCE_BWD:
      if (!a->labels || !a->lse || !a->coef) { set_err("opk_gemm: lce bwd buffers required"); return -1; }
      if (key == 0) return launch<false, false, 256, opk::EPI_LCE_BWD>(ta, tb, p, mc, st);
      break;
    default: break;
  }
  set_err("opk_gemm: unsupported (layout, epilogue) combination");
  return -3;
}

// ------------------------------------------------------------------------------------------------ wait self-test
// One CTA waits on an mbarrier that nothing ever completes, with a short cycle budget. The wait gives up, the abort
// flag is raised and the error word is set: the same unwinding path every pipeline role of the real kernels takes
// when a producer or peer never shows up. The kernel returns normally and the context stays usable.
namespace {
__global__ void wait_selftest_kernel(int* err, long long budget_cycles, long long* waited_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    opk::mbar_init(&bar, 1);
    abort_flag = 0;
    opk::fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool ok = opk::mbar_wait(&bar, 0, &abort_flag, budget_cycles);
    if (waited_cycles) *waited_cycles = clock64() - t0;
    if (!ok && err) atomicExch(err, 1);
  }
  __syncthreads();
  // every other thread sees the flag the waiting role raised
  if (threadIdx.x == 1 && abort_flag && err) atomicOr(err, 2);
}
}  // namespace

extern "C" int opk_wait_selftest(int32_t* err, int64_t budget_cycles, int64_t* waited_cycles, void* stream) {
  if (budget_cycles <= 0 || budget_cycles > 4000000000LL) return -1;
  wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(err, budget_cycles,
                                                                           reinterpret_cast<long long*>(waited_cycles));
  return (int)cudaGetLastError();
}
