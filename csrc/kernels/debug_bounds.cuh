// Debug-build index checks for data-dependent addresses (token ids, labels, expert ids, row maps).
//
// Built with -DOPK_DEBUG_BOUNDS (the `libopake_kernels_debug.so` variant), `OPK_IDX_OK(i, n)` tests 0 <= i < n; a
// failing index is RECORDED (count, source line, index, bound of the first failure, per translation unit) and the macro
// yields false, so the caller skips the access. Nothing traps and no kernel aborts: the context stays usable and the
// host reads the record with `opk_debug_bounds_read`. In the release build the macro is the constant `true` and the
// checks cost nothing.
#pragma once
#include <cuda_runtime.h>

#ifdef OPK_DEBUG_BOUNDS
namespace opk { namespace dbg {

static __device__ unsigned long long g_rec[4];   // [failures, line of the first, its index, its bound]

__device__ __forceinline__ bool idx_ok(long long i, long long n, int line) {
  if (i >= 0 && i < n) return true;
  if (atomicAdd(&g_rec[0], 1ULL) == 0ULL) {
    g_rec[1] = (unsigned long long)line;
    g_rec[2] = (unsigned long long)i;
    g_rec[3] = (unsigned long long)n;
  }
  return false;
}

typedef int (*ReadFn)(unsigned long long* out4, int reset);
void register_unit(ReadFn fn, const char* file);     // defined once, in gemm_sm100.cu

// reads (and optionally clears) this translation unit's record; cudaGetSymbolAddress needs the symbol's own unit
static int read_unit(unsigned long long* out4, int reset) {
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_rec);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemcpy(out4, p, 4 * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return (int)e;
  if (reset) e = cudaMemset(p, 0, 4 * sizeof(unsigned long long));
  return (int)e;
}

struct Registrar {
  explicit Registrar(const char* file) { register_unit(&read_unit, file); }
};

}}  // namespace opk::dbg
#define OPK_IDX_OK(i, n) (::opk::dbg::idx_ok((long long)(i), (long long)(n), __LINE__))
#define OPK_DEBUG_BOUNDS_UNIT() static ::opk::dbg::Registrar opk_dbg_registrar_(__FILE__)
#else
#define OPK_IDX_OK(i, n) (true)
#define OPK_DEBUG_BOUNDS_UNIT() static_assert(true, "")
#endif
