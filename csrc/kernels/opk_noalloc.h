// Allocation-free entry point of libopake_kernels.so.
//
// This entry point has no counterpart in the reference implementation. It exists for callers that are not allowed
// to allocate device memory at the point where they need the kernel: code running between the begin and end of a
// memory-pool snapshot, plugins embedded in a host application that owns the allocator and hands out only fixed
// input/output buffers, and late-stage error or teardown paths where cudaMalloc may fail or synchronise the device.
// Such callers can still pass inputs and outputs, but cannot provide (or size) scratch space.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest vocabulary the built-in scratch table covers (one int32 per vocabulary entry = 1 MiB, held by every GPU that
// loads the library until the process exits).
#define OPK_NOALLOC_MAX_VOCAB 262144

// Same computation as opk_embedding_bwd_compact (per-example embedding gradient summed onto the row of each token's
// first occurrence), but the first-occurrence table lives in a static device array inside the library instead of a
// caller-provided scratch buffer.
//
//   tok   int32 [T]      token ids; an id outside [0, vocab) is skipped (rep[t] = -1, no row written)
//   dx    bf16  [T][D]   gradient with respect to the embedding output
//   rep   int32 [T]      out: first position holding the same token
//   gc    fp32  [T][D]   out: summed rows (row rep[t] holds the sum; other rows are zero)
//   sumsq fp64  [1]      out (accumulated into; may be NULL): sum of squares of the bf16-rounded rows
//
// Returns 0 on success, -1 for invalid sizes, -2 when vocab exceeds OPK_NOALLOC_MAX_VOCAB, otherwise a cudaError_t.
// Calls no cudaMalloc / cudaFree and no allocating library routine.
//
// The device that owns `stream` must be the current device (cudaSetDevice) when the call is made: the scratch
// array is looked up per current device. The first call on a device looks up the device address of the scratch array (cudaGetSymbolAddress) and fills it
// with its idle value; make that first call before starting a stream capture. Every call shares the one scratch array
// of its device and leaves it in the idle state again, so calls must not overlap on the GPU (two streams, or two host
// threads on different streams, would race on the table).
int opk_embedding_bwd_compact_noalloc(const int32_t* tok, const void* dx, int32_t* rep, float* gc, double* sumsq, int T,
                                      int D, int vocab, void* stream);

#ifdef __cplusplus
}
#endif
