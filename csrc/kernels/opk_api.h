// C ABI of libopake_kernels.so. Every entry point takes raw device pointers and a CUDA stream, allocates
// nothing unless stated, and returns a cudaError_t-compatible int (0 = success; negative = argument error).
// The Python side (opake_b200/ops/_lib.py) binds these with ctypes.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct OpkGemmArgs {
  const void* A;       // bf16
  const void* B;       // bf16
  void* C;             // bf16 output (unused for epilogue 3)
  const void* R;       // optional residual (same layout as C)
  const void* bias;    // optional bf16 [N]
  int32_t M, N, K, batch;
  int32_t a_mn;        // 0: A is [M][K] (lda = row pitch); 1: A is [K][M]
  int32_t b_mn;        // 0: B is [N][K];                   1: B is [K][N]
  int32_t epilogue;    // GemmEpilogue
  int32_t b_batch_div; // B batch index = b / b_batch_div
  int64_t lda, ldb, ldc;                 // row pitches in elements
  int64_t strideA, strideB, strideC;     // batch strides in elements
  float alpha;
  float softcap;
  double* sumsq;       // epilogue 1
  void* act;           // epilogue 2
  int64_t ld_act;
  const int32_t* labels;  // epilogue 3/4
  float* pmax;
  float* psum;
  float* tgt;
  const float* lse;
  const float* coef;
  int32_t* err;        // device int, set to 1 if a bounded wait expired
  int32_t max_ctas;    // 0 = one per SM
} OpkGemmArgs;

int opk_gemm(const OpkGemmArgs* args, void* stream);
int opk_gemm_tiles_n(int N, int epilogue);  // number of column tiles the kernel uses (LCE partial buffers)
int opk_num_sms(void);
const char* opk_last_error(void);

#ifdef __cplusplus
}
#endif
