// Micro-benchmark: SM cycles per `tcgen05.mma` (kind::f16, bf16 operands, M = 128) issued back to back by one thread,
// for several widths and operand sources, alone and with background traffic from four other warps (shared-memory
// stores, TMEM loads). One CTA per SM on 148 SMs; the figure is taken on CTA 0 with clock64 around 512 instructions
// plus their completion. It gives the floor that the attention and GEMM kernels are compared against: whatever a
// kernel adds to these figures is waiting, not tensor-core work.
//
// Build and run (one B200):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -Icsrc/kernels benchmarks/tcgen05_rate.cu \
//        -o benchmarks/tcgen05_rate && ./benchmarks/tcgen05_rate
#include <cstdio>
#include <cuda_runtime.h>
#include "../csrc/kernels/ptx_sm100.cuh"
using namespace opk;

__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

template <int N, bool B_MN, bool A_TMEM, int EXTRA>
__global__ void __launch_bounds__(160, 1) rate_kernel(long long* out, int iters) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // zero operands (A: 32 KB at 0, B: 64 KB at 32 KB)
  for (int i = threadIdx.x; i < (96 * 1024) / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag = 0; fence_barrier_init(); }
  if (warp == 0) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = slot;
  if (warp == 0 && lane == 0) {
    const uint32_t a_s = smem_u32(smem), b_s = smem_u32(smem + 32768);
    const uint32_t idesc = make_idesc_bf16(128, N, false, B_MN);
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int k = 0; k < 128; k += 16) {
        const uint64_t ad = make_smem_desc(a_s + (k >> 6) * 128 * 128 + (k & 63) * 2, 16, 1024);
        const uint64_t bd = B_MN ? make_smem_desc(b_s + k * 128, 128 * 128, 1024)
                                 : make_smem_desc(b_s + (k >> 6) * N * 128 + (k & 63) * 2, 16, 1024);
        if (A_TMEM) umma_bf16_ts(tmem + (it & 1) * 128, tmem + 256 + k / 2, bd, idesc, 1u);
        else umma_bf16(tmem + (it & 1) * 128, ad, bd, idesc, 1u);
      }
    }
    umma_commit(&bar);
    mbar_wait(&bar, 0, &abort_flag);
    const long long t1 = clock64();
    if (blockIdx.x == 0) out[0] = t1 - t0;
  } else if (warp >= 1 && EXTRA) {
    // optional background traffic: EXTRA=1: shared-memory stores; EXTRA=2: TMEM loads
    uint32_t x[32];
    for (int it = 0; it < iters * 4; ++it) {
      if (EXTRA == 1) {
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<uint4*>(smem + 98304 + ((threadIdx.x * 16 + q * 2048 + it * 64) & 32767)) = make_uint4(it, q, 0, 0);
      } else {
        tmem_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + 384 + (it & 1) * 32, x);
        tc_wait_ld();
        if (x[0] == 0x12345678u) out[1] = x[1];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

template <int N, bool B_MN, bool A_TMEM, int EXTRA>
void run(const char* name, long long* d_out) {
  auto kern = rate_kernel<N, B_MN, A_TMEM, EXTRA>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  const int iters = 64;
  for (int rep = 0; rep < 2; ++rep) kern<<<148, 160, 200 * 1024>>>(d_out, iters);
  cudaError_t e = cudaDeviceSynchronize();
  long long h = 0;
  cudaMemcpy(&h, d_out, 8, cudaMemcpyDeviceToHost);
  printf("%-44s %s cycles/mma %.1f\n", name, cudaGetErrorString(e), (double)h / (iters * 8));
}

int main() {
  long long* d_out;
  cudaMalloc(&d_out, 64);
  run<128, false, false, 0>("SS 128x128x16 B K-major", d_out);
  run<128, true, false, 0>("SS 128x128x16 B MN-major", d_out);
  run<256, false, false, 0>("SS 128x256x16 B K-major", d_out);
  run<64, false, false, 0>("SS 128x64x16 B K-major", d_out);
  run<128, false, true, 0>("TS 128x128x16 B K-major (A in TMEM)", d_out);
  run<128, true, true, 0>("TS 128x128x16 B MN-major (A in TMEM)", d_out);
  run<256, false, true, 0>("TS 128x256x16 B K-major (A in TMEM)", d_out);
  run<128, false, false, 1>("SS 128x128x16 + shared stores", d_out);
  run<128, false, false, 2>("SS 128x128x16 + TMEM loads", d_out);
  run<128, true, true, 2>("TS 128x128x16 B MN + TMEM loads", d_out);
  return 0;
}
