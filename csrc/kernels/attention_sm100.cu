// Host side of the tcgen05 flash-attention kernels: tensor maps over the fused projection buffer and launches.
#include "attention_sm100.cuh"
#include "opk_api.h"

#include <cudaTypedefs.h>
#include <mutex>

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encoder() {
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

// {cols, rows} bf16 map with a {64, box_rows} box and 128-byte swizzle
bool map2d(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t ld, uint32_t box_rows) {
  EncodeFn enc = encoder();
  if (!enc || (reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t es[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// fp32 [slices][rows][cols] map with a {32 floats, 32 rows, 1} box and 128-byte swizzle (partial dK / dV stores)
bool map3d_f32(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t slices) {
  EncodeFn enc = encoder();
  if (!enc || (reinterpret_cast<uintptr_t>(base) & 15) || (cols * 4) % 16) return false;
  cuuint64_t dims[3] = {cols, rows, slices};
  cuuint64_t strides[2] = {cols * 4, rows * cols * 4};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t es[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <class K>
bool set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
}

}  // namespace

extern "C" int opk_attn_fwd(const void* qkv, void* out, float* lse, int T, int H, int KV, int hd, int64_t ld, int64_t ldo,
                            float scale, int32_t* err, void* stream) {
  if (T <= 0 || H <= 0 || KV <= 0 || H % KV || (hd != 64 && hd != 128)) return -1;
  if ((ldo % 8) || (reinterpret_cast<uintptr_t>(out) & 15)) return -1;
  CUtensorMap tm;
  if (!map2d(&tm, qkv, (uint64_t)(H + 2 * KV) * hd, (uint64_t)T, (uint64_t)ld, 128)) return -2;
  CUtensorMap tm_out;   // output rows leave through TMA stores of {64 columns, 32 rows} boxes (head_dim 128)
  if (!map2d(&tm_out, out, (uint64_t)H * hd, (uint64_t)T, (uint64_t)ldo, 32)) return -2;
  opk::AttnParams p{};
  p.T = T; p.H = H; p.KV = KV; p.hd = hd; p.ld = ld; p.ldo = ldo; p.out = out; p.lse = lse; p.scale = scale; p.err = err;
  // persistent CTAs, one per SM, each walking its share of the (query tile, head) items
  static const int n_sm = [] {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 0;
    return n;
  }();
  if (n_sm <= 0) return -3;
  const int n_items = ((T + 127) / 128) * H;
  const int grid = n_items < n_sm ? n_items : n_sm;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (hd == 128) {
    static bool once = set_smem(opk::attn_fwd_kernel<128>, opk::FwdSmem<128>::BYTES);
    if (!once) return -3;
    opk::attn_fwd_kernel<128><<<grid, opk::kFwdThreads, opk::FwdSmem<128>::BYTES, st>>>(tm, tm_out, p);
  } else {
    static bool once = set_smem(opk::attn_fwd_kernel<64>, opk::FwdSmem<64>::BYTES);
    if (!once) return -3;
    opk::attn_fwd_kernel<64><<<grid, opk::kFwdThreads, opk::FwdSmem<64>::BYTES, st>>>(tm, tm_out, p);
  }
  return (int)cudaGetLastError();
}

extern "C" int opk_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse, float* dsum, void* dqkv,
                            float* part, int T, int H, int KV, int hd, int64_t ld, int64_t ldo, float scale, int32_t* err,
                            void* stream) {
  if (T <= 0 || H <= 0 || KV <= 0 || H % KV || (hd != 64 && hd != 128)) return -1;
  if ((ld % 8) || (ldo % 8) || (reinterpret_cast<uintptr_t>(dqkv) & 15) || (reinterpret_cast<uintptr_t>(dsum) & 15))
    return -1;
  const int T64 = (T + 63) / 64 * 64;
  const uint64_t cols = (uint64_t)(H + 2 * KV) * hd;
  CUtensorMap tm128, tm64, tmdo64, tmdo128;
  if (!map2d(&tm128, qkv, cols, (uint64_t)T, (uint64_t)ld, 128)) return -2;
  if (!map2d(&tm64, qkv, cols, (uint64_t)T, (uint64_t)ld, 64)) return -2;
  if (!map2d(&tmdo64, dout, (uint64_t)H * hd, (uint64_t)T, (uint64_t)ldo, 64)) return -2;
  if (!map2d(&tmdo128, dout, (uint64_t)H * hd, (uint64_t)T, (uint64_t)ldo, 128)) return -2;
  opk::AttnParams p{};
  p.T = T; p.H = H; p.KV = KV; p.hd = hd; p.ld = ld; p.ldo = ldo; p.lse = const_cast<float*>(lse); p.dsum = dsum;
  p.nlse2 = dsum + (long long)H * T64; p.T64 = T64;
  if (part && (reinterpret_cast<uintptr_t>(part) & 15)) return -1;
  p.part = (H > KV) ? part : nullptr;       // without grouping every CTA already owns its dK / dV tile
  const int dkv_grid = ((T + 127) / 128) * (p.part ? H : KV);
  CUtensorMap tm_o128;                      // O tiles for the row sums of dO * O (taken in the dQ kernel)
  if (!map2d(&tm_o128, out, (uint64_t)H * hd, (uint64_t)T, (uint64_t)ldo, 128)) return -2;
  CUtensorMap tm_dq;                        // dQ rows leave through TMA stores of {64 columns, 32 rows} boxes (head_dim 128)
  if (!map2d(&tm_dq, dqkv, cols, (uint64_t)T, (uint64_t)ld, 32)) return -2;
  CUtensorMap tm_part = tm128;              // placeholder when there is no partial buffer (never dereferenced then)
  if (p.part && !map3d_f32(&tm_part, p.part, (uint64_t)KV * hd, (uint64_t)T, (uint64_t)2 * (H / KV))) return -2;
  p.dout = dout; p.dqkv = dqkv; p.scale = scale; p.err = err;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(dout) & 15)) return -1;
  const int n_kt = (T + 127) / 128;
  if (hd == 128) {
    static bool once = set_smem(opk::attn_dkv_kernel<128>, opk::DkvSmem<128>::BYTES) &&
                       set_smem(opk::attn_dq128_kernel<128>, opk::Dq128Smem<128>::BYTES);
    if (!once) return -3;
    // the dQ kernel goes first: it also writes the row statistics (dsum, nlse2) that the dK/dV kernel reads
    opk::attn_dq128_kernel<128><<<n_kt * H, opk::kBwdThreads, opk::Dq128Smem<128>::BYTES, st>>>(tm128, tm128, tmdo128, tm_dq, tm_o128, p);
    opk::attn_dkv_kernel<128><<<dkv_grid, opk::kBwdThreads, opk::DkvSmem<128>::BYTES, st>>>(tm128, tm64, tmdo64, tm_part, p);
  } else {
    static bool once = set_smem(opk::attn_dkv_kernel<64>, opk::DkvSmem<64>::BYTES) &&
                       set_smem(opk::attn_dq128_kernel<64>, opk::Dq128Smem<64>::BYTES);
    if (!once) return -3;
    opk::attn_dq128_kernel<64><<<n_kt * H, opk::kBwdThreads, opk::Dq128Smem<64>::BYTES, st>>>(tm128, tm128, tmdo128, tm_dq, tm_o128, p);
    opk::attn_dkv_kernel<64><<<dkv_grid, opk::kBwdThreads, opk::DkvSmem<64>::BYTES, st>>>(tm128, tm64, tmdo64, tm_part, p);
  }
  if (p.part) {
    const int kvw = KV * hd;
    const long long n8 = (long long)T * (kvw / 8) * 2;
    const unsigned blocks = (unsigned)((n8 + 255) / 256 < 148 * 8 ? (n8 + 255) / 256 : 148 * 8);
    opk::attn_dkv_reduce_kernel<<<blocks, 256, 0, st>>>(p.part, reinterpret_cast<__nv_bfloat16*>(dqkv), T, H / KV, kvw, ld,
                                                         H * hd);
  }
  return (int)cudaGetLastError();
}
