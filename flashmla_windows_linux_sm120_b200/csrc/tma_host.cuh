// Host-side construction of TMA tensor maps (driver entry point fetched through the runtime, so
// that the library does not link libcuda directly).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace fmla {
namespace tmah {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// bf16 tensor [tokens][heads][d] with element strides (stride_t, stride_h, 1);
// box = `box_rows` tokens x 64 columns of one head, 128-byte swizzle, zero fill outside the tensor
inline bool make_map_thd(CUtensorMap* m, const void* base, int d, int heads, int tokens, int64_t stride_h, int64_t stride_t,
                         int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(tokens)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(stride_h) * 2, static_cast<cuuint64_t>(stride_t) * 2};
  cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tmah
}  // namespace fmla
