// Pieces shared by the tensor-core attention kernels (forward and backward): the TMA
// descriptor builder and the 16-bit pair packing.
#pragma once

#include "t5b_common.cuh"

#include <cuda.h>

namespace t5b {
namespace sm100 {

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (kBf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
    if (qres != cudaDriverEntryPointSuccess) return nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// (D, rows, H, B) view with element strides; box = one [box_rows][64 dims] sub-tile.
inline int make_tmap(CUtensorMap* map, const void* ptr, bool bf16, int HD, int box_rows, int64_t rows, int H, int B,
                     int64_t stride_row, int64_t stride_h, int64_t stride_b) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return T5B_ERR_DRIVER;
  cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)rows, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)stride_row * 2, (cuuint64_t)stride_h * 2,
                           (cuuint64_t)(B > 1 ? stride_b : (int64_t)HD) * 2};
  // unit dims may carry any stride in the caller's tensor; give them a legal one
  if (H == 1) strides[1] = (cuuint64_t)HD * 2;
  if (rows == 1) strides[0] = (cuuint64_t)HD * 2;
  cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? T5B_OK : T5B_ERR_DRIVER;
}

}  // namespace sm100
}  // namespace t5b
