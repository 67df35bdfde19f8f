// Host helpers of the tcgen05 kernels: the driver's tensor-map encoder, looked up at run
// time so that the library does not link libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "common.h"

namespace annc {
namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 2-D fp32 tensor [rows, cols] with row pitch ld floats; box = 32 columns x box_rows rows;
// out-of-range elements read as zero.  `n_major` picks the 128-byte swizzle with 32-byte
// atoms that an N-major tf32 operand needs, else the plain 128-byte swizzle.
inline int make_map(CUtensorMap* map, const float* ptr, long long rows, long long cols, long long ld,
             int box_rows, bool n_major) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(ANNC_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
  const cuuint32_t box[2] = {32u, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  n_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ANNC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return ANNC_OK;
}

// 3-D variant for strided batches: [batch, rows, cols], box = 32 columns x box_rows rows x 1.
inline int make_map3(CUtensorMap* map, const float* ptr, long long batch, long long rows,
                     long long cols, long long ld, long long batch_stride, int box_rows,
                     bool n_major) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(ANNC_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)ld * sizeof(float),
                                 (cuuint64_t)batch_stride * sizeof(float)};
  const cuuint32_t box[3] = {32u, (cuuint32_t)box_rows, 1u};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  n_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ANNC_ERR_CUDA, "cuTensorMapEncodeTiled(3d) failed (%d)", (int)r);
  return ANNC_OK;
}

}  // namespace tc
}  // namespace annc
