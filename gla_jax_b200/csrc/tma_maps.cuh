// Host-side construction of TMA tensor maps for the arrays of the chunk path.
#pragma once
#include "gla_common.cuh"
#include <cuda.h>

namespace gla {

// ---- TMA descriptors -------------------------------------------------------------------------
// cuTensorMapEncodeTiled is fetched through the runtime so that the library has no link-time
// dependency on libcuda (it must load on machines without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}
// (B,T,H,128) array seen as 3-d (d, h, b*T + t); box = (box_cols, 1, box_rows); float32 or bf16.
inline int make_map_bthd(CUtensorMap* m, const void* ptr, int is_f32, int64_t B, int64_t T, int64_t H, int box_cols,
                         int swizzle128, int box_rows = 128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return GLA_ERR_NO_DEVICE;
  const cuuint64_t es = is_f32 ? 4 : 2;
  cuuint64_t dims[3] = {(cuuint64_t)128, (cuuint64_t)H, (cuuint64_t)(B * T)};
  cuuint64_t strides[2] = {(cuuint64_t)128 * es, (cuuint64_t)H * 128 * es};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, 1, (cuuint32_t)box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)ptr, dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GLA_OK : GLA_ERR_LAUNCH;
}
// dense bf16 matrix of `rows` rows x 128 columns; box = (box_cols, box_rows), 128-byte swizzle.
inline int make_map_rows(CUtensorMap* m, const void* ptr, int64_t rows, int box_cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return GLA_ERR_NO_DEVICE;
  cuuint64_t dims[2] = {(cuuint64_t)128, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)128 * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)ptr, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GLA_OK : GLA_ERR_LAUNCH;
}


}  // namespace gla
