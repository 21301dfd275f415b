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
// A descriptor depends only on (address, extents, box, swizzle), and callers hand the library the same buffers
// step after step (a training loop's allocator returns the same blocks), so every host thread keeps the last
// few it built: encoding one costs a driver call, looking one up a few compares.
struct MapKey {
  const void* ptr; int64_t a, b; int kind, c, d, e;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && a == o.a && b == o.b && kind == o.kind && c == o.c && d == o.d && e == o.e; }
};
struct MapCache {
  static constexpr int N = 48;
  MapKey key[N];
  CUtensorMap map[N];
  int used = 0, next = 0;
  const CUtensorMap* find(const MapKey& k) const {
    for (int i = 0; i < used; ++i) if (key[i] == k) return &map[i];
    return nullptr;
  }
  void put(const MapKey& k, const CUtensorMap& m) {
    const int i = used < N ? used++ : (next = (next + 1) % N);
    key[i] = k; map[i] = m;
  }
};
inline MapCache& map_cache() { static thread_local MapCache c; return c; }

// (B,T,H,128) array seen as 3-d (d, h, b*T + t); box = (box_cols, 1, box_rows); float32 or bf16.
inline int make_map_bthd(CUtensorMap* m, const void* ptr, int is_f32, int64_t B, int64_t T, int64_t H, int box_cols,
                         int swizzle128, int box_rows = 128) {
  const MapKey key{ptr, B * T, H, 1 + is_f32, box_cols, swizzle128, box_rows};
  if (const CUtensorMap* hit = map_cache().find(key)) { *m = *hit; return GLA_OK; }
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
  if (r != CUDA_SUCCESS) return GLA_ERR_LAUNCH;
  map_cache().put(key, *m);
  return GLA_OK;
}
// dense bf16 matrix of `rows` rows x 128 columns; box = (box_cols, box_rows), 128-byte swizzle.
inline int make_map_rows(CUtensorMap* m, const void* ptr, int64_t rows, int box_cols, int box_rows) {
  const MapKey key{ptr, rows, 0, 0, box_cols, box_rows, 0};
  if (const CUtensorMap* hit = map_cache().find(key)) { *m = *hit; return GLA_OK; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return GLA_ERR_NO_DEVICE;
  cuuint64_t dims[2] = {(cuuint64_t)128, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)128 * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)ptr, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return GLA_ERR_LAUNCH;
  map_cache().put(key, *m);
  return GLA_OK;
}

// float32 array (N, T, D) seen as 3-d (d, t, n); box = (128, box_rows, 1), no swizzle: the box's rows lie 512 bytes
// apart in shared memory.  Rows past T and columns past D are zero-filled by loads and skipped by stores, so a box
// never touches the next n.  D must be a multiple of 4 (strides in multiples of 16 bytes).
inline int make_map_ntd_f32(CUtensorMap* m, const void* ptr, int64_t N, int64_t T, int64_t D, int box_rows) {
  if (T > 0x7fffffffLL || D > 0x7fffffffLL || N > 0x7fffffffLL) return GLA_ERR_TOO_LARGE;
  const MapKey key{ptr, N, T, 3, (int)D, box_rows, 0};
  if (const CUtensorMap* hit = map_cache().find(key)) { *m = *hit; return GLA_OK; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return GLA_ERR_NO_DEVICE;
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)N};
  cuuint64_t strides[2] = {(cuuint64_t)D * 4, (cuuint64_t)T * D * 4};
  cuuint32_t box[3] = {128, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return GLA_ERR_LAUNCH;
  map_cache().put(key, *m);
  return GLA_OK;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device) instead of on every call.
struct SmemAttrOnce {
  unsigned long long done = 0;       // bit per device; a lost update only repeats an idempotent call
  template <typename K>
  int ensure(K kern, size_t bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return GLA_ERR_NO_DEVICE;
    if (dev >= 0 && dev < 64 && ((done >> dev) & 1ull)) return GLA_OK;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev >= 0 && dev < 64) done |= 1ull << dev;
    return GLA_OK;
  }
};


}  // namespace gla
