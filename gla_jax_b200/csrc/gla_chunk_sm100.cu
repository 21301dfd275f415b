// tcgen05 tensor-core chunk path (placeholder until the kernels land).
#include "gla_common.cuh"
namespace gla {
bool tc_supported(int64_t, int64_t, int) { return false; }
size_t tc_saved_bytes(int64_t, int64_t, int64_t, int64_t, int64_t) { return 0; }
size_t tc_fwd_ws_bytes(int64_t, int64_t, int64_t, int64_t, int64_t) { return 0; }
size_t tc_bwd_ws_bytes(int64_t, int64_t, int64_t, int64_t, int64_t) { return 0; }
int tc_chunk_fwd(cudaStream_t, int64_t, int64_t, int64_t, int64_t, int64_t, const void*, const float*, const void*,
                 const void*, const void*, void*, void*, void*, void*, int, float*, float*) { return GLA_ERR_UNSUPPORTED; }
int tc_chunk_bwd(cudaStream_t, int64_t, int64_t, int64_t, int64_t, int64_t, const float*, const void*, const void*,
                 const void*, const void*, const void*, const void*, void*, float*, void*, void*, void*, void*) { return GLA_ERR_UNSUPPORTED; }
}  // namespace gla
