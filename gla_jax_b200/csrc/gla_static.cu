// gla_chunk_fwd_static: a forward-only chunk_gla entry point that performs no allocation.
//
// Some callers cannot hand this library a workspace because they cannot allocate device
// memory at the point of the call: code running under a framework that owns the allocator
// and forbids raw cudaMalloc (an XLA custom call, a plugin inside an inference server), or
// code inside a region where allocation is illegal or would serialise the device.  For them
// the scratch that gla_chunk_fwd takes from the caller lives here, in a fixed device array
// that every GPU holds from the moment the library is loaded on it until the process exits.
#include "gla_common.cuh"
#include <mutex>

namespace gla {

constexpr size_t kStaticScratchBytes = 32u << 20;    // 32 MiB per device

// File-scope device array.  In HOST code this name is only a handle for the runtime's symbol
// table, never a device address: the address is looked up per device below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_scratch_ptr[kMaxDevices];      // device address of the array, per device ordinal
static std::mutex g_scratch_mutex;

// Device address of this device's copy of the array; looked up once per device with that
// device current, then cached.
static int static_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda_error(e);
  if (dev < 0 || dev >= kMaxDevices) return GLA_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (p == nullptr) return GLA_ERR_NO_DEVICE;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return GLA_OK;
}

}  // namespace gla

using namespace gla;

extern "C" {

GLA_API size_t gla_chunk_fwd_static_max_bytes(void) { return kStaticScratchBytes; }

GLA_API int gla_chunk_fwd_static(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype,
                                 int impl, const void* hidden_init, const float* log_fgate, const void* value,
                                 const void* key, const void* query, void* hidden_final, void* out) {
  if (!hidden_init || !log_fgate || !value || !key || !query || !hidden_final || !out) return GLA_ERR_NULL_POINTER;
  const size_t need = gla_chunk_fwd_workspace_bytes(B, T, H, D, chunk, dtype, impl);
  if (need == 0)   // invalid or unsupported sizes: the ordinary entry point reports which, before any launch
    return gla_chunk_fwd(stream, B, T, H, D, chunk, dtype, impl, hidden_init, log_fgate, value, key, query,
                         hidden_final, out, nullptr, nullptr, 0);
  if (need > kStaticScratchBytes) return GLA_ERR_TOO_LARGE;
  void* scratch = nullptr;
  GLA_TRY(static_scratch(&scratch));
  return gla_chunk_fwd(stream, B, T, H, D, chunk, dtype, impl, hidden_init, log_fgate, value, key, query, hidden_final,
                       out, /*saved=*/nullptr, scratch, kStaticScratchBytes);
}

}  // extern "C"
