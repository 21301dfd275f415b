// C ABI of libgla_b200.so: argument validation and dispatch.  See include/gla_b200.h for
// the contract of every entry point and the reference operator it replaces.
#include <atomic>
#include "gla_common.cuh"
#include <cstdio>

namespace gla {

static thread_local int g_last_cuda_error = 0;

int record_cuda_error(cudaError_t e) {
  if (e == cudaSuccess) return GLA_OK;
  g_last_cuda_error = (int)e;
  return GLA_ERR_LAUNCH;
}

// ---- launch counter and optional per-kernel event timing (thread-local) -----------------
static std::atomic<long long> g_launches{0};   // process-wide: autograd runs backward launches on its own thread
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

struct ProfRec { const char* name; cudaEvent_t a, b; };
static thread_local bool g_prof_on = false;
static thread_local ProfRec g_prof[4096];
static thread_local int g_prof_n = 0, g_prof_created = 0;

ProfScope::ProfScope(const char* name, cudaStream_t stream) : slot(-1), st(stream) {
  if (!g_prof_on || g_prof_n >= 4096) return;
  slot = g_prof_n++;
  if (slot >= g_prof_created) {
    cudaEventCreate(&g_prof[slot].a);
    cudaEventCreate(&g_prof[slot].b);
    g_prof_created = slot + 1;
  }
  g_prof[slot].name = name;
  cudaEventRecord(g_prof[slot].a, st);
}
ProfScope::~ProfScope() {
  if (slot >= 0) cudaEventRecord(g_prof[slot].b, st);
}

static int check_dtype(int dt) { return (dt == GLA_F32 || dt == GLA_BF16) ? GLA_OK : GLA_ERR_UNSUPPORTED; }

static int check_chunk_dims(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C, int dtype) {
  if (B <= 0 || T <= 0 || H <= 0 || D <= 0 || C <= 0) return GLA_ERR_BAD_DIMS;
  if (T % C != 0 || !is_pow2(C)) return GLA_ERR_BAD_DIMS;
  if (C < 16 || C > 256 || D < 16 || D > 256 || D % 8 != 0) return GLA_ERR_UNSUPPORTED;
  return check_dtype(dtype);
}

// Resolve GLA_IMPL_AUTO; returns a negative status (as -status) if the request is invalid.  The option bits
// above the low byte are passed on to the tensor-core path as they are.
constexpr int OPT_BITS = GLA_OPT_STATE_TWO_KERNELS | GLA_OPT_STATE_ONE_PASS | GLA_OPT_NO_EARLY_START | GLA_OPT_ALL_SCALES |
                         GLA_OPT_NO_L2_PREFETCH | GLA_OPT_STATE_SEGMENTS;
static int resolve_impl(int impl_and_opts, int64_t D, int64_t C, int dtype) {
  if (impl_and_opts < 0 || (impl_and_opts & ~(0xff | OPT_BITS)) != 0) return -GLA_ERR_UNSUPPORTED;
  const int impl = impl_and_opts & 0xff;
  if (impl == GLA_IMPL_AUTO) return (tc_auto_default() && tc_supported(D, C, dtype)) ? GLA_IMPL_TCGEN05 : GLA_IMPL_FP32_SIMT;
  if (impl == GLA_IMPL_TCGEN05) return tc_supported(D, C, dtype) ? GLA_IMPL_TCGEN05 : -GLA_ERR_UNSUPPORTED;
  if (impl == GLA_IMPL_FP32_SIMT) return GLA_IMPL_FP32_SIMT;
  return -GLA_ERR_UNSUPPORTED;
}

}  // namespace gla

using namespace gla;

extern "C" {

const char* gla_status_string(int status) {
  switch (status) {
    case GLA_OK: return "ok";
    case GLA_ERR_NULL_POINTER: return "a required pointer is NULL";
    case GLA_ERR_BAD_DIMS: return "bad dimensions (sizes must be positive, T a multiple of chunk, chunk a power of two)";
    case GLA_ERR_UNSUPPORTED: return "unsupported dtype or size for this build";
    case GLA_ERR_ALIGNMENT: return "pointer not 16-byte aligned";
    case GLA_ERR_WORKSPACE: return "workspace missing or too small";
    case GLA_ERR_LAUNCH: return "CUDA launch failed (see gla_last_cuda_error)";
    case GLA_ERR_NO_DEVICE: return "no usable sm_100 device";
    case GLA_ERR_TOO_LARGE: return "size beyond a fixed maximum";
    default: return "unknown status";
  }
}

const char* gla_version(void) { return "gla_b200 0.1 (sm_100a)"; }

int gla_last_cuda_error(void) { return g_last_cuda_error; }

long long gla_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

unsigned int gla_device_wait_timeouts(void) { return tc_read_wait_timeouts() + tc_state_read_wait_timeouts() + scan_read_wait_timeouts(); }

unsigned int gla_device_bad_offsets(void) { return tc_state_read_bad_offsets(); }

void gla_profile_enable(int on) {
  g_prof_on = on != 0;
  if (on) g_prof_n = 0;
}

// Writes "name launches total_ms\n" per kernel for the launches recorded since
// gla_profile_enable(1); synchronises on the recorded events.  Returns bytes written.
size_t gla_profile_report(char* buf, size_t cap) {
  struct Agg { const char* name; int n; double ms; } agg[64];
  int na = 0;
  for (int i = 0; i < g_prof_n; ++i) {
    float ms = 0.f;
    cudaEventSynchronize(g_prof[i].b);
    cudaEventElapsedTime(&ms, g_prof[i].a, g_prof[i].b);
    int j = 0;
    for (; j < na; ++j) if (agg[j].name == g_prof[i].name) break;
    if (j == na) { if (na == 64) continue; agg[na++] = {g_prof[i].name, 0, 0.0}; }
    agg[j].n += 1; agg[j].ms += ms;
  }
  size_t off = 0;
  for (int j = 0; j < na && off + 128 < cap; ++j)
    off += (size_t)snprintf(buf + off, cap - off, "%s %d %.6f\n", agg[j].name, agg[j].n, agg[j].ms);
  g_prof_n = 0;
  if (off < cap) buf[off] = 0;
  return off;
}

int gla_cumsum(void* stream, int64_t N, int64_t T, int64_t D, const void* src, const void* init, void* dst,
               int reverse, int in_dtype, int out_dtype) {
  if (!src || !dst) return GLA_ERR_NULL_POINTER;
  if (N <= 0 || T <= 0 || D <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(in_dtype));
  GLA_TRY(check_dtype(out_dtype));
  return launch_cumsum((cudaStream_t)stream, N, T, D, src, init, dst, reverse, in_dtype == GLA_BF16,
                       out_dtype == GLA_BF16);
}

int gla_scan(void* stream, int op, int64_t N, int64_t T, int64_t D, const void* src, const void* init, void* dst,
             int reverse, int in_dtype, int out_dtype) {
  if (!src || !dst) return GLA_ERR_NULL_POINTER;
  if (N <= 0 || T <= 0 || D <= 0) return GLA_ERR_BAD_DIMS;
  if (op < GLA_SCAN_ADD || op > GLA_SCAN_LOGADDEXP) return GLA_ERR_UNSUPPORTED;
  GLA_TRY(check_dtype(in_dtype));
  GLA_TRY(check_dtype(out_dtype));
  return launch_cumsum((cudaStream_t)stream, N, T, D, src, init, dst, reverse, in_dtype == GLA_BF16,
                       out_dtype == GLA_BF16, nullptr, nullptr, op);
}

int gla_rnn_scan(void* stream, int64_t batch, int64_t T, int64_t K, int64_t V, const float* log_fgate,
                 const void* kv, const float* init_log_fgate, const void* init_kv, float* out_log,
                 void* out_state, int reverse, int last_only, int kv_dtype) {
  if (!log_fgate || !kv || !out_log || !out_state) return GLA_ERR_NULL_POINTER;
  if ((init_log_fgate == nullptr) != (init_kv == nullptr)) return GLA_ERR_NULL_POINTER;
  if (batch <= 0 || T <= 0 || K <= 0 || V <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(kv_dtype));
  return launch_rnn_scan((cudaStream_t)stream, batch, T, K, V, log_fgate, kv, init_log_fgate, init_kv, out_log,
                         out_state, reverse, last_only, kv_dtype == GLA_BF16);
}

size_t gla_rnn_scan_workspace_bytes(int64_t batch, int64_t T, int64_t K, int64_t V) {
  if (batch <= 0 || T <= 0 || K <= 0 || V <= 0) return 0;
  return rnn_scan_ws_bytes(batch, T, K, V);
}

int gla_rnn_scan_ws(void* stream, int64_t batch, int64_t T, int64_t K, int64_t V, const float* log_fgate,
                    const void* kv, const float* init_log_fgate, const void* init_kv, float* out_log,
                    void* out_state, int reverse, int last_only, int kv_dtype, void* workspace, size_t workspace_bytes) {
  if (!log_fgate || !kv || !out_log || !out_state) return GLA_ERR_NULL_POINTER;
  if ((init_log_fgate == nullptr) != (init_kv == nullptr)) return GLA_ERR_NULL_POINTER;
  if (batch <= 0 || T <= 0 || K <= 0 || V <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(kv_dtype));
  return launch_rnn_scan((cudaStream_t)stream, batch, T, K, V, log_fgate, kv, init_log_fgate, init_kv, out_log,
                         out_state, reverse, last_only, kv_dtype == GLA_BF16, (float*)workspace, workspace_bytes);
}

int gla_recurrent_fwd(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int dtype, const void* hidden_init,
                      const float* log_fgate, const void* value, const void* key, const void* query,
                      void* hidden_final, void* out, int out_dtype, int reverse) {
  if (!hidden_init || !log_fgate || !value || !key || !query || !hidden_final || !out) return GLA_ERR_NULL_POINTER;
  if (B <= 0 || T <= 0 || H <= 0 || D <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(dtype));
  GLA_TRY(check_dtype(out_dtype));
  return recurrent_fwd((cudaStream_t)stream, B, T, H, D, dtype == GLA_BF16, hidden_init, log_fgate, value, key,
                       query, hidden_final, out, out_dtype == GLA_BF16, reverse);
}

int gla_decode_step(void* stream, int64_t B, int64_t H, int64_t D, int dtype, float* state, const float* log_fgate,
                    const void* value, const void* key, const void* query, void* out, int out_dtype) {
  if (!state || !log_fgate || !value || !key || !query || !out) return GLA_ERR_NULL_POINTER;
  if (B <= 0 || H <= 0 || D <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(dtype));
  GLA_TRY(check_dtype(out_dtype));
  return decode_step((cudaStream_t)stream, B, H, D, dtype == GLA_BF16, state, log_fgate, value, key, query, out,
                     out_dtype == GLA_BF16);
}

int gla_layer_gate_fwd(void* stream, int64_t n, int dtype, const void* z, float inv_tau, float* log_fgate) {
  if (!z || !log_fgate) return GLA_ERR_NULL_POINTER;
  if (n <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(dtype));
  return layer_gate_fwd((cudaStream_t)stream, n, dtype == GLA_BF16, z, inv_tau, log_fgate);
}

int gla_layer_gate_bwd(void* stream, int64_t n, int dtype, const void* z, const float* dlog_fgate, float inv_tau,
                       void* dz) {
  if (!z || !dlog_fgate || !dz) return GLA_ERR_NULL_POINTER;
  if (n <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(dtype));
  return layer_gate_bwd((cudaStream_t)stream, n, dtype == GLA_BF16, z, dlog_fgate, inv_tau, dz);
}

static int check_head_dim(int64_t D) { return (D == 32 || D == 64 || D == 128 || D == 256) ? GLA_OK : GLA_ERR_UNSUPPORTED; }

int gla_layer_headnorm_gate_fwd(void* stream, int64_t rows, int64_t D, int dtype, const void* x, const void* gate,
                                const float* weight, float eps, void* y, float* rstd) {
  if (!x || !gate || !y || !rstd) return GLA_ERR_NULL_POINTER;
  if (rows <= 0 || D <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(dtype));
  GLA_TRY(check_head_dim(D));
  if (!aligned16(x) || !aligned16(gate) || !aligned16(y)) return GLA_ERR_ALIGNMENT;
  return layer_headnorm_gate_fwd((cudaStream_t)stream, rows, D, dtype == GLA_BF16, x, gate, weight, eps, y, rstd);
}

size_t gla_layer_headnorm_gate_bwd_workspace_bytes(int64_t rows, int64_t D) {
  if (rows <= 0 || D <= 0) return 0;
  return layer_headnorm_gate_bwd_ws_bytes(rows, D);
}

int gla_layer_headnorm_gate_bwd(void* stream, int64_t rows, int64_t D, int dtype, const void* x, const void* gate,
                                const float* weight, const float* rstd, const void* dy, void* dx, void* dgate,
                                float* dweight, void* workspace, size_t workspace_bytes) {
  if (!x || !gate || !rstd || !dy || !dx || !dgate) return GLA_ERR_NULL_POINTER;
  if (rows <= 0 || D <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(dtype));
  GLA_TRY(check_head_dim(D));
  if (!aligned16(x) || !aligned16(gate) || !aligned16(dy) || !aligned16(dx) || !aligned16(dgate)) return GLA_ERR_ALIGNMENT;
  if (dweight && (!workspace || workspace_bytes < layer_headnorm_gate_bwd_ws_bytes(rows, D))) return GLA_ERR_WORKSPACE;
  return layer_headnorm_gate_bwd((cudaStream_t)stream, rows, D, dtype == GLA_BF16, x, gate, weight, rstd, dy, dx, dgate,
                                 dweight, workspace);
}

size_t gla_recurrent_bwd_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int dtype) {
  (void)dtype;
  if (B <= 0 || T <= 0 || H <= 0 || D <= 0) return 0;
  return recurrent_bwd_ws_bytes(B, T, H, D);
}

int gla_recurrent_bwd(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int dtype, const void* hidden_init,
                      const float* log_fgate, const void* value, const void* key, const void* query,
                      const void* dhidden_final, const void* dout, int dout_dtype, void* dhidden_init,
                      float* dlog_fgate, void* dvalue, void* dkey, void* dquery, int reverse, void* workspace,
                      size_t workspace_bytes) {
  if (!hidden_init || !log_fgate || !value || !key || !query || !dhidden_final || !dout || !dhidden_init ||
      !dlog_fgate || !dvalue || !dkey || !dquery)
    return GLA_ERR_NULL_POINTER;
  if (B <= 0 || T <= 0 || H <= 0 || D <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(dtype));
  GLA_TRY(check_dtype(dout_dtype));
  if (!workspace || workspace_bytes < recurrent_bwd_ws_bytes(B, T, H, D)) return GLA_ERR_WORKSPACE;
  if (!aligned16(workspace)) return GLA_ERR_ALIGNMENT;
  return recurrent_bwd((cudaStream_t)stream, B, T, H, D, dtype == GLA_BF16, hidden_init, log_fgate, value, key,
                       query, dhidden_final, dout, dout_dtype == GLA_BF16, dhidden_init, dlog_fgate, dvalue, dkey,
                       dquery, reverse, workspace);
}

size_t gla_chunk_saved_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int impl) {
  if (check_chunk_dims(B, T, H, D, chunk, dtype) != GLA_OK) return 0;
  int r = resolve_impl(impl, D, chunk, dtype);
  if (r < 0) return 0;
  return r == GLA_IMPL_TCGEN05 ? tc_saved_bytes(B, T, H, D, chunk) : simt_saved_bytes(B, T, H, D, chunk);
}
size_t gla_chunk_fwd_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int impl) {
  if (check_chunk_dims(B, T, H, D, chunk, dtype) != GLA_OK) return 0;
  int r = resolve_impl(impl, D, chunk, dtype);
  if (r < 0) return 0;
  return r == GLA_IMPL_TCGEN05 ? tc_fwd_ws_bytes(B, T, H, D, chunk) : simt_fwd_ws_bytes(B, T, H, D, chunk);
}
size_t gla_chunk_bwd_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int impl) {
  if (check_chunk_dims(B, T, H, D, chunk, dtype) != GLA_OK) return 0;
  int r = resolve_impl(impl, D, chunk, dtype);
  if (r < 0) return 0;
  return r == GLA_IMPL_TCGEN05 ? tc_bwd_ws_bytes(B, T, H, D, chunk) : simt_bwd_ws_bytes(B, T, H, D, chunk);
}

int gla_chunk_fwd(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int impl,
                  const void* hidden_init, const float* log_fgate, const void* value, const void* key,
                  const void* query, void* hidden_final, void* out, void* saved, void* workspace,
                  size_t workspace_bytes) {
  if (!hidden_init || !log_fgate || !value || !key || !query || !hidden_final || !out) return GLA_ERR_NULL_POINTER;
  GLA_TRY(check_chunk_dims(B, T, H, D, chunk, dtype));
  int r = resolve_impl(impl, D, chunk, dtype);
  if (r < 0) return -r;
  const size_t need = r == GLA_IMPL_TCGEN05 ? tc_fwd_ws_bytes(B, T, H, D, chunk) : simt_fwd_ws_bytes(B, T, H, D, chunk);
  if (!workspace || workspace_bytes < need) return GLA_ERR_WORKSPACE;
  const void* ptrs[] = {hidden_init, log_fgate, value, key, query, hidden_final, out, saved, workspace};
  for (const void* p : ptrs)
    if (p && !aligned16(p)) return GLA_ERR_ALIGNMENT;
  // the tensor-core kernels write rows with 32-byte vector stores
  if (r == GLA_IMPL_TCGEN05 && (!aligned32(out) || !aligned32(workspace))) return GLA_ERR_ALIGNMENT;
  if (r == GLA_IMPL_TCGEN05)
    return tc_chunk_fwd((cudaStream_t)stream, B, T, H, D, chunk, hidden_init, log_fgate, value, key, query,
                        hidden_final, out, saved, workspace, 0, nullptr, nullptr, impl & OPT_BITS);
  return simt_chunk_fwd((cudaStream_t)stream, B, T, H, D, chunk, dtype == GLA_BF16, hidden_init, log_fgate, value, key,
                        query, hidden_final, out, saved, workspace, 0, nullptr, nullptr);
}

int gla_chunk_bwd(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int impl,
                  const float* log_fgate, const void* value, const void* key, const void* query, const void* saved,
                  const void* dhidden_final, const void* dout, void* dhidden_init, float* dlog_fgate, void* dvalue,
                  void* dkey, void* dquery, void* workspace, size_t workspace_bytes) {
  if (!log_fgate || !value || !key || !query || !saved || !dhidden_final || !dout || !dhidden_init || !dlog_fgate ||
      !dvalue || !dkey || !dquery)
    return GLA_ERR_NULL_POINTER;
  GLA_TRY(check_chunk_dims(B, T, H, D, chunk, dtype));
  int r = resolve_impl(impl, D, chunk, dtype);
  if (r < 0) return -r;
  const size_t need = r == GLA_IMPL_TCGEN05 ? tc_bwd_ws_bytes(B, T, H, D, chunk) : simt_bwd_ws_bytes(B, T, H, D, chunk);
  if (!workspace || workspace_bytes < need) return GLA_ERR_WORKSPACE;
  const void* ptrs[] = {log_fgate, value, key, query, saved, dhidden_final, dout, dhidden_init, dlog_fgate,
                        dvalue, dkey, dquery, workspace};
  for (const void* p : ptrs)
    if (!aligned16(p)) return GLA_ERR_ALIGNMENT;
  if (r == GLA_IMPL_TCGEN05 && (!aligned32(dvalue) || !aligned32(workspace))) return GLA_ERR_ALIGNMENT;
  if (r == GLA_IMPL_TCGEN05)
    return tc_chunk_bwd((cudaStream_t)stream, B, T, H, D, chunk, log_fgate, value, key, query, saved, dhidden_final,
                        dout, dhidden_init, dlog_fgate, dvalue, dkey, dquery, workspace, impl & OPT_BITS);
  return simt_chunk_bwd((cudaStream_t)stream, B, T, H, D, chunk, dtype == GLA_BF16, log_fgate, value, key, query, saved,
                        dhidden_final, dout, dhidden_init, dlog_fgate, dvalue, dkey, dquery, workspace);
}

int gla_chunk_fwd_packed(void* stream, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int64_t nseq,
                         const int32_t* cu_seqlens, const void* hidden_init, const float* log_fgate, const void* value,
                         const void* key, const void* query, void* hidden_final, void* out, void* saved,
                         void* workspace, size_t workspace_bytes) {
  if (!cu_seqlens || !hidden_init || !log_fgate || !value || !key || !query || !hidden_final || !out)
    return GLA_ERR_NULL_POINTER;
  if (nseq <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_chunk_dims(1, T, H, D, chunk, dtype));
  if (!tc_supported_local_state(D, 128, dtype) || chunk % 128 != 0) return GLA_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < tc_fwd_ws_bytes(1, T, H, D, chunk)) return GLA_ERR_WORKSPACE;
  const void* ptrs[] = {hidden_init, log_fgate, value, key, query, hidden_final, out, saved, workspace};
  for (const void* p : ptrs)
    if (p && !aligned16(p)) return GLA_ERR_ALIGNMENT;
  if (!aligned32(out)) return GLA_ERR_ALIGNMENT;
  return tc_chunk_fwd((cudaStream_t)stream, 1, T, H, D, chunk, hidden_init, log_fgate, value, key, query, hidden_final,
                      out, saved, workspace, 0, nullptr, nullptr, 0, nseq, cu_seqlens);
}

int gla_chunk_bwd_packed(void* stream, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int64_t nseq,
                         const int32_t* cu_seqlens, const float* log_fgate, const void* value, const void* key,
                         const void* query, const void* saved, const void* dhidden_final, const void* dout,
                         void* dhidden_init, float* dlog_fgate, void* dvalue, void* dkey, void* dquery,
                         void* workspace, size_t workspace_bytes) {
  if (!cu_seqlens || !log_fgate || !value || !key || !query || !saved || !dhidden_final || !dout || !dhidden_init ||
      !dlog_fgate || !dvalue || !dkey || !dquery)
    return GLA_ERR_NULL_POINTER;
  if (nseq <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_chunk_dims(1, T, H, D, chunk, dtype));
  if (!tc_supported_local_state(D, 128, dtype) || chunk % 128 != 0) return GLA_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < tc_bwd_ws_bytes(1, T, H, D, chunk)) return GLA_ERR_WORKSPACE;
  const void* ptrs[] = {log_fgate, value, key, query, saved, dhidden_final, dout, dhidden_init, dlog_fgate, dvalue, dkey,
                        dquery, workspace};
  for (const void* p : ptrs)
    if (!aligned16(p)) return GLA_ERR_ALIGNMENT;
  if (!aligned32(dvalue)) return GLA_ERR_ALIGNMENT;
  return tc_chunk_bwd((cudaStream_t)stream, 1, T, H, D, chunk, log_fgate, value, key, query, saved, dhidden_final, dout,
                      dhidden_init, dlog_fgate, dvalue, dkey, dquery, workspace, 0, nseq, cu_seqlens);
}

int gla_chunk_local_state(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype,
                          int impl, const float* log_fgate, const void* value, const void* key, float* G_total,
                          float* S_local, void* workspace, size_t workspace_bytes) {
  if (!log_fgate || !value || !key || !G_total || !S_local) return GLA_ERR_NULL_POINTER;
  GLA_TRY(check_chunk_dims(B, T, H, D, chunk, dtype));
  int r = resolve_impl(impl, D, chunk, dtype);
  if (r < 0) return -r;
  if (r == GLA_IMPL_TCGEN05 && !tc_supported_local_state(D, chunk, dtype)) {
    if (impl == GLA_IMPL_TCGEN05) return GLA_ERR_UNSUPPORTED;
    r = GLA_IMPL_FP32_SIMT;
  }
  const size_t need = r == GLA_IMPL_TCGEN05 ? tc_fwd_ws_bytes(B, T, H, D, chunk) : simt_fwd_ws_bytes(B, T, H, D, chunk);
  if (!workspace || workspace_bytes < need) return GLA_ERR_WORKSPACE;
  if (r == GLA_IMPL_TCGEN05)
    return tc_chunk_fwd((cudaStream_t)stream, B, T, H, D, chunk, nullptr, log_fgate, value, key, nullptr, nullptr,
                        nullptr, nullptr, workspace, 1, G_total, S_local, impl & OPT_BITS);
  return simt_chunk_fwd((cudaStream_t)stream, B, T, H, D, chunk, dtype == GLA_BF16, nullptr, log_fgate, value, key,
                        nullptr, nullptr, nullptr, nullptr, workspace, 1, G_total, S_local);
}

int gla_chunk_local_dstate(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype,
                           int impl, const float* log_fgate, const void* query, const void* dout, float* dS_local,
                           void* workspace, size_t workspace_bytes) {
  if (!log_fgate || !query || !dout || !dS_local) return GLA_ERR_NULL_POINTER;
  GLA_TRY(check_chunk_dims(B, T, H, D, chunk, dtype));
  int r = resolve_impl(impl, D, chunk, dtype);
  if (r < 0) return -r;
  if (r == GLA_IMPL_TCGEN05 && !tc_supported_local_state(D, chunk, dtype)) {
    if (impl == GLA_IMPL_TCGEN05) return GLA_ERR_UNSUPPORTED;
    r = GLA_IMPL_FP32_SIMT;
  }
  const size_t need = r == GLA_IMPL_TCGEN05 ? tc_bwd_ws_bytes(B, T, H, D, chunk) : simt_bwd_ws_bytes(B, T, H, D, chunk);
  if (!workspace || workspace_bytes < need) return GLA_ERR_WORKSPACE;
  if (r == GLA_IMPL_TCGEN05)
    return tc_local_dstate((cudaStream_t)stream, B, T, H, log_fgate, query, dout, dS_local, workspace);
  return simt_chunk_dstate_only((cudaStream_t)stream, B, T, H, D, chunk, dtype == GLA_BF16, log_fgate, query, dout,
                                dS_local, workspace);
}

// ---- sequence parallelism without repeated work: the chunk states of a slice are computed once ----------------
static int sp_check(int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int impl) {
  GLA_TRY(check_chunk_dims(B, T, H, D, chunk, dtype));
  int r = resolve_impl(impl, D, chunk, dtype);
  if (r < 0) return -r;
  if (r != GLA_IMPL_TCGEN05 || D != 128) return GLA_ERR_UNSUPPORTED;
  return GLA_OK;
}

int gla_chunk_sp_fwd_local(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int impl,
                           const float* log_fgate, const void* value, const void* key, float* G_total, float* S_local,
                           void* saved, void* workspace, size_t workspace_bytes) {
  if (!log_fgate || !value || !key || !G_total || !S_local || !saved) return GLA_ERR_NULL_POINTER;
  GLA_TRY(sp_check(B, T, H, D, chunk, dtype, impl));
  if (!workspace || workspace_bytes < tc_fwd_ws_bytes(B, T, H, D, chunk)) return GLA_ERR_WORKSPACE;
  const void* ptrs[] = {log_fgate, value, key, G_total, S_local, saved, workspace};
  for (const void* p : ptrs)
    if (!aligned16(p)) return GLA_ERR_ALIGNMENT;
  return tc_chunk_fwd((cudaStream_t)stream, B, T, H, D, chunk, nullptr, log_fgate, value, key, nullptr, nullptr, nullptr,
                      saved, workspace, 0, G_total, S_local, impl & OPT_BITS, 0, nullptr, 1, nullptr);
}

int gla_chunk_sp_fwd_finish(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int impl,
                            const float* H_in, const float* log_fgate, const void* value, const void* key,
                            const void* query, void* out, void* saved, void* workspace, size_t workspace_bytes) {
  if (!H_in || !log_fgate || !value || !key || !query || !out || !saved) return GLA_ERR_NULL_POINTER;
  GLA_TRY(sp_check(B, T, H, D, chunk, dtype, impl));
  if (!workspace || workspace_bytes < tc_fwd_ws_bytes(B, T, H, D, chunk)) return GLA_ERR_WORKSPACE;
  const void* ptrs[] = {H_in, log_fgate, value, key, query, out, saved, workspace};
  for (const void* p : ptrs)
    if (!aligned16(p)) return GLA_ERR_ALIGNMENT;
  if (!aligned32(out)) return GLA_ERR_ALIGNMENT;
  return tc_chunk_fwd((cudaStream_t)stream, B, T, H, D, chunk, nullptr, log_fgate, value, key, query, nullptr, out, saved,
                      workspace, 0, nullptr, nullptr, impl & OPT_BITS, 0, nullptr, 2, H_in);
}

int gla_chunk_sp_bwd_local(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int impl,
                           const float* log_fgate, const void* query, const void* dout, const void* saved,
                           float* A_local, void* workspace, size_t workspace_bytes) {
  if (!log_fgate || !query || !dout || !saved || !A_local) return GLA_ERR_NULL_POINTER;
  GLA_TRY(sp_check(B, T, H, D, chunk, dtype, impl));
  if (!workspace || workspace_bytes < tc_bwd_ws_bytes(B, T, H, D, chunk)) return GLA_ERR_WORKSPACE;
  const void* ptrs[] = {log_fgate, query, dout, saved, A_local, workspace};
  for (const void* p : ptrs)
    if (!aligned16(p)) return GLA_ERR_ALIGNMENT;
  return tc_chunk_bwd((cudaStream_t)stream, B, T, H, D, chunk, log_fgate, nullptr, nullptr, query, saved, nullptr, dout,
                      nullptr, nullptr, nullptr, nullptr, nullptr, workspace, impl & OPT_BITS, 0, nullptr, 1, A_local, nullptr);
}

int gla_chunk_sp_bwd_finish(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype, int impl,
                            const float* dH_out, const float* log_fgate, const void* value, const void* key,
                            const void* query, const void* saved, const void* dout, float* dlog_fgate, void* dvalue,
                            void* dkey, void* dquery, void* workspace, size_t workspace_bytes) {
  if (!dH_out || !log_fgate || !value || !key || !query || !saved || !dout || !dlog_fgate || !dvalue || !dkey || !dquery)
    return GLA_ERR_NULL_POINTER;
  GLA_TRY(sp_check(B, T, H, D, chunk, dtype, impl));
  if (!workspace || workspace_bytes < tc_bwd_ws_bytes(B, T, H, D, chunk)) return GLA_ERR_WORKSPACE;
  const void* ptrs[] = {dH_out, log_fgate, value, key, query, saved, dout, dlog_fgate, dvalue, dkey, dquery, workspace};
  for (const void* p : ptrs)
    if (!aligned16(p)) return GLA_ERR_ALIGNMENT;
  if (!aligned32(dvalue)) return GLA_ERR_ALIGNMENT;
  return tc_chunk_bwd((cudaStream_t)stream, B, T, H, D, chunk, log_fgate, value, key, query, saved, nullptr, dout, nullptr,
                      dlog_fgate, dvalue, dkey, dquery, workspace, impl & OPT_BITS, 0, nullptr, 2, nullptr, dH_out);
}

int gla_sp_combine(void* stream, int64_t R, int64_t rank, int64_t BH, int64_t D, const float* all_G,
                   const float* all_S, const void* init, int init_dtype, void* result, int result_dtype,
                   int reverse) {
  if (!all_G || !all_S || !result) return GLA_ERR_NULL_POINTER;
  if (R <= 0 || rank < -1 || rank > R || BH <= 0 || D <= 0) return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(init_dtype));
  GLA_TRY(check_dtype(result_dtype));
  return launch_sp_combine((cudaStream_t)stream, R, rank, BH, D, all_G, all_S, init, init_dtype == GLA_BF16, result,
                           result_dtype == GLA_BF16, reverse);
}

int gla_sp_combine2(void* stream, int64_t R, int64_t rank, int64_t BH, int64_t D, const float* all_G, int64_t g_rank_stride,
                    const float* all_S, int64_t s_rank_stride, const void* init, int init_dtype, float* entering,
                    void* total, int total_dtype, int reverse) {
  if (!all_G || !all_S || (!entering && !total)) return GLA_ERR_NULL_POINTER;
  if (R <= 0 || rank < 0 || rank >= R || BH <= 0 || D <= 0 || g_rank_stride < BH * D || s_rank_stride < BH * D * D)
    return GLA_ERR_BAD_DIMS;
  GLA_TRY(check_dtype(init_dtype));
  GLA_TRY(check_dtype(total_dtype));
  return launch_sp_combine2((cudaStream_t)stream, R, rank, BH, D, all_G, g_rank_stride, all_S, s_rank_stride, init,
                            init_dtype == GLA_BF16, entering, total, total_dtype == GLA_BF16, reverse);
}

}  // extern "C"
