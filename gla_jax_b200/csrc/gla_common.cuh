// Shared helpers for the GLA kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/gla_b200.h"

namespace gla {

typedef __nv_bfloat16 bf16;

// Element (b, t, h, d) of a dense (B, T, H, D) array.
__host__ __device__ __forceinline__ int64_t idx_bthd(int64_t b, int64_t t, int64_t h, int64_t d,
                                                     int64_t T, int64_t H, int64_t D) {
  return ((b * T + t) * H + h) * D + d;
}

__device__ __forceinline__ float ld_f(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ float ld_f(const bf16* p, int64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st_f(float* p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void st_f(bf16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// Typed load/store through a void pointer and a runtime dtype flag (used by the generic
// fp32 kernels whose operands may be either type).
__device__ __forceinline__ float ld_any(const void* p, int is_bf16, int64_t i) {
  return is_bf16 ? __bfloat162float(((const bf16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ void st_any(void* p, int is_bf16, int64_t i, float v) {
  if (is_bf16) ((bf16*)p)[i] = __float2bfloat16_rn(v); else ((float*)p)[i] = v;
}

// Host-side: record and translate launch errors.
int record_cuda_error(cudaError_t e);   // returns GLA_OK or GLA_ERR_LAUNCH
void count_launch();
#define GLA_CHECK_LAUNCH()                                   \
  do {                                                       \
    ::gla::count_launch();                                   \
    int _s = ::gla::record_cuda_error(cudaGetLastError());   \
    if (_s != GLA_OK) return _s;                             \
  } while (0)
#define GLA_TRY(expr)                                        \
  do {                                                       \
    int _s = (expr);                                         \
    if (_s != GLA_OK) return _s;                             \
  } while (0)

// Optional per-kernel timing (off by default): while enabled on the calling thread, every
// kernel launch site is bracketed by a pair of CUDA events on its stream.
struct ProfScope {
  int slot;
  cudaStream_t st;
  ProfScope(const char* name, cudaStream_t stream);
  ~ProfScope();
};

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline bool is_pow2(int64_t x) { return x > 0 && (x & (x - 1)) == 0; }
static inline bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }
static inline bool aligned32(const void* p) { return (((uintptr_t)p) & 31) == 0; }

// ---- internal launchers shared between translation units -------------------------------

// Inclusive cumsum along the middle axis of (N, T, D), fp32 math.  `sub`, when given, has src's
// shape and type and is subtracted from it element-wise before the scan.  With `scratch` of
// cumsum_scratch_bytes(N, T, D) the scan axis is cut into segments that run as separate blocks
// (segment sums first, then the scans), which fills the device when N * D alone is small.
int launch_cumsum(cudaStream_t st, int64_t N, int64_t T, int64_t D, const void* src, const void* init,
                  void* dst, int reverse, int in_bf16, int out_bf16, const void* sub = nullptr,
                  float* scratch = nullptr, int op = GLA_SCAN_ADD);
size_t cumsum_scratch_bytes(int64_t N, int64_t T, int64_t D);

// Exclusive state scan over chunks: for every (bh): S <- init; for n in order:
// before[n] = S; S = exp(G[n]) (x) S + X[n].  final = S.  X, before: (BH, N, D, D);
// G: (BH, N, D); init/final: (BH, D, D).  `before` may alias X (in place).
int launch_state_scan(cudaStream_t st, int64_t BH, int64_t N, int64_t D, const float* G, const void* X,
                      int x_bf16, const void* init, int init_bf16, void* before, int before_bf16,
                      void* final_state, int final_bf16, int reverse);

// Single-token step with a persistent float32 state.
int decode_step(cudaStream_t st, int64_t B, int64_t H, int64_t D, int bf, float* state, const float* g, const void* v,
                const void* k, const void* q, void* out, int out_bf);

// Element-wise stages of a GLA layer either side of the op.
int layer_gate_fwd(cudaStream_t st, int64_t n, int bf, const void* z, float inv_tau, float* g);
int layer_gate_bwd(cudaStream_t st, int64_t n, int bf, const void* z, const float* dg, float inv_tau, void* dz);
int layer_headnorm_gate_fwd(cudaStream_t st, int64_t rows, int64_t D, int bf, const void* x, const void* gate,
                            const float* w, float eps, void* y, float* rstd);
size_t layer_headnorm_gate_bwd_ws_bytes(int64_t rows, int64_t D);
int layer_headnorm_gate_bwd(cudaStream_t st, int64_t rows, int64_t D, int bf, const void* x, const void* gate,
                            const float* w, const float* rstd, const void* dy, void* dx, void* dgate, float* dweight,
                            void* ws);

// fp32 CUDA-core chunk path.
size_t simt_saved_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C);
size_t simt_fwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C);
size_t simt_bwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C);
int simt_chunk_fwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C, int bf,
                   const void* hidden_init, const float* g, const void* v, const void* k, const void* q,
                   void* hidden_final, void* out, void* saved, void* ws, int state_only,
                   float* G_total, float* S_local);
int simt_chunk_bwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C, int bf,
                   const float* g, const void* v, const void* k, const void* q, const void* saved,
                   const void* dhidden_final, const void* dout, void* dhidden_init, float* dg,
                   void* dv, void* dk, void* dq, void* ws);

int simt_chunk_dstate_only(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C, int bf,
                           const float* g, const void* q, const void* dout, float* dS_local, void* ws);

// tcgen05 tensor-core chunk path (bf16, D = 128 or 256, chunk a multiple of 128).
bool tc_supported(int64_t D, int64_t C, int dtype);
bool tc_supported_local_state(int64_t D, int64_t C, int dtype);
int tc_local_dstate(cudaStream_t st, int64_t B, int64_t T, int64_t H, const float* g, const void* q, const void* dout,
                    float* dS_local, void* ws);
bool tc_auto_default();
unsigned int tc_read_wait_timeouts();
size_t tc_saved_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C);
size_t tc_fwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C);
size_t tc_bwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C);
int tc_chunk_fwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C,
                 const void* hidden_init, const float* g, const void* v, const void* k, const void* q,
                 void* hidden_final, void* out, void* saved, void* ws, int state_only,
                 float* G_total, float* S_local, int opts = 0, int64_t nseq = 0, const int* cu = nullptr,
                 int sp_phase = 0, const float* H_in = nullptr);
// One-pass chunk states (product and recurrence fused); mode 0 forward states, mode 1 gradient states.
bool tc_state_fused_preferred(int64_t BH, int64_t N, int opts);
int tc_state_fused(cudaStream_t st, int mode, int64_t B, int64_t T, int64_t H, int R, const float* g, const void* x,
                   const void* y, const void* init, void* states, void* fin, float* Gc, int64_t nseq = 0,
                   const int* cu = nullptr, unsigned int* done = nullptr, unsigned int* done_target = nullptr,
                   float* fin32 = nullptr, int nsegs = 1);
int tc_state_segments(int64_t BH, int64_t N, int opts);
unsigned int tc_state_read_wait_timeouts();
unsigned int scan_read_wait_timeouts();
unsigned int tc_state_read_bad_offsets();
int tc_chunk_bwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C,
                 const float* g, const void* v, const void* k, const void* q, const void* saved,
                 const void* dhidden_final, const void* dout, void* dhidden_init, float* dg,
                 void* dv, void* dk, void* dq, void* ws, int opts = 0, int64_t nseq = 0, const int* cu = nullptr,
                 int sp_phase = 0, float* A_local = nullptr, const float* dH_out = nullptr);

}  // namespace gla

namespace gla {
int launch_rnn_scan(cudaStream_t st, int64_t batch, int64_t T, int64_t K, int64_t V, const float* g,
                    const void* kv, const float* ig, const void* ikv, float* out_log, void* out_state,
                    int reverse, int last_only, int kv_bf16, float* ws = nullptr, size_t ws_bytes = 0);
size_t rnn_scan_ws_bytes(int64_t batch, int64_t T, int64_t K, int64_t V);
int launch_sp_combine(cudaStream_t st, int64_t R, int64_t rank, int64_t BH, int64_t D, const float* all_G,
                      const float* all_S, const void* init, int init_bf16, void* result, int result_bf16,
                      int reverse);
int launch_sp_combine2(cudaStream_t st, int64_t R, int64_t rank, int64_t BH, int64_t D, const float* all_G, int64_t gstride,
                       const float* all_S, int64_t sstride, const void* init, int init_bf16, float* entering, void* total,
                       int total_bf16, int reverse);
int recurrent_fwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int bf, const void* hidden_init,
                  const float* g, const void* v, const void* k, const void* q, void* hidden_final, void* out,
                  int out_bf, int reverse);
size_t recurrent_bwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D);
int recurrent_bwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int bf, const void* hidden_init,
                  const float* g, const void* v, const void* k, const void* q, const void* dhidden_final,
                  const void* dout, int do_bf, void* dhidden_init, float* dg, void* dv, void* dk, void* dq,
                  int reverse, void* ws);
}  // namespace gla
