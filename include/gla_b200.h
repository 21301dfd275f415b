/*
 * gla_b200.h — C ABI of libgla_b200.so: gated linear attention (GLA) kernels for NVIDIA B200
 * (sm_100a).  This is the drop-in boundary for the hot path of zhixuan-lin/gla-jax: every
 * entry point below replaces one Python-level operator of the reference, whose device code
 * is Pallas/Triton JIT-compiled inside jaxlib (the reference has no C interface of its
 * own; the cited file:line is the operator each function stands in for).
 *
 * Conventions (all entry points)
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless stated;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); all
 *     work is enqueued on it, on the CURRENT device; nothing synchronises and nothing allocates
 *     device memory.  What the library keeps between calls: on the host, a per-thread cache of
 *     TMA descriptors keyed by address and shape (a few KB), one "attribute set" bit per kernel
 *     and device, the launch counter and the optional per-thread kernel timer below; on each
 *     device, two error counters (gla_device_wait_timeouts, gla_device_bad_offsets) and the fixed
 *     scratch array of gla_chunk_fwd_static.  No call's result depends on any of it;
 *   - the caller owns every buffer, including the workspace whose size the matching
 *     *_workspace_bytes() function reports;
 *   - arrays are dense row-major with the reference's axis order and an optional leading
 *     batch axis B (the reference adds it with jax.vmap, gla.py:1335; pass B = 1 for the
 *     per-sequence API):
 *         log_fgate, value, key, query, out, and their gradients : (B, T, H, D)
 *         hidden_init, hidden_final and their gradients          : (B, H, D, D)  [key, value]
 *   - `dtype` is the element type of value/key/query/hidden/out and their gradients;
 *     log_fgate and its gradient are always float32 (as in every configuration of the
 *     reference harness, gla.py:1391);
 *   - the return value is GLA_OK (0) or a gla_status code; nothing throws across the ABI.
 *     Dimension and alignment problems are reported before anything is launched (the
 *     reference raises Python asserts at trace time instead: gla.py:120-127, 499-500,
 *     975-977; ops.py:195-207, 348-364).
 *   - every function is thread-safe and reentrant: the cached state above is per thread or
 *     idempotent, and work is ordered by the stream the caller passes (the one exception, the shared
 *     scratch of gla_chunk_fwd_static, is documented there).
 */
#ifndef GLA_B200_H_
#define GLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define GLA_API __attribute__((visibility("default")))
#else
#define GLA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum gla_status {
  GLA_OK = 0,
  GLA_ERR_NULL_POINTER = 1,   /* a required pointer is NULL */
  GLA_ERR_BAD_DIMS = 2,       /* non-positive size, T % chunk != 0, chunk not a power of two, ... */
  GLA_ERR_UNSUPPORTED = 3,    /* dtype / size combination this build has no kernel for */
  GLA_ERR_ALIGNMENT = 4,      /* a pointer is not 16-byte aligned (32-byte for out, dvalue and the workspace of the
                                 tensor-core chunk path, whose kernels store rows with 32-byte vector stores) */
  GLA_ERR_WORKSPACE = 5,      /* workspace missing or smaller than *_workspace_bytes() */
  GLA_ERR_LAUNCH = 6,         /* the CUDA runtime rejected a launch (see gla_last_cuda_error) */
  GLA_ERR_NO_DEVICE = 7,      /* no usable sm_100 device / driver */
  GLA_ERR_TOO_LARGE = 8       /* size beyond a documented fixed maximum */
} gla_status;

typedef enum gla_dtype {
  GLA_F32 = 0,
  GLA_BF16 = 1
} gla_dtype;

/* Which implementation gla_chunk_fwd/bwd use. AUTO picks the tcgen05 tensor-core kernels
 * when the shape has one (bf16, D = 128 or 256, chunk a multiple of 128) and the fp32 CUDA-core kernels otherwise. */
typedef enum gla_chunk_impl {
  GLA_IMPL_AUTO = 0,
  GLA_IMPL_FP32_SIMT = 1,     /* fp32 math on CUDA cores: every dtype, D <= 256, chunk 16..256 */
  GLA_IMPL_TCGEN05 = 2        /* bf16 operands, fp32 TMEM accumulators (sm_100a tensor cores) */
} gla_chunk_impl;

/* Options that may be OR-ed into the `impl` argument of the chunk entry points (the low byte is the
 * gla_chunk_impl).  They select between equivalent ways of running the tensor-core path; results agree to
 * rounding.  Tests and benchmarks use them to pin a path; callers normally pass none.
 *   STATE_TWO_KERNELS / STATE_ONE_PASS  how the per-chunk states (gla.py:705-723) are produced: a batched
 *       k_hat^T v product followed by a streaming scan, or one kernel that keeps the state on chip.  Default:
 *       chosen from the shape.
 *   NO_EARLY_START   keep the forward chunk kernel strictly behind the state kernel (default: it is launched as
 *       a programmatic dependent and its first blocks start on the SMs the state kernel leaves idle).
 *   ALL_SCALES       always run every level of the secondary chunking (gla.py:843-852, 985-1027).  Default: a
 *       chunk whose total |log decay| is at most 60 for every feature uses a single anchor, because all its decay
 *       weights then lie within exp(+-60); up to 140 a single anchor in the middle of the decay (weights within
 *       exp(+-70), the state tile rescaled to match); sharper chunks take all levels.  The choice is made per chunk
 *       on the device from the gates themselves.
 *   NO_L2_PREFETCH   no L2 prefetch of the next chunk's operands in the chunk kernels.
 *   STATE_SEGMENTS   cut every head's chunks into runs that separate thread blocks walk from a zero state, then
 *       correct the stored states with the state that really enters each run (the recurrence is linear in it).
 *       Default: done when (batch x heads) alone gives the one-pass state kernel too few blocks for the device
 *       and the sequence is long; this bit forces it for any shape. */
typedef enum gla_chunk_option {
  GLA_OPT_STATE_TWO_KERNELS = 0x100,
  GLA_OPT_STATE_ONE_PASS = 0x200,
  GLA_OPT_NO_EARLY_START = 0x400,
  GLA_OPT_ALL_SCALES = 0x800,
  GLA_OPT_NO_L2_PREFETCH = 0x1000,
  GLA_OPT_STATE_SEGMENTS = 0x2000
} gla_chunk_option;

/* Human-readable text for a status code. Never NULL. (Reference: Python assert messages.) */
GLA_API const char* gla_status_string(int status);

/* Library version string, e.g. "gla_b200 0.1 (sm_100a)". */
GLA_API const char* gla_version(void);

/* cudaError_t value of the most recent failed launch on the calling thread (0 if none). */
GLA_API int gla_last_cuda_error(void);

/* Number of kernels this library has launched since load, from all threads (monotonic).
 * Diagnostic; the reference has no counterpart. */
GLA_API long long gla_launch_count(void);

/* Every device-side wait in this library (on an mbarrier that a tensor-core operation
 * completes) is bounded: a wait that runs out makes its thread block skip its output and
 * increments a device counter instead of spinning forever.  An entry point cannot report this in
 * its own return value, because it returns before its kernels have run (nothing synchronises);
 * a caller that wants to know polls this counter after synchronising the stream: it reads the
 * count of waits that gave up since the library was loaded, on the current device
 * (synchronises the device).  0 means no wait has ever given up; a value that grew since the
 * previous poll means outputs written in between are incomplete.  The Python package wraps the
 * poll as gla_jax_b200.check_device(). */
GLA_API unsigned int gla_device_wait_timeouts(void);

/* gla_chunk_fwd_packed / gla_chunk_bwd_packed take their sequence offsets from device memory and cannot check
 * them on the host without synchronising.  The kernels therefore clamp every sequence to chunks inside the arrays
 * (no access ever leaves the buffers) and count the sequences whose offsets were not rising multiples of 128
 * within [0, T]; such a sequence is cut short or skipped, so its results are not meaningful.  This reads the
 * count since the library was loaded, for the current device (synchronises the device).  0 means every offset
 * array seen so far was valid.  No counterpart in the reference. */
GLA_API unsigned int gla_device_bad_offsets(void);

/* Per-kernel device timing for benchmarks (diagnostic; no counterpart in the reference, whose
 * harness times whole calls with timeit, gla.py:1430-1434).  While enabled on the calling
 * thread, each internal kernel launch is bracketed by CUDA events on its stream;
 * gla_profile_report waits for them and writes one line "kernel_name launches total_ms" per
 * kernel into buf (NUL-terminated), returning the bytes written.  At most 4096 launches are
 * recorded between enable(1) and report. */
GLA_API void gla_profile_enable(int on);
GLA_API size_t gla_profile_report(char* buf, size_t capacity);

/* ------------------------------------------------------------------------------------
 * decode step — one token of gla.py:26-47 (recurrent_gla_naive's loop body) for a batch of
 * requests, with the state kept on the device between calls.  No counterpart in the reference,
 * whose callers would run recurrent_gla with T = 1 and carry hidden_final to the next call
 * (gla.py:405-416); T calls of this step equal one recurrent_gla call over T tokens.
 *   state (B, H, D, D) float32, updated IN PLACE:  S <- exp(log_fgate) (.) S + key (x) value
 *   out   (B, H, D) in out_dtype:                  out = query S
 * log_fgate (B, H, D) float32; value, key, query (B, H, D) in dtype.  D in {32, 64, 128, 256}.
 * ---------------------------------------------------------------------------------- */
GLA_API int gla_decode_step(void* stream, int64_t B, int64_t H, int64_t D, int dtype,
                    float* state, const float* log_fgate, const void* value, const void* key,
                    const void* query, void* out, int out_dtype);

/* ------------------------------------------------------------------------------------
 * layer stages — the element-wise steps a gated-linear-attention layer runs either side of the
 * op.  No counterpart in the reference, which ships the op only (gla.py:657); they produce the
 * float32 log_fgate the op takes (gla.py:483) and consume its `out`.
 *   gate:          log_fgate[i] = inv_tau * log_sigmoid(z[i])      z in dtype, log_fgate float32
 *                  dz[i]        = dlog_fgate[i] * inv_tau * sigmoid(-z[i])
 *   headnorm_gate: rows of D elements (rows = B*T*H, D in {32, 64, 128, 256}), x/gate/y in dtype:
 *                  rstd[r] = rsqrt(mean_d x[r,d]^2 + eps)
 *                  y[r,d]  = x[r,d] * rstd[r] * weight[d] * gate[r,d] * sigmoid(gate[r,d])
 *                  weight (D) float32 or NULL (= 1); rstd (rows) float32 is kept for the backward.
 *                  The backward returns dx, dgate (dtype) and, if dweight (D, float32) is not NULL,
 *                  the weight gradient (deterministic: per-block partial sums in `workspace`).
 * x, gate, y, dy, dx, dgate must be 16-byte aligned.
 * ---------------------------------------------------------------------------------- */
GLA_API int gla_layer_gate_fwd(void* stream, int64_t n, int dtype, const void* z, float inv_tau,
                       float* log_fgate);
GLA_API int gla_layer_gate_bwd(void* stream, int64_t n, int dtype, const void* z,
                       const float* dlog_fgate, float inv_tau, void* dz);
GLA_API int gla_layer_headnorm_gate_fwd(void* stream, int64_t rows, int64_t D, int dtype,
                                const void* x, const void* gate, const float* weight, float eps,
                                void* y, float* rstd);
GLA_API size_t gla_layer_headnorm_gate_bwd_workspace_bytes(int64_t rows, int64_t D);
GLA_API int gla_layer_headnorm_gate_bwd(void* stream, int64_t rows, int64_t D, int dtype,
                                const void* x, const void* gate, const float* weight,
                                const float* rstd, const void* dy, void* dx, void* dgate,
                                float* dweight, void* workspace, size_t workspace_bytes);

/* ------------------------------------------------------------------------------------
 * cumsum — replaces ops.py:234 cumsum_recursive / ops.py:166 cumsum_pallas /
 * ops.py:152 cumsum_kernel.
 * Inclusive cumulative sum along the middle axis of src (N, T, D); `init` (N, D), if not
 * NULL, is added to every element (ops.py:91-103); reverse != 0 scans from the end.
 * Math is float32 (ops.py:159-160).  Any T (the reference's 16384-item and 2048-block
 * limits, ops.py:195-207,239, do not apply).  `init` has dtype in_dtype.
 * ---------------------------------------------------------------------------------- */
GLA_API int gla_cumsum(void* stream, int64_t N, int64_t T, int64_t D,
               const void* src, const void* init, void* dst,
               int reverse, int in_dtype, int out_dtype);

/* ------------------------------------------------------------------------------------
 * scan — the generic associative scan of ops.py:82 triton_scan for single-array operands, with the combine
 * function chosen from a fixed set instead of traced from Python (the reference lowers an arbitrary function
 * through Triton, ops.py:18-80; a precompiled library can only offer named rules):
 *     dst[n, t, d] = init[n, d] (op) src[n, 0, d] (op) ... (op) src[n, t, d]      (init omitted when NULL)
 * along the middle axis of src (N, T, D); reverse != 0 scans from the end.  Math is float32; any T.
 * GLA_SCAN_ADD is gla_cumsum.  The two-array log-space rule of ops.py:286 is gla_rnn_scan.
 * ---------------------------------------------------------------------------------- */
typedef enum gla_scan_op {
  GLA_SCAN_ADD = 0,
  GLA_SCAN_MUL = 1,
  GLA_SCAN_MAX = 2,
  GLA_SCAN_MIN = 3,
  GLA_SCAN_LOGADDEXP = 4      /* log(exp(a) + exp(b)) */
} gla_scan_op;
GLA_API int gla_scan(void* stream, int op, int64_t N, int64_t T, int64_t D,
             const void* src, const void* init, void* dst,
             int reverse, int in_dtype, int out_dtype);

/* ------------------------------------------------------------------------------------
 * rnn_scan — replaces ops.py:396 rnn_recursive / ops.py:338 rnn_pallas / ops.py:299
 * rnn_kernel with ops.py:286 binary_operator.
 * For each of `batch` independent problems: inclusive scan over the leading axis of
 * (log_fgate (T, K) float32, kv (T, K, V)) under
 *     (A_i, b_i) o (A_j, b_j) = (A_i + A_j, exp(A_j) * b_i + b_j),
 * with the optional pair (init_log_fgate (K) float32, init_kv (K, V)) combined in front
 * (both NULL or both set, ops.py:351).  Outputs: out_log (T, K) float32 cumulative log
 * decay, out_state (T, K, V) in kv_dtype.  reverse != 0 scans from the end.  With
 * last_only != 0 only the final row (row 0 when reversed) of both outputs is written
 * (ops.py:330-334); the other rows are left untouched.  Any T (no 8192-item limit).
 * ---------------------------------------------------------------------------------- */
GLA_API int gla_rnn_scan(void* stream, int64_t batch, int64_t T, int64_t K, int64_t V,
                 const float* log_fgate, const void* kv,
                 const float* init_log_fgate, const void* init_kv,
                 float* out_log, void* out_state,
                 int reverse, int last_only, int kv_dtype);

/* The same scan with scratch for long axes with few rows (the case ops.py:396-456 rnn_recursive serves by
 * recursion): when batch x K x V alone gives the device too few threads and T >= 512, the axis is cut into runs
 * that separate thread blocks scan from the identity, a small kernel scans the runs' last rows and one pass adds
 * exp(local log decay) x (state entering the run) to every row after the first run.  workspace:
 * gla_rnn_scan_workspace_bytes (0 when the plain scan is used anyway; a NULL or short workspace also selects it).
 * Results agree with gla_rnn_scan to rounding (the order of the additions differs). */
GLA_API size_t gla_rnn_scan_workspace_bytes(int64_t batch, int64_t T, int64_t K, int64_t V);
GLA_API int gla_rnn_scan_ws(void* stream, int64_t batch, int64_t T, int64_t K, int64_t V,
                 const float* log_fgate, const void* kv,
                 const float* init_log_fgate, const void* init_kv,
                 float* out_log, void* out_state,
                 int reverse, int last_only, int kv_dtype, void* workspace, size_t workspace_bytes);

/* ------------------------------------------------------------------------------------
 * recurrent_gla — replaces gla.py:405 recurrent_gla (forward: gla.py:99, kernel gla.py:50)
 * and, with out_dtype = GLA_F32, gla.py:26 recurrent_gla_naive.
 * Exact step recurrence S_t = exp(g_t) * S_{t-1} + k_t (x) v_t, o_t = q_t S_t with the
 * state held on chip in float32 and never written to memory.  reverse != 0 runs the
 * recurrence from the last token to the first (gla.py:421-423,437-438).
 * `out` has dtype out_dtype (the reference's recurrent_gla returns value's dtype,
 * recurrent_gla_naive returns float32).
 * ---------------------------------------------------------------------------------- */
GLA_API int gla_recurrent_fwd(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int dtype,
                      const void* hidden_init, const float* log_fgate,
                      const void* value, const void* key, const void* query,
                      void* hidden_final, void* out, int out_dtype, int reverse);

/* Bytes of workspace gla_recurrent_bwd needs for these sizes. */
GLA_API size_t gla_recurrent_bwd_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int dtype);

/* Backward of recurrent_gla — replaces gla.py:172 recurrent_gla_backward (kernel
 * gla.py:271): a recompute pass for dquery, a reverse pass for dvalue, dkey and
 * dhidden_init, and dlog_fgate = reverse_cumsum_T(q*dq - k*dk) + sum_v(dS_T * S_T)
 * (gla.py:263).  `dout` has dtype dout_dtype.  Gradients have dtype `dtype`
 * (dlog_fgate float32).
 */
GLA_API int gla_recurrent_bwd(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int dtype,
                      const void* hidden_init, const float* log_fgate,
                      const void* value, const void* key, const void* query,
                      const void* dhidden_final, const void* dout, int dout_dtype,
                      void* dhidden_init, float* dlog_fgate,
                      void* dvalue, void* dkey, void* dquery,
                      int reverse, void* workspace, size_t workspace_bytes);

/* ------------------------------------------------------------------------------------
 * chunk_gla — replaces gla.py:657 chunk_gla, gla.py:483 chunk_gla_forward (with
 * gla.py:695 compute_inter_contrib, gla.py:792 compute_intra_contrib, gla.py:1242
 * compute_score) and gla.py:552 chunk_gla_backward (with gla.py:731, 857, 1191).
 *
 * Requirements: T % chunk == 0; chunk a power of two, 16 <= chunk <= 256; 16 <= D <= 256
 * and D % 8 == 0.  `impl` is a gla_chunk_impl.
 *
 * The forward writes the residuals the backward needs into `saved` (size
 * gla_chunk_saved_bytes): the state entering every chunk, the per-chunk total log decay
 * and the intra-chunk score matrices (the reference keeps `state` and `score_list`,
 * gla.py:542-549).  Pass saved = NULL for a forward that will not be differentiated.
 * ---------------------------------------------------------------------------------- */
GLA_API size_t gla_chunk_saved_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                             int dtype, int impl);
GLA_API size_t gla_chunk_fwd_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                                     int dtype, int impl);
GLA_API size_t gla_chunk_bwd_workspace_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                                     int dtype, int impl);

GLA_API int gla_chunk_fwd(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                  int dtype, int impl,
                  const void* hidden_init, const float* log_fgate,
                  const void* value, const void* key, const void* query,
                  void* hidden_final, void* out,
                  void* saved, void* workspace, size_t workspace_bytes);

GLA_API int gla_chunk_bwd(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                  int dtype, int impl,
                  const float* log_fgate,
                  const void* value, const void* key, const void* query,
                  const void* saved,
                  const void* dhidden_final, const void* dout,
                  void* dhidden_init, float* dlog_fgate,
                  void* dvalue, void* dkey, void* dquery,
                  void* workspace, size_t workspace_bytes);

/* gla_chunk_fwd_static: the forward of gla_chunk_fwd (no residuals, so not differentiable)
 * for callers that cannot give the library a workspace.  (No counterpart in the reference,
 * where XLA owns all memory.)
 *
 * Who needs it: code that runs where device allocation is not available to it - a custom
 * call inside a runtime that owns the allocator and exposes no scratch to the callee, a
 * plugin in a serving process whose memory pool is closed, a callback in a region where
 * cudaMalloc would fail or stall the device.  Such a caller still passes inputs and outputs,
 * but the scratch comes from a fixed array inside the library image:
 *   - the array is gla_chunk_fwd_static_max_bytes() = 32 MiB of device memory PER GPU, held
 *     from the first use of the library on that GPU until the process exits;
 *   - a problem whose gla_chunk_fwd_workspace_bytes() exceeds it returns GLA_ERR_TOO_LARGE
 *     and launches nothing (32 MiB covers, e.g., one sequence of T=4096, H=6, D=128);
 *   - the function allocates nothing and frees nothing, on host or device.  The first call
 *     on each device looks up the array's device address (a symbol query, with that device
 *     current); make that first call outside any stream capture;
 *   - every call on a device uses the SAME array, and it keeps whatever the previous call
 *     left there.  Nothing in it has to start at zero (each launch sequence writes every
 *     word before reading it), but two calls whose kernels overlap on the GPU - different
 *     streams, or different host threads - race on it: serialise them on one stream.
 * Arguments, layouts, validation and status codes otherwise match gla_chunk_fwd. */
GLA_API size_t gla_chunk_fwd_static_max_bytes(void);
GLA_API int gla_chunk_fwd_static(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                         int dtype, int impl,
                         const void* hidden_init, const float* log_fgate,
                         const void* value, const void* key, const void* query,
                         void* hidden_final, void* out);

/* ------------------------------------------------------------------------------------
 * Packed (variable-length) sequences — no counterpart in the reference, which asserts one
 * length per call (gla.py:499-500, 674).
 * The arrays hold ONE time axis of T tokens with nseq sequences laid end to end:
 * log_fgate/value/key/query/out are (T, H, D); cu_seqlens is a DEVICE array of nseq + 1 int32
 * token offsets (cu_seqlens[0] = 0, cu_seqlens[nseq] = T), every offset a multiple of 128;
 * hidden_init / hidden_final (and their gradients) are (nseq, H, D, D).  Results equal nseq
 * separate gla_chunk_fwd / gla_chunk_bwd calls.  Tensor-core path only: bf16, D = 128, chunk
 * a multiple of 128; other shapes return GLA_ERR_UNSUPPORTED.  saved / workspace sizes:
 * gla_chunk_saved_bytes / gla_chunk_{fwd,bwd}_workspace_bytes with B = 1 and impl GLA_IMPL_TCGEN05.
 * ---------------------------------------------------------------------------------- */
GLA_API int gla_chunk_fwd_packed(void* stream, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype,
                         int64_t nseq, const int32_t* cu_seqlens,
                         const void* hidden_init, const float* log_fgate, const void* value,
                         const void* key, const void* query, void* hidden_final, void* out,
                         void* saved, void* workspace, size_t workspace_bytes);
GLA_API int gla_chunk_bwd_packed(void* stream, int64_t T, int64_t H, int64_t D, int64_t chunk, int dtype,
                         int64_t nseq, const int32_t* cu_seqlens,
                         const float* log_fgate, const void* value, const void* key, const void* query,
                         const void* saved, const void* dhidden_final, const void* dout,
                         void* dhidden_init, float* dlog_fgate, void* dvalue, void* dkey, void* dquery,
                         void* workspace, size_t workspace_bytes);

/* ------------------------------------------------------------------------------------
 * Sequence-parallel support (no counterpart in the reference, which is single-device; the
 * algebra is ops.py:286 binary_operator applied across ranks and the exact chaining of
 * hidden_init -> hidden_final, gla.py:720-723).
 *
 * gla_chunk_local_state: for a slice of the sequence, the total log decay
 * G (B, H, D) float32 = sum_t log_fgate and the state S (B, H, D, D) float32 reached from
 * a ZERO initial state (only the K^T V products and the state scan run).
 * Workspace: gla_chunk_fwd_workspace_bytes.
 *
 * gla_sp_combine: given every rank's (G_r, S_r) gathered as all_G (R, B, H, D) and
 * all_S (R, B, H, D, D) float32, computes for rank `rank`
 *   forward  (reverse == 0): H_in = sum_{p<rank} exp(sum_{p<s<rank} G_s) * S_p
 *                                   + exp(sum_{s<rank} G_s) * init
 *   backward (reverse != 0): the mirror image over ranks p > rank, used for dhidden_final,
 * where `init` (B, H, D, D) has dtype init_dtype (hidden_init on the forward pass,
 * dhidden_final of the whole sequence on the backward pass) and `result` has dtype
 * result_dtype.  The decay multiplies along the key axis.  rank may also be R (forward: the
 * state after the last rank = hidden_final of the whole sequence) or -1 (backward: the
 * gradient reaching hidden_init of the whole sequence).
 * ---------------------------------------------------------------------------------- */
GLA_API int gla_chunk_local_state(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                          int dtype, int impl,
                          const float* log_fgate, const void* value, const void* key,
                          float* G_total, float* S_local,
                          void* workspace, size_t workspace_bytes);

/* gla_chunk_local_dstate: the backward counterpart of gla_chunk_local_state.  For a slice of
 * the sequence, A (B, H, D, D) float32 = the gradient reaching the slice's initial state
 * when the gradient of its final state is ZERO: sum_n exp(sum_{m<n} G_m) * (q_hat_n^T dO_n).
 * The slice's dhidden_init for a non-zero dhidden_final is A + exp(G_total) * dhidden_final
 * (the scan is linear), which is what gla_sp_combine evaluates across ranks with
 * reverse != 0.  Workspace: gla_chunk_bwd_workspace_bytes for the same impl. */
GLA_API int gla_chunk_local_dstate(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                           int dtype, int impl,
                           const float* log_fgate, const void* query, const void* dout,
                           float* dS_local, void* workspace, size_t workspace_bytes);

/* ------------------------------------------------------------------------------------
 * Sequence parallelism in two phases per direction, so that a slice's chunk states are computed ONCE (no
 * counterpart in the reference; the algebra is the linearity of the state scan, ops.py:286-297).  Tensor-core
 * path only (bf16, D = 128, chunk a multiple of 128); other shapes return GLA_ERR_UNSUPPORTED and the caller
 * falls back to gla_chunk_local_state + gla_chunk_fwd.  `saved` (gla_chunk_saved_bytes) and `workspace`
 * (gla_chunk_fwd_workspace_bytes / gla_chunk_bwd_workspace_bytes, impl GLA_IMPL_TCGEN05) must be the SAME buffers,
 * untouched, in the local and the finish call of a direction; `saved` also goes from the forward to the backward.
 *
 *   gla_chunk_sp_fwd_local   the slice's chunk states from a ZERO initial state (left in `saved` with the
 *                            per-chunk log decays), its total log decay G_total (B, H, D) float32 and its final
 *                            state S_local (B, H, D, D) float32 (unrounded) for the exchange between ranks.
 *   gla_chunk_sp_fwd_finish  given H_in (B, H, D, D) float32, the true state entering the slice
 *                            (gla_sp_combine), adds exp(sum of the log decays of the chunks before n) (.) H_in to
 *                            the state entering chunk n, then runs the chunk kernel: `out` of the slice.
 *   gla_chunk_sp_bwd_local   gradient states from a ZERO final-state gradient (left in `workspace`) and
 *                            A_local (B, H, D, D) float32, the gradient reaching the slice's initial state.
 *   gla_chunk_sp_bwd_finish  given dH_out (B, H, D, D) float32, the true gradient of the slice's final state,
 *                            corrects the gradient states the same way (chunks after n) and runs the backward
 *                            chunk kernel: dlog_fgate, dvalue, dkey, dquery of the slice.
 * hidden_final and dhidden_init of the whole sequence come from gla_sp_combine (rank = R and rank = -1).
 * ---------------------------------------------------------------------------------- */
GLA_API int gla_chunk_sp_fwd_local(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                           int dtype, int impl, const float* log_fgate, const void* value, const void* key,
                           float* G_total, float* S_local, void* saved, void* workspace, size_t workspace_bytes);
GLA_API int gla_chunk_sp_fwd_finish(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                            int dtype, int impl, const float* H_in, const float* log_fgate, const void* value,
                            const void* key, const void* query, void* out, void* saved, void* workspace,
                            size_t workspace_bytes);
GLA_API int gla_chunk_sp_bwd_local(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                           int dtype, int impl, const float* log_fgate, const void* query, const void* dout,
                           const void* saved, float* A_local, void* workspace, size_t workspace_bytes);
GLA_API int gla_chunk_sp_bwd_finish(void* stream, int64_t B, int64_t T, int64_t H, int64_t D, int64_t chunk,
                            int dtype, int impl, const float* dH_out, const float* log_fgate, const void* value,
                            const void* key, const void* query, const void* saved, const void* dout,
                            float* dlog_fgate, void* dvalue, void* dkey, void* dquery, void* workspace,
                            size_t workspace_bytes);

GLA_API int gla_sp_combine(void* stream, int64_t R, int64_t rank, int64_t BH, int64_t D,
                   const float* all_G, const float* all_S,
                   const void* init, int init_dtype,
                   void* result, int result_dtype, int reverse);

/* The two results a rank needs from the gathered pairs, in one launch: `entering` (BH, D, D) float32, the state that
 * enters the slice of `rank` (0 <= rank < R; what gla_chunk_sp_fwd_finish / _bwd_finish take), and `total`, the state
 * that leaves the last slice in scan order (hidden_final of the whole sequence; with reverse != 0 dhidden_init).
 * Either may be NULL.  all_G / all_S need not be separate arrays: g_rank_stride / s_rank_stride are the distances
 * between consecutive ranks in floats, so one all-gather of a packed [G | S] record per rank serves
 * (all_S = all_G + BH * D, both strides BH * D * (D + 1)).  No counterpart in the reference (single device). */
GLA_API int gla_sp_combine2(void* stream, int64_t R, int64_t rank, int64_t BH, int64_t D,
                    const float* all_G, int64_t g_rank_stride, const float* all_S, int64_t s_rank_stride,
                    const void* init, int init_dtype, float* entering, void* total, int total_dtype, int reverse);

#ifdef __cplusplus
}
#endif
#endif /* GLA_B200_H_ */
