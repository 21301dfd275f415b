// Single-token step of gated linear attention with a persistent state (serving / decode path).
//
// One step of the reference's definitional recurrence (gla.py:26-47) for a batch of requests:
//     S <- exp(g) (.) S + k (x) v         (the decay multiplies along the key axis)
//     o  = q S
// with the state (B, H, D, D) kept in float32 in device memory between calls and updated in place;
// hidden_init -> hidden_final chaining of recurrent_gla is exact (gla.py:720-723), so T calls of this
// step equal one recurrent_gla call over T tokens.  The reference has no such entry point: its callers
// would run recurrent_gla with T = 1.
//
// The step is pure HBM streaming: 2 * 4 * D * D bytes of state per (request, head) against 5 D bytes of
// everything else.  A block owns 32 value columns of one head's state: 256 threads = 32 columns x 8 row
// lanes, each thread walks D / 8 key rows (coalesced 128-byte rows, loads of a whole 8-row group issued
// before they are used), keeps its partial of o, and the 8 row lanes are summed through shared memory.
#include "gla_common.cuh"

namespace gla {

constexpr int DC = 32;       // value columns per block
constexpr int DR = 8;        // row lanes

template <int D>
__global__ void __launch_bounds__(DC * DR) decode_step_kernel(float* __restrict__ S, const float* __restrict__ g,
                                                              const void* __restrict__ v, const void* __restrict__ k,
                                                              const void* __restrict__ q, void* __restrict__ out,
                                                              int bf, int out_bf) {
  constexpr int RPT = D / DR;                   // key rows per thread
  __shared__ float red[DR][DC];
  __shared__ float fk[3][D];                    // exp(g), k, q of this (request, head)
  const int col = threadIdx.x % DC, rl = threadIdx.x / DC;
  const int64_t bh = blockIdx.y;
  const int c0 = blockIdx.x * DC;
  for (int i = threadIdx.x; i < D; i += DC * DR) {
    fk[0][i] = expf(g[bh * D + i]);
    fk[1][i] = ld_any(k, bf, bh * D + i);
    fk[2][i] = ld_any(q, bf, bh * D + i);
  }
  const float vv = ld_any(v, bf, bh * D + c0 + col);
  float* Sp = S + (bh * D + rl) * (int64_t)D + c0 + col;     // rows rl, rl + 8, ...
  float s[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) s[i] = Sp[(int64_t)i * DR * D];
  __syncthreads();
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = rl + i * DR;
    const float ns = fmaf(fk[0][r], s[i], fk[1][r] * vv);
    Sp[(int64_t)i * DR * D] = ns;
    acc = fmaf(fk[2][r], ns, acc);
  }
  red[rl][col] = acc;
  __syncthreads();
  if (rl == 0) {
    float o = 0.f;
#pragma unroll
    for (int j = 0; j < DR; ++j) o += red[j][col];
    st_any(out, out_bf, bh * D + c0 + col, o);
  }
}

template <int D>
static int launch_decode(cudaStream_t st, int64_t BH, float* S, const float* g, const void* v, const void* k,
                         const void* q, void* out, int bf, int out_bf) {
  if (BH > 65535) return GLA_ERR_TOO_LARGE;
  ProfScope ps("decode_step_kernel", st);
  decode_step_kernel<D><<<dim3(D / DC, (unsigned)BH), DC * DR, 0, st>>>(S, g, v, k, q, out, bf, out_bf);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

int decode_step(cudaStream_t st, int64_t B, int64_t H, int64_t D, int bf, float* state, const float* g, const void* v,
                const void* k, const void* q, void* out, int out_bf) {
  const int64_t BH = B * H;
  switch (D) {
    case 32: return launch_decode<32>(st, BH, state, g, v, k, q, out, bf, out_bf);
    case 64: return launch_decode<64>(st, BH, state, g, v, k, q, out, bf, out_bf);
    case 128: return launch_decode<128>(st, BH, state, g, v, k, q, out, bf, out_bf);
    case 256: return launch_decode<256>(st, BH, state, g, v, k, q, out, bf, out_bf);
    default: return GLA_ERR_UNSUPPORTED;
  }
}

}  // namespace gla
