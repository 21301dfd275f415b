// Element-wise stages either side of the GLA op in a gated-linear-attention layer.
//
// The reference ships the op only (gla.py:657 chunk_gla); a caller wraps it as
//     log_fgate = log_sigmoid(z) / tau            z = low-rank projection of the layer input
//     o         = rmsnorm_per_head(out) * w * swish(gate)
// Both stages are pure HBM streaming, so each is one pass: the forget gate goes straight from the
// projection's dtype to the float32 log-gate the op takes (gla.py:483 wants log_fgate in float32),
// and the normalisation, its weight and the output gate are applied in the same pass over `out`.
//
//   gate_*          : flat arrays of n elements, grid-stride (consecutive threads, consecutive elements).
//   headnorm_gate_* : rows = B*T*H rows of D; one warp per row, D / 32 elements per lane held in
//                     registers between the sum of squares and the scaling; the weight gradient is
//                     reduced per block (registers -> shared memory) into a (blocks, D) partial
//                     array and summed by a second small launch, so that the result is deterministic.
#include "gla_common.cuh"

namespace gla {

namespace {

constexpr int LY_THREADS = 256;
constexpr int LY_WARPS = LY_THREADS / 32;

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(__expf(-fabsf(z))); }
__device__ __forceinline__ float sigmoid(float z) { return 1.f / (1.f + __expf(-z)); }

// EPL consecutive elements of a row, as the widest loads/stores the element count allows (the row
// base is 16-byte aligned: checked at the entry points).
template <int EPL>
__device__ __forceinline__ void ld_vec(const float* p, float (&o)[EPL]) {
  if constexpr (EPL % 4 == 0) {
#pragma unroll
    for (int e = 0; e < EPL; e += 4) {
      const float4 t = *reinterpret_cast<const float4*>(p + e);
      o[e] = t.x; o[e + 1] = t.y; o[e + 2] = t.z; o[e + 3] = t.w;
    }
  } else if constexpr (EPL == 2) {
    const float2 t = *reinterpret_cast<const float2*>(p);
    o[0] = t.x; o[1] = t.y;
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[e] = p[e];
  }
}
template <int EPL>
__device__ __forceinline__ void ld_vec(const bf16* p, float (&o)[EPL]) {
  if constexpr (EPL % 2 == 0) {
    uint32_t raw[EPL / 2];
    if constexpr (EPL == 8) {
      const uint4 t = *reinterpret_cast<const uint4*>(p);
      raw[0] = t.x; raw[1] = t.y; raw[2] = t.z; raw[3] = t.w;
    } else if constexpr (EPL == 4) {
      const uint2 t = *reinterpret_cast<const uint2*>(p);
      raw[0] = t.x; raw[1] = t.y;
    } else {
      raw[0] = *reinterpret_cast<const uint32_t*>(p);
    }
#pragma unroll
    for (int e = 0; e < EPL / 2; ++e) {
      o[2 * e] = __uint_as_float(raw[e] << 16);
      o[2 * e + 1] = __uint_as_float(raw[e] & 0xffff0000u);
    }
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[e] = __bfloat162float(p[e]);
  }
}
template <int EPL>
__device__ __forceinline__ void st_vec(float* p, const float (&v)[EPL]) {
  if constexpr (EPL % 4 == 0) {
#pragma unroll
    for (int e = 0; e < EPL; e += 4) *reinterpret_cast<float4*>(p + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
  } else if constexpr (EPL == 2) {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) p[e] = v[e];
  }
}
template <int EPL>
__device__ __forceinline__ void st_vec(bf16* p, const float (&v)[EPL]) {
  if constexpr (EPL % 2 == 0) {
    uint32_t raw[EPL / 2];
#pragma unroll
    for (int e = 0; e < EPL / 2; ++e) {
      const __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
      raw[e] = *reinterpret_cast<const uint32_t*>(&t);
    }
    if constexpr (EPL == 8) *reinterpret_cast<uint4*>(p) = make_uint4(raw[0], raw[1], raw[2], raw[3]);
    else if constexpr (EPL == 4) *reinterpret_cast<uint2*>(p) = make_uint2(raw[0], raw[1]);
    else *reinterpret_cast<uint32_t*>(p) = raw[0];
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) p[e] = __float2bfloat16_rn(v[e]);
  }
}

// Eight consecutive elements per thread and iteration (one 16-byte load of bfloat16, two of float32);
// the n % 8 tail, or everything when a pointer is not 16-byte aligned (n8 = 0), goes element by element.
template <typename TZ>
__global__ void __launch_bounds__(LY_THREADS) gate_fwd_kernel(int64_t n, int64_t n8, const TZ* __restrict__ z,
                                                              float inv_tau, float* __restrict__ g) {
  const int64_t stride = (int64_t)gridDim.x * LY_THREADS;
  const int64_t tid = (int64_t)blockIdx.x * LY_THREADS + threadIdx.x;
  for (int64_t i = tid; i < n8; i += stride) {
    float v[8];
    ld_vec<8>(z + 8 * i, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = inv_tau * log_sigmoid(v[e]);
    st_vec<8>(g + 8 * i, v);
  }
  for (int64_t i = 8 * n8 + tid; i < n; i += stride) g[i] = inv_tau * log_sigmoid(ld_f(z, i));
}

// d log_sigmoid(z) / dz = sigmoid(-z)
template <typename TZ>
__global__ void __launch_bounds__(LY_THREADS) gate_bwd_kernel(int64_t n, int64_t n8, const TZ* __restrict__ z,
                                                              const float* __restrict__ dg, float inv_tau,
                                                              TZ* __restrict__ dz) {
  const int64_t stride = (int64_t)gridDim.x * LY_THREADS;
  const int64_t tid = (int64_t)blockIdx.x * LY_THREADS + threadIdx.x;
  for (int64_t i = tid; i < n8; i += stride) {
    float v[8], d[8];
    ld_vec<8>(z + 8 * i, v);
    ld_vec<8>(dg + 8 * i, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = d[e] * inv_tau * sigmoid(-v[e]);
    st_vec<8>(dz + 8 * i, v);
  }
  for (int64_t i = 8 * n8 + tid; i < n; i += stride) st_f(dz, i, dg[i] * inv_tau * sigmoid(-ld_f(z, i)));
}

// y = x * rstd * w * swish(gate), rstd = rsqrt(mean_d x^2 + eps); EPL = D / 32 elements per lane,
// lane l owns the EPL consecutive elements starting at l * EPL.
template <typename TX, int EPL>
__global__ void __launch_bounds__(LY_THREADS) headnorm_gate_fwd_kernel(int64_t rows, const TX* __restrict__ x,
                                                                       const TX* __restrict__ gate,
                                                                       const float* __restrict__ w, float eps,
                                                                       TX* __restrict__ y, float* __restrict__ rstd_out) {
  constexpr int D = EPL * 32;
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  float wv[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) wv[e] = w ? w[lane * EPL + e] : 1.f;
  // two rows per warp and iteration, both rows' loads issued before either is used
  const int64_t stride = (int64_t)gridDim.x * LY_WARPS;
  for (int64_t r = (int64_t)blockIdx.x * LY_WARPS + warp; r < rows; r += 2 * stride) {
    const bool two = r + stride < rows;
    const int64_t o0 = r * D + lane * EPL, o1 = (two ? r + stride : r) * D + lane * EPL;
    float xv[2][EPL], gv[2][EPL];
    ld_vec<EPL>(x + o0, xv[0]);
    ld_vec<EPL>(gate + o0, gv[0]);
    ld_vec<EPL>(x + o1, xv[1]);
    ld_vec<EPL>(gate + o1, gv[1]);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u == 1 && !two) break;
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) ss = fmaf(xv[u][e], xv[u][e], ss);
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
      const float rs = rsqrtf(ss * (1.f / D) + eps);
      float yv[EPL];
#pragma unroll
      for (int e = 0; e < EPL; ++e) yv[e] = xv[u][e] * rs * wv[e] * gv[u][e] * sigmoid(gv[u][e]);
      st_vec<EPL>(y + (u ? o1 : o0), yv);
      if (lane == 0) rstd_out[u ? r + stride : r] = rs;
    }
  }
}

// With n = x * rstd, s = swish(gate), t = dy * s * w:
//   dx    = rstd * (t - n * mean_d(t n))
//   dgate = dy * n * w * sigmoid(gate) * (1 + gate * (1 - sigmoid(gate)))
//   dw    = sum over rows of dy * s * n        (per-block partials here)
template <typename TX, int EPL>
__global__ void __launch_bounds__(LY_THREADS) headnorm_gate_bwd_kernel(int64_t rows, const TX* __restrict__ x,
                                                                       const TX* __restrict__ gate,
                                                                       const float* __restrict__ w,
                                                                       const float* __restrict__ rstd,
                                                                       const TX* __restrict__ dy, TX* __restrict__ dx,
                                                                       TX* __restrict__ dgate,
                                                                       float* __restrict__ dw_partial) {
  constexpr int D = EPL * 32;
  __shared__ float red[LY_WARPS][D];
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  float wv[EPL], dwv[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    wv[e] = w ? w[lane * EPL + e] : 1.f;
    dwv[e] = 0.f;
  }
  // two rows per warp and iteration, both rows' loads issued before either is used
  const int64_t stride = (int64_t)gridDim.x * LY_WARPS;
  for (int64_t r = (int64_t)blockIdx.x * LY_WARPS + warp; r < rows; r += 2 * stride) {
    const bool two = r + stride < rows;
    const int64_t r1 = two ? r + stride : r;
    const int64_t o0 = r * D + lane * EPL, o1 = r1 * D + lane * EPL;
    float nv[2][EPL], gvv[2][EPL], dyv[2][EPL];
    ld_vec<EPL>(x + o0, nv[0]);
    ld_vec<EPL>(gate + o0, gvv[0]);
    ld_vec<EPL>(dy + o0, dyv[0]);
    ld_vec<EPL>(x + o1, nv[1]);
    ld_vec<EPL>(gate + o1, gvv[1]);
    ld_vec<EPL>(dy + o1, dyv[1]);
    const float rsv[2] = {rstd[r], rstd[r1]};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u == 1 && !two) break;
      const int64_t o = u ? o1 : o0;
      const float rs = rsv[u];
      float tv[EPL], outv[EPL];
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float gv = gvv[u][e];
        const float sg = sigmoid(gv);
        nv[u][e] *= rs;
        const float sw = gv * sg;
        tv[e] = dyv[u][e] * sw * wv[e];
        dot = fmaf(tv[e], nv[u][e], dot);
        dwv[e] = fmaf(dyv[u][e] * sw, nv[u][e], dwv[e]);
        outv[e] = dyv[u][e] * nv[u][e] * wv[e] * sg * (1.f + gv * (1.f - sg));
      }
      st_vec<EPL>(dgate + o, outv);
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
      const float m = dot * (1.f / D);
#pragma unroll
      for (int e = 0; e < EPL; ++e) outv[e] = rs * (tv[e] - nv[u][e] * m);
      st_vec<EPL>(dx + o, outv);
    }
  }
  if (dw_partial) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) red[warp][lane * EPL + e] = dwv[e];
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += LY_THREADS) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < LY_WARPS; ++k) s += red[k][d];
      dw_partial[(int64_t)blockIdx.x * D + d] = s;
    }
  }
}

// out[d] = sum over the rows of partial (nrows, D): a block owns 32 columns, its 8 row lanes walk
// the rows eight apart (four loads in flight each) and are summed through shared memory.
__global__ void __launch_bounds__(LY_THREADS) column_sum_kernel(int nrows, int D, const float* __restrict__ partial,
                                                               float* __restrict__ out) {
  __shared__ float red[LY_WARPS][33];
  const int tx = threadIdx.x % 32, rl = threadIdx.x / 32;
  const int d = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (d < D) {
    int r = rl;
    for (; r + 3 * LY_WARPS < nrows; r += 4 * LY_WARPS) {
      const float a = partial[(int64_t)r * D + d], b = partial[(int64_t)(r + LY_WARPS) * D + d];
      const float c = partial[(int64_t)(r + 2 * LY_WARPS) * D + d], e = partial[(int64_t)(r + 3 * LY_WARPS) * D + d];
      s += (a + b) + (c + e);
    }
    for (; r < nrows; r += LY_WARPS) s += partial[(int64_t)r * D + d];
  }
  red[rl][tx] = s;
  __syncthreads();
  if (rl == 0 && d < D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < LY_WARPS; ++k) t += red[k][tx];
    out[d] = t;
  }
}

int stream_grid(int64_t units_per_block_total) {
  // enough blocks to fill 148 SMs eight deep, never more than the work
  const int64_t cap = 148 * 8;
  return (int)(units_per_block_total < cap ? (units_per_block_total < 1 ? 1 : units_per_block_total) : cap);
}

int headnorm_blocks(int64_t rows) { return stream_grid((rows + LY_WARPS - 1) / LY_WARPS); }
// the backward leaves one row of weight-gradient partials per block: four blocks per SM keep that array short
int headnorm_bwd_blocks(int64_t rows) {
  const int64_t want = (rows + LY_WARPS - 1) / LY_WARPS;
  return (int)(want < 148 * 4 ? want : 148 * 4);
}

template <typename TX>
int headnorm_fwd_t(cudaStream_t st, int64_t rows, int64_t D, const void* x, const void* gate, const float* w, float eps,
                   void* y, float* rstd) {
  const int grid = headnorm_blocks(rows);
#define GLA_HN_FWD(E)                                                                                           \
  headnorm_gate_fwd_kernel<TX, E><<<grid, LY_THREADS, 0, st>>>(rows, (const TX*)x, (const TX*)gate, w, eps, (TX*)y, rstd)
  switch (D) {
    case 32: GLA_HN_FWD(1); break;
    case 64: GLA_HN_FWD(2); break;
    case 128: GLA_HN_FWD(4); break;
    case 256: GLA_HN_FWD(8); break;
    default: return GLA_ERR_UNSUPPORTED;
  }
#undef GLA_HN_FWD
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

template <typename TX>
int headnorm_bwd_t(cudaStream_t st, int64_t rows, int64_t D, const void* x, const void* gate, const float* w,
                   const float* rstd, const void* dy, void* dx, void* dgate, float* dw_partial) {
  const int grid = headnorm_bwd_blocks(rows);
#define GLA_HN_BWD(E)                                                                                          \
  headnorm_gate_bwd_kernel<TX, E><<<grid, LY_THREADS, 0, st>>>(rows, (const TX*)x, (const TX*)gate, w, rstd,   \
                                                               (const TX*)dy, (TX*)dx, (TX*)dgate, dw_partial)
  switch (D) {
    case 32: GLA_HN_BWD(1); break;
    case 64: GLA_HN_BWD(2); break;
    case 128: GLA_HN_BWD(4); break;
    case 256: GLA_HN_BWD(8); break;
    default: return GLA_ERR_UNSUPPORTED;
  }
#undef GLA_HN_BWD
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

}  // namespace

int layer_gate_fwd(cudaStream_t st, int64_t n, int bf, const void* z, float inv_tau, float* g) {
  const int64_t n8 = (aligned16(z) && aligned16(g)) ? n / 8 : 0;
  const int grid = stream_grid((n8 + (n - 8 * n8) + LY_THREADS - 1) / LY_THREADS);
  ProfScope ps("gate_fwd_kernel", st);
  if (bf) gate_fwd_kernel<bf16><<<grid, LY_THREADS, 0, st>>>(n, n8, (const bf16*)z, inv_tau, g);
  else gate_fwd_kernel<float><<<grid, LY_THREADS, 0, st>>>(n, n8, (const float*)z, inv_tau, g);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

int layer_gate_bwd(cudaStream_t st, int64_t n, int bf, const void* z, const float* dg, float inv_tau, void* dz) {
  const int64_t n8 = (aligned16(z) && aligned16(dg) && aligned16(dz)) ? n / 8 : 0;
  const int grid = stream_grid((n8 + (n - 8 * n8) + LY_THREADS - 1) / LY_THREADS);
  ProfScope ps("gate_bwd_kernel", st);
  if (bf) gate_bwd_kernel<bf16><<<grid, LY_THREADS, 0, st>>>(n, n8, (const bf16*)z, dg, inv_tau, (bf16*)dz);
  else gate_bwd_kernel<float><<<grid, LY_THREADS, 0, st>>>(n, n8, (const float*)z, dg, inv_tau, (float*)dz);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

int layer_headnorm_gate_fwd(cudaStream_t st, int64_t rows, int64_t D, int bf, const void* x, const void* gate,
                            const float* w, float eps, void* y, float* rstd) {
  ProfScope ps("headnorm_gate_fwd_kernel", st);
  return bf ? headnorm_fwd_t<bf16>(st, rows, D, x, gate, w, eps, y, rstd)
            : headnorm_fwd_t<float>(st, rows, D, x, gate, w, eps, y, rstd);
}

size_t layer_headnorm_gate_bwd_ws_bytes(int64_t rows, int64_t D) {
  return (size_t)headnorm_bwd_blocks(rows) * (size_t)D * sizeof(float);
}

int layer_headnorm_gate_bwd(cudaStream_t st, int64_t rows, int64_t D, int bf, const void* x, const void* gate,
                            const float* w, const float* rstd, const void* dy, void* dx, void* dgate, float* dweight,
                            void* ws) {
  float* partial = dweight ? (float*)ws : nullptr;
  {
    ProfScope ps("headnorm_gate_bwd_kernel", st);
    GLA_TRY(bf ? headnorm_bwd_t<bf16>(st, rows, D, x, gate, w, rstd, dy, dx, dgate, partial)
               : headnorm_bwd_t<float>(st, rows, D, x, gate, w, rstd, dy, dx, dgate, partial));
  }
  if (dweight) {
    ProfScope ps("column_sum_kernel", st);
    column_sum_kernel<<<(unsigned)((D + 31) / 32), LY_THREADS, 0, st>>>(headnorm_bwd_blocks(rows), (int)D,
                                                                                           partial, dweight);
    GLA_CHECK_LAUNCH();
  }
  return GLA_OK;
}

}  // namespace gla
