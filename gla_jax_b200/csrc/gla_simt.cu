// fp32 CUDA-core implementation of chunk_gla forward and backward.
//
// This is the precision path: every product is accumulated in float32 from float32 (or
// widened bf16) operands, so float32 inputs meet a 1e-4 relative-L2 tolerance, which the
// bf16 tensor-core path cannot.  It serves float32 callers, every (D, chunk) the
// tensor-core path has no kernel for, and it is the on-device cross-check of that path.
//
// Algorithm (reference: gla.py:483-625 chunk_gla_forward/backward, gla.py:695-790 inter-chunk
// terms, gla.py:792-960 intra-chunk terms):
//   lam    = within-chunk inclusive cumsum of log_fgate,  G = lam[last row]
//   k_hat  = k exp(G - lam),  q_hat = q exp(lam)
//   kv_n   = k_hat^T v ;  S_n = exp(G_n) S_{n-1} + kv_n ;  out = P v + q_hat S_{n-1}
//   P[i,j] = sum_d q[i,d] k[j,d] exp(lam[i,d] - lam[j,d])  (j <= i)
// The reference evaluates P through dyadic anchors (gla.py:985-1027) because it needs
// matmul-shaped work; with one thread group per (i, j) pair the exponent lam_i - lam_j <= 0
// is applied directly, which is the limit of that secondary chunking (anchor distance 0)
// and is unconditionally stable.  The dense products run through one generic tiled SGEMM.
#include "gla_common.cuh"

namespace gla {

// ---------------------------------------------------------------------------------------
// Generic batched SGEMM with strided, typed operands: for batch (b, h, n)
//   C(m, n) = sum_p sum_k A_p(m, k) B_p(k, n),   p < nprod <= 2
// 64 x 64 tile, K slab 16, 256 threads, 4 x 4 micro-tile.
// ---------------------------------------------------------------------------------------
struct Mat {
  const void* p;
  int bf;                 // 1 = bf16 elements, 0 = float32
  int64_t sb, sh, sn;     // element offsets per batch / head / chunk
  int64_t s0, s1;         // element strides of the two logical indices
};
struct GemmArgs {
  Mat A[2], B[2];
  int K[2];
  int nprod;
  void* C;
  int c_bf;
  int64_t csb, csh, csn, cm, cn;
  int M, N;
  int H, NC;              // batch decomposition: blockIdx.z = (b * H + h) * NC + n
  int tril;               // zero entries with column > row
};

constexpr int GT = 64, GK = 16, GP = 4;

__global__ void __launch_bounds__(256) gemm_kernel(GemmArgs a) {
  __shared__ __align__(16) float As[GK][GT + GP];
  __shared__ __align__(16) float Bs[GK][GT + GP];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int64_t z = blockIdx.z;
  const int64_t n_ = z % a.NC, h_ = (z / a.NC) % a.H, b_ = z / ((int64_t)a.NC * a.H);
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int p = 0; p < a.nprod; ++p) {
    const Mat& A = a.A[p];
    const Mat& B = a.B[p];
    const int64_t aoff = b_ * A.sb + h_ * A.sh + n_ * A.sn;
    const int64_t boff = b_ * B.sb + h_ * B.sh + n_ * B.sn;
    const bool a_kfast = (A.s1 == 1), b_kfast = (B.s0 == 1);
    const int K = a.K[p];
    for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        int idx = tid + 256 * r;
        int mm, kk;
        if (a_kfast) { mm = idx / GK; kk = idx % GK; } else { kk = idx / GT; mm = idx % GT; }
        float v = 0.f;
        if (m0 + mm < a.M && k0 + kk < K) v = ld_any(A.p, A.bf, aoff + (int64_t)(m0 + mm) * A.s0 + (int64_t)(k0 + kk) * A.s1);
        As[kk][mm] = v;
        int nn;
        if (b_kfast) { nn = idx / GK; kk = idx % GK; } else { kk = idx / GT; nn = idx % GT; }
        v = 0.f;
        if (n0 + nn < a.N && k0 + kk < K) v = ld_any(B.p, B.bf, boff + (int64_t)(k0 + kk) * B.s0 + (int64_t)(n0 + nn) * B.s1);
        Bs[kk][nn] = v;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < GK; ++kk) {
        const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
        const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
        const float ar[4] = {av.x, av.y, av.z, av.w};
        const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
  const int64_t coff = b_ * a.csb + h_ * a.csh + n_ * a.csn;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= a.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= a.N) continue;
      float v = acc[i][j];
      if (a.tril && n > m) v = 0.f;
      st_any(a.C, a.c_bf, coff + (int64_t)m * a.cm + (int64_t)n * a.cn, v);
    }
  }
}

static int launch_gemm(cudaStream_t st, const GemmArgs& a, int64_t batches) {
  ProfScope ps("simt_gemm_kernel", st);
  dim3 grid((a.N + GT - 1) / GT, (a.M + GT - 1) / GT, (unsigned)batches);
  if (batches > 65535) return GLA_ERR_TOO_LARGE;
  gemm_kernel<<<grid, 256, 0, st>>>(a);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

// Shape bundle used to build operand descriptors.
struct Dims {
  int64_t B, T, H, D, C, N;
  __host__ __device__ int64_t HD() const { return H * D; }
};
static Mat mat_bthd(const void* p, int bf, const Dims& d, bool transposed) {
  // chunk matrix (C rows of time, D columns); transposed swaps the logical indices
  Mat m{p, bf, d.T * d.H * d.D, d.D, d.C * d.H * d.D, d.H * d.D, 1};
  if (transposed) { m.s0 = 1; m.s1 = d.H * d.D; }
  return m;
}
static Mat mat_sq(const void* p, const Dims& d, int64_t R, bool transposed) {
  // per-chunk R x R float32 matrix in a (B*H, N, R, R) array
  Mat m{p, 0, d.H * d.N * R * R, d.N * R * R, R * R, R, 1};
  if (transposed) { m.s0 = 1; m.s1 = R; }
  return m;
}

// ---------------------------------------------------------------------------------------
// prep: k_hat = k exp(G - lam), q_hat = q exp(lam) (float32), and the compact per-chunk
// total log decay Gc (B*H, N, D).  One thread per element.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prep_kernel(Dims d, const float* __restrict__ lam, const void* k, const void* q,
                                                   int bf, float* __restrict__ khat, float* __restrict__ qhat,
                                                   float* __restrict__ Gc) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t total = d.B * d.T * d.H * d.D;
  if (e >= total) return;
  const int64_t dd = e % d.D, h = (e / d.D) % d.H, t = (e / (d.D * d.H)) % d.T, b = e / (d.D * d.H * d.T);
  const int64_t n = t / d.C;
  const float l = lam[e];
  const float G = lam[idx_bthd(b, n * d.C + d.C - 1, h, dd, d.T, d.H, d.D)];
  if (khat) khat[e] = ld_any(k, bf, e) * expf(G - l);
  if (qhat) qhat[e] = ld_any(q, bf, e) * expf(l);
  if (Gc && (t % d.C) == d.C - 1) Gc[((b * d.H + h) * d.N + n) * d.D + dd] = G;
}

// ---------------------------------------------------------------------------------------
// Intra-chunk gated score: P[i, j] = sum_d q[i,d] k[j,d] exp(lam[i,d] - lam[j,d]) for j <= i,
// 0 above the diagonal (gla.py:964-1029).  One warp per query row i; lanes stride over d
// (coalesced), the row's q and lam live in registers; a shuffle reduction per (i, j).
// grid = (C / 8, N, B*H), block = 256 (8 warps = 8 rows).  Supports D <= 256.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) score_kernel(Dims d, const float* __restrict__ lam, const void* k, const void* q,
                                                    int bf, float* __restrict__ P) {
  const int lane = threadIdx.x % 32, w = threadIdx.x / 32;
  const int i = blockIdx.x * 8 + w;
  const int64_t n = blockIdx.y, bh = blockIdx.z, b = bh / d.H, h = bh % d.H;
  const int64_t row0 = idx_bthd(b, n * d.C, h, 0, d.T, d.H, d.D);
  const int64_t HD = d.HD();
  float qi[8], li[8];
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const int dd = lane + 32 * m;
    qi[m] = dd < d.D ? ld_any(q, bf, row0 + i * HD + dd) : 0.f;
    li[m] = dd < d.D ? lam[row0 + i * HD + dd] : 0.f;
  }
  float* Pr = P + ((bh * d.N + n) * d.C + i) * d.C;
  for (int j = 0; j < d.C; ++j) {
    float s = 0.f;
    if (j <= i) {
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const int dd = lane + 32 * m;
        if (dd < d.D) {
          const float kj = ld_any(k, bf, row0 + j * HD + dd);
          const float lj = lam[row0 + j * HD + dd];
          s = fmaf(qi[m] * kj, expf(li[m] - lj), s);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    }
    if (lane == 0) Pr[j] = s;
  }
}

// ---------------------------------------------------------------------------------------
// Backward of the intra-chunk score plus the final assembly of dq, dk and dlam
// (gla.py:1036-1189, 892-901, 753-754, 778-786), one block per (chunk, row r), one thread
// per feature d:
//   dq[r,d] = sum_{j<=r} dP[r,j] k[j,d] e^{lam[r,d]-lam[j,d]} + dqh[r,d] e^{lam[r,d]}
//   dk[r,d] = sum_{i>=r} dP[i,r] q[i,d] e^{lam[i,d]-lam[r,d]} + dkh[r,d] e^{G[d]-lam[r,d]}
//   dlam    = q dq - k dk
// dqh = dO S_prev^T and dkh = V dS_next^T are precomputed by the SGEMM.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) intra_bwd_kernel(Dims d, const float* __restrict__ lam, const void* k,
                                                        const void* q, int bf, const float* __restrict__ dP,
                                                        const float* __restrict__ dqh, const float* __restrict__ dkh,
                                                        void* dq_out, void* dk_out, float* __restrict__ dlam) {
  const int dd = threadIdx.x;
  const int r = blockIdx.x;
  const int64_t n = blockIdx.y, bh = blockIdx.z, b = bh / d.H, h = bh % d.H;
  if (dd >= d.D) return;
  const int64_t row0 = idx_bthd(b, n * d.C, h, 0, d.T, d.H, d.D);
  const int64_t HD = d.HD();
  const float* dPc = dP + (bh * d.N + n) * d.C * d.C;
  const int64_t er = row0 + r * HD + dd;
  const float lr = lam[er];
  const float qr = ld_any(q, bf, er), kr = ld_any(k, bf, er);
  const float G = lam[row0 + (d.C - 1) * HD + dd];
  float dq = 0.f, dk = 0.f;
  for (int j = 0; j <= r; ++j) {
    const int64_t ej = row0 + j * HD + dd;
    dq = fmaf(dPc[r * d.C + j] * ld_any(k, bf, ej), expf(lr - lam[ej]), dq);
  }
  for (int i = r; i < d.C; ++i) {
    const int64_t ei = row0 + i * HD + dd;
    dk = fmaf(dPc[i * d.C + r] * ld_any(q, bf, ei), expf(lam[ei] - lr), dk);
  }
  dq = fmaf(dqh[er], expf(lr), dq);
  dk = fmaf(dkh[er], expf(G - lr), dk);
  st_any(dq_out, bf, er, dq);
  st_any(dk_out, bf, er, dk);
  dlam[er] = qr * dq - kr * dk;
}

// dG[bh, n, d] = sum_c dkh[c,d] k_hat[c,d] + sum_v S_prev[d,v] exp(G[d]) dS_next[d,v]  (gla.py:782)
// One warp per (bh, n, d): lanes stride over c then over v.
__global__ void __launch_bounds__(256) dG_kernel(Dims d, const float* __restrict__ dkh, const float* __restrict__ khat,
                                                 const float* __restrict__ Gc, const float* __restrict__ S_prev,
                                                 const float* __restrict__ dS_next, float* __restrict__ dG) {
  const int lane = threadIdx.x % 32;
  const int64_t wid = (int64_t)blockIdx.x * 8 + threadIdx.x / 32;
  const int64_t total = d.B * d.H * d.N * d.D;
  if (wid >= total) return;
  const int64_t dd = wid % d.D, n = (wid / d.D) % d.N, bh = wid / (d.D * d.N), b = bh / d.H, h = bh % d.H;
  const int64_t row0 = idx_bthd(b, n * d.C, h, dd, d.T, d.H, d.D);
  float s = 0.f;
  for (int c = lane; c < d.C; c += 32) s = fmaf(dkh[row0 + c * d.HD()], khat[row0 + c * d.HD()], s);
  const float eg = expf(Gc[(bh * d.N + n) * d.D + dd]);
  const int64_t so = ((bh * d.N + n) * d.D + dd) * d.D;
  float s2 = 0.f;
  for (int v = lane; v < d.D; v += 32) s2 = fmaf(S_prev[so + v], dS_next[so + v], s2);
  s = fmaf(eg, s2, s);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) dG[wid] = s;
}

// Sum of G over the chunks of a slice: G_total (B*H, D) = sum_n Gc[bh, n, d].
__global__ void __launch_bounds__(256) gsum_kernel(int64_t BH, int64_t N, int64_t D, const float* __restrict__ Gc,
                                                   float* __restrict__ Gt) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= BH * D) return;
  const int64_t bh = e / D, dd = e % D;
  float s = 0.f;
  for (int64_t n = 0; n < N; ++n) s += Gc[(bh * N + n) * D + dd];
  Gt[e] = s;
}

// ---------------------------------------------------------------------------------------
// Buffer layouts.
//   saved     : S_prev (BH,N,D,D) f32 | Gc (BH,N,D) f32 | P (BH,N,C,C) f32
//   fwd ws    : lam (BTHD) | khat | qhat | kv (BH,N,D,D)          all f32
//   bwd ws    : lam | khat | qhat | dstate->dS_next (BH,N,D,D) | dP (BH,N,C,C) | dqh | dkh | dG (BH,N,D)
//               (dlam overwrites qhat once qhat is dead)
// ---------------------------------------------------------------------------------------
static size_t f32b(int64_t n) { return align_up((size_t)n * 4, 256); }

size_t simt_saved_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C) {
  int64_t N = T / C, BH = B * H;
  return f32b(BH * N * D * D) + f32b(BH * N * D) + f32b(BH * N * C * C);
}
// The k_hat region doubles as the score buffer of a forward without residuals: (BH, N, C, C) floats, which is
// larger than (B, T, H, D) when chunk > D, so the region is sized for the larger of the two.
static int64_t khat_region_elems(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C) { return B * T * H * (D > C ? D : C); }
size_t simt_fwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C) {
  int64_t N = T / C, BH = B * H, E = B * T * H * D;
  return 2 * f32b(E) + f32b(khat_region_elems(B, T, H, D, C)) + f32b(BH * N * D * D) + f32b(BH * N * D);
}
size_t simt_bwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C) {
  int64_t N = T / C, BH = B * H, E = B * T * H * D;
  return 5 * f32b(E) + f32b(BH * N * D * D) + f32b(BH * N * C * C) + f32b(BH * N * D);
}

int simt_chunk_fwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C, int bf,
                   const void* hidden_init, const float* g, const void* v, const void* k, const void* q,
                   void* hidden_final, void* out, void* saved, void* ws, int state_only,
                   float* G_total, float* S_local) {
  Dims d{B, T, H, D, C, T / C};
  const int64_t N = d.N, BH = B * H, E = B * T * H * D;
  // every size limit of the launches below, before the first of them
  if (N > 65535 || BH > 65535 || BH * N > 65535) return GLA_ERR_TOO_LARGE;
  char* w = (char*)ws;
  float* lam = (float*)w;  w += f32b(E);
  float* khat = (float*)w; w += f32b(khat_region_elems(B, T, H, D, C));
  float* qhat = (float*)w; w += f32b(E);
  float* kv = (float*)w;   w += f32b(BH * N * D * D);
  float* Gc_ws = (float*)w;
  float *S_prev = nullptr, *Gc = Gc_ws, *P = nullptr;
  if (saved) {
    char* s = (char*)saved;
    S_prev = (float*)s; s += f32b(BH * N * D * D);
    Gc = (float*)s;     s += f32b(BH * N * D);
    P = (float*)s;
  }
  // lam: within-chunk cumsum, viewing g as (B*N, C, H*D)
  GLA_TRY(launch_cumsum(st, B * N, C, H * D, g, nullptr, lam, 0, 0, 0));
  {
    ProfScope ps_prep_kernel("simt_prep_kernel", st);
    prep_kernel<<<(unsigned)((E + 255) / 256), 256, 0, st>>>(d, lam, k, q, bf, khat, state_only ? nullptr : qhat, Gc);
  }
  GLA_CHECK_LAUNCH();
  {  // kv = k_hat^T v
    GemmArgs a{};
    a.nprod = 1; a.A[0] = mat_bthd(khat, 0, d, true); a.B[0] = mat_bthd(v, bf, d, false); a.K[0] = (int)C;
    a.C = kv; a.c_bf = 0; a.csb = H * N * D * D; a.csh = N * D * D; a.csn = D * D; a.cm = D; a.cn = 1;
    a.M = (int)D; a.N = (int)D; a.H = (int)H; a.NC = (int)N; a.tril = 0;
    GLA_TRY(launch_gemm(st, a, BH * N));
  }
  if (state_only) {
    GLA_TRY(launch_state_scan(st, BH, N, D, Gc, kv, 0, nullptr, 0, nullptr, 0, S_local, 0, 0));
    ProfScope ps_gsum_kernel("simt_gsum_kernel", st);
    gsum_kernel<<<(unsigned)((BH * D + 255) / 256), 256, 0, st>>>(BH, N, D, Gc, G_total);
    GLA_CHECK_LAUNCH();
    return GLA_OK;
  }
  // states entering each chunk (in place over kv when nothing is saved) and hidden_final
  float* before = S_prev ? S_prev : kv;
  GLA_TRY(launch_state_scan(st, BH, N, D, Gc, kv, 0, hidden_init, bf, before, 0, hidden_final, bf, 0));
  // scores; without a residual buffer they go to the (dead) k_hat region, which is sized for them
  float* Pbuf = P ? P : khat;
  {
    dim3 grid((unsigned)(C / 8), (unsigned)N, (unsigned)BH);
    ProfScope ps_score_kernel("simt_score_kernel", st);
    score_kernel<<<grid, 256, 0, st>>>(d, lam, k, q, bf, Pbuf);
    GLA_CHECK_LAUNCH();
  }
  {  // out = P v + q_hat S_prev
    GemmArgs a{};
    a.nprod = 2;
    a.A[0] = mat_sq(Pbuf, d, C, false); a.B[0] = mat_bthd(v, bf, d, false); a.K[0] = (int)C;
    a.A[1] = mat_bthd(qhat, 0, d, false); a.B[1] = mat_sq(before, d, D, false); a.K[1] = (int)D;
    a.C = out; a.c_bf = bf; a.csb = T * H * D; a.csh = D; a.csn = C * H * D; a.cm = H * D; a.cn = 1;
    a.M = (int)C; a.N = (int)D; a.H = (int)H; a.NC = (int)N; a.tril = 0;
    GLA_TRY(launch_gemm(st, a, BH * N));
  }
  return GLA_OK;
}

__global__ void __launch_bounds__(256) dG_transpose_kernel(int64_t B, int64_t H, int64_t N, int64_t D,
                                                           const float* __restrict__ in, float* __restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= B * H * N * D) return;
  const int64_t dd = e % D, h = (e / D) % H, n = (e / (D * H)) % N, b = e / (D * H * N);
  out[e] = in[((b * H + h) * N + n) * D + dd];
}
static int launch_dG_transpose(cudaStream_t st, int64_t B, int64_t H, int64_t N, int64_t D, const float* in, float* out) {
  const int64_t n = B * H * N * D;
  ProfScope ps_dG_transpose_kernel("simt_dG_transpose_kernel", st);
  dG_transpose_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(B, H, N, D, in, out);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

int simt_chunk_bwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C, int bf,
                   const float* g, const void* v, const void* k, const void* q, const void* saved,
                   const void* dhidden_final, const void* dout, void* dhidden_init, float* dg,
                   void* dv, void* dk, void* dq, void* ws) {
  Dims d{B, T, H, D, C, T / C};
  const int64_t N = d.N, BH = B * H, E = B * T * H * D;
  if (N > 65535 || BH > 65535 || BH * N > 65535) return GLA_ERR_TOO_LARGE;
  char* w = (char*)ws;
  float* lam = (float*)w;  w += f32b(E);
  float* khat = (float*)w; w += f32b(E);
  float* qhat = (float*)w; w += f32b(E);
  float* dqh = (float*)w;  w += f32b(E);
  float* dkh = (float*)w;  w += f32b(E);
  float* dS = (float*)w;   w += f32b(BH * N * D * D);
  float* dP = (float*)w;   w += f32b(BH * N * C * C);
  float* dG = (float*)w;
  const char* s = (const char*)saved;
  const float* S_prev = (const float*)s; s += f32b(BH * N * D * D);
  const float* Gc = (const float*)s;     s += f32b(BH * N * D);
  const float* P = (const float*)s;

  GLA_TRY(launch_cumsum(st, B * N, C, H * D, g, nullptr, lam, 0, 0, 0));
  {
    ProfScope ps_prep_kernel("simt_prep_kernel", st);
    prep_kernel<<<(unsigned)((E + 255) / 256), 256, 0, st>>>(d, lam, k, q, bf, khat, qhat, nullptr);
  }
  GLA_CHECK_LAUNCH();
  auto sq_out = [&](GemmArgs& a, float* C_, int64_t R) {
    a.C = C_; a.c_bf = 0; a.csb = H * N * R * R; a.csh = N * R * R; a.csn = R * R; a.cm = R; a.cn = 1;
    a.H = (int)H; a.NC = (int)N;
  };
  auto bthd_out = [&](GemmArgs& a, void* C_, int cbf) {
    a.C = C_; a.c_bf = cbf; a.csb = T * H * D; a.csh = D; a.csn = C * H * D; a.cm = H * D; a.cn = 1;
    a.H = (int)H; a.NC = (int)N;
  };
  {  // dstate = q_hat^T dO
    GemmArgs a{};
    a.nprod = 1; a.A[0] = mat_bthd(qhat, 0, d, true); a.B[0] = mat_bthd(dout, bf, d, false); a.K[0] = (int)C;
    sq_out(a, dS, D); a.M = (int)D; a.N = (int)D;
    GLA_TRY(launch_gemm(st, a, BH * N));
  }
  // reverse scan in place: dS[n] <- y_{n+1}; dhidden_init = y_0
  GLA_TRY(launch_state_scan(st, BH, N, D, Gc, dS, 0, dhidden_final, bf, dS, 0, dhidden_init, bf, 1));
  {  // dP = tril(dO v^T)
    GemmArgs a{};
    a.nprod = 1; a.A[0] = mat_bthd(dout, bf, d, false); a.B[0] = mat_bthd(v, bf, d, true); a.K[0] = (int)D;
    sq_out(a, dP, C); a.M = (int)C; a.N = (int)C; a.tril = 1;
    GLA_TRY(launch_gemm(st, a, BH * N));
  }
  {  // dv = P^T dO + k_hat dS_next
    GemmArgs a{};
    a.nprod = 2;
    a.A[0] = mat_sq(P, d, C, true); a.B[0] = mat_bthd(dout, bf, d, false); a.K[0] = (int)C;
    a.A[1] = mat_bthd(khat, 0, d, false); a.B[1] = mat_sq(dS, d, D, false); a.K[1] = (int)D;
    bthd_out(a, dv, bf); a.M = (int)C; a.N = (int)D;
    GLA_TRY(launch_gemm(st, a, BH * N));
  }
  {  // dqh = dO S_prev^T
    GemmArgs a{};
    a.nprod = 1; a.A[0] = mat_bthd(dout, bf, d, false); a.B[0] = mat_sq(S_prev, d, D, true); a.K[0] = (int)D;
    bthd_out(a, dqh, 0); a.M = (int)C; a.N = (int)D;
    GLA_TRY(launch_gemm(st, a, BH * N));
  }
  {  // dkh = v dS_next^T
    GemmArgs a{};
    a.nprod = 1; a.A[0] = mat_bthd(v, bf, d, false); a.B[0] = mat_sq(dS, d, D, true); a.K[0] = (int)D;
    bthd_out(a, dkh, 0); a.M = (int)C; a.N = (int)D;
    GLA_TRY(launch_gemm(st, a, BH * N));
  }
  {
    const int64_t nw = BH * N * D;
    ProfScope ps_dG_kernel("simt_dG_kernel", st);
    dG_kernel<<<(unsigned)((nw + 7) / 8), 256, 0, st>>>(d, dkh, khat, Gc, S_prev, dS, dG);
    GLA_CHECK_LAUNCH();
  }
  float* dlam = qhat;   // q_hat is dead from here on
  {
    dim3 grid((unsigned)C, (unsigned)N, (unsigned)BH);
    ProfScope ps_intra_bwd_kernel("simt_intra_bwd_kernel", st);
    intra_bwd_kernel<<<grid, 256, 0, st>>>(d, lam, k, q, bf, dP, dqh, dkh, dq, dk, dlam);
    GLA_CHECK_LAUNCH();
  }
  // dg = reverse within-chunk cumsum of dlam + dG.  dG is (BH, N, D); the cumsum view is
  // (B*N, C, H*D) whose init must be laid out (B, N, H, D): re-order while summing.
  // The init for batch row (b, n) and column (h, d) is dG[(b*H + h), n, d]; the cumsum
  // kernel indexes init as init[(b*N + n) * (H*D) + h*D + d], so transpose first.
  {
    float* dGt = dqh;   // dqh is dead; holds (B, N, H, D)
    GLA_TRY(launch_dG_transpose(st, B, H, N, D, dG, dGt));
    GLA_TRY(launch_cumsum(st, B * N, C, H * D, dlam, dGt, dg, 1, 0, 0));
  }
  return GLA_OK;
}

// Gradient reaching the slice's initial state for a zero final-state gradient (used by the
// sequence-parallel backward): only dstate = q_hat^T dO and the reverse scan run.
int simt_chunk_dstate_only(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C, int bf,
                           const float* g, const void* q, const void* dout, float* dS_local, void* ws) {
  Dims d{B, T, H, D, C, T / C};
  const int64_t N = d.N, BH = B * H, E = B * T * H * D;
  if (N > 65535 || BH > 65535 || BH * N > 65535) return GLA_ERR_TOO_LARGE;
  char* w = (char*)ws;
  float* lam = (float*)w;  w += f32b(E);
  w += f32b(E);
  float* qhat = (float*)w; w += f32b(E);
  w += 2 * f32b(E);
  float* dS = (float*)w;   w += f32b(BH * N * D * D);
  w += f32b(BH * N * C * C);
  float* Gc = (float*)w;
  GLA_TRY(launch_cumsum(st, B * N, C, H * D, g, nullptr, lam, 0, 0, 0));
  {
    ProfScope ps_prep_kernel("simt_prep_kernel", st);
    prep_kernel<<<(unsigned)((E + 255) / 256), 256, 0, st>>>(d, lam, nullptr, q, bf, nullptr, qhat, Gc);
  }
  GLA_CHECK_LAUNCH();
  GemmArgs a{};
  a.nprod = 1; a.A[0] = mat_bthd(qhat, 0, d, true); a.B[0] = mat_bthd(dout, bf, d, false); a.K[0] = (int)C;
  a.C = dS; a.c_bf = 0; a.csb = H * N * D * D; a.csh = N * D * D; a.csn = D * D; a.cm = D; a.cn = 1;
  a.M = (int)D; a.N = (int)D; a.H = (int)H; a.NC = (int)N;
  GLA_TRY(launch_gemm(st, a, BH * N));
  return launch_state_scan(st, BH, N, D, Gc, dS, 0, nullptr, 0, nullptr, 0, dS_local, 0, 1);
}

}  // namespace gla
