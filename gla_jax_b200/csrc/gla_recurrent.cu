// recurrent_gla forward and backward: the exact step recurrence with the state tile held in
// registers and never written to memory.
//
// Reference: gla.py:50-96 (forward kernel), gla.py:271-360 (backward kernel), gla.py:99-170,
// 172-269 (wrappers).  The reference tiles the state over (head, key block, value block)
// programs of one warp each and sums per-block partial outputs afterwards (gla.py:140,166,
// 210-214,257-259).  Here the state is SLICED along one axis only, so that the reduction
// each pass needs runs over the axis a thread block holds completely, and no partial sums
// ever reach memory:
//
//   pass      slice axis   per step                                         reduction
//   FWD       value        S = f (.) S + k (x) v_s                          o_s  = sum_k q S
//   DQ        key          S = f_s S + k_s v            (recompute)         dq_s = sum_v dO S
//   DV        value        dS = dC + q (x) dO_s ; dC = f (.) dS  (reverse)  dv_s = sum_k k dS
//   DK        key          dS = dC + q_s dO     ; dC = f_s dS    (reverse)  dk_s = sum_v v dS
//
// A block owns a 16-wide slice and all D entries of the other ("long") axis.  The kernel is bound by
// the shared-memory / shuffle pipe, not by FMAs, so the thread layout is chosen to reuse what a thread
// reads: LP = min(32, D/4) lanes span the long axis (a warp's 16-byte loads cover a whole row of a
// staged tile), and each thread carries the state of its D/LP long entries for FOUR slice entries, so
// every tile value it loads feeds four recurrences.  The four per-step sums are reduced over the
// lanes by a transposing butterfly (2 + 1 + log2(LP/4) shuffles instead of 4 log2(LP)).
// Time is processed in blocks of 32 steps staged through shared memory in
// float32 (gate already exponentiated), with the next block's global loads in flight
// during the current block's arithmetic.  dlog_fgate follows gla.py:263:
//   dg = cumsum over the remaining tokens of (q dq - k dk) + sum_v(dS_T * S_T).
#include "gla_common.cuh"

namespace gla {

constexpr int RB = 32;      // time steps per staged block
constexpr int RS = 16;      // slice width
constexpr int NSI = 4;      // slice entries per thread (4 or 2)
constexpr int rec_lanes(int D) { return D / 4 < 32 ? D / 4 : 32; }     // lanes along the long axis
constexpr int rec_threads(int D) { return (RS / NSI) * rec_lanes(D); }

enum RecMode { REC_FWD = 0, REC_DQ = 1, REC_DV = 2, REC_DK = 3 };

struct RecParams {
  int64_t B, T, H;
  int bf, do_bf, out_bf;     // element types: inputs/hidden/grads, dout, out
  const void* hidden_init;
  const float* g;
  const void *v, *k, *q;
  const void* dhidden_final;
  const void* dout;
  void* hidden_final;
  void* out;
  void *dq, *dk, *dv, *dhidden_init;
  float* E;                  // (B,T,H,D) float32: q dq
  float* F;                  // (B,T,H,D) float32: k dk  (dlog_fgate is a suffix sum of E - F)
  float* boundary;           // (B,H,D) float32: sum_v dS_T * S_T
  int time_reversed;         // process tokens from last to first
};

// Packed pairs of float32 in one 64-bit register: Blackwell's two-wide FMA halves the issue slots
// of the state update, which is what bounds these kernels (few warps per SM, long straight-line steps).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 x2_pack(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void x2_unpack(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 x2_fma(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 x2_mul(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// Sum over the LP consecutive lanes of a lane group.
template <int LP>
__device__ __forceinline__ float reduce_lanes(float x) {
#pragma unroll
  for (int o = 1; o < LP; o <<= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
// Four sums at once: after two exchange stages each lane holds one of the four values summed over its
// group of four lanes, the remaining stages sum that value over the other lanes.  On return lane lp
// (lp < 4) of the group holds the total of v[rec_which(lp)].
template <int LP>
__device__ __forceinline__ float reduce4_lanes(const float (&v)[4], int lp) {
  const bool o1 = (lp & 1) != 0, o2 = (lp & 2) != 0;
  float a0 = o1 ? v[2] : v[0], a1 = o1 ? v[3] : v[1];
  a0 += __shfl_xor_sync(0xffffffffu, o1 ? v[0] : v[2], 1);
  a1 += __shfl_xor_sync(0xffffffffu, o1 ? v[1] : v[3], 1);
  float b = o2 ? a1 : a0;
  b += __shfl_xor_sync(0xffffffffu, o2 ? a0 : a1, 2);
#pragma unroll
  for (int o = 4; o < LP; o <<= 1) b += __shfl_xor_sync(0xffffffffu, b, o);
  return b;
}
__device__ __forceinline__ int rec_which(int lp) { return NSI == 4 ? 2 * (lp & 1) + ((lp >> 1) & 1) : (lp & 1); }
template <int LP>
__device__ __forceinline__ float reduce2_lanes(const float (&v)[2], int lp) {
  const bool o1 = (lp & 1) != 0;
  float b = o1 ? v[1] : v[0];
  b += __shfl_xor_sync(0xffffffffu, o1 ? v[0] : v[1], 1);
#pragma unroll
  for (int o = 2; o < LP; o <<= 1) b += __shfl_xor_sync(0xffffffffu, b, o);
  return b;
}
template <int LP, int N>
__device__ __forceinline__ float reduceN_lanes(const float (&v)[N], int lp) {
  if constexpr (N == 4) return reduce4_lanes<LP>(v, lp); else return reduce2_lanes<LP>(v, lp);
}

// A staged tile source: column window [c0, c0 + W) of a (B,T,H,D) array for one (b, h).
struct TileSrc {
  const void* p;
  int bf;
  int do_exp;
};

// A staged tile of RB rows x W columns is fetched in groups of four consecutive elements (one 8- or
// 16-byte load per group; group index = threadIdx.x + RTHREADS * i).  The fetch only issues the
// loads and parks the RAW bits in registers: nothing in it consumes a loaded value, so all of a
// thread's loads are in flight together (a conversion right behind each load would stall the
// in-order warp for a full memory latency per load).  tile_commit converts and stores to smem.
template <int W, int NG, int RTHREADS>
__device__ __forceinline__ void tile_fetch(uint4 (&raw)[NG], const TileSrc& s, int64_t base, int64_t row_stride,
                                           int64_t step0, int64_t T, int time_reversed, int c0) {
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    const int e = (threadIdx.x + RTHREADS * i) * 4;
    const int row = e / W, col = e % W;
    const int64_t sidx = step0 + row;
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (e < RB * W && sidx < T) {
      const int64_t t = time_reversed ? (T - 1 - sidx) : sidx;
      const int64_t off = base + t * row_stride + c0 + col;
      if (s.bf) {
        const uint2 w = __ldg(reinterpret_cast<const uint2*>((const bf16*)s.p + off));
        u.x = w.x; u.y = w.y;
      } else {
        u = __ldg(reinterpret_cast<const uint4*>((const float*)s.p + off));
      }
    }
    raw[i] = u;
  }
}
template <int W, int NG, int RTHREADS>
__device__ __forceinline__ void tile_commit(float* sm, const uint4 (&raw)[NG], int is_bf16, int do_exp) {
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    const int e = (threadIdx.x + RTHREADS * i) * 4;
    if (e < RB * W) {
      const uint4 u = raw[i];
      float4 o;
      if (is_bf16) {
        o.x = __uint_as_float(u.x << 16); o.y = __uint_as_float(u.x & 0xffff0000u);
        o.z = __uint_as_float(u.y << 16); o.w = __uint_as_float(u.y & 0xffff0000u);
      } else {
        o.x = __uint_as_float(u.x); o.y = __uint_as_float(u.y); o.z = __uint_as_float(u.z); o.w = __uint_as_float(u.w);
      }
      if (do_exp) { o.x = expf(o.x); o.y = expf(o.y); o.z = expf(o.z); o.w = expf(o.w); }
      *reinterpret_cast<float4*>(sm + e) = o;
    }
  }
}

template <int D, int MODE>
__device__ __forceinline__ void rec_body(const RecParams& p, const int64_t b) {
  constexpr int LP = rec_lanes(D), RTHREADS = rec_threads(D);
  constexpr int KP = D / LP;                      // long entries per thread (x NSI slice entries of state)
  constexpr int NL = (MODE == REC_FWD || MODE == REC_DV) ? 3 : 2;   // long tiles
  constexpr int NS = (MODE == REC_FWD || MODE == REC_DV) ? 1 : 3;   // slice tiles
  constexpr int LG = RB * D / RTHREADS / 4;       // long-tile groups of four elements per thread
  constexpr int SG = (RB * RS / 4 + RTHREADS - 1) / RTHREADS;       // slice-tile groups per thread
  extern __shared__ __align__(16) float smem[];
  // tile offsets inside the one shared array (plain offsets, not pointer tables, so that every
  // access is compiled as a shared-memory access)
  constexpr int L_OFF = RB * D, S_BASE = NL * RB * D, S_OFF = RB * RS, R_BASE = NL * RB * D + NS * RB * RS;

  const int lp = threadIdx.x % LP, sg = threadIdx.x / LP;     // lane on the long axis, group of NSI slice entries
  const int c0 = blockIdx.x * RS;                 // slice window
  const int64_t h = blockIdx.y;
  const int64_t T = p.T, HD = p.H * D;
  const int64_t base = (b * T * p.H + h) * D;     // element (b, 0, h, 0)
  const int64_t hbase = (b * p.H + h) * (int64_t)D * D;
  const bool bwd_pass = (MODE == REC_DV || MODE == REC_DK);
  const int trev = p.time_reversed ^ (bwd_pass ? 1 : 0);
  const bool slice_is_value = (MODE == REC_FWD || MODE == REC_DV);

  // long / slice tile sources per mode
  TileSrc Lsrc[3], Ssrc[3];
  if (MODE == REC_FWD) {
    Lsrc[0] = {p.g, 0, 1}; Lsrc[1] = {p.k, p.bf, 0}; Lsrc[2] = {p.q, p.bf, 0};
    Ssrc[0] = {p.v, p.bf, 0};
  } else if (MODE == REC_DQ) {
    Lsrc[0] = {p.v, p.bf, 0}; Lsrc[1] = {p.dout, p.do_bf, 0};
    Ssrc[0] = {p.g, 0, 1}; Ssrc[1] = {p.k, p.bf, 0}; Ssrc[2] = {p.q, p.bf, 0};
  } else if (MODE == REC_DV) {
    Lsrc[0] = {p.g, 0, 1}; Lsrc[1] = {p.k, p.bf, 0}; Lsrc[2] = {p.q, p.bf, 0};
    Ssrc[0] = {p.dout, p.do_bf, 0};
  } else {
    Lsrc[0] = {p.v, p.bf, 0}; Lsrc[1] = {p.dout, p.do_bf, 0};
    Ssrc[0] = {p.g, 0, 1}; Ssrc[1] = {p.k, p.bf, 0}; Ssrc[2] = {p.q, p.bf, 0};
  }

  // state: element (long index L(i), slice index c0 + NSI sg + j); memory layout [key][value]
  auto long_index = [&](int i) { return 4 * lp + 4 * LP * (i / 4) + (i % 4); };
  auto state_addr = [&](int i, int j) -> int64_t {
    const int L = long_index(i), c = c0 + NSI * sg + j;
    return slice_is_value ? hbase + (int64_t)L * D + c : hbase + (int64_t)c * D + L;
  };
  float st[KP][NSI];
  {
    const void* init = bwd_pass ? p.dhidden_final : p.hidden_init;
#pragma unroll
    for (int i = 0; i < KP; ++i)
#pragma unroll
      for (int j = 0; j < NSI; ++j) st[i][j] = init ? ld_any(init, p.bf, state_addr(i, j)) : 0.f;
  }

  uint4 lreg[NL][LG];
  uint4 sreg[NS][SG];
  auto fetch = [&](int64_t step0) {
#pragma unroll
    for (int a = 0; a < NL; ++a) tile_fetch<D, LG, RTHREADS>(lreg[a], Lsrc[a], base, HD, step0, T, trev, 0);
#pragma unroll
    for (int a = 0; a < NS; ++a) tile_fetch<RS, SG, RTHREADS>(sreg[a], Ssrc[a], base, HD, step0, T, trev, c0);
  };
  fetch(0);
  // the state as pairs along the long axis: st2[i][j] = (st[2i][j], st[2i+1][j])
  f32x2 st2[KP / 2][NSI];
#pragma unroll
  for (int i = 0; i < KP / 2; ++i)
#pragma unroll
    for (int j = 0; j < NSI; ++j) st2[i][j] = x2_pack(st[2 * i][j], st[2 * i + 1][j]);
  for (int64_t step0 = 0; step0 < T; step0 += RB) {
    __syncthreads();   // previous block's readers of the tiles and of Rs are done
#pragma unroll
    for (int a = 0; a < NL; ++a) tile_commit<D, LG, RTHREADS>(smem + a * L_OFF, lreg[a], Lsrc[a].bf, Lsrc[a].do_exp);
#pragma unroll
    for (int a = 0; a < NS; ++a) tile_commit<RS, SG, RTHREADS>(smem + S_BASE + a * S_OFF, sreg[a], Ssrc[a].bf, Ssrc[a].do_exp);
    __syncthreads();
    if (step0 + RB < T) fetch(step0 + RB);
    const int nt = (int)((T - step0) < RB ? (T - step0) : RB);
    // One step of the recurrence for this thread's state; returns the four per-step sums (not yet reduced).
    auto step = [&](int tt, float (&red)[NSI]) {
      f32x2 red2[NSI], s0d[NSI], s1d[NSI], s2d[NSI];
      // the step's slice-axis scalars, each broadcast to both halves of a pair (duplicating them in
      // shared memory instead costs more in extra shared-memory loads than the moves do here)
#pragma unroll
      for (int j = 0; j < NSI; ++j) {
        red2[j] = 0ull;
        const float s0 = smem[S_BASE + tt * RS + NSI * sg + j];
        s0d[j] = x2_pack(s0, s0);
        if (NS == 3) {
          const float s1 = smem[S_BASE + S_OFF + tt * RS + NSI * sg + j];
          const float s2 = smem[S_BASE + 2 * S_OFF + tt * RS + NSI * sg + j];
          s1d[j] = x2_pack(s1, s1);
          s2d[j] = x2_pack(s2, s2);
        } else {
          s1d[j] = 0ull; s2d[j] = 0ull;
        }
      }
#pragma unroll
      for (int m = 0; m < KP / 4; ++m) {
        const int off = tt * D + 4 * LP * m + 4 * lp;
        const ulonglong2 a4 = *reinterpret_cast<const ulonglong2*>(smem + off);
        const ulonglong2 b4 = *reinterpret_cast<const ulonglong2*>(smem + L_OFF + off);
        ulonglong2 c4 = make_ulonglong2(0ull, 0ull);
        if (NL == 3) c4 = *reinterpret_cast<const ulonglong2*>(smem + 2 * L_OFF + off);
        const f32x2 av[2] = {a4.x, a4.y};
        const f32x2 bv[2] = {b4.x, b4.y};
        const f32x2 cv[2] = {c4.x, c4.y};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
#pragma unroll
          for (int j = 0; j < NSI; ++j) {
            f32x2& S = st2[2 * m + e][j];
            if (MODE == REC_FWD) {          // a = f, b = k, c = q ; s0 = v
              S = x2_fma(av[e], S, x2_mul(bv[e], s0d[j]));
              red2[j] = x2_fma(cv[e], S, red2[j]);
            } else if (MODE == REC_DQ) {    // a = v, b = dO ; s0 = f, s1 = k
              S = x2_fma(s0d[j], S, x2_mul(s1d[j], av[e]));
              red2[j] = x2_fma(bv[e], S, red2[j]);
            } else if (MODE == REC_DV) {    // a = f, b = k, c = q ; s0 = dO
              const f32x2 tmp = x2_fma(cv[e], s0d[j], S);
              red2[j] = x2_fma(bv[e], tmp, red2[j]);
              S = x2_mul(av[e], tmp);
            } else {                        // a = v, b = dO ; s0 = f, s1 = k, s2 = q
              const f32x2 tmp = x2_fma(s2d[j], bv[e], S);
              red2[j] = x2_fma(av[e], tmp, red2[j]);
              S = x2_mul(s0d[j], tmp);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < NSI; ++j) {
        float lo, hi;
        x2_unpack(red2[j], lo, hi);
        red[j] = lo + hi;
      }
    };
    // The block's steps are fully unrolled with the reduced sums kept in registers until the end: with no
    // shared-memory store between the steps the compiler is free to issue a step's loads and FMAs while the
    // previous step's shuffle chain is still in flight (an in-order warp otherwise waits out every chain).
    float res[RB];
    if (nt == RB) {
#pragma unroll
      for (int tt = 0; tt < RB; ++tt) {
        float red[NSI];
        step(tt, red);
        res[tt] = reduceN_lanes<LP, NSI>(red, lp);
      }
    } else {
#pragma unroll
      for (int tt = 0; tt < RB; ++tt) res[tt] = 0.f;
      for (int tt = 0; tt < nt; ++tt) {
        float red[NSI];
        step(tt, red);
        const float tot = reduceN_lanes<LP, NSI>(red, lp);
#pragma unroll
        for (int u = 0; u < RB; ++u) if (u == tt) res[u] = tot;
      }
    }
    if (lp < NSI) {
#pragma unroll
      for (int tt = 0; tt < RB; ++tt) smem[R_BASE + tt * RS + NSI * sg + rec_which(lp)] = res[tt];
    }
    __syncthreads();
    // write the block's results: RB x RS values
    for (int e = threadIdx.x; e < RB * RS; e += RTHREADS) {
      const int row = e / RS, col = e % RS;
      const int64_t sidx = step0 + row;
      if (sidx < T) {
        const int64_t t = trev ? (T - 1 - sidx) : sidx;
        const int64_t addr = base + t * HD + c0 + col;
        const float r = smem[R_BASE + e];
        if (MODE == REC_FWD) {
          st_any(p.out, p.out_bf, addr, r);
        } else if (MODE == REC_DQ) {
          st_any(p.dq, p.bf, addr, r);
          p.E[addr] = smem[S_BASE + 2 * S_OFF + e] * r;
        } else if (MODE == REC_DV) {
          st_any(p.dv, p.bf, addr, r);
        } else {
          st_any(p.dk, p.bf, addr, r);
          p.F[addr] = smem[S_BASE + S_OFF + e] * r;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < KP / 2; ++i)
#pragma unroll
    for (int j = 0; j < NSI; ++j) x2_unpack(st2[i][j], st[2 * i][j], st[2 * i + 1][j]);
  // final state
  if (MODE == REC_FWD) {
    if (p.hidden_final) {
#pragma unroll
      for (int i = 0; i < KP; ++i)
#pragma unroll
        for (int j = 0; j < NSI; ++j) st_any(p.hidden_final, p.bf, state_addr(i, j), st[i][j]);
    }
  } else if (MODE == REC_DQ) {
    float s[NSI] = {};
    if (p.dhidden_final) {
#pragma unroll
      for (int i = 0; i < KP; ++i)
#pragma unroll
        for (int j = 0; j < NSI; ++j) s[j] = fmaf(ld_any(p.dhidden_final, p.bf, state_addr(i, j)), st[i][j], s[j]);
    }
#pragma unroll
    for (int j = 0; j < NSI; ++j) {
      const float t = reduce_lanes<LP>(s[j]);
      if (lp == 0) p.boundary[(b * p.H + h) * D + c0 + NSI * sg + j] = t;
    }
  } else if (MODE == REC_DV) {
#pragma unroll
    for (int i = 0; i < KP; ++i)
#pragma unroll
      for (int j = 0; j < NSI; ++j) st_any(p.dhidden_init, p.bf, state_addr(i, j), st[i][j]);
  }
}

template <int D, int MODE>
__global__ void __launch_bounds__(rec_threads(D)) rec_kernel(RecParams p) {
  rec_body<D, MODE>(p, blockIdx.z);
}

// The three passes of the backward in one grid (blockIdx.z = 3 b + pass).  They are independent of
// one another, and one pass alone leaves each scheduler with one or two warps: side by side, two
// CTAs of different passes share an SM and fill each other's issue gaps.
template <int D>
__global__ void __launch_bounds__(rec_threads(D)) rec_bwd_kernel(RecParams p) {
  const int pass = blockIdx.z % 3;
  const int64_t b = blockIdx.z / 3;
  if (pass == 0) rec_body<D, REC_DV>(p, b);
  else if (pass == 1) rec_body<D, REC_DQ>(p, b);
  else rec_body<D, REC_DK>(p, b);
}

template <int MODE>
constexpr size_t rec_smem_bytes(int D) {
  return (size_t)(((MODE == REC_FWD || MODE == REC_DV) ? 3 : 2) * RB * D +
                  ((MODE == REC_FWD || MODE == REC_DV) ? 1 : 3) * RB * RS + RB * RS) * sizeof(float);
}

template <int D>
static int launch_rec_fwd(cudaStream_t st, const RecParams& p) {
  const size_t smem = rec_smem_bytes<REC_FWD>(D);
  if (p.H > 65535 || p.B > 65535) return GLA_ERR_TOO_LARGE;
  cudaError_t e = cudaFuncSetAttribute(rec_kernel<D, REC_FWD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return record_cuda_error(e);
  dim3 grid(D / RS, (unsigned)p.H, (unsigned)p.B);
  ProfScope ps("rec_kernel_fwd", st);
  rec_kernel<D, REC_FWD><<<grid, rec_threads(D), smem, st>>>(p);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

template <int D>
static int launch_rec_bwd(cudaStream_t st, const RecParams& p) {
  const size_t a = rec_smem_bytes<REC_DV>(D), c = rec_smem_bytes<REC_DQ>(D);
  const size_t smem = a > c ? a : c;
  if (p.H > 65535 || 3 * p.B > 65535) return GLA_ERR_TOO_LARGE;
  cudaError_t e = cudaFuncSetAttribute(rec_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return record_cuda_error(e);
  dim3 grid(D / RS, (unsigned)p.H, (unsigned)(3 * p.B));
  ProfScope ps("rec_bwd_kernel", st);
  rec_bwd_kernel<D><<<grid, rec_threads(D), smem, st>>>(p);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

#define REC_DISPATCH_D(fn, st, D, p)          \
  switch (D) {                                \
    case 32: return fn<32>(st, p);            \
    case 64: return fn<64>(st, p);            \
    case 128: return fn<128>(st, p);          \
    case 256: return fn<256>(st, p);          \
    default: return GLA_ERR_UNSUPPORTED;      \
  }
static int launch_rec_fwd_d(cudaStream_t st, int D, const RecParams& p) { REC_DISPATCH_D(launch_rec_fwd, st, D, p) }
static int launch_rec_bwd_d(cudaStream_t st, int D, const RecParams& p) { REC_DISPATCH_D(launch_rec_bwd, st, D, p) }

int recurrent_fwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int bf, const void* hidden_init,
                  const float* g, const void* v, const void* k, const void* q, void* hidden_final, void* out,
                  int out_bf, int reverse) {
  RecParams p{};
  p.B = B; p.T = T; p.H = H; p.bf = bf; p.out_bf = out_bf;
  p.hidden_init = hidden_init; p.g = g; p.v = v; p.k = k; p.q = q;
  p.hidden_final = hidden_final; p.out = out; p.time_reversed = reverse;
  return launch_rec_fwd_d(st, (int)D, p);
}

size_t recurrent_bwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D) {
  return 2 * align_up((size_t)B * T * H * D * 4, 256) + align_up((size_t)B * H * D * 4, 256) +
         align_up(cumsum_scratch_bytes(B, T, H * D), 256);
}

int recurrent_bwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int bf, const void* hidden_init,
                  const float* g, const void* v, const void* k, const void* q, const void* dhidden_final,
                  const void* dout, int do_bf, void* dhidden_init, float* dg, void* dv, void* dk, void* dq,
                  int reverse, void* ws) {
  RecParams p{};
  p.B = B; p.T = T; p.H = H; p.bf = bf; p.do_bf = do_bf;
  p.hidden_init = hidden_init; p.g = g; p.v = v; p.k = k; p.q = q;
  p.dhidden_final = dhidden_final; p.dout = dout;
  p.dq = dq; p.dk = dk; p.dv = dv; p.dhidden_init = dhidden_init;
  const size_t plane = align_up((size_t)B * T * H * D * 4, 256);
  p.E = (float*)ws;
  p.F = (float*)((char*)ws + plane);
  p.boundary = (float*)((char*)ws + 2 * plane);
  float* seg_sums = (float*)((char*)ws + 2 * plane + align_up((size_t)B * H * D * 4, 256));
  p.time_reversed = reverse;
  GLA_TRY(launch_rec_bwd_d(st, (int)D, p));
  // dg[t] = sum over the tokens processed at or after t of (E - F), plus the boundary term
  return launch_cumsum(st, B, T, H * D, p.E, p.boundary, dg, reverse ? 0 : 1, 0, 0, p.F, seg_sums);
}

}  // namespace gla
