// tcgen05 tensor-core implementation of chunk_gla for bf16, head dim 128, chunk 128 (sm_100a).
//
// Reference algorithm: gla.py:483-625 (chunk forward/backward), gla.py:695-790 (inter-chunk
// terms), gla.py:792-960 and gla.py:964-1189 (intra-chunk scores with dyadic secondary
// chunking).  Every dense contraction runs on tcgen05.mma with bf16 operands staged in
// shared memory in the 128-byte-swizzled canonical layout and float32 accumulators in tensor
// memory; the decay weights are formed in float32 registers.
//
// Thread layout of the element-wise stages ("column-pair layout"): 512 threads = 8 row groups
// x 64 column pairs; thread (rg, cp) owns rows [16 rg, 16 rg + 16) and columns 2cp, 2cp+1 of
// the chunk's 128 x 128 tiles.  A warp covers 64 consecutive columns of one row, so global
// loads are 128/256-byte coalesced and operand-tile stores hit one 128-byte swizzle row.
// Every decay weight is a product of per-step gates f = exp(g) <= 1:
//   pre[r]  = prod_{t in [16 rg, r]} f_t      (inclusive, within the thread's 16 rows)
//   suf[r]  = prod_{t in (r, 16 rg + 15]} f_t (exclusive)
//   tot[rg] = pre[last]                        (shared between row groups through smem)
// so only C*D exponentials are evaluated per chunk and no exponent is ever positive.
#include "gla_common.cuh"
#include "tc_ptx.cuh"
#include "tma_maps.cuh"
#include <type_traits>
#include <cuda.h>
#include <cstdlib>

namespace gla {

using namespace tc;

constexpr int TC = 128;          // chunk length
constexpr int TD = 128;          // head dim
constexpr int TTHREADS = 512;
constexpr uint32_t TILE_BYTES = 128 * 128;     // one SW128 tile of 128 rows

__device__ unsigned int g_tc_wait_timeouts = 0;   // incremented when a bounded wait gives up

// K slice ks of an operand whose slice-0 descriptor is d0 (K-major: 32 bytes per slice, next 64-column
// block after four; MN-major: 2048 bytes per slice).  One 32-bit add instead of a descriptor rebuild, which
// matters because the issuing thread's instruction stream is serial and on the critical path.
__device__ __forceinline__ uint64_t kslice_kmajor(uint64_t d0, uint32_t tile_stride, int ks) {
  return desc_advance(d0, (uint32_t)(ks >> 2) * tile_stride + (uint32_t)(ks & 3) * 32u);
}
__device__ __forceinline__ uint64_t kslice_mnmajor(uint64_t d0, int ks) { return desc_advance(d0, (uint32_t)ks * 2048u); }

// smem carve-up helper: dynamic shared memory aligned to 1024 bytes
__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return (uint8_t*)(((uintptr_t)p + 1023) & ~(uintptr_t)1023);
}

// Copy a raw 128 x 128 bf16 matrix (row stride ld elements) into two SW128 tiles.
__device__ __forceinline__ void copy_tile_128x128(uint8_t* dst, const bf16* __restrict__ src, int64_t ld) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int id = threadIdx.x + TTHREADS * j;        // 2048 chunks of 16 bytes
    const int row = id >> 4, ch = id & 15;
    const uint4 val = *reinterpret_cast<const uint4*>(src + (int64_t)row * ld + ch * 8);
    *reinterpret_cast<uint4*>(dst + (ch >> 3) * TILE_BYTES + sw128_chunk(row, ch & 7)) = val;
  }
}

// ---------------------------------------------------------------------------------------
// kv / dstate kernel: out[dk][dv] = sum_c W[c][dk] Y[c][dv] for one chunk, where
//   MODE 0: W = k exp(G - lam)  (k_hat), Y = v      -> kv     (gla.py:705-708)
//   MODE 1: W = q exp(lam)      (q_hat), Y = dO     -> dstate (gla.py:748-750)
// Also writes the chunk's total log decay G[d] (MODE 0).  One CTA per chunk.
// MMA: M = dk (128), N = dv (128), K = c (128); both operands MN-major.
// ---------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(TTHREADS, 1)
tc_kv_kernel(int64_t T, int64_t H, int64_t N, const float* __restrict__ g, const bf16* __restrict__ x,
             const bf16* __restrict__ y, float* __restrict__ out, float* __restrict__ Gc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* sA = sm;                         // 2 tiles: W (rows = c, cols = dk)
  uint8_t* sB = sm + 2 * TILE_BYTES;        // 2 tiles: Y (rows = c, cols = dv)
  float* tot = reinterpret_cast<float*>(sm + 4 * TILE_BYTES);        // [8][128]
  float* gsum = tot + 8 * TD;                                         // [8][128]
  uint64_t* bar = reinterpret_cast<uint64_t*>(gsum + 8 * TD);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = tid >> 6, cp = tid & 63;
  const int64_t n = blockIdx.x % N, bh = blockIdx.x / N, b = bh / H, h = bh % H;
  const int64_t HD = H * TD;
  const int64_t row0 = ((b * T + n * TC) * H + h) * TD;     // element (b, n*C, h, 0)

  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 128);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(smem_u32(bar), 1);
    mbar_fence_init();
  }

  // ---- element-wise stage ------------------------------------------------------------------
  // All loads of the stage are issued before anything consumes one; the weights overwrite the gates.
  float2 f[16];
  uint32_t xv[16];
  {
    const int64_t e0 = row0 + (int64_t)(rg * 16) * HD + 2 * cp;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      f[i] = __ldg(reinterpret_cast<const float2*>(g + e0 + (int64_t)i * HD));
      xv[i] = __ldg(reinterpret_cast<const unsigned int*>(x + e0 + (int64_t)i * HD));
    }
  }
  float2 gs = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    gs.x += f[i].x; gs.y += f[i].y;
    f[i] = make_float2(__expf(f[i].x), __expf(f[i].y));
  }
  // f[i] becomes w[i]: MODE 0 exclusive suffix product, MODE 1 inclusive prefix product, within the 16 rows
  float2 (&w)[16] = f;
  if (MODE == 0) {
    float2 run = make_float2(1.f, 1.f);
#pragma unroll
    for (int i = 15; i >= 0; --i) { const float2 t = f[i]; w[i] = run; run.x *= t.x; run.y *= t.y; }
    *reinterpret_cast<float2*>(tot + rg * TD + 2 * cp) = run;
  } else {
    float2 run = make_float2(1.f, 1.f);
#pragma unroll
    for (int i = 0; i < 16; ++i) { run.x *= f[i].x; run.y *= f[i].y; w[i] = run; }
    *reinterpret_cast<float2*>(tot + rg * TD + 2 * cp) = run;
  }
  *reinterpret_cast<float2*>(gsum + rg * TD + 2 * cp) = gs;
  copy_tile_128x128(sB, y + row0, HD);
  __syncthreads();
  float2 cross = make_float2(1.f, 1.f);
  if (MODE == 0) {
    for (int r2 = rg + 1; r2 < 8; ++r2) {
      const float2 t = *reinterpret_cast<const float2*>(tot + r2 * TD + 2 * cp);
      cross.x *= t.x; cross.y *= t.y;
    }
  } else {
    for (int r2 = 0; r2 < rg; ++r2) {
      const float2 t = *reinterpret_cast<const float2*>(tot + r2 * TD + 2 * cp);
      cross.x *= t.x; cross.y *= t.y;
    }
  }
  if (Gc != nullptr && rg == 0) {
    float2 s = make_float2(0.f, 0.f);
#pragma unroll
    for (int r2 = 0; r2 < 8; ++r2) {
      const float2 t = *reinterpret_cast<const float2*>(gsum + r2 * TD + 2 * cp);
      s.x += t.x; s.y += t.y;
    }
    *reinterpret_cast<float2*>(Gc + (bh * N + n) * TD + 2 * cp) = s;
  }
  {
    uint8_t* tile = sA + (cp >> 5) * TILE_BYTES;
    const int c = (2 * cp) & 63;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 xf = unpack_bf16x2(xv[i]);
      const int r = rg * 16 + i;
      *reinterpret_cast<uint32_t*>(tile + sw128_off(r, c)) =
          pack_bf16x2(xf.x * w[i].x * cross.x, xf.y * w[i].y * cross.y);
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // ---- MMA ---------------------------------------------------------------------------------
  if (tid == 0) {
    constexpr uint32_t idesc = idesc_bf16(128, 128, 1, 1);
    const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      umma_bf16(tmem, desc_mnmajor(a0, TILE_BYTES, ks), desc_mnmajor(b0, TILE_BYTES, ks), idesc, ks > 0);
    umma_commit(smem_u32(bar));
  }
  const bool ok = mbar_wait(smem_u32(bar), 0);
  tc_fence_after();

  // ---- epilogue: TMEM -> global float32 (lane = dk, columns = dv) -----------------------------
  if (ok) {
    const int q4 = warp & 3, cg = warp >> 2;
    uint32_t r[32];
    tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(cg * 32), r);
    tmem_ld_wait();
    float* o = out + ((bh * N + n) * TD + (q4 * 32 + lane)) * TD + cg * 32;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<float4*>(o + 4 * j) = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                          __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
  } else if (tid == 0) {
    atomicAdd(&g_tc_wait_timeouts, 1u);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

// Number of thread blocks resident at a time (SMs x blocks per SM) = how far ahead in block index the
// block that follows on the same SM lies; 0 disables the L2 prefetch.
static int prefetch_distance(int blocks_per_sm) {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 0;
    sms[dev] = n;
  }
  return sms[dev] * blocks_per_sm;
}

constexpr size_t KV_SMEM = 1024 + 4 * TILE_BYTES + 2 * 8 * TD * sizeof(float) + 64;

template <int MODE>
static int launch_tc_kv(cudaStream_t st, int64_t B, int64_t T, int64_t H, const float* g, const void* x, const void* y,
                        float* out, float* Gc) {
  const int64_t N = T / TC;
  static SmemAttrOnce attr;
  GLA_TRY(attr.ensure(tc_kv_kernel<MODE>, KV_SMEM));
  ProfScope ps(MODE == 0 ? "tc_kv_kernel" : "tc_dstate_kernel", st);
  tc_kv_kernel<MODE><<<(unsigned)(B * H * N), TTHREADS, KV_SMEM, st>>>(T, H, N, g, (const bf16*)x, (const bf16*)y, out, Gc);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

// ---------------------------------------------------------------------------------------
// Forward chunk kernel: scores with dyadic secondary chunking, out = P V + q_hat S_prev.
//
// Dyadic levels (gla.py:985-1027, 843-852): for half size h in {1,2,...,64} the chunk splits
// into blocks of 2h rows; queries in the right half of a block meet keys in its left half with
// the anchor at the last row of the left half:
//   q~[i] = q[i] * prod_{t in (anchor, i]} f_t,   k~[j] = k[j] * prod_{t in (j, anchor]} f_t.
// One level = ONE MMA: A = all 128 rows of q~ (left-half rows hold stale data and are never
// read back), B = the 64 left-half rows of k~ packed densely ("compact" index
// c(j) = (j / 2h) h + j mod h), M = 128, N = 64, K = 128, result in TMEM columns
// [64 s, 64 s + 64) for level slot s.  Entry (i, c(j)) is meaningful iff i and j share a block.
// The seven slots fill 448 of the 512 TMEM columns; after they are read back into the bf16
// P tile, columns [0, 128) are reused for the output accumulator.
// ---------------------------------------------------------------------------------------
struct FwdSmem {
  static constexpr uint32_t Q = 0;                         // 2 buffers x 32 KB   (q~ / q_hat); TMA lands g here first
  static constexpr uint32_t K = Q + 2 * 2 * TILE_BYTES;    // 2 buffers x 16 KB   (compact k~);  TMA lands raw q here first
  static constexpr uint32_t V = K + 2 * TILE_BYTES;        // 32 KB
  static constexpr uint32_t S = V + 2 * TILE_BYTES;        // 32 KB
  static constexpr uint32_t P = S + 2 * TILE_BYTES;        // 32 KB;               TMA lands raw k here first
  static constexpr uint32_t TOT = P + 2 * TILE_BYTES;      // 8 x 128 float
  static constexpr uint32_t DIAG = TOT + 8 * TD * 4;       // 2 x 128 float
  static constexpr uint32_t GAB = DIAG + 2 * TC * 4;       // 8 x 128 float: sums of |g| per 16 rows
  static constexpr uint32_t BAR = GAB + 8 * TD * 4;        // 5 mbarriers + tmem slot
  static constexpr uint32_t END = BAR + 64;
};
// A chunk whose gates satisfy sum_rows |g| <= ONE_SCALE_LIMIT for every feature needs no secondary chunking: with
// one anchor for the whole chunk every decay weight stays within exp(+-limit), far inside the range of bf16 and
// float32, so the dyadic levels (which exist to keep exponents non-positive, gla.py:986-993) collapse into one.
constexpr float ONE_SCALE_LIMIT = 60.f;
// Between the two limits the single anchor still serves if it is put in the MIDDLE of the chunk's decay instead of
// at an end: every feature d gets the anchor value m_d = -(sum_rows |g|) / 2, q~ = q exp(lam - m) and
// k~ = k exp(m - lam) then stay within exp(+-limit / 2), and the one operand per side that must be anchored at the
// chunk's end for the inter-chunk products (q_hat in the forward, k_hat in the backward) is replaced by the
// balanced one with the factor exp(-m_d) moved onto the rows of the state tile (S_prev, resp. dS_next), which are
// rescaled in shared memory.  Sharp gates (log_sigmoid(N(0,1)): about -103 per chunk) run this way; chunks beyond
// the second limit take all levels.  In the backward the transposed accumulators then hold values up to
// exp(limit / 2) |k| |dP| 128, which is what bounds the limit (float32 overflows at exp(88.7)).
constexpr float BALANCED_LIMIT = 140.f;
constexpr uint32_t KC_TILE = 64 * 128;    // one SW128 tile of 64 rows

// TMA descriptors of one launch (built on the host per call, passed by value).
struct FwdMaps { CUtensorMap g, q, k, v, s; };


// Operands of level slot S (half size 2^S) for the thread's 16 rows x 2 columns, with the decay
// weights formed on the fly as running products of the gates f (no weight arrays are kept):
// rows in a right half write q~ (inclusive prefix from the half's first row), rows in a left
// half write k~ at their compact index (exclusive suffix to the half's last row).
template <int S>
__device__ __forceinline__ void fwd_emit(const float2 (&f)[16], const uint32_t (&qv)[16], const uint32_t (&kv)[16],
                                         uint8_t* sQb, uint8_t* sKb, int rg, int cp, const float* tot) {
  constexpr int HH = 1 << S;
  const int tile = cp >> 5, col = (2 * cp) & 63;
  uint8_t* qb = sQb + tile * TILE_BYTES;
  uint8_t* kb = sKb + tile * KC_TILE;
  if (S < 4) {
    float2 run = make_float2(1.f, 1.f);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (i % HH == 0) run = f[i]; else { run.x *= f[i].x; run.y *= f[i].y; }
      if (i & HH) {
        const float2 x = unpack_bf16x2(qv[i]);
        *reinterpret_cast<uint32_t*>(qb + sw128_off(rg * 16 + i, col)) = pack_bf16x2(x.x * run.x, x.y * run.y);
      }
    }
#pragma unroll
    for (int i = 15; i >= 0; --i) {
      if (i % HH == HH - 1) run = make_float2(1.f, 1.f);
      if (!(i & HH)) {
        const float2 x = unpack_bf16x2(kv[i]);
        const int r = rg * 16 + i;
        const int c = ((r >> (S + 1)) << S) + (r & (HH - 1));
        *reinterpret_cast<uint32_t*>(kb + sw128_off(c, col)) = pack_bf16x2(x.x * run.x, x.y * run.y);
      }
      run.x *= f[i].x; run.y *= f[i].y;
    }
  } else {
    auto tot_at = [&](int r2) { return *reinterpret_cast<const float2*>(tot + r2 * TD + 2 * cp); };
    bool right;
    float2 run = make_float2(1.f, 1.f);
    if (S == 4) {
      right = (rg & 1) != 0;
    } else if (S == 5) {
      const int m = rg & 3;
      right = m >= 2;
      if (m == 3) run = tot_at(rg - 1);
      if (m == 0) run = tot_at(rg + 1);
    } else {
      right = rg >= 4;
      if (right) { for (int r2 = 4; r2 < rg; ++r2) { const float2 t = tot_at(r2); run.x *= t.x; run.y *= t.y; } }
      else       { for (int r2 = rg + 1; r2 < 4; ++r2) { const float2 t = tot_at(r2); run.x *= t.x; run.y *= t.y; } }
    }
    if (right) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        run.x *= f[i].x; run.y *= f[i].y;
        const float2 x = unpack_bf16x2(qv[i]);
        *reinterpret_cast<uint32_t*>(qb + sw128_off(rg * 16 + i, col)) = pack_bf16x2(x.x * run.x, x.y * run.y);
      }
    } else {
#pragma unroll
      for (int i = 15; i >= 0; --i) {
        const float2 x = unpack_bf16x2(kv[i]);
        const int r = rg * 16 + i;
        const int c = ((r >> (S + 1)) << S) + (r & (HH - 1));
        *reinterpret_cast<uint32_t*>(kb + sw128_off(c, col)) = pack_bf16x2(x.x * run.x, x.y * run.y);
        run.x *= f[i].x; run.y *= f[i].y;
      }
    }
  }
}


// Out of line on purpose (the forward kernel's straight-line code is sensitive to anything added to it): the
// late path of a block that started beside the state kernel.  It blocks on the grid dependency itself
// (griddepcontrol.wait returns once the state kernel has completed and its writes are visible; no polling of
// memory between the two grids), then issues the state tile's two TMA loads.  The counter is read once more
// only to report a dependency that did not hold.
__device__ __noinline__ bool fwd_load_state_late(const unsigned int* state_done, unsigned int state_target,
                                                 const CUtensorMap* map_s, uint32_t dst, int row, uint32_t bar) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const bool done = ld_acquire_u32(state_done) >= state_target;
  fence_proxy_async_global();
  tma_load_2d(dst, map_s, 0, row, bar);
  tma_load_2d(dst + TILE_BYTES, map_s, 64, row, bar);
  return done;
}

__global__ void __launch_bounds__(TTHREADS, 1)
tc_chunk_fwd_kernel(const __grid_constant__ FwdMaps maps, int64_t T, int64_t H, int R, int64_t N, bf16* __restrict__ out,
                    bf16* __restrict__ P_saved, const unsigned int* __restrict__ state_done, unsigned int state_target,
                    int all_scales, int pf_dist) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  float* tot = reinterpret_cast<float*>(sm + FwdSmem::TOT);
  float* diag = reinterpret_cast<float*>(sm + FwdSmem::DIAG);
  float* gab = reinterpret_cast<float*>(sm + FwdSmem::GAB);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + FwdSmem::BAR);   // [0],[1]: level buffers, [2]: output, [3]: g,q,k loads, [4]: v,S loads
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile uint32_t* s_pending_sm = tmem_slot + 1;     // thread 0's note to itself: the state tile's load is still to be issued

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = tid >> 6, cp = tid & 63;
  // H counts VIRTUAL heads of size 128: a head of size 128 R is R x R independent (key block a, value block c)
  // problems, virtual head (h R + a) R + c, whose results the caller sums over a.  In the (B, T, H_real R, 128) view
  // of the inputs the key-side tensors of a virtual head are head h R + a, the value-side ones head h R + c; the
  // output is written per virtual head, (B, T, H, 128).  R = 1: everything coincides with the real layout.
  // Block order: chunk-major, LAST chunks first.  The state kernel that runs before this one walks the chunks of all
  // heads in step, first to last, so the inputs it read most recently (g, k, v of the late chunks) and the states
  // it wrote last are the ones most likely to be still in L2.
  const int64_t BHn = (int64_t)gridDim.x / N;
  const int64_t n = N - 1 - (int64_t)blockIdx.x / BHn, bh = (int64_t)blockIdx.x % BHn, b = bh / H, h_ = bh % H;
  const int64_t hk_ = (h_ / (R * R)) * R + (h_ % (R * R)) / R, hv_ = (h_ / (R * R)) * R + h_ % R;
  const int64_t HD = H * TD;
  const int64_t row0 = ((b * T + n * TC) * H + h_) * TD;
  const int64_t chunk_id = bh * N + n;

  if (tid == 0) {
    mbar_init(smem_u32(bars + 0), 1);
    mbar_init(smem_u32(bars + 1), 1);
    mbar_init(smem_u32(bars + 2), 1);
    mbar_init(smem_u32(bars + 3), 1);
    mbar_init(smem_u32(bars + 4), 1);
    mbar_fence_init();
    // ---- all global inputs of the chunk through TMA: 192 KB in flight.  g, q, k (needed at once) come first on
    // their own barrier; v and S_prev are only needed by the output product and land while the levels run.
    const uint32_t lb = smem_u32(bars + 3), lb2 = smem_u32(bars + 4);
    const int z = (int)(b * T + n * TC), y = (int)hk_, yv = (int)hv_;
    mbar_arrive_expect_tx(lb, 4 * 2 * TILE_BYTES);
    mbar_arrive_expect_tx(lb2, 2 * 2 * TILE_BYTES);
    tma_load_3d(smem_u32(sm + FwdSmem::Q), &maps.g, 0, y, z, lb);                       // 128 x 128 float, row pitch 512 B
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      tma_load_3d(smem_u32(sm + FwdSmem::K + half * TILE_BYTES), &maps.q, 64 * half, y, z, lb);
      tma_load_3d(smem_u32(sm + FwdSmem::P + half * TILE_BYTES), &maps.k, 64 * half, y, z, lb);
    }
    // state_done (optional): this grid was launched as a programmatic dependent of the state kernel and may be
    // running beside it, on SMs that kernel leaves idle.  One look at the counter (no waiting on it): if every
    // state block has finished, the state tile is loaded now; otherwise its load is left to thread 32 at the
    // point where the tile is needed, behind the grid dependency (everything before that needs no state).
    const bool s_pending = state_done != nullptr && ld_acquire_u32(state_done) < state_target;
    *s_pending_sm = s_pending ? 1u : 0u;
    if (!s_pending && state_done != nullptr) fence_proxy_async_global();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      tma_load_3d(smem_u32(sm + FwdSmem::V + half * TILE_BYTES), &maps.v, 64 * half, yv, z, lb2);
      if (!s_pending) tma_load_2d(smem_u32(sm + FwdSmem::S + half * TILE_BYTES), &maps.s, 64 * half, (int)(chunk_id * TD), lb2);
    }
    // The same boxes of the block that the scheduler starts on this SM when this one retires (pf_dist blocks
    // ahead), requested into L2 only: seven instructions of this one thread, so that the next block's load phase
    // is served from L2.
    const int64_t nb = (int64_t)blockIdx.x + pf_dist;
    if (pf_dist > 0 && nb < (int64_t)gridDim.x) {
      const int64_t n2 = N - 1 - nb / BHn, bh2 = nb % BHn, h2 = bh2 % H;
      const int y2 = (int)((h2 / (R * R)) * R + (h2 % (R * R)) / R), yv2 = (int)((h2 / (R * R)) * R + h2 % R);
      const int z2 = (int)((bh2 / H) * T + n2 * TC);
      tma_prefetch_l2_3d(&maps.g, 0, y2, z2);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        tma_prefetch_l2_3d(&maps.q, 64 * half, y2, z2);
        tma_prefetch_l2_3d(&maps.k, 64 * half, y2, z2);
        tma_prefetch_l2_3d(&maps.v, 64 * half, yv2, z2);
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();          // barrier inits and the TMEM address are visible
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool ok = mbar_wait(smem_u32(bars + 3), 0);
  // ---- gates, q, k of the thread's 16 rows x 2 columns from the landed tiles ---------------------
  float2 f[16];
  uint32_t qv[16], kv[16];
  float2 prod = make_float2(1.f, 1.f);          // product of the thread's 16 gates, per column
  {
    const uint8_t* gq = sm + FwdSmem::Q;
    const uint8_t* qt = sm + FwdSmem::K + (cp >> 5) * TILE_BYTES;
    const uint8_t* kt = sm + FwdSmem::P + (cp >> 5) * TILE_BYTES;
    const int col = (2 * cp) & 63;
    float2 gsum = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int r = rg * 16 + i;
      const float2 gg = *reinterpret_cast<const float2*>(gq + r * 512 + cp * 8);
      qv[i] = *reinterpret_cast<const uint32_t*>(qt + sw128_off(r, col));
      kv[i] = *reinterpret_cast<const uint32_t*>(kt + sw128_off(r, col));
      f[i] = make_float2(__expf(gg.x), __expf(gg.y));
      prod.x *= f[i].x; prod.y *= f[i].y;
      gsum.x += fabsf(gg.x); gsum.y += fabsf(gg.y);
    }
    *reinterpret_cast<float2*>(tot + rg * TD + 2 * cp) = prod;
    *reinterpret_cast<float2*>(gab + rg * TD + 2 * cp) = gsum;
  }
  __syncthreads();          // raw g, q, k have been consumed (their regions become operand buffers); tot and gab are visible
  // One scale or all of them: the chunk's total |log decay| per feature decides, the same way for every thread.
  bool one_scale, balanced;
  float2 anchor = make_float2(1.f, 1.f);
  {
    float2 tsum = make_float2(0.f, 0.f);
#pragma unroll
    for (int r2 = 0; r2 < 8; ++r2) {
      const float2 t = *reinterpret_cast<const float2*>(gab + r2 * TD + 2 * cp);
      tsum.x += t.x; tsum.y += t.y;
    }
    // (a NaN gate fails the comparisons and takes the general path)
    // (mild chunks, the common case, pay one block-wide vote; only a chunk that fails it takes the second)
    one_scale = __syncthreads_or(!(tsum.x <= ONE_SCALE_LIMIT && tsum.y <= ONE_SCALE_LIMIT) || all_scales != 0) == 0;
    balanced = false;
    if (!one_scale) balanced = one_scale = __syncthreads_or(!(tsum.x <= BALANCED_LIMIT && tsum.y <= BALANCED_LIMIT) || all_scales != 0) == 0;
    if (balanced) {
      // exp(-m_d) = exp(sum |g| / 2) for the thread's two features; row group 0 leaves exp(m_d) for the rescaling of
      // the state tile (the |g| sums have been read by everybody: two barriers back)
      anchor = make_float2(__expf(0.5f * tsum.x), __expf(0.5f * tsum.y));
      if (rg == 0) *reinterpret_cast<float2*>(gab + 2 * cp) = make_float2(1.f / anchor.x, 1.f / anchor.y);
    }
  }
  const uint32_t sQ0 = smem_u32(sm + FwdSmem::Q), sK0 = smem_u32(sm + FwdSmem::K);
  uint8_t* sQb[2] = {sm + FwdSmem::Q, sm + FwdSmem::Q + 2 * TILE_BYTES};
  uint8_t* sKb[2] = {sm + FwdSmem::K, sm + FwdSmem::K + 2 * KC_TILE};

  if (one_scale) {
    // ---- one anchor for the whole chunk (the row before its first): q_hat = q exp(lam) serves both the scores and
    // the inter-chunk product, k~ = k exp(-lam); P = q_hat k~^T is ONE 128 x 128 x 128 product into TMEM columns
    // [128, 256), masked to the lower triangle on the way back.  exp(-lam) is formed as
    // (1 / prod of the gates up to the end of the thread's run) x (running product back from that end),
    // so it costs two reciprocals per thread.
    {
      float2 crossq = anchor;                           // 1, or exp(-m_d) with the balanced anchor
      for (int r2 = 0; r2 < rg; ++r2) {
        const float2 t = *reinterpret_cast<const float2*>(tot + r2 * TD + 2 * cp);
        crossq.x *= t.x; crossq.y *= t.y;
      }
      const int tile = cp >> 5, col = (2 * cp) & 63;
      uint8_t* qb = sQb[1] + tile * TILE_BYTES;        // q_hat: where the output product expects it
      uint8_t* kb = sQb[0] + tile * TILE_BYTES;        // k~: 128 rows x 128 features, two tiles
      float2 run = crossq;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        run.x *= f[i].x; run.y *= f[i].y;
        const float2 x = unpack_bf16x2(qv[i]);
        *reinterpret_cast<uint32_t*>(qb + sw128_off(rg * 16 + i, col)) = pack_bf16x2(x.x * run.x, x.y * run.y);
      }
      run = make_float2(1.f / (crossq.x * prod.x), 1.f / (crossq.y * prod.y));
#pragma unroll
      for (int i = 15; i >= 0; --i) {
        const float2 x = unpack_bf16x2(kv[i]);
        *reinterpret_cast<uint32_t*>(kb + sw128_off(rg * 16 + i, col)) = pack_bf16x2(x.x * run.x, x.y * run.y);
        run.x *= f[i].x; run.y *= f[i].y;
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = idesc_bf16(128, 128, 0, 0);
      const uint64_t a0 = desc_kmajor(sQ0 + 2 * TILE_BYTES, TILE_BYTES, 0), b0 = desc_kmajor(sQ0, TILE_BYTES, 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_bf16(tmem + 128, kslice_kmajor(a0, TILE_BYTES, ks), kslice_kmajor(b0, TILE_BYTES, ks), idesc, ks > 0);
      umma_commit(smem_u32(bars + 0));
    }
    ok = mbar_wait(smem_u32(bars + 0), 0) && ok;
    tc_fence_after();
    // scores back into the bf16 P tile: row i = 32 q4 + lane, columns 32 cj + [0, 32); the diagonal entry
    // q_hat_i . k~_i = q_i . k_i comes out of the same product
    {
      const int q4 = warp & 3, cj = warp >> 2;
      const int i = 32 * q4 + lane;
      uint32_t r[32];
      if (cj <= q4) {
        tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + 128u + (uint32_t)(32 * cj), r);
        tmem_ld_wait();
      }
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        uint4 u = make_uint4(0u, 0u, 0u, 0u);
        if (cj <= q4) {
          float x[8];
#pragma unroll
          for (int m = 0; m < 8; ++m) x[m] = (cj < q4 || 8 * c8 + m <= lane) ? __uint_as_float(r[8 * c8 + m]) : 0.f;
          u.x = pack_bf16x2(x[0], x[1]); u.y = pack_bf16x2(x[2], x[3]);
          u.z = pack_bf16x2(x[4], x[5]); u.w = pack_bf16x2(x[6], x[7]);
        }
        const int col0 = 32 * cj + 8 * c8;
        *reinterpret_cast<uint4*>(sm + FwdSmem::P + (col0 >> 6) * TILE_BYTES + sw128_chunk(i, (col0 & 63) >> 3)) = u;
      }
    }
  } else {
  // diagonal: sum_d q k, reduced over the 64 column-pair threads of a row group (two warps)
  {
    float part[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 a = unpack_bf16x2(qv[i]), c = unpack_bf16x2(kv[i]);
      part[i] = a.x * c.x + a.y * c.y;
    }
    // Sum of each of the 16 values over the warp's 32 lanes by a transposing butterfly: at every stage a lane keeps
    // half of its values and hands the other half to its partner, so 16 + 8 + 4 + 2 + 1 shuffles do what
    // 16 x 5 would; lanes 2r and 2r + 1 end up with the total of row r.
    const bool h4 = (lane & 16) != 0, h3 = (lane & 8) != 0, h2 = (lane & 4) != 0, h1 = (lane & 2) != 0;
    float a8[8], a4[4], a2[2];
#pragma unroll
    for (int j = 0; j < 8; ++j) a8[j] = (h4 ? part[j + 8] : part[j]) + __shfl_xor_sync(0xffffffffu, h4 ? part[j] : part[j + 8], 16);
#pragma unroll
    for (int j = 0; j < 4; ++j) a4[j] = (h3 ? a8[j + 4] : a8[j]) + __shfl_xor_sync(0xffffffffu, h3 ? a8[j] : a8[j + 4], 8);
#pragma unroll
    for (int j = 0; j < 2; ++j) a2[j] = (h2 ? a4[j + 2] : a4[j]) + __shfl_xor_sync(0xffffffffu, h2 ? a4[j] : a4[j + 2], 4);
    float a1 = (h1 ? a2[1] : a2[0]) + __shfl_xor_sync(0xffffffffu, h1 ? a2[0] : a2[1], 2);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
    if ((lane & 1) == 0) diag[(warp & 1) * TC + rg * 16 + (lane >> 1)] = a1;     // read after the level barriers below
  }

  auto issue_level = [&](int slot) {
    const int bsel = slot & 1;
    constexpr uint32_t idesc = idesc_bf16(128, 64, 0, 0);
    const uint64_t a0 = desc_kmajor(sQ0 + bsel * 2 * TILE_BYTES, TILE_BYTES, 0), b0 = desc_kmajor(sK0 + bsel * 2 * KC_TILE, KC_TILE, 0);
    const uint32_t acc = tmem + 64 * slot;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      umma_bf16(acc, kslice_kmajor(a0, TILE_BYTES, ks), kslice_kmajor(b0, KC_TILE, ks), idesc, ks > 0);
    umma_commit(smem_u32(bars + bsel));
  };
  auto level_sync_and_issue = [&](int slot) {
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      issue_level(slot);
    }
  };
  auto wait_buffer_free = [&](int slot) {
    // before rebuilding buffer (slot & 1): the MMA of level slot-2 must have consumed it
    if (slot >= 2) ok = mbar_wait(smem_u32(bars + (slot & 1)), (uint32_t)(((slot - 2) >> 1) & 1)) && ok;
  };

  fwd_emit<0>(f, qv, kv, sQb[0], sKb[0], rg, cp, tot); level_sync_and_issue(0);
  fwd_emit<1>(f, qv, kv, sQb[1], sKb[1], rg, cp, tot); level_sync_and_issue(1);
  wait_buffer_free(2);
  fwd_emit<2>(f, qv, kv, sQb[0], sKb[0], rg, cp, tot); level_sync_and_issue(2);
  wait_buffer_free(3);
  fwd_emit<3>(f, qv, kv, sQb[1], sKb[1], rg, cp, tot); level_sync_and_issue(3);
  wait_buffer_free(4);
  fwd_emit<4>(f, qv, kv, sQb[0], sKb[0], rg, cp, tot); level_sync_and_issue(4);
  wait_buffer_free(5);
  fwd_emit<5>(f, qv, kv, sQb[1], sKb[1], rg, cp, tot); level_sync_and_issue(5);
  wait_buffer_free(6);
  fwd_emit<6>(f, qv, kv, sQb[0], sKb[0], rg, cp, tot); level_sync_and_issue(6);

  // ---- q_hat into Q buffer 1 (free once the MMA of level slot 5 has completed); overlaps slot 6's MMA
  ok = mbar_wait(smem_u32(bars + 1), 0) && ok;     // buffer 1, third use (level slot 5)
  {
    float2 run = make_float2(1.f, 1.f);
    for (int r2 = 0; r2 < rg; ++r2) {
      const float2 t = *reinterpret_cast<const float2*>(tot + r2 * TD + 2 * cp);
      run.x *= t.x; run.y *= t.y;
    }
    uint8_t* tile = sQb[1] + (cp >> 5) * TILE_BYTES;
    const int col = (2 * cp) & 63;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      run.x *= f[i].x; run.y *= f[i].y;
      const float2 x = unpack_bf16x2(qv[i]);
      *reinterpret_cast<uint32_t*>(tile + sw128_off(rg * 16 + i, col)) = pack_bf16x2(x.x * run.x, x.y * run.y);
    }
  }
  // all seven level MMAs done when the last commit (buffer 0, fourth use) completes
  ok = mbar_wait(smem_u32(bars + 0), 1) && ok;
  tc_fence_after();

  // ---- read the scores back into the bf16 P tile -----------------------------------------------------
  // Rows 32 q4 + lane belong to the four warps of TMEM quadrant q4; each of them (cj = 0..3) writes
  // 32 of the row's 128 columns in 16-byte chunks of 8: q4 chunks below the diagonal block (copied
  // from level slot 5 or 6), one chunk of the 32 x 32 diagonal block (assembled from slots 0..4 and
  // the q.k diagonal) and 3 - q4 chunks of zeros above it, so that the four warps are balanced.
  {
    const int q4 = warp & 3, cj = warp >> 2;
    const int li = lane, i = 32 * q4 + li;
    const uint32_t lane_base = tmem + ((uint32_t)(q4 * 32) << 16);
    auto put_chunk = [&](int col0, const float (&x)[8]) {
      uint4 u;
      u.x = pack_bf16x2(x[0], x[1]); u.y = pack_bf16x2(x[2], x[3]);
      u.z = pack_bf16x2(x[4], x[5]); u.w = pack_bf16x2(x[6], x[7]);
      *reinterpret_cast<uint4*>(sm + FwdSmem::P + (col0 >> 6) * TILE_BYTES + sw128_chunk(i, (col0 & 63) >> 3)) = u;
    };
    // below the diagonal block
    for (int ch = 0; ch < q4; ++ch) {
      const int col0 = 8 * (q4 * cj + ch), cb = col0 >> 5;
      const int tcol = ((q4 ^ cb) >= 2) ? (64 * 6 + col0) : (64 * 5 + (cb >> 1) * 32 + (col0 & 31));
      uint32_t r[8];
      tmem_ld8(lane_base + tcol, r);
      tmem_ld_wait();
      float x[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) x[m] = __uint_as_float(r[m]);
      put_chunk(col0, x);
    }
    // the diagonal block: local columns lj = 8 cj + m
    {
      float x[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) x[m] = 0.f;
      const int lj0 = 8 * cj;
#pragma unroll
      for (int s2 = 0; s2 < 3; ++s2) {
        const int hh = 1 << s2;
        uint32_t r[4];
        tmem_ld4(lane_base + 64 * s2 + 16 * q4 + 4 * cj, r);
        tmem_ld_wait();
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          if ((m & hh) == 0) {
            const int c = ((m >> (s2 + 1)) << s2) + (m & (hh - 1));
            if (((li ^ (lj0 + m)) >> s2) == 1) x[m] = __uint_as_float(r[c]);
          }
        }
      }
      if ((cj & 1) == 0) {            // half size 8: columns with bit 3 clear
        uint32_t r[8];
        tmem_ld8(lane_base + 64 * 3 + 16 * q4 + 8 * (cj >> 1), r);
        tmem_ld_wait();
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (((li ^ (lj0 + m)) >> 3) == 1) x[m] = __uint_as_float(r[m]);
      }
      if (cj < 2) {                   // half size 16: columns with bit 4 clear
        uint32_t r[8];
        tmem_ld8(lane_base + 64 * 4 + 16 * q4 + 8 * cj, r);
        tmem_ld_wait();
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (((li ^ (lj0 + m)) >> 4) == 1) x[m] = __uint_as_float(r[m]);
      }
      const float dgv = diag[i] + diag[TC + i];
#pragma unroll
      for (int m = 0; m < 8; ++m)
        if (lj0 + m == li) x[m] = dgv;
      put_chunk(32 * q4 + lj0, x);
    }
    // above the diagonal block
    {
      float z[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) z[m] = 0.f;
      for (int ch = 0; ch < 3 - q4; ++ch) put_chunk(32 * (q4 + 1) + 8 * ((3 - q4) * cj + ch), z);
    }
  }
  }   // all scales
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (balanced) {
    // the q_hat operand carries exp(-m_d): row d of the state tile takes exp(m_d) before the product.  Every thread
    // waits for the tile itself here (a block that started beside the state kernel requests it first).
    if (tid == 32 && *s_pending_sm != 0u) {
      if (!fwd_load_state_late(state_done, state_target, &maps.s, smem_u32(sm + FwdSmem::S), (int)(chunk_id * TD), smem_u32(bars + 4)))
        atomicAdd(&g_tc_wait_timeouts, 1u);
      *s_pending_sm = 0u;
    }
    __syncwarp();
    ok = mbar_wait(smem_u32(bars + 4), 0) && ok;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int id = tid + TTHREADS * j, row = id >> 4, ch = id & 15;
      const float w = gab[row];
      uint4* p4 = reinterpret_cast<uint4*>(sm + FwdSmem::S + (ch >> 3) * TILE_BYTES + sw128_chunk(row, ch & 7));
      uint4 u = *p4;
      float2 a = unpack_bf16x2(u.x), b2 = unpack_bf16x2(u.y), c2 = unpack_bf16x2(u.z), d2 = unpack_bf16x2(u.w);
      u.x = pack_bf16x2(a.x * w, a.y * w); u.y = pack_bf16x2(b2.x * w, b2.y * w);
      u.z = pack_bf16x2(c2.x * w, c2.y * w); u.w = pack_bf16x2(d2.x * w, d2.y * w);
      *p4 = u;
    }
    fence_async_smem();
    __syncthreads();
  }
  if (tid == 0) {
    ok = mbar_wait(smem_u32(bars + 4), 0) && ok;       // v and S_prev have landed (long ago, as a rule)
    tc_fence_after();
    constexpr uint32_t idesc = idesc_bf16(128, 128, 0, 1);
    const uint64_t aq = desc_kmajor(sQ0 + 2 * TILE_BYTES, TILE_BYTES, 0), bs = desc_mnmajor(smem_u32(sm + FwdSmem::S), TILE_BYTES, 0);
    const uint64_t ap = desc_kmajor(smem_u32(sm + FwdSmem::P), TILE_BYTES, 0), bv = desc_mnmajor(smem_u32(sm + FwdSmem::V), TILE_BYTES, 0);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      umma_bf16(tmem, kslice_kmajor(aq, TILE_BYTES, ks), kslice_mnmajor(bs, ks), idesc, ks > 0);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      umma_bf16(tmem, kslice_kmajor(ap, TILE_BYTES, ks), kslice_mnmajor(bv, ks), idesc, 1);
    umma_commit(smem_u32(bars + 2));
  } else if (tid == 32) {
    // a block that started beside the state kernel: the state tile's load, issued here by another warp than the
    // one that waits for it, so that the common path above carries nothing extra
    if (*s_pending_sm != 0u && !fwd_load_state_late(state_done, state_target, &maps.s, smem_u32(sm + FwdSmem::S), (int)(chunk_id * TD), smem_u32(bars + 4)))
      atomicAdd(&g_tc_wait_timeouts, 1u);
  }
  // The saved copy of P goes out from the assembled shared-memory tile while the output product runs: rows are
  // written whole (a warp stores two full 256-byte rows per instruction) instead of in 16-byte pieces of 32
  // different rows from the read-back above.
  if (P_saved) {
    bf16* pg = P_saved + chunk_id * TC * TC;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int id = tid + TTHREADS * j, row = id >> 4, ch = id & 15;
      const uint4 u = *reinterpret_cast<const uint4*>(sm + FwdSmem::P + (ch >> 3) * TILE_BYTES + sw128_chunk(row, ch & 7));
      *reinterpret_cast<uint4*>(pg + row * TC + ch * 8) = u;
    }
  }
  ok = mbar_wait(smem_u32(bars + 2), 0) && ok;
  tc_fence_after();
  if (ok) {
    const int q4 = warp & 3, cg = warp >> 2;
    uint32_t r[32];
    tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(cg * 32), r);
    tmem_ld_wait();
    bf16* o = out + row0 + (int64_t)(q4 * 32 + lane) * HD + cg * 32;
    // 64 contiguous bytes of one row per thread, rows of a warp far apart: two 32-byte stores
#pragma unroll
    for (int c8 = 0; c8 < 2; ++c8) {
      uint32_t u[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) u[m] = pack_bf16x2(__uint_as_float(r[16 * c8 + 2 * m]), __uint_as_float(r[16 * c8 + 2 * m + 1]));
      st_global_v8(o + 16 * c8, u);
    }
  } else if (tid == 0) {
    atomicAdd(&g_tc_wait_timeouts, 1u);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------
// Backward chunk kernel (gla.py:552-625, 731-790, 857-960, 1036-1189).
//
//   dP = dO V^T                      dV = P^T dO + k_hat dS_next
//   dq = (dO S_prev^T) exp(lam) + sum_levels (dP_l k~_l) wq_l + diag
//   dk = (V dS_next^T) exp(G-lam) + sum_levels (dP_l^T q~_l) wk_l + diag
//   dlam = q dq - k dk ;  dG = sum_c dk_hat k_hat + e^G sum_v S_prev dS_next
//   dg = reverse cumsum of dlam within the chunk + dG
//
// Everything that must be multiplied by a (row, feature)-dependent decay weight AFTER its
// contraction (the two inter-chunk terms and all level terms) is computed TRANSPOSED, with
// the feature index d on the TMEM lanes and the chunk rows on the TMEM columns.  A thread
// then owns one feature d and a run of rows ("column layout"): the accumulator it reads back
// with tcgen05.ld is exactly the slice whose weights it can form from its own gates by
// running products, and the final reverse cumsum over rows is a serial loop in registers.
//
// Register budget forces two passes over the rows (first rows 64..127, then 0..63): in a
// pass thread (d, rq) owns rows 64 p + 16 rq + [0, 16).  For half sizes h <= 32 a row's dyadic
// partners lie in the same 64-row half, so a level is M = 128 (d) x N = 64 (rows of the half)
// x K = 64 (partner rows): A = W_l (row r' holds q~ or k~ of that row, whichever side it is
// on), B = the 64 x 64 block of dP masked to the level, once as (n = i, k = j) and once as
// (n = j, k = i), both accumulating into one tile.  For h = 64 the partners are the other
// half; W_64 for all 128 rows is built before the passes.
// ---------------------------------------------------------------------------------------
struct BwdSmem {
  static constexpr uint32_t DO = 0;                        // dO   (rows i, cols dv)     -> later W64
  static constexpr uint32_t V = DO + 2 * TILE_BYTES;       // v    (rows j, cols dv)     -> later W_l x2
  static constexpr uint32_t SP = V + 2 * TILE_BYTES;       // S_prev (rows dk, cols dv)  -> later dP_l x2
  static constexpr uint32_t DS = SP + 2 * TILE_BYTES;      // dS_next (rows dk, cols dv)
  static constexpr uint32_t P = DS + 2 * TILE_BYTES;       // P    (rows i, cols j)
  static constexpr uint32_t KH = P + 2 * TILE_BYTES;       // k_hat (rows j, cols dk)
  static constexpr uint32_t TOT = KH + 2 * TILE_BYTES;     // [8][128] float: gate products per 16 rows
  static constexpr uint32_t GRP = TOT + 8 * TD * 4;        // [8][128] float: dlam totals per 16 rows
  static constexpr uint32_t DIAG = GRP + 8 * TD * 4;       // [128] float: dP[i][i]
  static constexpr uint32_t DG1 = DIAG + TC * 4;           // [4][128] float: partial sums of the two dG terms, one slot per
  static constexpr uint32_t DG2 = DG1 + 4 * TD * 4;        // [4][128] float  quarter of the rows (summed in a fixed order)
  static constexpr uint32_t GAB = DG2 + 4 * TD * 4;        // [4][128] float: sums of |g| per 32 rows
  static constexpr uint32_t BAR = GAB + 4 * TD * 4;        // 8 mbarriers + tmem slot
  static constexpr uint32_t END = BAR + 96;
  // After the phase-1 products have completed, dO, v and P are dead; after phase 1.5 the rest is.  Reuse:
  static constexpr uint32_t W64 = KH;                      // 32 KB: k~ / q~ at the h = 64 anchor, all 128 rows
  static constexpr uint32_t WL = DS;                       // 2 x 16 KB: per-level W_l
  static constexpr uint32_t DPL = SP;                      // 2 x 8 KB: per-level masked dP block
  static constexpr uint32_t DPD = V + 24576;               // [128][16] float: each row's 16 x 16 diagonal block of dP
  // TMA landing zones of g, q, k for the row passes (plain row-major, 64 rows each)
  static constexpr uint32_t GH = DO;                       // [64][128] float: gates of the pass's rows
  static constexpr uint32_t QH = P;                        // [64][128] bf16: q of the pass's rows
  static constexpr uint32_t K1 = P + 16384;                // [64][128] bf16: k of rows 64..127
  static constexpr uint32_t K0 = V;                        // [64][128] bf16: k of rows 0..63
  // TMA landing zones of the chunk's gates and raw q at the start of the block (raw k lands in KH)
  static constexpr uint32_t G0 = SP;                       // [128][128] float row-major (64 KB over S_prev and dS_next)
  static constexpr uint32_t Q0 = P;                        // [128][128] bf16 row-major
  // One-scale path (chunks whose gates need no secondary chunking), after the phase-1 products:
  static constexpr uint32_t ST0 = DO;                      // [16][512] u32: every thread's own (k | q << 16) of its rows 0..15
  static constexpr uint32_t ST1 = P;                       // [16][512] u32: ... of its rows 16..31
  static constexpr uint32_t DPM = V;                       // 32 KB: dP masked to the strict lower triangle (rows i, cols j)
  static constexpr uint32_t QT = SP;                       // 32 KB: q~ = q exp(lam - G), stored like k_hat (rows = feature)
  static constexpr uint32_t DLB = V;                       // [128][128] float row-major (64 KB over V and S_prev): dlam suffix sums
  static constexpr uint32_t DQT = DS;                      // [128][128] bf16 row-major: dq of the chunk, staged for whole-row stores
  static constexpr uint32_t DKT = KH;                      // [128][128] bf16 row-major: dk
};
struct BwdMaps {
  CUtensorMap g, q, k;          // boxes of 128 features x 64 rows, unswizzled (row passes)
  CUtensorMap dO, v;            // boxes of 64 features x 128 rows, 128-byte swizzle (operand tiles)
  CUtensorMap sp, ds, p;        // dense (rows, 128) matrices: boxes of 64 columns x 128 rows, 128-byte swizzle
};
constexpr uint32_t TM_DP = 0, TM_DQH = 128, TM_DKH = 256, TM_DV = 384, TM_T = 384;

// Decay weights of the thread's 16 rows at level slot S (half size 2^S), column layout.
// f[i] = gate of row i of the thread's run; rq = which 16-row run of the 64-row half; p = which half.
// right(i) tells which side row i is on; w[i] is wq (right side) or wk (left side).
template <int S>
__device__ __forceinline__ void level_weights(const float (&f)[16], int rq, int p, const float* tot, int d,
                                              float (&w)[16]) {
  if (S < 4) {
    constexpr int HH = 1 << S;
    float run = 1.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {          // inclusive prefix within aligned HH-blocks
      run = (i % HH == 0) ? f[i] : run * f[i];
      if (i & HH) w[i] = run;
    }
#pragma unroll
    for (int i = 15; i >= 0; --i) {         // exclusive suffix within aligned HH-blocks
      if (i % HH == HH - 1) run = 1.f;
      if (!(i & HH)) w[i] = run;
      run *= f[i];
    }
  } else {
    const int g = 4 * p + rq;
    bool right;
    float cross = 1.f;
    if (S == 4) {
      right = rq & 1;
    } else if (S == 5) {
      right = rq >= 2;
      if (rq == 3) cross = tot[(g - 1) * TD + d];
      if (rq == 0) cross = tot[(g + 1) * TD + d];
    } else {
      right = p == 1;
      if (right) { for (int b2 = 4; b2 < g; ++b2) cross *= tot[b2 * TD + d]; }
      else       { for (int b2 = g + 1; b2 < 4; ++b2) cross *= tot[b2 * TD + d]; }
    }
    if (right) {
      float run = cross;
#pragma unroll
      for (int i = 0; i < 16; ++i) { run *= f[i]; w[i] = run; }
    } else {
      float run = cross;
#pragma unroll
      for (int i = 15; i >= 0; --i) { w[i] = run; run *= f[i]; }
    }
  }
}
template <int S>
__device__ __forceinline__ bool row_is_right(int i, int rq, int p) {
  return S < 4 ? ((i >> S) & 1) : S == 4 ? (rq & 1) : S == 5 ? (rq >= 2) : (p == 1);
}

// Raw 16-bit global load (bf16 bits).  Loops below first issue ALL their loads into raw registers and
// only then convert / use them: an instruction consuming a loaded value right behind the load stalls
// the in-order warp for a full memory latency per load, which serialises the loads.
__device__ __forceinline__ uint32_t ldg_u16(const bf16* p) { return (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(p)); }
__device__ __forceinline__ float bf16_bits_to_float(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ void st_bf16(uint8_t* p, float v) { *reinterpret_cast<bf16*>(p) = __float2bfloat16_rn(v); }

// Out of line on purpose (inlined, even skipped, it cost the common path 5 us per launch): the balanced anchor's
// rescaling of the dS_next tile.  Row d of the tile takes w = 1 / A (this thread: its columns 32 wq + [0, 32)), so that
// k_hat dS_next and dS_next V^T come out as with the end anchor, the latter divided by A like the dk~ term that joins
// it.  Waits (bounded) for the tile to have landed first and leaves it alone if it has not.
__device__ __noinline__ void bwd_rescale_ds(uint8_t* ds, uint32_t bar, float w, int d, int wq) {
  if (!mbar_wait(bar, 0)) return;
  uint8_t* td = ds + (wq >> 1) * TILE_BYTES;
#pragma unroll
  for (int c4 = 0; c4 < 4; ++c4) {
    uint4* p4 = reinterpret_cast<uint4*>(td + sw128_chunk(d, (wq & 1) * 4 + c4));
    uint4 u = *p4;
    u.x = pack_bf16x2(bf16_lo(u.x) * w, bf16_hi(u.x) * w); u.y = pack_bf16x2(bf16_lo(u.y) * w, bf16_hi(u.y) * w);
    u.z = pack_bf16x2(bf16_lo(u.z) * w, bf16_hi(u.z) * w); u.w = pack_bf16x2(bf16_lo(u.w) * w, bf16_hi(u.w) * w);
    *p4 = u;
  }
}

__global__ void __launch_bounds__(TTHREADS, 1)
tc_chunk_bwd_kernel(const __grid_constant__ BwdMaps maps, int64_t T, int64_t H, int R, int64_t N, int pf_dist, const float* __restrict__ g, const bf16* __restrict__ v,
                    const bf16* __restrict__ k, const bf16* __restrict__ q, const bf16* __restrict__ dO,
                    const bf16* __restrict__ S_prev, const bf16* __restrict__ dS_next, const bf16* __restrict__ P_saved,
                    bf16* __restrict__ dq_out, bf16* __restrict__ dk_out, bf16* __restrict__ dv_out,
                    float* __restrict__ dg_out, int all_scales) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  float* tot = reinterpret_cast<float*>(sm + BwdSmem::TOT);
  float* grp = reinterpret_cast<float*>(sm + BwdSmem::GRP);
  float* diag = reinterpret_cast<float*>(sm + BwdSmem::DIAG);
  float* dG1 = reinterpret_cast<float*>(sm + BwdSmem::DG1);
  float* dG2 = reinterpret_cast<float*>(sm + BwdSmem::DG2);
  float* gab = reinterpret_cast<float*>(sm + BwdSmem::GAB);
  // mbarriers [0]: phase-1 products, [1],[2]: level buffers / the two closing products, [3],[4]: pass loads,
  // [5]: dO and v tiles, [6]: gates and raw q, k, [7]: the three late tiles; the TMEM address slot lies behind them
  constexpr int BWD_NBARS = 8;
  static_assert(BWD_NBARS * 8 + 8 <= 96, "barriers and the TMEM slot must fit the space reserved at BwdSmem::BAR");
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + BwdSmem::BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BWD_NBARS);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, wq_ = warp >> 2;        // TMEM lane quadrant, and which quarter of the columns
  const int d = 32 * q4 + lane;                     // column layout: feature index
  // H counts virtual heads (see the forward kernel).  Inputs are addressed in the (B, T, H / R, 128) view: key-side
  // tensors (g, q, k) at head hk_, value-side tensors (v, dO) at head hv_; the gradients are written per virtual
  // head, (B, T, H, 128), and the caller sums dq, dk, dg over the value blocks and dv over the key blocks.
  // Block order: chunk-major, FIRST chunks first: the gradient-state kernel before this one walks the chunks of all
  // heads last to first, so g, q, dO of the early chunks and the gradient states written last are freshest in L2.
  const int64_t BHn = (int64_t)gridDim.x / N;
  const int64_t n = (int64_t)blockIdx.x / BHn, bh = (int64_t)blockIdx.x % BHn, b = bh / H, h_ = bh % H;
  const int64_t hk_ = (h_ / (R * R)) * R + (h_ % (R * R)) / R, hv_ = (h_ / (R * R)) * R + h_ % R;
  const int64_t HD = H * TD;                                          // output row pitch (virtual heads)
  const int64_t row0 = ((b * T + n * TC) * H + h_) * TD;              // outputs
  const int64_t chunk_id = bh * N + n;

  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(smem_u32(bars + 0), 4);        // four issuing threads commit the phase-1 products
#pragma unroll
    for (int i = 1; i < BWD_NBARS; ++i) mbar_init(smem_u32(bars + i), 1);
    mbar_fence_init();
    // What the block needs first, the gates and raw q, k of the whole chunk (row-major, 128 KB), comes by TMA into
    // regions whose operand tiles are not needed until the products: g over the S_prev and dS_next regions, q over
    // the P region, k into the region that k_hat will occupy.  Every thread copies its 32 rows of one feature from
    // there into registers; after the barrier that follows, the three late tiles are requested.
    const int z = (int)(b * T + n * TC), yv = (int)hv_, yk = (int)hk_;
    {
      const uint32_t kb = smem_u32(bars + 6);
      mbar_arrive_expect_tx(kb, 8 * TILE_BYTES);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        tma_load_3d(smem_u32(sm + BwdSmem::G0 + half * 2 * TILE_BYTES), &maps.g, 0, yk, z + 64 * half, kb);
        tma_load_3d(smem_u32(sm + BwdSmem::Q0 + half * TILE_BYTES), &maps.q, 0, yk, z + 64 * half, kb);
        tma_load_3d(smem_u32(sm + BwdSmem::KH + half * TILE_BYTES), &maps.k, 0, yk, z + 64 * half, kb);
      }
    }
    // dO and v keep their own regions and land while the gates are processed
    const uint32_t lb = smem_u32(bars + 5);
    mbar_arrive_expect_tx(lb, 2 * 2 * TILE_BYTES);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      tma_load_3d(smem_u32(sm + BwdSmem::DO + half * TILE_BYTES), &maps.dO, 64 * half, yv, z, lb);
      tma_load_3d(smem_u32(sm + BwdSmem::V + half * TILE_BYTES), &maps.v, 64 * half, yv, z, lb);
    }
  }

  // The barriers must be initialised before any other thread waits on one (the first wait follows at once now that
  // the gates come through shared memory), and the TMEM address must be visible.
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // ---- phase 0: gate products per 16 rows; k_hat (the operand tiles are arriving by TMA) ------------------
  float f32r[32];                                   // gates of rows 32 wq_ + [0, 32), feature d
  uint32_t kraw[32];                                // k of the same rows and feature (low half), q above it
  bool ok = true;
  {
    const bool lok = mbar_wait(smem_u32(bars + 6), 0);
    ok = lok;
    const float* gs = reinterpret_cast<const float*>(sm + BwdSmem::G0) + (32 * wq_) * TD + d;
    const unsigned short* qs = reinterpret_cast<const unsigned short*>(sm + BwdSmem::Q0) + (32 * wq_) * TD + d;
    const unsigned short* ks = reinterpret_cast<const unsigned short*>(sm + BwdSmem::KH) + (32 * wq_) * TD + d;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      f32r[i] = lok ? gs[i * TD] : 0.f;
      kraw[i] = lok ? ((uint32_t)ks[i * TD] | ((uint32_t)qs[i * TD] << 16)) : 0u;
    }
    float p0 = 1.f, p1 = 1.f, ga = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      ga += fabsf(f32r[i]);
      f32r[i] = __expf(f32r[i]);
      if (i < 16) p0 *= f32r[i]; else p1 *= f32r[i];
    }
    tot[(2 * wq_) * TD + d] = p0;
    tot[(2 * wq_ + 1) * TD + d] = p1;
    gab[wq_ * TD + d] = ga;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // One scale or all of them (see ONE_SCALE_LIMIT): decided from the chunk's total |log decay| per feature, the
  // same way for every thread of the block.
  bool one_scale, balanced;
  float A = 1.f;
  {
    const float tsum = (gab[d] + gab[TD + d]) + (gab[2 * TD + d] + gab[3 * TD + d]);
    one_scale = __syncthreads_or(!(tsum <= ONE_SCALE_LIMIT) || all_scales != 0) == 0;
    balanced = false;
    if (!one_scale) balanced = one_scale = __syncthreads_or(!(tsum <= BALANCED_LIMIT) || all_scales != 0) == 0;
    // balanced anchor (see BALANCED_LIMIT): A = exp(-m_d) = exp(sum |g| / 2) rides on k_hat, its inverse on the rows
    // of the dS_next tile and on q~
    if (balanced) A = __expf(0.5f * tsum);
  }
  if (tid == 0) {
    // every thread holds its gates, q and k in registers (two barriers back): the landing zones take the three late
    // operand tiles, which arrive while k_hat is built
    const uint32_t lb = smem_u32(bars + 7);
    const int cr = (int)(chunk_id * TD);
    mbar_arrive_expect_tx(lb, 3 * 2 * TILE_BYTES);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      tma_load_2d(smem_u32(sm + BwdSmem::SP + half * TILE_BYTES), &maps.sp, 64 * half, cr, lb);
      tma_load_2d(smem_u32(sm + BwdSmem::DS + half * TILE_BYTES), &maps.ds, 64 * half, cr, lb);
      tma_load_2d(smem_u32(sm + BwdSmem::P + half * TILE_BYTES), &maps.p, 64 * half, cr, lb);
    }
  }
  {
    // k_hat[r][d] = k[r][d] * prod_{t > r} f_t   (rows of this thread: 32 wq_ + i), times A with the balanced anchor
    float run = A;
    for (int b2 = 2 * wq_ + 2; b2 < 8; ++b2) run *= tot[b2 * TD + d];
    // stored TRANSPOSED: row = feature dk, columns = chunk rows j, so the thread's 32 values are 64
    // contiguous bytes (four 16-byte stores instead of 32 two-byte ones)
    uint8_t* tile = sm + BwdSmem::KH + (wq_ >> 1) * TILE_BYTES;
    uint32_t pk[16];
#pragma unroll
    for (int i = 31; i >= 1; i -= 2) {
      const float hi = bf16_bits_to_float(kraw[i]) * run;
      run *= f32r[i];
      const float lo = bf16_bits_to_float(kraw[i - 1]) * run;
      run *= f32r[i - 1];
      pk[i >> 1] = pack_bf16x2(lo, hi);
    }
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4)
      *reinterpret_cast<uint4*>(tile + sw128_chunk(d, (wq_ & 1) * 4 + c4)) =
          make_uint4(pk[4 * c4], pk[4 * c4 + 1], pk[4 * c4 + 2], pk[4 * c4 + 3]);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (balanced) {
    // (its wait is not folded into `ok`: measured, that dependency alone cost the common path 3.5 us per launch; a
    // tile that never lands fails the issuing threads' wait on the same barrier below)
    bwd_rescale_ds(sm + BwdSmem::DS, smem_u32(bars + 7), 1.f / A, d, wq_);
    fence_async_smem();
    __syncthreads();
  }

  // ---- phase 1: the four dense products --------------------------------------------------------------
  // Issued by four threads of four warps on different schedulers (8 to 16 MMAs each instead of 40 from one): the
  // issuing thread's instruction stream is serial, so this shortens the wait of everybody else.  The two halves of
  // dV come from the same thread, in order.
  if (lane == 0 && (warp == 3 || warp == 6 || warp == 9 || warp == 12)) {
    ok = mbar_wait(smem_u32(bars + 5), 0) && ok;    // operand tiles landed
    ok = mbar_wait(smem_u32(bars + 7), 0) && ok;
    tc_fence_after();
    constexpr uint32_t iKK = idesc_bf16(128, 128, 0, 0), iMM = idesc_bf16(128, 128, 1, 1);
    const uint32_t aDO = smem_u32(sm + BwdSmem::DO), aV = smem_u32(sm + BwdSmem::V);
    if (warp == 3) {
      const uint64_t kDO = desc_kmajor(aDO, TILE_BYTES, 0), kV = desc_kmajor(aV, TILE_BYTES, 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)   // dP[i][j] = sum_dv dO[i][dv] v[j][dv]
        umma_bf16(tmem + TM_DP, kslice_kmajor(kDO, TILE_BYTES, ks), kslice_kmajor(kV, TILE_BYTES, ks), iKK, ks > 0);
    } else if (warp == 6) {
      const uint64_t kSP = desc_kmajor(smem_u32(sm + BwdSmem::SP), TILE_BYTES, 0), kDO = desc_kmajor(aDO, TILE_BYTES, 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)   // dQh^T[dk][i] = sum_dv S_prev[dk][dv] dO[i][dv]
        umma_bf16(tmem + TM_DQH, kslice_kmajor(kSP, TILE_BYTES, ks), kslice_kmajor(kDO, TILE_BYTES, ks), iKK, ks > 0);
    } else if (warp == 9) {
      const uint64_t kDS = desc_kmajor(smem_u32(sm + BwdSmem::DS), TILE_BYTES, 0), kV = desc_kmajor(aV, TILE_BYTES, 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)   // dKh^T[dk][j] = sum_dv dS_next[dk][dv] v[j][dv]
        umma_bf16(tmem + TM_DKH, kslice_kmajor(kDS, TILE_BYTES, ks), kslice_kmajor(kV, TILE_BYTES, ks), iKK, ks > 0);
    } else {
      const uint64_t mP = desc_mnmajor(smem_u32(sm + BwdSmem::P), TILE_BYTES, 0), mDO = desc_mnmajor(aDO, TILE_BYTES, 0);
      const uint64_t mKH = desc_mnmajor(smem_u32(sm + BwdSmem::KH), TILE_BYTES, 0), mDS = desc_mnmajor(smem_u32(sm + BwdSmem::DS), TILE_BYTES, 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)   // dV[j][dv] = sum_i P[i][j] dO[i][dv]
        umma_bf16(tmem + TM_DV, kslice_mnmajor(mP, ks), kslice_mnmajor(mDO, ks), iMM, ks > 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)   //          + sum_dk k_hat[j][dk] dS_next[dk][dv]
        umma_bf16(tmem + TM_DV, kslice_mnmajor(mKH, ks), kslice_mnmajor(mDS, ks), iMM, 1);
    }
    umma_commit(smem_u32(bars + 0));
  }
  __syncwarp();
  // This chunk's operands have landed: ask L2 for those of the chunk that the block scheduler will
  // start on this SM when this block retires (pf_dist blocks ahead), so that its load phase streams
  // from L2 while DRAM is busy during everybody's compute phases instead of everybody's load phases.
  // One thread requests the same boxes the next block will load (tensor prefetches: one instruction per
  // box, where per-line prefetches cost every thread three instructions and measured 1 us slower).
  {
    const int64_t nb = (int64_t)blockIdx.x + pf_dist;
    if (pf_dist > 0 && nb < (int64_t)gridDim.x && tid == 0) {
      const int64_t n2 = nb / BHn, bh2 = nb % BHn, h2 = bh2 % H;
      const int y2 = (int)((h2 / (R * R)) * R + (h2 % (R * R)) / R), yv2 = (int)((h2 / (R * R)) * R + h2 % R);
      const int z2 = (int)((bh2 / H) * T + n2 * TC);
      const int64_t c2 = (bh2 * N + n2) * TD * TD;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        tma_prefetch_l2_3d(&maps.g, 0, y2, z2 + 64 * half);
        tma_prefetch_l2_3d(&maps.q, 0, y2, z2 + 64 * half);
        tma_prefetch_l2_3d(&maps.k, 0, y2, z2 + 64 * half);
        tma_prefetch_l2_3d(&maps.dO, 64 * half, yv2, z2);
        tma_prefetch_l2_3d(&maps.v, 64 * half, yv2, z2);
      }
      // contiguous 32 KB tiles: one bulk request each
      l2_prefetch_bulk(S_prev + c2, 2 * TD * TD);
      l2_prefetch_bulk(dS_next + c2, 2 * TD * TD);
      l2_prefetch_bulk(P_saved + (bh2 * N + n2) * TC * TC, 2 * TC * TC);
    }
  }
  ok = mbar_wait(smem_u32(bars + 0), 0) && ok;
  ok = mbar_wait(smem_u32(bars + 5), 0) && ok;      // every thread observes the tiles' arrival itself before reading them
  ok = mbar_wait(smem_u32(bars + 7), 0) && ok;
  tc_fence_after();
  // dO, v and P have been consumed by the products: their regions take g, q, k of rows 64..127 and k of rows
  // 0..63 by TMA while phase 1.5 runs, so that the W64 build and the first pass read them from shared memory.
  const int zrow = (int)(b * T + n * TC), yh = (int)hk_;
  if (one_scale) {
    // every thread parks the raw k and q of its 32 rows in the regions the products have released; it alone reads
    // them back (for the q~ operand and in the closing pass), so no barrier is involved
    uint32_t* st0 = reinterpret_cast<uint32_t*>(sm + BwdSmem::ST0) + tid;
    uint32_t* st1 = reinterpret_cast<uint32_t*>(sm + BwdSmem::ST1) + tid;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      st0[i * TTHREADS] = kraw[i];
      st1[i * TTHREADS] = kraw[16 + i];
    }
  } else if (tid == 0) {
    const uint32_t lb = smem_u32(bars + 3);
    mbar_arrive_expect_tx(lb, 32768 + 3 * 16384);
    tma_load_3d(smem_u32(sm + BwdSmem::GH), &maps.g, 0, yh, zrow + 64, lb);
    tma_load_3d(smem_u32(sm + BwdSmem::QH), &maps.q, 0, yh, zrow + 64, lb);
    tma_load_3d(smem_u32(sm + BwdSmem::K1), &maps.k, 0, yh, zrow + 64, lb);
    tma_load_3d(smem_u32(sm + BwdSmem::K0), &maps.k, 0, yh, zrow, lb);
  }

  // ---- phase 1.5: dV out, dP diagonal, the two dG sums ---------------------------------------------------
  {
    // three accumulator slices per thread; the first two loads are in flight together, the third (dP) follows
    // while their values are being used
    uint32_t r[32], r2[32];
    const uint32_t lane_base = tmem + ((uint32_t)(q4 * 32) << 16);
    tmem_ld32(lane_base + TM_DV + 32 * wq_, r);       // row j = d here (row layout)
    tmem_ld32(lane_base + TM_DKH + 32 * wq_, r2);     // feature d, rows 32 wq_ + m (column layout)
    tmem_ld_wait();
    if (ok) {
      bf16* o = dv_out + row0 + (int64_t)d * HD + 32 * wq_;
      // a thread owns 64 contiguous bytes of one row; the rows of a warp are far apart, so what counts is the
      // number of store requests: two 32-byte stores instead of four 16-byte ones
#pragma unroll
      for (int c8 = 0; c8 < 2; ++c8) {
        uint32_t u[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) u[m] = pack_bf16x2(__uint_as_float(r[16 * c8 + 2 * m]), __uint_as_float(r[16 * c8 + 2 * m + 1]));
        st_global_v8(o + 16 * c8, u);
      }
    }
    // the thread's slice of dP (row i = d, columns 32 wq_ + [0, 32)): the single-anchor path masks all of it into an
    // operand tile; every path needs the diagonal entries, which lie in the slices with wq_ == q4
    const bool need_dp = one_scale || wq_ == q4;
    if (need_dp) tmem_ld32(lane_base + TM_DP + 32 * wq_, r);
    // dG1[d] = sum_r dKh^T[d][r] k_hat[r][d]   (this thread: rows 32 wq_ + m)
    {
      float s1 = 0.f;
      const uint8_t* tile = sm + BwdSmem::KH + (wq_ >> 1) * TILE_BYTES;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const uint4 a = *reinterpret_cast<const uint4*>(tile + sw128_chunk(d, (wq_ & 1) * 4 + c4));
        s1 = fmaf(__uint_as_float(r2[8 * c4 + 0]), bf16_lo(a.x), s1); s1 = fmaf(__uint_as_float(r2[8 * c4 + 1]), bf16_hi(a.x), s1);
        s1 = fmaf(__uint_as_float(r2[8 * c4 + 2]), bf16_lo(a.y), s1); s1 = fmaf(__uint_as_float(r2[8 * c4 + 3]), bf16_hi(a.y), s1);
        s1 = fmaf(__uint_as_float(r2[8 * c4 + 4]), bf16_lo(a.z), s1); s1 = fmaf(__uint_as_float(r2[8 * c4 + 5]), bf16_hi(a.z), s1);
        s1 = fmaf(__uint_as_float(r2[8 * c4 + 6]), bf16_lo(a.w), s1); s1 = fmaf(__uint_as_float(r2[8 * c4 + 7]), bf16_hi(a.w), s1);
      }
      dG1[wq_ * TD + d] = s1;
    }
    if (need_dp) tmem_ld_wait();
    if (wq_ == q4) {          // the 32 x 32 diagonal block of dP: pick dP[i][i]
      float dv_ = 0.f;
#pragma unroll
      for (int m = 0; m < 32; ++m)
        if (m == lane) dv_ = __uint_as_float(r[m]);
      diag[d] = dv_;
      if (!one_scale) {
        // this row's 16 x 16 diagonal block of dP in float32, for the small levels done on the CUDA cores
        // (the v tile this overwrites was last read by the phase-1 products, which have completed)
        float4* dpd = reinterpret_cast<float4*>(sm + BwdSmem::DPD + d * 64);
        const bool hi = (lane & 16) != 0;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4)
          dpd[c4] = make_float4(__uint_as_float(hi ? r[16 + 4 * c4 + 0] : r[4 * c4 + 0]), __uint_as_float(hi ? r[16 + 4 * c4 + 1] : r[4 * c4 + 1]),
                                __uint_as_float(hi ? r[16 + 4 * c4 + 2] : r[4 * c4 + 2]), __uint_as_float(hi ? r[16 + 4 * c4 + 3] : r[4 * c4 + 3]));
      }
    }
    if (one_scale) {
      // dP restricted to j < i as a bf16 operand tile (row i = d here, columns 32 wq_ + [0, 32)); the v tile it
      // overwrites was last read by the phase-1 products
      uint8_t* tile = sm + BwdSmem::DPM + (wq_ >> 1) * TILE_BYTES;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t pk[4];
#pragma unroll
        for (int m = 0; m < 8; m += 2) {
          const int j = 32 * wq_ + 8 * c4 + m;
          pk[m >> 1] = pack_bf16x2(j < d ? __uint_as_float(r[8 * c4 + m]) : 0.f, j + 1 < d ? __uint_as_float(r[8 * c4 + m + 1]) : 0.f);
        }
        *reinterpret_cast<uint4*>(tile + sw128_chunk(d, (wq_ & 1) * 4 + c4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }
    // dG2[d] = sum_v S_prev[d][v] dS_next[d][v]    (this thread: v in 32 wq_ + [0, 32))
    float s2 = 0.f;
    const uint8_t* ts = sm + BwdSmem::SP + (wq_ >> 1) * TILE_BYTES;
    const uint8_t* td = sm + BwdSmem::DS + (wq_ >> 1) * TILE_BYTES;
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      const uint4 a = *reinterpret_cast<const uint4*>(ts + sw128_chunk(d, (wq_ & 1) * 4 + c4));
      const uint4 c = *reinterpret_cast<const uint4*>(td + sw128_chunk(d, (wq_ & 1) * 4 + c4));
      s2 += bf16_lo(a.x) * bf16_lo(c.x) + bf16_hi(a.x) * bf16_hi(c.x) + bf16_lo(a.y) * bf16_lo(c.y) + bf16_hi(a.y) * bf16_hi(c.y) +
            bf16_lo(a.z) * bf16_lo(c.z) + bf16_hi(a.z) * bf16_hi(c.z) + bf16_lo(a.w) * bf16_lo(c.w) + bf16_hi(a.w) * bf16_hi(c.w);
    }
    dG2[wq_ * TD + d] = s2;
  }
  tc_fence_before();
  __syncthreads();      // all readers of the phase-1 tiles are done: the regions can be reused
  tc_fence_after();

  // (A is formed again from the |g| sums here rather than kept in a register across the products and phase 1.5)
  const float A2 = balanced ? __expf(0.5f * ((gab[d] + gab[TD + d]) + (gab[2 * TD + d] + gab[3 * TD + d]))) : 1.f;
  float eG = A2;          // exp(G), times A with the balanced anchor (dG2 was formed from the rescaled dS_next tile)
#pragma unroll
  for (int b2 = 0; b2 < 8; ++b2) eG *= tot[b2 * TD + d];
  // the four partial sums of each dG term in a fixed order: the result does not depend on which warp came first
  const float dG = ((dG1[d] + dG1[TD + d]) + (dG1[2 * TD + d] + dG1[3 * TD + d])) +
                   eG * ((dG2[d] + dG2[TD + d]) + (dG2[2 * TD + d] + dG2[3 * TD + d]));

  if (one_scale) {
    // ---- one anchor (the chunk's last row) for all intra-chunk terms:
    //   dq~^T[d][i] = sum_j k_hat[j][d] dPm[i][j],   dq_intra = dq~ exp(lam_i - G)
    //   dk~^T[d][j] = sum_i q~[i][d]   dPm[i][j],   dk_intra = dk~ exp(G - lam_j),   q~ = q exp(lam - G)
    // two 128 x 128 x 128 products; a thread (feature d, rows 32 wq_ + [0, 32)) then finishes its rows in one pass.
    const uint32_t lane_base = tmem + ((uint32_t)(q4 * 32) << 16);
    const float t0 = tot[(2 * wq_) * TD + d], t1 = tot[(2 * wq_ + 1) * TD + d];
    // gate products of the rows before / after this thread's 32; with the balanced anchor Ck and 1 / eG carry A and
    // 1 / A, which keeps every running product below within exp(+-limit / 2)
    const float invG = 1.f / eG;
    float Cq = 1.f, Cqi = invG, Ck = A2;      // Cqi: the same product as Cq started from 1 / eG (see the closing pass)
    for (int b2 = 0; b2 < 2 * wq_; ++b2) { const float t = tot[b2 * TD + d]; Cq *= t; Cqi *= t; }
    for (int b2 = 2 * wq_ + 2; b2 < 8; ++b2) Ck *= tot[b2 * TD + d];
    const uint32_t* st0 = reinterpret_cast<const uint32_t*>(sm + BwdSmem::ST0) + tid;     // this thread's parked (k | q << 16)
    const uint32_t* st1 = reinterpret_cast<const uint32_t*>(sm + BwdSmem::ST1) + tid;
    {
      uint32_t qr[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) { qr[i] = st0[i * TTHREADS]; qr[16 + i] = st1[i * TTHREADS]; }
      // q~[r] = q[r] / prod_{t > r} f_t = q[r] * (prod_{first <= t <= r} f_t) / (prod_{t >= first} f_t): one reciprocal
      float run = 1.f / (t0 * t1 * Ck);
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        run *= f32r[i];
        const float lo = bf16_hi(qr[i]) * run;
        run *= f32r[i + 1];
        const float hi = bf16_hi(qr[i + 1]) * run;
        pk[i >> 1] = pack_bf16x2(lo, hi);
      }
      uint8_t* tile = sm + BwdSmem::QT + (wq_ >> 1) * TILE_BYTES;       // transposed like k_hat: row = feature
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4)
        *reinterpret_cast<uint4*>(tile + sw128_chunk(d, (wq_ & 1) * 4 + c4)) =
            make_uint4(pk[4 * c4], pk[4 * c4 + 1], pk[4 * c4 + 2], pk[4 * c4 + 3]);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t iK = idesc_bf16(128, 128, 0, 0);
      const uint64_t kA = desc_kmajor(smem_u32(sm + BwdSmem::KH), TILE_BYTES, 0), kB = desc_kmajor(smem_u32(sm + BwdSmem::DPM), TILE_BYTES, 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)     // dq~^T[d][i] = sum_j k_hat^T[d][j] dPm[i][j]
        umma_bf16(tmem + TM_DV, kslice_kmajor(kA, TILE_BYTES, ks), kslice_kmajor(kB, TILE_BYTES, ks), iK, ks > 0);
      umma_commit(smem_u32(bars + 1));
    } else if (tid == 32) {
      tc_fence_after();
      constexpr uint32_t iM = idesc_bf16(128, 128, 0, 1);
      const uint64_t kA = desc_kmajor(smem_u32(sm + BwdSmem::QT), TILE_BYTES, 0), mB = desc_mnmajor(smem_u32(sm + BwdSmem::DPM), TILE_BYTES, 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)     // dk~^T[d][j] = sum_i q~^T[d][i] dPm[i][j], on top of the inter-chunk term:
        umma_bf16(tmem + TM_DKH, kslice_kmajor(kA, TILE_BYTES, ks), kslice_mnmajor(mB, ks), iM, 1);   // same weight exp(G - lam_j)
      umma_commit(smem_u32(bars + 2));
    }
    ok = mbar_wait(smem_u32(bars + 1), 0) && ok;
    ok = mbar_wait(smem_u32(bars + 2), 0) && ok;
    tc_fence_after();
    // The operands of the two products are consumed: their regions stage the chunk's dq, dk (bf16) and the dlam suffix
    // sums (float32) row-major, so that they leave for global memory as whole rows instead of two or four bytes per
    // thread and row.
    float* dlb = reinterpret_cast<float*>(sm + BwdSmem::DLB);
    unsigned short* dqt = reinterpret_cast<unsigned short*>(sm + BwdSmem::DQT);
    unsigned short* dkt = reinterpret_cast<unsigned short*>(sm + BwdSmem::DKT);
    float carry = 0.f;            // sum of dlam over this thread's rows after the current half
#pragma unroll
    for (int hh = 1; hh >= 0; --hh) {
      const int rb = 32 * wq_ + 16 * hh;
      uint32_t a[16], c[16], qk[16];     // qk: k in the low half, q in the high half
      float dl[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) qk[i] = (hh ? st1 : st0)[i * TTHREADS];
      tmem_ld16(lane_base + TM_DQH + rb, a);
      tmem_ld16(lane_base + TM_DV + rb, c);
      tmem_ld_wait();
      // run = exp(lam_r) for the inter-chunk term (may underflow to zero in a sharp chunk, as the term itself does);
      // runi = exp(lam_r) / eG for the intra-chunk term, kept as a product of its own so that it never leaves the range
      float run = hh ? Cq * t0 : Cq, runi = hh ? Cqi * t0 : Cqi;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        run *= f32r[16 * hh + i];
        runi *= f32r[16 * hh + i];
        const float dqv = fmaf(runi, __uint_as_float(c[i]), run * __uint_as_float(a[i])) + diag[rb + i] * bf16_lo(qk[i]);
        dl[i] = bf16_hi(qk[i]) * dqv;
        dqt[(rb + i) * TD + d] = __bfloat16_as_ushort(__float2bfloat16_rn(dqv));
      }
      tmem_ld16(lane_base + TM_DKH + rb, a);
      tmem_ld_wait();
      run = hh ? Ck : Ck * t1;
#pragma unroll
      for (int i = 15; i >= 0; --i) {      // run = exp(G - lam_r)
        const float dkv = run * __uint_as_float(a[i]) + diag[rb + i] * bf16_hi(qk[i]);
        run *= f32r[16 * hh + i];
        dl[i] -= bf16_lo(qk[i]) * dkv;
        dkt[(rb + i) * TD + d] = __bfloat16_as_ushort(__float2bfloat16_rn(dkv));
      }
#pragma unroll
      for (int i = 14; i >= 0; --i) dl[i] += dl[i + 1];
#pragma unroll
      for (int i = 0; i < 16; ++i) dlb[(rb + i) * TD + d] = dl[i] + carry;
      carry += dl[0];
    }
    grp[wq_ * TD + d] = carry;
    if (wq_ == 0) gab[d] = dG;             // (the |g| sums kept here were last read at the path decision)
    tc_fence_before();
    __syncthreads();
    if (ok) {
      // dq, dk: 2048 pieces of 16 bytes each; a warp writes two whole 256-byte rows per instruction
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int id = tid + TTHREADS * j, row = id >> 4, ch = id & 15;
        const int64_t e = row0 + (int64_t)row * HD + ch * 8;
        *reinterpret_cast<uint4*>(dq_out + e) = *reinterpret_cast<const uint4*>(dqt + row * TD + ch * 8);
        *reinterpret_cast<uint4*>(dk_out + e) = *reinterpret_cast<const uint4*>(dkt + row * TD + ch * 8);
      }
      // dg = suffix sum inside the thread's rows + the totals of the later quarters of the chunk + dG: 4096 pieces of
      // four floats; a warp writes one whole 512-byte row per instruction
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int id = tid + TTHREADS * j, row = id >> 5, d0 = 4 * (id & 31), w = row >> 5;
        float4 x = *reinterpret_cast<const float4*>(dlb + row * TD + d0);
        float4 o = *reinterpret_cast<const float4*>(gab + d0);
#pragma unroll
        for (int w2 = 1; w2 < 4; ++w2) {
          if (w2 > w) {
            const float4 t = *reinterpret_cast<const float4*>(grp + w2 * TD + d0);
            o.x += t.x; o.y += t.y; o.z += t.z; o.w += t.w;
          }
        }
        x.x += o.x; x.y += o.y; x.z += o.z; x.w += o.w;
        *reinterpret_cast<float4*>(dg_out + row0 + (int64_t)row * HD + d0) = x;
      }
    }
  } else {
  // ---- phase 1.9: W64 for all 128 rows (rows < 64: k~, rows >= 64: q~, anchor row 63) ----------------------
  {
    uint8_t* tile = sm + BwdSmem::W64 + (wq_ >> 1) * TILE_BYTES;       // transposed like k_hat: row = feature
    ok = mbar_wait(smem_u32(bars + 3), 0) && ok;
    // rows 32 wq_ + i: k of rows 0..63 (K0) for wq_ < 2, q of rows 64..127 (QH) otherwise; 256-byte rows
    const unsigned short* xp = reinterpret_cast<const unsigned short*>(sm + (wq_ < 2 ? BwdSmem::K0 : BwdSmem::QH)) +
                               (32 * (wq_ & 1)) * TD + d;
    uint32_t xraw[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) xraw[i] = xp[i * TD];
    uint32_t pk[16];
    if (wq_ < 2) {
      float run = (wq_ == 0) ? tot[2 * TD + d] * tot[3 * TD + d] : 1.f;
#pragma unroll
      for (int i = 31; i >= 1; i -= 2) {
        const float hi = bf16_bits_to_float(xraw[i]) * run;
        run *= f32r[i];
        const float lo = bf16_bits_to_float(xraw[i - 1]) * run;
        run *= f32r[i - 1];
        pk[i >> 1] = pack_bf16x2(lo, hi);
      }
    } else {
      float run = (wq_ == 3) ? tot[4 * TD + d] * tot[5 * TD + d] : 1.f;
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        run *= f32r[i];
        const float lo = bf16_bits_to_float(xraw[i]) * run;
        run *= f32r[i + 1];
        const float hi = bf16_bits_to_float(xraw[i + 1]) * run;
        pk[i >> 1] = pack_bf16x2(lo, hi);
      }
    }
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4)
      *reinterpret_cast<uint4*>(tile + sw128_chunk(d, (wq_ & 1) * 4 + c4)) =
          make_uint4(pk[4 * c4], pk[4 * c4 + 1], pk[4 * c4 + 2], pk[4 * c4 + 3]);
  }

  // ---- phase 2: two passes over the rows ----------------------------------------------------------------------
  uint32_t ph1 = 0, ph2 = 0;      // completed-phase counters of bars[1], bars[2]
  const uint32_t aW64 = smem_u32(sm + BwdSmem::W64), aWL = smem_u32(sm + BwdSmem::WL), aDPL = smem_u32(sm + BwdSmem::DPL);
  const int rq = wq_;
  float later = 0.f;              // sum of dlam over all rows after this thread's run (filled per pass)
#pragma unroll 1
  for (int p = 1; p >= 0; --p) {
    const int rbase = 64 * p + 16 * rq;
    const int gi = 4 * p + rq;
    float f[16], dq[16], dk[16];
    uint32_t qk[16];
    {
      if (p == 0) ok = mbar_wait(smem_u32(bars + 4), 0) && ok;      // pass 0's g and q have landed (pass 1: waited above)
      const float* gs_ = reinterpret_cast<const float*>(sm + BwdSmem::GH) + (16 * rq) * TD + d;
      const unsigned short* qs_ = reinterpret_cast<const unsigned short*>(sm + BwdSmem::QH) + (16 * rq) * TD + d;
      const unsigned short* ks_ = reinterpret_cast<const unsigned short*>(sm + (p ? BwdSmem::K1 : BwdSmem::K0)) + (16 * rq) * TD + d;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        f[i] = gs_[i * TD];
        qk[i] = (uint32_t)qs_[i * TD] | ((uint32_t)ks_[i * TD] << 16);
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = __expf(f[i]);
    }
    // inter-chunk terms and the diagonal
    {
      float crossq = 1.f, crossk = 1.f;
      for (int b2 = 0; b2 < gi; ++b2) crossq *= tot[b2 * TD + d];
      for (int b2 = gi + 1; b2 < 8; ++b2) crossk *= tot[b2 * TD + d];
      uint32_t r[16];
      tmem_ld16(tmem + ((uint32_t)(q4 * 32) << 16) + TM_DQH + rbase, r);
      tmem_ld_wait();
      float run = crossq;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        run *= f[i];
        dq[i] = __uint_as_float(r[i]) * run + diag[rbase + i] * bf16_hi(qk[i]);
      }
      tmem_ld16(tmem + ((uint32_t)(q4 * 32) << 16) + TM_DKH + rbase, r);
      tmem_ld_wait();
      run = crossk;
#pragma unroll
      for (int i = 15; i >= 0; --i) {
        dk[i] = __uint_as_float(r[i]) * run + diag[rbase + i] * bf16_lo(qk[i]);
        run *= f[i];
      }
    }

    // one level: build operands, issue; the accumulate of the previous level overlaps the MMA
    auto build_and_issue = [&](auto SC) {
      constexpr int S = decltype(SC)::value;
      const int bsel = S & 1;
      if (S < 6) {
        // W_l stored transposed (row = feature d, columns = the 64 rows of the half): this thread's 16
        // values are 32 contiguous bytes
        float w[16];
        level_weights<S>(f, rq, p, tot, d, w);
        uint8_t* tile = sm + BwdSmem::WL + bsel * TILE_BYTES;
        const uint32_t sh = (S < 4) ? 0u : (row_is_right<S>(0, rq, p) ? 16u : 0u);
        uint32_t pk[8];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          float x0, x1;
          if (S < 4) {
            x0 = row_is_right<S>(i, rq, p) ? bf16_lo(qk[i]) : bf16_hi(qk[i]);
            x1 = row_is_right<S>(i + 1, rq, p) ? bf16_lo(qk[i + 1]) : bf16_hi(qk[i + 1]);
          } else {
            x0 = __uint_as_float((qk[i] << sh) & 0xffff0000u);
            x1 = __uint_as_float((qk[i + 1] << sh) & 0xffff0000u);
          }
          pk[i >> 1] = pack_bf16x2(x0 * w[i], x1 * w[i + 1]);
        }
        *reinterpret_cast<uint4*>(tile + sw128_chunk(d, 2 * rq)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        *reinterpret_cast<uint4*>(tile + sw128_chunk(d, 2 * rq + 1)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      }
      // masked 64 x 64 block of dP (row layout): rows i, columns j = jbase + 16 wq_ + m
      {
        const int ibase = (S == 6) ? 64 : 64 * p;
        const int jbase = (S == 6) ? 0 : 64 * p;
        if ((q4 >> 1) == (ibase >> 6)) {
          const int i = 32 * q4 + lane;
          // Level membership: i and j in the same block of 2^(S+1) rows, i in its right half, j in its
          // left half.  The 16 columns of this thread start at a multiple of 16, so for S < 4 the test
          // splits into a per-thread part (sel) and a compile-time part (m); for S >= 4 it is per-thread.
          int sel;          // S < 4: the value (m >> (S+1)) must have, or -1; S >= 4: 0 keep all, -1 none
          if (S < 4)       sel = (((i >> 4) == ((jbase >> 4) + wq_)) && ((i >> S) & 1)) ? ((i & 15) >> (S + 1)) : -1;
          else if (S == 4) sel = (((i >> 5) == ((jbase >> 5) + (wq_ >> 1))) && ((i >> 4) & 1) && !(wq_ & 1)) ? 0 : -1;
          else if (S == 5) sel = (((i >> 5) & 1) && (wq_ < 2)) ? 0 : -1;
          else             sel = 0;
          uint32_t r[16];
          tmem_ld16(tmem + ((uint32_t)(q4 * 32) << 16) + TM_DP + jbase + 16 * wq_, r);
          tmem_ld_wait();
          uint32_t pk[8];
#pragma unroll
          for (int m = 0; m < 16; m += 2) {
            bool k0, k1;
            if (S < 4) {
              k0 = !((m >> S) & 1) && (sel == (m >> (S + 1)));
              k1 = !(((m + 1) >> S) & 1) && (sel == ((m + 1) >> (S + 1)));
            } else {
              k0 = k1 = (sel == 0);
            }
            pk[m >> 1] = pack_bf16x2(k0 ? __uint_as_float(r[m]) : 0.f, k1 ? __uint_as_float(r[m + 1]) : 0.f);
          }
          uint8_t* tile = sm + BwdSmem::DPL + bsel * (KC_TILE);
          *reinterpret_cast<uint4*>(tile + sw128_chunk(i - ibase, 2 * wq_)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(tile + sw128_chunk(i - ibase, 2 * wq_ + 1)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      }
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        if (S == 3 && p == 1) {
          // every thread has read its pass-1 gates and q (they are past the barrier above): the landing zones
          // take g and q of rows 0..63, which arrive while this pass runs
          const uint32_t lb = smem_u32(bars + 4);
          mbar_arrive_expect_tx(lb, 32768 + 16384);
          tma_load_3d(smem_u32(sm + BwdSmem::GH), &maps.g, 0, yh, zrow, lb);
          tma_load_3d(smem_u32(sm + BwdSmem::QH), &maps.q, 0, yh, zrow, lb);
        }
        tc_fence_after();
        const uint32_t tacc = tmem + TM_T + 64 * bsel;
        const uint64_t kD = desc_kmajor(aDPL + bsel * KC_TILE, KC_TILE, 0), mD = desc_mnmajor(aDPL + bsel * KC_TILE, KC_TILE, 0);
        constexpr uint32_t iK = idesc_bf16(128, 64, 0, 0), iM = idesc_bf16(128, 64, 0, 1);
        if (S < 6) {
          const uint64_t kW = desc_kmajor(aWL + bsel * TILE_BYTES, TILE_BYTES, 0);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)    // rows i of the half on the columns: dq side
            umma_bf16(tacc, kslice_kmajor(kW, TILE_BYTES, ks), kslice_kmajor(kD, KC_TILE, ks), iK, ks > 0);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)    // rows j on the columns: dk side
            umma_bf16(tacc, kslice_kmajor(kW, TILE_BYTES, ks), kslice_mnmajor(mD, ks), iM, 1);
        } else if (p == 1) {
          const uint64_t kW = desc_kmajor(aW64, TILE_BYTES, 0);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)    // T[d][i-64] = sum_{j<64} k~64[j][d] dP[i][j]
            umma_bf16(tacc, kslice_kmajor(kW, TILE_BYTES, ks), kslice_kmajor(kD, KC_TILE, ks), iK, ks > 0);
        } else {
          const uint64_t kW = desc_kmajor(aW64 + TILE_BYTES, TILE_BYTES, 0);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)    // T[d][j] = sum_{i>=64} q~64[i][d] dP[i][j]
            umma_bf16(tacc, kslice_kmajor(kW, TILE_BYTES, ks), kslice_mnmajor(mD, ks), iM, ks > 0);
        }
        umma_commit(smem_u32(bars + 1 + bsel));
      }
    };
    auto accumulate = [&](auto SC) {
      constexpr int S = decltype(SC)::value;
      const int bsel = S & 1;
      if (bsel == 0) { ok = mbar_wait(smem_u32(bars + 1), ph1 & 1) && ok; ++ph1; }
      else           { ok = mbar_wait(smem_u32(bars + 2), ph2 & 1) && ok; ++ph2; }
      tc_fence_after();
      uint32_t r[16];
      tmem_ld16(tmem + ((uint32_t)(q4 * 32) << 16) + TM_T + 64 * bsel + 16 * rq, r);
      tmem_ld_wait();
      float w[16];
      level_weights<S>(f, rq, p, tot, d, w);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float t = __uint_as_float(r[i]) * w[i];
        if (row_is_right<S>(i, rq, p)) dq[i] += t; else dk[i] += t;
      }
    };
    using I3 = std::integral_constant<int, 3>;
    using I4 = std::integral_constant<int, 4>; using I5 = std::integral_constant<int, 5>;
    using I6 = std::integral_constant<int, 6>;
    build_and_issue(I3{});
    build_and_issue(I4{});
    // Half sizes 1, 2, 4 together are all pairs i > j inside each block of 8 rows.  Their partners are this
    // thread's own rows, so they need no contraction across threads: float32 FMAs with the exact pairwise decay
    // prod_{t in (j, i]} f_t, run while the tensor core works on the two products just issued.
    {
      const float* dpd = reinterpret_cast<const float*>(sm + BwdSmem::DPD) + rbase * 16;
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
        for (int i = 1; i < 8; ++i) {
          const int ri = 8 * blk + i;
          float pv[8];
          {
            const float4 a = *reinterpret_cast<const float4*>(dpd + ri * 16 + 8 * blk);
            pv[0] = a.x; pv[1] = a.y; pv[2] = a.z; pv[3] = a.w;
            if (i > 4) {
              const float4 b4 = *reinterpret_cast<const float4*>(dpd + ri * 16 + 8 * blk + 4);
              pv[4] = b4.x; pv[5] = b4.y; pv[6] = b4.z; pv[7] = b4.w;
            }
          }
          const float qi = bf16_lo(qk[ri]);
          float D = 1.f;
#pragma unroll
          for (int j = i - 1; j >= 0; --j) {
            const int rj = 8 * blk + j;
            D *= f[rj + 1];
            const float t = pv[j] * D;
            dq[ri] = fmaf(t, bf16_hi(qk[rj]), dq[ri]);
            dk[rj] = fmaf(t, qi, dk[rj]);
          }
        }
      }
    }
    accumulate(I3{});
    build_and_issue(I5{});
    accumulate(I4{});
    build_and_issue(I6{});
    accumulate(I5{});
    accumulate(I6{});

    // ---- outputs of this pass ---------------------------------------------------------------------------
    float dl[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int64_t e = row0 + (int64_t)(rbase + i) * HD + d;
      dl[i] = bf16_lo(qk[i]) * dq[i] - bf16_hi(qk[i]) * dk[i];
      if (ok) {
        dq_out[e] = __float2bfloat16_rn(dq[i]);
        dk_out[e] = __float2bfloat16_rn(dk[i]);
      }
    }
#pragma unroll
    for (int i = 14; i >= 0; --i) dl[i] += dl[i + 1];      // inclusive suffix sums within the run
    grp[gi * TD + d] = dl[0];
    tc_fence_before();
    __syncthreads();
    float off = dG + later;
    for (int g2 = gi + 1; g2 < 4 * p + 4; ++g2) off += grp[g2 * TD + d];
    if (ok) {
#pragma unroll
      for (int i = 0; i < 16; ++i) dg_out[row0 + (int64_t)(rbase + i) * HD + d] = dl[i] + off;
    }
    if (p == 1) {
      later = 0.f;
      for (int g2 = 4; g2 < 8; ++g2) later += grp[g2 * TD + d];
    }
  }
  }   // all scales
  if (!ok && tid == 0) atomicAdd(&g_tc_wait_timeouts, 1u);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// Sum of G over the chunks of a slice: G_total (B*H, D) = sum_n Gc[bh, n, d].
__global__ void __launch_bounds__(256) tc_gsum_kernel(int64_t BH, int64_t N, const float* __restrict__ Gc,
                                                      float* __restrict__ Gt) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= BH * TD) return;
  const int64_t bh = e / TD, dd = e % TD;
  float s = 0.f;
  for (int64_t n = 0; n < N; ++n) s += Gc[(bh * N + n) * TD + dd];
  Gt[e] = s;
}

// ---- chunk states computed from a zero state, corrected once the true incoming state is known -------------------
// The state recurrence is linear: with S0[n] the state entering chunk n when a run of chunks starts from zero, the
// state entering it when the run starts from H_in is S0[n] + exp(sum_{m<n} G_m) (.) H_in (decay along the key axis;
// ops.py:286-297 applied to the run's prefix).  The gradient states mirror it with the chunks after n.  Two callers:
// sequence parallelism (the run is a rank's slice, H_in arrives from the other ranks) and the segmented one-pass
// state kernel (the runs are `nsegs` pieces of every head's chunks, `Ns` chunks each, H_in of a run follows from
// the runs before it).  nsegs = 1, Ns = N is the single-run form.
//
// E[bh][n][d] = exp(sum of Gc over the chunks of n's run before n (reverse == 0) or after n (reverse != 0)); one
// block per (batch, head, run), one thread per feature.  live[bh][n] = 1 while any feature's factor is non-zero: once
// the accumulated log decay has underflowed for all 128 features, the incoming state contributes exactly nothing to
// the chunk and the correction pass skips it (a long run with ordinary gates needs its first few dozen chunks).
__global__ void __launch_bounds__(TD) sp_cum_gate_kernel(int64_t N, int nsegs, int64_t Ns, const float* __restrict__ Gc,
                                                         float* __restrict__ E, int* __restrict__ live,
                                                         float* __restrict__ Gs, int reverse) {
  const int64_t bh = blockIdx.x / nsegs, n0 = (blockIdx.x % nsegs) * Ns, n1 = n0 + Ns < N ? n0 + Ns : N;
  const int dd = threadIdx.x;
  // the flags start at zero and every thread with a non-zero factor raises its chunk's: one barrier for the whole
  // walk instead of a block-wide vote per chunk (the walk is a chain of additions; the loads do not depend on it)
  for (int64_t n = n0 + dd; n < n1; n += TD) live[bh * N + n] = 0;
  __syncthreads();
  float acc = 0.f;
  for (int64_t i0 = 0; i0 < n1 - n0; i0 += 8) {
    float gq[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {          // eight loads in flight; the chain below is additions only
      const int64_t i = i0 + u < n1 - n0 ? i0 + u : n1 - n0 - 1;
      gq[u] = __ldg(Gc + (bh * N + (reverse ? n1 - 1 - i : n0 + i)) * TD + dd);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int64_t i = i0 + u;
      if (i < n1 - n0) {
        const int64_t n = reverse ? n1 - 1 - i : n0 + i;
        const float w = __expf(acc);
        E[(bh * N + n) * TD + dd] = w;
        if (w != 0.f) live[bh * N + n] = 1;
        acc += gq[u];
      }
    }
  }
  if (Gs != nullptr) Gs[(int64_t)blockIdx.x * TD + dd] = acc;       // the run's total log decay, (bh, run, feature)
}
// states[bh][n][dk][dv] += E[bh][n][dk] * Hin[bh][run of n][dk][dv]; one thread per 8 consecutive dv (16 bytes of
// bf16).  skip_seg: a run whose incoming correction is known to be zero (it started from the true state), or -1.
__global__ void __launch_bounds__(256) sp_fix_states_kernel(int64_t BH, int64_t N, int nsegs, int64_t Ns, int skip_seg,
                                                            const float* __restrict__ E, const int* __restrict__ live,
                                                            const float* __restrict__ Hin, bf16* __restrict__ states) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= BH * N * TD * (TD / 8)) return;
  const int j = (int)(e % (TD / 8));
  const int dk = (int)((e / (TD / 8)) % TD);
  const int64_t bhn = e / (TD / 8) / TD, bh = bhn / N, seg = (bhn % N) / Ns;
  if (live[bhn] == 0 || seg == skip_seg) return;          // 8 blocks share a chunk-head: the whole block leaves together
  const float w = E[bhn * TD + dk];
  const float4* hp = reinterpret_cast<const float4*>(Hin + ((bh * nsegs + seg) * TD + dk) * TD + j * 8);
  const float4 h0 = __ldg(hp), h1 = __ldg(hp + 1);
  uint4* sp = reinterpret_cast<uint4*>(states + (bhn * TD + dk) * TD + j * 8);
  uint4 u = *sp;
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d2 = unpack_bf16x2(u.w);
  u.x = pack_bf16x2(fmaf(w, h0.x, a.x), fmaf(w, h0.y, a.y));
  u.y = pack_bf16x2(fmaf(w, h0.z, b.x), fmaf(w, h0.w, b.y));
  u.z = pack_bf16x2(fmaf(w, h1.x, c.x), fmaf(w, h1.y, c.y));
  u.w = pack_bf16x2(fmaf(w, h1.z, d2.x), fmaf(w, h1.w, d2.y));
  *sp = u;
}
// The scan over the runs of one head, in walk order (time order, or its reverse for the gradient states):
//   Cin[first run] = init32 (or 0),  Cin[next run] = F[run] + exp(sum of the run's Gc) (.) Cin[run],
// F[run] being the run's final state computed from its own start and Cin[run] the correction its stored states
// need, i.e. the part of the true incoming state that its start did not contain.  What leaves the last run is the
// final state of the whole walk (fin32 float32 and / or fin16 bf16).  One thread per four consecutive dv.
__global__ void __launch_bounds__(256) seg_scan_kernel(int64_t BH, int nsegs, const float* __restrict__ Gs,
                                                       const float* __restrict__ F, const float* __restrict__ init32,
                                                       float* __restrict__ Cin, bf16* __restrict__ fin16,
                                                       float* __restrict__ fin32, int reverse) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= BH * TD * (TD / 4)) return;
  const int j = (int)(e % (TD / 4));
  const int dk = (int)((e / (TD / 4)) % TD);
  const int64_t bh = e / (TD / 4) / TD;
  const int64_t el = (bh * TD + dk) * TD + j * 4;
  float4 c = init32 ? *reinterpret_cast<const float4*>(init32 + el) : make_float4(0.f, 0.f, 0.f, 0.f);
  // the chain is only the multiply-add: the loads of the runs ahead do not depend on it and are kept in flight
  constexpr int AHEAD = 4;
  float4 f[AHEAD];
  float gs[AHEAD];
  auto run_of = [&](int w) { return (int64_t)(reverse ? nsegs - 1 - w : w); };
#pragma unroll
  for (int a = 0; a < AHEAD; ++a)
    if (a < nsegs) {
      f[a] = __ldg(reinterpret_cast<const float4*>(F + ((bh * nsegs + run_of(a)) * TD + dk) * TD + j * 4));
      gs[a] = __ldg(Gs + (bh * nsegs + run_of(a)) * TD + dk);
    }
  for (int w0 = 0; w0 < nsegs; w0 += AHEAD) {
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
      const int w = w0 + a;
      if (w < nsegs) {
        const float4 fw = f[a];
        const float dec = __expf(gs[a]);
        if (w + AHEAD < nsegs) {
          f[a] = __ldg(reinterpret_cast<const float4*>(F + ((bh * nsegs + run_of(w + AHEAD)) * TD + dk) * TD + j * 4));
          gs[a] = __ldg(Gs + (bh * nsegs + run_of(w + AHEAD)) * TD + dk);
        }
        *reinterpret_cast<float4*>(Cin + ((bh * nsegs + run_of(w)) * TD + dk) * TD + j * 4) = c;
        c = make_float4(fmaf(dec, c.x, fw.x), fmaf(dec, c.y, fw.y), fmaf(dec, c.z, fw.z), fmaf(dec, c.w, fw.w));
      }
    }
  }
  if (fin32) *reinterpret_cast<float4*>(fin32 + el) = c;
  if (fin16) {
    uint2 u;
    u.x = pack_bf16x2(c.x, c.y); u.y = pack_bf16x2(c.z, c.w);
    *reinterpret_cast<uint2*>(fin16 + el) = u;
  }
}
// Scratch of a correction, carved from the float32 product area of the workspace (BH * N * 128 * 128 floats, unused
// whenever the one-pass state kernel runs): with runs, F and Cin, BH * nsegs * 128 * 128 floats each (nsegs <= N / 4,
// so they take at most half of the area); then E, BH * N * 128 floats, the runs' total log decays Gs, BH * nsegs * 128
// floats, and the live flags, BH * N ints.
struct FixScratch {
  float *F, *Cin, *E, *Gs;
  int* live;
  FixScratch(float* area, int64_t BH, int64_t N, int nsegs) {
    const int64_t per = nsegs > 1 ? BH * nsegs * TD * TD : 0;
    F = area;
    Cin = F + per;
    E = Cin + per;
    Gs = E + BH * N * TD;
    live = reinterpret_cast<int*>(Gs + (nsegs > 1 ? BH * nsegs * TD : 0));
  }
};
// E, live and the runs' totals Gs from the chunks' log decays (they depend on nothing else).
static int launch_cum_gate(cudaStream_t st, int64_t BH, int64_t N, int nsegs, const float* Gc, const FixScratch& fx, int reverse) {
  const int64_t Ns = (N + nsegs - 1) / nsegs;
  ProfScope ps("sp_cum_gate_kernel", st);
  sp_cum_gate_kernel<<<(unsigned)(BH * nsegs), TD, 0, st>>>(N, nsegs, Ns, Gc, fx.E, fx.live, nsegs > 1 ? fx.Gs : nullptr, reverse);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}
static int launch_seg_scan(cudaStream_t st, int64_t BH, int nsegs, const FixScratch& fx, const float* init32, void* fin16,
                           float* fin32, int reverse) {
  const int64_t n = BH * TD * (TD / 4);
  ProfScope ps("seg_scan_kernel", st);
  seg_scan_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(BH, nsegs, fx.Gs, fx.F, init32, fx.Cin, (bf16*)fin16, fin32, reverse);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}
// Hin: (BH, nsegs, 128, 128) float32, the correction entering every run; E and live from launch_cum_gate.
static int launch_fix_states(cudaStream_t st, int64_t BH, int64_t N, int nsegs, int skip_seg, const FixScratch& fx,
                             const float* Hin, bf16* states) {
  const int64_t Ns = (N + nsegs - 1) / nsegs;
  const int64_t n = BH * N * TD * (TD / 8);
  if ((n + 255) / 256 > 2147483647LL) return GLA_ERR_TOO_LARGE;
  ProfScope ps("sp_fix_states_kernel", st);
  sp_fix_states_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(BH, N, nsegs, Ns, skip_seg, fx.E, fx.live, Hin, states);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
// bf16; head size 128 or 256 (a head of 256 runs as 2 x 2 independent blocks of 128, see the kernels); any chunk
// size that is a multiple of 128: the result does not depend on the chunk size, so the kernels always use 128.
bool tc_supported(int64_t D, int64_t C, int dtype) {
  return (D == TD || D == 2 * TD) && C >= TC && C % TC == 0 && dtype == GLA_BF16;
}
// the entry points that produce a rank's local state for sequence parallelism keep to the original shape
bool tc_supported_local_state(int64_t D, int64_t C, int dtype) { return D == TD && C == TC && dtype == GLA_BF16; }
bool tc_auto_default() { return true; }

static size_t f32b(int64_t n) { return align_up((size_t)n * 4, 256); }
static size_t b16b(int64_t n) { return align_up((size_t)n * 2, 256); }

// ---- head sizes above 128: layout changes around the kernels --------------------------------------------------
// (BH, 128 R, 128 R) <-> (BH, R, R, 128, 128): the state of a head as R x R tiles, one per virtual head.
__global__ void __launch_bounds__(256) state_block_kernel(const bf16* __restrict__ in, bf16* __restrict__ out,
                                                          int64_t BH, int R, int to_blocked) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;      // one 16-byte piece (8 elements)
  if (e >= BH * R * R * TD * (TD / 8)) return;
  const int j = (int)(e % (TD / 8));
  const int r = (int)((e / (TD / 8)) % TD);
  const int c = (int)((e / (TD / 8) / TD) % R);
  const int a = (int)((e / (TD / 8) / TD / R) % R);
  const int64_t bh = e / (TD / 8) / TD / R / R;
  const int64_t real = ((bh * TD * R + a * TD + r) * (int64_t)(TD * R) + c * TD + j * 8);
  const int64_t blocked = ((((bh * R + a) * R + c) * TD + r) * (int64_t)TD + j * 8);
  if (to_blocked) *reinterpret_cast<uint4*>(out + blocked) = *reinterpret_cast<const uint4*>(in + real);
  else            *reinterpret_cast<uint4*>(out + real) = *reinterpret_cast<const uint4*>(in + blocked);
}
// Per-virtual-head results (rows, H R R, 128) summed into (rows, H, 128 R): key-side arrays (dq, dk, dg) keep the
// key block a and sum over the value blocks c; value-side arrays (out, dv) keep c and sum over a.  Float32 sums.
// Eight consecutive features of one array as floats, through 16-byte accesses.
__device__ __forceinline__ void ld8_f32(const bf16* p, float (&x)[8]) {
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16x2(w[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void ld8_f32(const float* p, float (&x)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void st8_f32(bf16* p, const float (&x)[8]) {
  uint4 u;
  u.x = pack_bf16x2(x[0], x[1]); u.y = pack_bf16x2(x[2], x[3]); u.z = pack_bf16x2(x[4], x[5]); u.w = pack_bf16x2(x[6], x[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void st8_f32(float* p, const float (&x)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(x[0], x[1], x[2], x[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(x[4], x[5], x[6], x[7]);
}
template <typename T, int KEYSIDE>
__global__ void __launch_bounds__(256) sum_blocks_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows,
                                                         int64_t H, int R) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;      // eight consecutive features
  if (e >= rows * H * R * (TD / 8)) return;
  const int j = (int)(e % (TD / 8));
  const int keep = (int)((e / (TD / 8)) % R);
  const int64_t h = (e / (TD / 8) / R) % H, row = e / (TD / 8) / R / H;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int s2 = 0; s2 < R; ++s2) {
    const int a = KEYSIDE ? keep : s2, c = KEYSIDE ? s2 : keep;
    float x[8];
    ld8_f32(in + ((row * H * R * R + (h * R + a) * R + c) * (int64_t)TD + j * 8), x);
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[u] += x[u];
  }
  st8_f32(out + ((row * H + h) * (int64_t)(TD * R) + keep * TD + j * 8), acc);
}
static int launch_state_block(cudaStream_t st, const void* in, void* out, int64_t BH, int R, int to_blocked) {
  const int64_t n = BH * R * R * TD * (TD / 8);
  ProfScope ps("state_block_kernel", st);
  state_block_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const bf16*)in, (bf16*)out, BH, R, to_blocked);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}
template <typename T, int KEYSIDE>
static int launch_sum_blocks(cudaStream_t st, const T* in, T* out, int64_t rows, int64_t H, int R) {
  const int64_t n = rows * H * R * (TD / 8);
  ProfScope ps("sum_blocks_kernel", st);
  sum_blocks_kernel<T, KEYSIDE><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(in, out, rows, H, R);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

// Sizes.  R = D / 128, HV = H R R virtual heads, N = T / 128 chunks whatever chunk size the caller named.
// saved: S_prev bf16 (B HV, N, 128, 128) | Gc f32 (B HV, N, 128) | P bf16 (B HV, N, 128, 128)
size_t tc_saved_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t) {
  const int64_t R = D / TD, N = T / TC, BHV = B * H * R * R;
  return b16b(BHV * N * TD * TD) + f32b(BHV * N * TD) + b16b(BHV * N * TC * TC);
}
// fwd workspace: kv f32 (R = 1 only: the product + scan pair) | Gc f32 | S_prev bf16 (used when nothing is saved)
//                | R > 1: blocked hidden_init, blocked hidden_final bf16 (B HV, 128, 128) | out per virtual head bf16
size_t tc_fwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t) {
  const int64_t R = D / TD, N = T / TC, BHV = B * H * R * R;
  size_t n = (R == 1 ? f32b(BHV * N * TD * TD) : 0) + f32b(BHV * N * TD) + b16b(BHV * N * TD * TD);
  if (R > 1) n += 2 * b16b(BHV * TD * TD) + b16b(B * T * H * R * R * TD);
  return n;
}
// bwd workspace: dstate f32 (R = 1 only) | dS_next bf16 | R > 1: blocked dhidden_final, dhidden_init |
//                dq, dk, dv per virtual head bf16 | dg per virtual head f32
size_t tc_bwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t) {
  const int64_t R = D / TD, N = T / TC, BHV = B * H * R * R;
  size_t n = (R == 1 ? f32b(BHV * N * TD * TD) : 0) + b16b(BHV * N * TD * TD);
  if (R > 1) n += 2 * b16b(BHV * TD * TD) + 3 * b16b(B * T * H * R * R * TD) + f32b(B * T * H * R * R * TD);
  return n;
}

constexpr size_t FWD_SMEM = 1024 + FwdSmem::END;

int tc_chunk_fwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C, const void* hidden_init,
                 const float* g, const void* v, const void* k, const void* q, void* hidden_final, void* out,
                 void* saved, void* ws, int state_only, float* G_total, float* S_local, int opts, int64_t nseq,
                 const int* cu, int sp_phase, const float* H_in) {
  (void)C;
  const int R = (int)(D / TD);
  const int64_t N = T / TC, HV = H * R * R, HK = H * R, BHV = B * HV;
  if (state_only && R != 1) return GLA_ERR_UNSUPPORTED;
  // sequence-parallel phases (sp_phase 1: states from a zero state, kept in `saved`; 2: correct them with H_in, then
  // the chunk kernel) exist for the plain head size and need the residual buffer to carry the states between them
  if (sp_phase != 0 && (R != 1 || saved == nullptr || cu != nullptr || state_only)) return GLA_ERR_UNSUPPORTED;
  if (cu != nullptr && (B != 1 || R != 1 || state_only || nseq <= 0)) return GLA_ERR_UNSUPPORTED;   // packed sequences
  char* w = (char*)ws;
  float* kv = (float*)w; w += (R == 1 ? f32b(BHV * N * TD * TD) : 0);
  float* Gc = (float*)w; w += f32b(BHV * N * TD);
  bf16* S_prev = (bf16*)w; w += b16b(BHV * N * TD * TD);
  bf16 *hib = nullptr, *hfb = nullptr, *out_v = nullptr;
  if (R > 1) {
    hib = (bf16*)w; w += b16b(BHV * TD * TD);
    hfb = (bf16*)w; w += b16b(BHV * TD * TD);
    out_v = (bf16*)w;
  }
  bf16* P = nullptr;
  if (saved) {
    char* s = (char*)saved;
    S_prev = (bf16*)s; s += b16b(BHV * N * TD * TD);
    Gc = (float*)s;    s += f32b(BHV * N * TD);
    P = (bf16*)s;
  }
  const void* init_v = hidden_init;
  void* fin_v = hidden_final;
  if (R > 1) {
    GLA_TRY(launch_state_block(st, hidden_init, hib, B * H, R, 1));
    init_v = hib; fin_v = hfb;
  }
  const bool fused_states = !state_only && (R > 1 || cu != nullptr || tc_state_fused_preferred(BHV, N, opts));
  // runs of chunks walked by separate blocks and corrected afterwards (plain head size, dense batches)
  const int nsegs = (fused_states && R == 1 && cu == nullptr) ? tc_state_segments(BHV, N, opts) : 1;
  const FixScratch fx(kv, BHV, N, nsegs);
  if (sp_phase == 1) {
    if (nsegs > 1) {
      // every run from zero; the scan over the runs gives the slice's final state (its corrections are recomputed
      // in the finish phase, which knows the state entering the slice; the runs' final states stay in the workspace)
      GLA_TRY(tc_state_fused(st, 0, B, T, HV, R, g, k, v, nullptr, S_prev, nullptr, Gc, 0, nullptr, nullptr, nullptr, fx.F, nsegs));
      GLA_TRY(launch_cum_gate(st, BHV, N, nsegs, Gc, fx, 0));          // stays in the workspace for the finish phase
      GLA_TRY(launch_seg_scan(st, BHV, nsegs, fx, nullptr, nullptr, S_local, 0));
    } else if (fused_states) {
      GLA_TRY(tc_state_fused(st, 0, B, T, HV, R, g, k, v, nullptr, S_prev, nullptr, Gc, 0, nullptr, nullptr, nullptr, S_local));
    } else {
      GLA_TRY((launch_tc_kv<0>(st, B, T, H, g, k, v, kv, Gc)));
      GLA_TRY(launch_state_scan(st, BHV, N, TD, Gc, kv, 0, nullptr, 0, S_prev, 1, S_local, 0, 0));
    }
    ProfScope ps("tc_gsum_kernel", st);
    tc_gsum_kernel<<<(unsigned)((BHV * TD + 255) / 256), 256, 0, st>>>(BHV, N, Gc, G_total);
    GLA_CHECK_LAUNCH();
    return GLA_OK;
  }
  // The chunk kernel may start beside the one-pass state kernel (which fills only 4 x batch x heads SMs) when it
  // is the very next launch: plain head size, and the kv area of the workspace, unused then, holds the counter.
  unsigned int* early_flag = (sp_phase == 0 && fused_states && R == 1 && nsegs == 1 && !(opts & GLA_OPT_NO_EARLY_START)) ? (unsigned int*)kv : nullptr;
  unsigned int early_target = 0;
  if (sp_phase == 2 && nsegs > 1) {
    // the corrections of all runs, now from the state that enters the slice, in one pass over the stored states
    GLA_TRY(launch_seg_scan(st, BHV, nsegs, fx, H_in, nullptr, nullptr, 0));
    GLA_TRY(launch_fix_states(st, BHV, N, nsegs, -1, fx, fx.Cin, S_prev));
  } else if (sp_phase == 2) {
    // the product area of the workspace is dead by now: it takes the cumulative decays
    GLA_TRY(launch_cum_gate(st, BHV, N, 1, Gc, fx, 0));
    GLA_TRY(launch_fix_states(st, BHV, N, 1, -1, fx, H_in, S_prev));
  } else if (nsegs > 1) {
    // the first run starts from hidden_init and needs no correction; the others get theirs from the scan over runs
    GLA_TRY(tc_state_fused(st, 0, B, T, HV, R, g, k, v, init_v, S_prev, nullptr, Gc, 0, nullptr, nullptr, nullptr, fx.F, nsegs));
    GLA_TRY(launch_cum_gate(st, BHV, N, nsegs, Gc, fx, 0));
    GLA_TRY(launch_seg_scan(st, BHV, nsegs, fx, nullptr, fin_v, nullptr, 0));
    GLA_TRY(launch_fix_states(st, BHV, N, nsegs, 0, fx, fx.Cin, S_prev));
  } else if (fused_states) {
    GLA_TRY(tc_state_fused(st, 0, B, T, HV, R, g, k, v, init_v, S_prev, fin_v, Gc, nseq, cu, early_flag, &early_target));
  } else {
    GLA_TRY((launch_tc_kv<0>(st, B, T, H, g, k, v, kv, Gc)));
  }
  if (state_only) {
    GLA_TRY(launch_state_scan(st, BHV, N, TD, Gc, kv, 0, nullptr, 0, nullptr, 0, S_local, 0, 0));
    ProfScope ps("tc_gsum_kernel", st);
    tc_gsum_kernel<<<(unsigned)((BHV * TD + 255) / 256), 256, 0, st>>>(BHV, N, Gc, G_total);
    GLA_CHECK_LAUNCH();
    return GLA_OK;
  }
  if (!fused_states && sp_phase == 0) GLA_TRY(launch_state_scan(st, BHV, N, TD, Gc, kv, 0, hidden_init, 1, S_prev, 1, hidden_final, 1, 0));
  static SmemAttrOnce fwd_attr;
  GLA_TRY(fwd_attr.ensure(tc_chunk_fwd_kernel, FWD_SMEM));
  cudaError_t e;
  const int all_scales = (opts & GLA_OPT_ALL_SCALES) ? 1 : 0;
  FwdMaps maps;
  GLA_TRY(make_map_bthd(&maps.g, g, 1, B, T, HK, 128, 0));
  GLA_TRY(make_map_bthd(&maps.q, q, 0, B, T, HK, 64, 1));
  GLA_TRY(make_map_bthd(&maps.k, k, 0, B, T, HK, 64, 1));
  GLA_TRY(make_map_bthd(&maps.v, v, 0, B, T, HK, 64, 1));
  GLA_TRY(make_map_rows(&maps.s, S_prev, BHV * N * TD, 64, 128));
  {
    ProfScope ps("tc_chunk_fwd_kernel", st);
    bf16* out_p = R > 1 ? out_v : (bf16*)out;
    const int pf_dist = (opts & GLA_OPT_NO_L2_PREFETCH) ? 0 : prefetch_distance(1);
    if (early_flag != nullptr) {
      // programmatic dependent of the state kernel launched just before: may start while that one runs
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)(BHV * N));
      cfg.blockDim = dim3(TTHREADS);
      cfg.dynamicSmemBytes = FWD_SMEM;
      cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      e = cudaLaunchKernelEx(&cfg, tc_chunk_fwd_kernel, maps, T, HV, R, N, out_p, P, (const unsigned int*)early_flag,
                             early_target, all_scales, pf_dist);
      if (e != cudaSuccess) return record_cuda_error(e);
    } else {
      tc_chunk_fwd_kernel<<<(unsigned)(BHV * N), TTHREADS, FWD_SMEM, st>>>(maps, T, HV, R, N, out_p, P, nullptr, 0u, all_scales, pf_dist);
    }
  }
  GLA_CHECK_LAUNCH();
  if (R > 1) {
    GLA_TRY((launch_sum_blocks<bf16, 0>(st, out_v, (bf16*)out, B * T, H, R)));
    GLA_TRY(launch_state_block(st, hfb, hidden_final, B * H, R, 0));
  }
  return GLA_OK;
}

constexpr size_t BWD_SMEM = 1024 + BwdSmem::END;

// Gradient reaching a slice's initial state when the gradient of its final state is zero (sequence parallelism):
// q_hat^T dO per chunk on the tensor cores, then the reverse scan keeping only its last value.
// ws: the backward workspace (dstate f32 | Gc in the region of dS_next).
int tc_local_dstate(cudaStream_t st, int64_t B, int64_t T, int64_t H, const float* g, const void* q, const void* dout,
                    float* dS_local, void* ws) {
  const int64_t N = T / TC, BH = B * H;
  char* w = (char*)ws;
  float* dstate = (float*)w; w += f32b(BH * N * TD * TD);
  float* Gc = (float*)w;
  GLA_TRY((launch_tc_kv<1>(st, B, T, H, g, q, dout, dstate, Gc)));
  return launch_state_scan(st, BH, N, TD, Gc, dstate, 0, nullptr, 0, nullptr, 0, dS_local, 0, 1);
}

int tc_chunk_bwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C, const float* g,
                 const void* v, const void* k, const void* q, const void* saved, const void* dhidden_final,
                 const void* dout, void* dhidden_init, float* dg, void* dv, void* dk, void* dq, void* ws, int opts,
                 int64_t nseq, const int* cu, int sp_phase, float* A_local, const float* dH_out) {
  (void)C;
  const int R = (int)(D / TD);
  const int64_t N = T / TC, HV = H * R * R, HK = H * R, BHV = B * HV;
  if (cu != nullptr && (B != 1 || R != 1 || nseq <= 0)) return GLA_ERR_UNSUPPORTED;   // packed sequences
  // sequence-parallel phases: 1 = gradient states from a zero final gradient (kept in the workspace) and the
  // gradient reaching the slice's initial state; 2 = correct them with dH_out, then the chunk kernel
  if (sp_phase != 0 && (R != 1 || cu != nullptr)) return GLA_ERR_UNSUPPORTED;
  char* w = (char*)ws;
  float* dstate = (float*)w; w += (R == 1 ? f32b(BHV * N * TD * TD) : 0);
  bf16* dS_next = (bf16*)w; w += b16b(BHV * N * TD * TD);
  bf16 *dhfb = nullptr, *dhib = nullptr, *dq_v = (bf16*)dq, *dk_v = (bf16*)dk, *dv_v = (bf16*)dv;
  float* dg_v = dg;
  if (R > 1) {
    dhfb = (bf16*)w; w += b16b(BHV * TD * TD);
    dhib = (bf16*)w; w += b16b(BHV * TD * TD);
    dq_v = (bf16*)w; w += b16b(B * T * HV * TD);
    dk_v = (bf16*)w; w += b16b(B * T * HV * TD);
    dv_v = (bf16*)w; w += b16b(B * T * HV * TD);
    dg_v = (float*)w;
  }
  const char* s = (const char*)saved;
  const bf16* S_prev = (const bf16*)s; s += b16b(BHV * N * TD * TD);
  const float* Gc = (const float*)s;   s += f32b(BHV * N * TD);
  const bf16* P = (const bf16*)s;
  const void* dfin_v = dhidden_final;
  void* dinit_v = dhidden_init;
  if (R > 1) {
    GLA_TRY(launch_state_block(st, dhidden_final, dhfb, B * H, R, 1));
    dfin_v = dhfb; dinit_v = dhib;
  }
  const bool fused_states = R > 1 || cu != nullptr || tc_state_fused_preferred(BHV, N, opts);
  const int nsegs = (fused_states && R == 1 && cu == nullptr) ? tc_state_segments(BHV, N, opts) : 1;
  const FixScratch fx(dstate, BHV, N, nsegs);
  if (sp_phase == 1) {
    if (nsegs > 1) {
      GLA_TRY(tc_state_fused(st, 1, B, T, HV, R, g, q, dout, nullptr, dS_next, nullptr, nullptr, 0, nullptr, nullptr, nullptr, fx.F, nsegs));
      GLA_TRY(launch_cum_gate(st, BHV, N, nsegs, Gc, fx, 1));
      GLA_TRY(launch_seg_scan(st, BHV, nsegs, fx, nullptr, nullptr, A_local, 1));
    } else if (fused_states) {
      GLA_TRY(tc_state_fused(st, 1, B, T, HV, R, g, q, dout, nullptr, dS_next, nullptr, nullptr, 0, nullptr, nullptr, nullptr, A_local));
    } else {
      GLA_TRY((launch_tc_kv<1>(st, B, T, H, g, q, dout, dstate, nullptr)));
      GLA_TRY(launch_state_scan(st, BHV, N, TD, Gc, dstate, 0, nullptr, 0, dS_next, 1, A_local, 0, 1));
    }
    return GLA_OK;
  }
  if (sp_phase == 2 && nsegs > 1) {
    GLA_TRY(launch_seg_scan(st, BHV, nsegs, fx, dH_out, nullptr, nullptr, 1));
    GLA_TRY(launch_fix_states(st, BHV, N, nsegs, -1, fx, fx.Cin, dS_next));
  } else if (sp_phase == 2) {
    GLA_TRY(launch_cum_gate(st, BHV, N, 1, Gc, fx, 1));
    GLA_TRY(launch_fix_states(st, BHV, N, 1, -1, fx, dH_out, dS_next));
  } else if (nsegs > 1) {
    // the run that is walked first (the last in time) starts from dhidden_final and needs no correction
    GLA_TRY(tc_state_fused(st, 1, B, T, HV, R, g, q, dout, dfin_v, dS_next, nullptr, nullptr, 0, nullptr, nullptr, nullptr, fx.F, nsegs));
    GLA_TRY(launch_cum_gate(st, BHV, N, nsegs, Gc, fx, 1));
    GLA_TRY(launch_seg_scan(st, BHV, nsegs, fx, nullptr, dinit_v, nullptr, 1));
    GLA_TRY(launch_fix_states(st, BHV, N, nsegs, nsegs - 1, fx, fx.Cin, dS_next));
  } else if (fused_states) {
    GLA_TRY(tc_state_fused(st, 1, B, T, HV, R, g, q, dout, dfin_v, dS_next, dinit_v, nullptr, nseq, cu));
  } else {
    GLA_TRY((launch_tc_kv<1>(st, B, T, H, g, q, dout, dstate, nullptr)));
    GLA_TRY(launch_state_scan(st, BHV, N, TD, Gc, dstate, 0, dhidden_final, 1, dS_next, 1, dhidden_init, 1, 1));
  }
  static SmemAttrOnce bwd_attr;
  GLA_TRY(bwd_attr.ensure(tc_chunk_bwd_kernel, BWD_SMEM));
  BwdMaps bmaps;
  GLA_TRY(make_map_bthd(&bmaps.g, g, 1, B, T, HK, 128, 0, 64));
  GLA_TRY(make_map_bthd(&bmaps.q, q, 0, B, T, HK, 128, 0, 64));
  GLA_TRY(make_map_bthd(&bmaps.k, k, 0, B, T, HK, 128, 0, 64));
  GLA_TRY(make_map_bthd(&bmaps.dO, dout, 0, B, T, HK, 64, 1));
  GLA_TRY(make_map_bthd(&bmaps.v, v, 0, B, T, HK, 64, 1));
  GLA_TRY(make_map_rows(&bmaps.sp, S_prev, BHV * N * TD, 64, 128));
  GLA_TRY(make_map_rows(&bmaps.ds, dS_next, BHV * N * TD, 64, 128));
  GLA_TRY(make_map_rows(&bmaps.p, P, BHV * N * TC, 64, 128));
  {
    ProfScope ps("tc_chunk_bwd_kernel", st);
    tc_chunk_bwd_kernel<<<(unsigned)(BHV * N), TTHREADS, BWD_SMEM, st>>>(
        bmaps, T, HV, R, N, (opts & GLA_OPT_NO_L2_PREFETCH) ? 0 : prefetch_distance(1), g, (const bf16*)v, (const bf16*)k,
        (const bf16*)q, (const bf16*)dout, S_prev, dS_next, P, dq_v, dk_v, dv_v, dg_v, (opts & GLA_OPT_ALL_SCALES) ? 1 : 0);
  }
  GLA_CHECK_LAUNCH();
  if (R > 1) {
    GLA_TRY((launch_sum_blocks<bf16, 1>(st, dq_v, (bf16*)dq, B * T, H, R)));
    GLA_TRY((launch_sum_blocks<bf16, 1>(st, dk_v, (bf16*)dk, B * T, H, R)));
    GLA_TRY((launch_sum_blocks<float, 1>(st, dg_v, dg, B * T, H, R)));
    GLA_TRY((launch_sum_blocks<bf16, 0>(st, dv_v, (bf16*)dv, B * T, H, R)));
    GLA_TRY(launch_state_block(st, dhib, dhidden_init, B * H, R, 0));
  }
  return GLA_OK;
}

unsigned int tc_read_wait_timeouts() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_wait_timeouts, sizeof(v));
  return v;
}

}  // namespace gla
