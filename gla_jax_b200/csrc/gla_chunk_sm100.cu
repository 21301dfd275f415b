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

namespace gla {

using namespace tc;

constexpr int TC = 128;          // chunk length
constexpr int TD = 128;          // head dim
constexpr int TTHREADS = 512;
constexpr uint32_t TILE_BYTES = 128 * 128;     // one SW128 tile of 128 rows

__device__ unsigned int g_tc_wait_timeouts = 0;   // incremented when a bounded wait gives up

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
  float2 f[16];
  uint32_t xv[16];
  float2 gs = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t e = row0 + (int64_t)(rg * 16 + i) * HD + 2 * cp;
    const float2 gg = *reinterpret_cast<const float2*>(g + e);
    xv[i] = *reinterpret_cast<const uint32_t*>(x + e);
    gs.x += gg.x; gs.y += gg.y;
    f[i] = make_float2(__expf(gg.x), __expf(gg.y));
  }
  // w[i]: MODE 0 exclusive suffix product, MODE 1 inclusive prefix product, within the 16 rows
  float2 w[16];
  if (MODE == 0) {
    float2 run = make_float2(1.f, 1.f);
#pragma unroll
    for (int i = 15; i >= 0; --i) { w[i] = run; run.x *= f[i].x; run.y *= f[i].y; }
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
  if (MODE == 0 && Gc != nullptr && rg == 0) {
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

constexpr size_t KV_SMEM = 1024 + 4 * TILE_BYTES + 2 * 8 * TD * sizeof(float) + 64;

template <int MODE>
static int launch_tc_kv(cudaStream_t st, int64_t B, int64_t T, int64_t H, const float* g, const void* x, const void* y,
                        float* out, float* Gc) {
  const int64_t N = T / TC;
  cudaError_t e = cudaFuncSetAttribute(tc_kv_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)KV_SMEM);
  if (e != cudaSuccess) return record_cuda_error(e);
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
  static constexpr uint32_t Q = 0;                         // 2 buffers x 32 KB   (q~ / q_hat)
  static constexpr uint32_t K = Q + 2 * 2 * TILE_BYTES;    // 2 buffers x 16 KB   (compact k~)
  static constexpr uint32_t V = K + 2 * TILE_BYTES;        // 32 KB
  static constexpr uint32_t S = V + 2 * TILE_BYTES;        // 32 KB
  static constexpr uint32_t P = S + 2 * TILE_BYTES;        // 32 KB
  static constexpr uint32_t TOT = P + 2 * TILE_BYTES;      // 8 x 128 float
  static constexpr uint32_t DIAG = TOT + 8 * TD * 4;       // 2 x 128 float
  static constexpr uint32_t BAR = DIAG + 2 * TC * 4;       // 3 mbarriers + tmem slot
  static constexpr uint32_t END = BAR + 64;
};
constexpr uint32_t KC_TILE = 64 * 128;    // one SW128 tile of 64 rows

template <int HH>
__device__ __forceinline__ void emit_level_local(const float2 (&pre)[16], const float2 (&suf)[16],
                                                 const uint32_t (&qv)[16], const uint32_t (&kv)[16], uint8_t* sQb,
                                                 uint8_t* sKb, int rg, int cp) {
  constexpr int LG = HH == 1 ? 0 : HH == 2 ? 1 : HH == 4 ? 2 : 3;
  const int tile = cp >> 5, col = (2 * cp) & 63;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int r = rg * 16 + i;
    if (i & HH) {
      const float2 x = unpack_bf16x2(qv[i]);
      *reinterpret_cast<uint32_t*>(sQb + tile * TILE_BYTES + sw128_off(r, col)) = pack_bf16x2(x.x * pre[i].x, x.y * pre[i].y);
    } else {
      const float2 x = unpack_bf16x2(kv[i]);
      const int c = ((r >> (LG + 1)) << LG) + (r & (HH - 1));
      *reinterpret_cast<uint32_t*>(sKb + tile * KC_TILE + sw128_off(c, col)) = pack_bf16x2(x.x * suf[i].x, x.y * suf[i].y);
    }
  }
}
// pre/suf for half size HH -> half size 2 HH (in place)
template <int HH>
__device__ __forceinline__ void widen_products(float2 (&pre)[16], float2 (&suf)[16]) {
#pragma unroll
  for (int s0 = 0; s0 < 16; s0 += 2 * HH) {
    const float2 tf = pre[s0 + HH - 1], ts = pre[s0 + 2 * HH - 1];
#pragma unroll
    for (int i = 0; i < HH; ++i) {
      suf[s0 + i].x *= ts.x; suf[s0 + i].y *= ts.y;
      pre[s0 + HH + i].x *= tf.x; pre[s0 + HH + i].y *= tf.y;
    }
  }
}
// Level with half size >= 16: every row of the thread is on the same side.
__device__ __forceinline__ void emit_level_wide(int h, int lg, bool right, float2 cross, const float2 (&pre)[16],
                                                const float2 (&suf)[16], const uint32_t (&qv)[16],
                                                const uint32_t (&kv)[16], uint8_t* sQb, uint8_t* sKb, int rg, int cp) {
  const int tile = cp >> 5, col = (2 * cp) & 63;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int r = rg * 16 + i;
    if (right) {
      const float2 x = unpack_bf16x2(qv[i]);
      *reinterpret_cast<uint32_t*>(sQb + tile * TILE_BYTES + sw128_off(r, col)) =
          pack_bf16x2(x.x * pre[i].x * cross.x, x.y * pre[i].y * cross.y);
    } else {
      const float2 x = unpack_bf16x2(kv[i]);
      const int c = ((r >> (lg + 1)) << lg) + (r & (h - 1));
      *reinterpret_cast<uint32_t*>(sKb + tile * KC_TILE + sw128_off(c, col)) =
          pack_bf16x2(x.x * suf[i].x * cross.x, x.y * suf[i].y * cross.y);
    }
  }
}

__global__ void __launch_bounds__(TTHREADS, 1)
tc_chunk_fwd_kernel(int64_t T, int64_t H, int64_t N, const float* __restrict__ g, const bf16* __restrict__ v,
                    const bf16* __restrict__ k, const bf16* __restrict__ q, const bf16* __restrict__ S_prev,
                    bf16* __restrict__ out, bf16* __restrict__ P_saved) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  float* tot = reinterpret_cast<float*>(sm + FwdSmem::TOT);
  float* diag = reinterpret_cast<float*>(sm + FwdSmem::DIAG);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + FwdSmem::BAR);   // [0],[1]: level buffers, [2]: output
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = tid >> 6, cp = tid & 63;
  const int64_t n = blockIdx.x % N, bh = blockIdx.x / N, b = bh / H, h_ = bh % H;
  const int64_t HD = H * TD;
  const int64_t row0 = ((b * T + n * TC) * H + h_) * TD;
  const int64_t chunk_id = bh * N + n;

  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(smem_u32(bars + 0), 1);
    mbar_init(smem_u32(bars + 1), 1);
    mbar_init(smem_u32(bars + 2), 1);
    mbar_fence_init();
  }

  // ---- loads -----------------------------------------------------------------------------------
  float2 pre[16], suf[16];
  uint32_t qv[16], kv[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t e = row0 + (int64_t)(rg * 16 + i) * HD + 2 * cp;
    const float2 gg = *reinterpret_cast<const float2*>(g + e);
    qv[i] = *reinterpret_cast<const uint32_t*>(q + e);
    kv[i] = *reinterpret_cast<const uint32_t*>(k + e);
    pre[i] = make_float2(__expf(gg.x), __expf(gg.y));
    suf[i] = make_float2(1.f, 1.f);
  }
  copy_tile_128x128(sm + FwdSmem::V, v + row0, HD);
  copy_tile_128x128(sm + FwdSmem::S, S_prev + chunk_id * TD * TD, TD);
  // diagonal: sum_d q k, reduced over the 64 column-pair threads of a row group (two warps)
  {
    float part[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 a = unpack_bf16x2(qv[i]), c = unpack_bf16x2(kv[i]);
      part[i] = a.x * c.x + a.y * c.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int i = 0; i < 16; ++i) part[i] += __shfl_xor_sync(0xffffffffu, part[i], o);
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < 16; ++i) diag[(warp & 1) * TC + rg * 16 + i] = part[i];
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t sQ0 = smem_u32(sm + FwdSmem::Q), sK0 = smem_u32(sm + FwdSmem::K);

  auto issue_level = [&](int slot) {
    // executed by thread 0 after the block-wide barrier that follows the operand build
    const int bsel = slot & 1;
    constexpr uint32_t idesc = idesc_bf16(128, 64, 0, 0);
    const uint32_t a0 = sQ0 + bsel * 2 * TILE_BYTES, b0 = sK0 + bsel * 2 * KC_TILE;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      umma_bf16(tmem + 64 * slot, desc_kmajor(a0, TILE_BYTES, ks), desc_kmajor(b0, KC_TILE, ks), idesc, ks > 0);
    umma_commit(smem_u32(bars + bsel));
  };
  bool ok = true;
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

  // ---- levels h = 1, 2, 4, 8: rows of one block all belong to this thread -----------------------
  emit_level_local<1>(pre, suf, qv, kv, sm + FwdSmem::Q, sm + FwdSmem::K, rg, cp);
  level_sync_and_issue(0);
  widen_products<1>(pre, suf);
  emit_level_local<2>(pre, suf, qv, kv, sm + FwdSmem::Q + 2 * TILE_BYTES, sm + FwdSmem::K + 2 * KC_TILE, rg, cp);
  level_sync_and_issue(1);
  widen_products<2>(pre, suf);
  wait_buffer_free(2);
  emit_level_local<4>(pre, suf, qv, kv, sm + FwdSmem::Q, sm + FwdSmem::K, rg, cp);
  level_sync_and_issue(2);
  widen_products<4>(pre, suf);
  wait_buffer_free(3);
  emit_level_local<8>(pre, suf, qv, kv, sm + FwdSmem::Q + 2 * TILE_BYTES, sm + FwdSmem::K + 2 * KC_TILE, rg, cp);
  widen_products<8>(pre, suf);     // now pre/suf span the thread's 16 rows
  *reinterpret_cast<float2*>(tot + rg * TD + 2 * cp) = pre[15];
  level_sync_and_issue(3);         // the barrier inside also publishes tot

  // ---- levels h = 16, 32, 64 ------------------------------------------------------------------------
  auto tot_at = [&](int r2) { return *reinterpret_cast<const float2*>(tot + r2 * TD + 2 * cp); };
  {
    wait_buffer_free(4);
    emit_level_wide(16, 4, (rg & 1) != 0, make_float2(1.f, 1.f), pre, suf, qv, kv, sm + FwdSmem::Q, sm + FwdSmem::K, rg, cp);
    level_sync_and_issue(4);
  }
  {
    const int m = rg & 3;
    float2 cross = make_float2(1.f, 1.f);
    if (m == 3) cross = tot_at(rg - 1);
    if (m == 0) cross = tot_at(rg + 1);
    wait_buffer_free(5);
    emit_level_wide(32, 5, m >= 2, cross, pre, suf, qv, kv, sm + FwdSmem::Q + 2 * TILE_BYTES, sm + FwdSmem::K + 2 * KC_TILE, rg, cp);
    level_sync_and_issue(5);
  }
  float2 cross_q = make_float2(1.f, 1.f);      // prod of tot over row groups before rg (for q_hat)
  {
    float2 cross = make_float2(1.f, 1.f);
    if (rg >= 4) {
      for (int r2 = 4; r2 < rg; ++r2) { const float2 t = tot_at(r2); cross.x *= t.x; cross.y *= t.y; }
    } else {
      for (int r2 = rg + 1; r2 < 4; ++r2) { const float2 t = tot_at(r2); cross.x *= t.x; cross.y *= t.y; }
    }
    for (int r2 = 0; r2 < rg; ++r2) { const float2 t = tot_at(r2); cross_q.x *= t.x; cross_q.y *= t.y; }
    wait_buffer_free(6);
    emit_level_wide(64, 6, rg >= 4, cross, pre, suf, qv, kv, sm + FwdSmem::Q, sm + FwdSmem::K, rg, cp);
    level_sync_and_issue(6);
  }
  // all seven level MMAs done when the last commit (buffer 0, fourth use) completes
  ok = mbar_wait(smem_u32(bars + 0), 1) && ok;
  ok = mbar_wait(smem_u32(bars + 1), 0) && ok;     // buffer 1, third use (level slot 5)
  tc_fence_after();

  // ---- read the scores back into the bf16 P tile -----------------------------------------------------
  {
    const int q4 = warp & 3, cj = warp >> 2;
    const int li = lane;
    const uint32_t lane_base = tmem + ((uint32_t)(q4 * 32) << 16);
    float pr[32];
    if (cj > q4) {
#pragma unroll
      for (int m = 0; m < 32; ++m) pr[m] = 0.f;
    } else if (cj < q4) {
      const int slot = ((q4 ^ cj) >= 2) ? 6 : 5;
      const int col = (slot == 6) ? 32 * cj : 16 * cj;
      uint32_t r[32];
      tmem_ld32(lane_base + 64 * slot + col, r);
      tmem_ld_wait();
#pragma unroll
      for (int m = 0; m < 32; ++m) pr[m] = __uint_as_float(r[m]);
    } else {
#pragma unroll
      for (int m = 0; m < 32; ++m) pr[m] = 0.f;
#pragma unroll
      for (int s = 0; s < 5; ++s) {
        const int hh = 1 << s;
        uint32_t r[16];
        tmem_ld16(lane_base + 64 * s + 16 * q4, r);
        tmem_ld_wait();
#pragma unroll
        for (int lj = 0; lj < 32; ++lj) {
          if ((lj & hh) == 0) {
            const int c = ((lj >> (s + 1)) << s) + (lj & (hh - 1));
            if (((li ^ lj) >> s) == 1) pr[lj] = __uint_as_float(r[c]);
          }
        }
      }
      const float dg = diag[32 * q4 + li] + diag[TC + 32 * q4 + li];
#pragma unroll
      for (int lj = 0; lj < 32; ++lj)
        if (lj == li) pr[lj] = dg;
    }
    const int i = 32 * q4 + li;
    uint8_t* tile = sm + FwdSmem::P + (cj >> 1) * TILE_BYTES;
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      uint4 u;
      u.x = pack_bf16x2(pr[8 * c4 + 0], pr[8 * c4 + 1]);
      u.y = pack_bf16x2(pr[8 * c4 + 2], pr[8 * c4 + 3]);
      u.z = pack_bf16x2(pr[8 * c4 + 4], pr[8 * c4 + 5]);
      u.w = pack_bf16x2(pr[8 * c4 + 6], pr[8 * c4 + 7]);
      *reinterpret_cast<uint4*>(tile + sw128_chunk(i, (cj & 1) * 4 + c4)) = u;
      if (P_saved)
        *reinterpret_cast<uint4*>(P_saved + (chunk_id * TC + i) * TC + 32 * cj + 8 * c4) = u;
    }
  }
  // ---- q_hat into Q buffer 0 (all level MMAs have completed) ------------------------------------------
  {
    uint8_t* tile = sm + FwdSmem::Q + (cp >> 5) * TILE_BYTES;
    const int col = (2 * cp) & 63;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 x = unpack_bf16x2(qv[i]);
      *reinterpret_cast<uint32_t*>(tile + sw128_off(rg * 16 + i, col)) =
          pack_bf16x2(x.x * pre[i].x * cross_q.x, x.y * pre[i].y * cross_q.y);
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    tc_fence_after();
    constexpr uint32_t idesc = idesc_bf16(128, 128, 0, 1);
    const uint32_t aq = sQ0, bs = smem_u32(sm + FwdSmem::S), ap = smem_u32(sm + FwdSmem::P), bv = smem_u32(sm + FwdSmem::V);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      umma_bf16(tmem, desc_kmajor(aq, TILE_BYTES, ks), desc_mnmajor(bs, TILE_BYTES, ks), idesc, ks > 0);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      umma_bf16(tmem, desc_kmajor(ap, TILE_BYTES, ks), desc_mnmajor(bv, TILE_BYTES, ks), idesc, 1);
    umma_commit(smem_u32(bars + 2));
  }
  ok = mbar_wait(smem_u32(bars + 2), 0) && ok;
  tc_fence_after();
  if (ok) {
    const int q4 = warp & 3, cg = warp >> 2;
    uint32_t r[32];
    tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(cg * 32), r);
    tmem_ld_wait();
    bf16* o = out + row0 + (int64_t)(q4 * 32 + lane) * HD + cg * 32;
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      uint4 u;
      u.x = pack_bf16x2(__uint_as_float(r[8 * c4 + 0]), __uint_as_float(r[8 * c4 + 1]));
      u.y = pack_bf16x2(__uint_as_float(r[8 * c4 + 2]), __uint_as_float(r[8 * c4 + 3]));
      u.z = pack_bf16x2(__uint_as_float(r[8 * c4 + 4]), __uint_as_float(r[8 * c4 + 5]));
      u.w = pack_bf16x2(__uint_as_float(r[8 * c4 + 6]), __uint_as_float(r[8 * c4 + 7]));
      *reinterpret_cast<uint4*>(o + 8 * c4) = u;
    }
  } else if (tid == 0) {
    atomicAdd(&g_tc_wait_timeouts, 1u);
  }
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

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
bool tc_supported(int64_t D, int64_t C, int dtype) { return D == TD && C == TC && dtype == GLA_BF16; }
bool tc_auto_default() { return false; }

static size_t f32b(int64_t n) { return align_up((size_t)n * 4, 256); }

static size_t b16b(int64_t n) { return align_up((size_t)n * 2, 256); }

// saved: S_prev bf16 (BH,N,D,D) | Gc f32 (BH,N,D) | P bf16 (BH,N,C,C)
size_t tc_saved_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C) {
  const int64_t N = T / C, BH = B * H;
  return b16b(BH * N * D * D) + f32b(BH * N * D) + b16b(BH * N * C * C);
}
// fwd workspace: kv f32 (BH,N,D,D) | Gc f32 | S_prev bf16 (used when nothing is saved)
size_t tc_fwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C) {
  const int64_t N = T / C, BH = B * H;
  return f32b(BH * N * D * D) + f32b(BH * N * D) + b16b(BH * N * D * D);
}
size_t tc_bwd_ws_bytes(int64_t B, int64_t T, int64_t H, int64_t D, int64_t C) { return simt_bwd_ws_bytes(B, T, H, D, C); }

constexpr size_t FWD_SMEM = 1024 + FwdSmem::END;

int tc_chunk_fwd(cudaStream_t st, int64_t B, int64_t T, int64_t H, int64_t D, int64_t C, const void* hidden_init,
                 const float* g, const void* v, const void* k, const void* q, void* hidden_final, void* out,
                 void* saved, void* ws, int state_only, float* G_total, float* S_local) {
  const int64_t N = T / C, BH = B * H;
  char* w = (char*)ws;
  float* kv = (float*)w; w += f32b(BH * N * D * D);
  float* Gc = (float*)w; w += f32b(BH * N * D);
  bf16* S_prev = (bf16*)w;
  bf16* P = nullptr;
  if (saved) {
    char* s = (char*)saved;
    S_prev = (bf16*)s; s += b16b(BH * N * D * D);
    Gc = (float*)s;    s += f32b(BH * N * D);
    P = (bf16*)s;
  }
  GLA_TRY((launch_tc_kv<0>(st, B, T, H, g, k, v, kv, Gc)));
  if (state_only) {
    GLA_TRY(launch_state_scan(st, BH, N, D, Gc, kv, 0, nullptr, 0, nullptr, 0, S_local, 0, 0));
    ProfScope ps("tc_gsum_kernel", st);
    tc_gsum_kernel<<<(unsigned)((BH * D + 255) / 256), 256, 0, st>>>(BH, N, Gc, G_total);
    GLA_CHECK_LAUNCH();
    return GLA_OK;
  }
  GLA_TRY(launch_state_scan(st, BH, N, D, Gc, kv, 0, hidden_init, 1, S_prev, 1, hidden_final, 1, 0));
  cudaError_t e = cudaFuncSetAttribute(tc_chunk_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FWD_SMEM);
  if (e != cudaSuccess) return record_cuda_error(e);
  {
    ProfScope ps("tc_chunk_fwd_kernel", st);
    tc_chunk_fwd_kernel<<<(unsigned)(BH * N), TTHREADS, FWD_SMEM, st>>>(T, H, N, g, (const bf16*)v, (const bf16*)k,
                                                                       (const bf16*)q, S_prev, (bf16*)out, P);
  }
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

int tc_chunk_bwd(cudaStream_t, int64_t, int64_t, int64_t, int64_t, int64_t, const float*, const void*, const void*,
                 const void*, const void*, const void*, const void*, void*, float*, void*, void*, void*, void*) {
  return GLA_ERR_UNSUPPORTED;
}

unsigned int tc_read_wait_timeouts() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_wait_timeouts, sizeof(v));
  return v;
}

}  // namespace gla
