// Memory-bound scan kernels: cumsum along time, the log-space linear-RNN scan, the D x D
// state scan over chunks and the cross-rank state combine.  All math in float32.
//
// Reference operators restated here: ops.py:152-284 (cumsum), ops.py:286-456 (linear-RNN
// scan).  The reference lowers these to a generic Triton `tt.scan` (ops.py:18-104) and
// needs a host-side hierarchy for long axes; here a thread block walks the time axis in
// tiles, scanning within a tile in registers and carrying the running total, so any length
// is one launch with fully coalesced 128-byte row segments.
#include "gla_common.cuh"
#include "tc_ptx.cuh"
#include "tma_maps.cuh"

namespace gla {

// ---------------------------------------------------------------------------------------
// cumsum: src (N, T, D) -> dst (N, T, D), inclusive along T, + init (N, D).
// Block = 32 column lanes x 8 row lanes; a tile is 64 rows; each thread scans 8
// consecutive rows of one column in registers, row lanes are combined through shared memory.
// ---------------------------------------------------------------------------------------
constexpr int CS_RPT = 8;    // rows per thread
constexpr int CS_RL = 8;     // row lanes

// The combine rules of the scan library (gla_scan_op): each is associative with an identity element, which is what
// the tiled scan needs (padding, carries, segment totals).  ops.py:82-104 scans with an arbitrary traced function;
// here the function is one of these, picked by the caller.
struct OpAdd { static __device__ __forceinline__ float id() { return 0.f; }
               static __device__ __forceinline__ float f(float a, float b) { return a + b; } };
struct OpMul { static __device__ __forceinline__ float id() { return 1.f; }
               static __device__ __forceinline__ float f(float a, float b) { return a * b; } };
struct OpMax { static __device__ __forceinline__ float id() { return -INFINITY; }
               static __device__ __forceinline__ float f(float a, float b) { return fmaxf(a, b); } };
struct OpMin { static __device__ __forceinline__ float id() { return INFINITY; }
               static __device__ __forceinline__ float f(float a, float b) { return fminf(a, b); } };
struct OpLogAddExp {      // log(exp(a) + exp(b)), evaluated around the larger argument
  static __device__ __forceinline__ float id() { return -INFINITY; }
  static __device__ __forceinline__ float f(float a, float b) {
    const float m = fmaxf(a, b), n = fminf(a, b);
    return m == -INFINITY ? m : m + log1pf(__expf(n - m));
  }
};

// The scan axis may be cut into `nseg` segments of `seg_len` positions (in scan order) that run
// as separate blocks: a first launch with TOTALS = true leaves every segment's column sums in
// `totals` (N, nseg, D); the second adds the sums of the segments before its own to its carry.
// nseg = 1 with totals = nullptr is the plain one-pass scan.
template <typename TI, typename TO, bool TOTALS, typename OP>
__global__ void __launch_bounds__(256) cumsum_kernel(const TI* __restrict__ src, const TI* __restrict__ sub,
                                                     const TI* __restrict__ init, TO* __restrict__ dst, int64_t T,
                                                     int64_t D, int reverse, int nseg, int64_t seg_len,
                                                     float* __restrict__ totals) {
  __shared__ float tot[CS_RL][33];
  const int64_t n = blockIdx.x / nseg;
  const int seg = (int)(blockIdx.x % nseg);
  const int tx = threadIdx.x, rl = threadIdx.y;
  const int64_t c = (int64_t)blockIdx.y * 32 + tx;
  const bool cvalid = c < D;
  float carry = (!TOTALS && init != nullptr && cvalid) ? ld_f(init, n * D + c) : OP::id();
  if (!TOTALS && totals != nullptr && cvalid)
    for (int s2 = 0; s2 < seg; ++s2) carry = OP::f(carry, totals[(n * nseg + s2) * D + c]);
  const TI* s = src + n * T * D;
  const TI* s2 = sub ? sub + n * T * D : nullptr;   // optional second source, subtracted element-wise
  TO* o = dst + n * T * D;
  const int64_t tbeg = (int64_t)seg * seg_len;
  const int64_t tend = tbeg + seg_len < T ? tbeg + seg_len : T;
  // The loads of the NEXT tile are issued before the current one is combined: a block walks its rows in order, so
  // without this every tile would wait out a full memory latency with nothing in flight.
  auto fetch = [&](int64_t t0, float (&y)[CS_RPT]) {
#pragma unroll
    for (int r = 0; r < CS_RPT; ++r) {
      int64_t tt = t0 + rl * CS_RPT + r;
      int64_t tp = reverse ? (T - 1 - tt) : tt;
      y[r] = (cvalid && tt < tend) ? ld_f(s, tp * D + c) : OP::id();
      if (s2 && cvalid && tt < tend) y[r] -= ld_f(s2, tp * D + c);
    }
  };
  float xn[CS_RPT];
  fetch(tbeg, xn);
  for (int64_t t0 = tbeg; t0 < tend; t0 += CS_RPT * CS_RL) {
    float x[CS_RPT];
#pragma unroll
    for (int r = 0; r < CS_RPT; ++r) x[r] = xn[r];
    if (t0 + CS_RPT * CS_RL < tend) fetch(t0 + CS_RPT * CS_RL, xn);
#pragma unroll
    for (int r = 1; r < CS_RPT; ++r) x[r] = OP::f(x[r - 1], x[r]);
    if (TOTALS) {
      // the row lanes hold consecutive pieces of the tile: combined in order after the loop (each lane keeps the
      // running combination of ITS pieces, which is only order-safe for commutative rules; all rules here are)
      carry = OP::f(carry, x[CS_RPT - 1]);
      continue;
    }
    tot[rl][tx] = x[CS_RPT - 1];
    __syncthreads();
    float off = carry, total = OP::id();
#pragma unroll
    for (int r2 = 0; r2 < CS_RL; ++r2) {
      float v = tot[r2][tx];
      if (r2 < rl) off = OP::f(off, v);
      total = OP::f(total, v);
    }
#pragma unroll
    for (int r = 0; r < CS_RPT; ++r) {
      int64_t tt = t0 + rl * CS_RPT + r;
      int64_t tp = reverse ? (T - 1 - tt) : tt;
      if (cvalid && tt < tend) st_f(o, tp * D + c, OP::f(off, x[r]));
    }
    carry = OP::f(carry, total);
    __syncthreads();
  }
  if (TOTALS) {
    tot[rl][tx] = carry;
    __syncthreads();
    if (rl == 0 && cvalid) {
      float total = OP::id();
#pragma unroll
      for (int r2 = 0; r2 < CS_RL; ++r2) total = OP::f(total, tot[r2][tx]);
      totals[(n * nseg + seg) * D + c] = total;
    }
  }
}

__device__ __forceinline__ float4 ld4_f(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 ld4_f(const bf16* p) {
  const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}
__device__ __forceinline__ void st4_f(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4_f(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}


// The same scan with FOUR consecutive columns per thread (16-byte accesses: a warp reads 512 contiguous bytes of a
// row) and 16 row lanes: a block covers 128 columns and walks the axis in tiles of 128 rows, 64 KB of float32 per
// tile with the next tile's loads already in flight.  Rows this wide keep the memory system busy from few blocks,
// which is what a long scan axis with few rows offers.  Serves D % 4 == 0 with suitably aligned pointers.
constexpr int C4_RL = 16;    // row lanes
template <typename OP> __device__ __forceinline__ float4 op4(float4 a, float4 b) {
  return make_float4(OP::f(a.x, b.x), OP::f(a.y, b.y), OP::f(a.z, b.z), OP::f(a.w, b.w));
}
template <typename TI, typename TO, bool TOTALS, typename OP>
__global__ void __launch_bounds__(32 * C4_RL) cumsum_v4_kernel(const TI* __restrict__ src, const TI* __restrict__ sub,
                                                               const TI* __restrict__ init, TO* __restrict__ dst,
                                                               int64_t T, int64_t D, int reverse, int nseg,
                                                               int64_t seg_len, float* __restrict__ totals) {
  // both arrays are double-buffered by tile parity, which is what lets a tile get by with ONE block barrier: a
  // buffer is rewritten two tiles later, after a barrier that every reader of it has passed
  __shared__ float4 tot[2][C4_RL][32];
  __shared__ float4 car[2][32];
  const int64_t n = blockIdx.x / nseg;
  const int seg = (int)(blockIdx.x % nseg);
  const int tx = threadIdx.x, rl = threadIdx.y;
  const int64_t c = ((int64_t)blockIdx.y * 32 + tx) * 4;
  const bool cvalid = c < D;
  const float4 ident = make_float4(OP::id(), OP::id(), OP::id(), OP::id());
  float4 carry = (!TOTALS && init != nullptr && cvalid) ? ld4_f(init + n * D + c) : ident;
  if (!TOTALS && totals != nullptr && cvalid)
    for (int s2 = 0; s2 < seg; ++s2)
      carry = op4<OP>(carry, *reinterpret_cast<const float4*>(totals + (n * nseg + s2) * D + c));
  const int64_t tbeg = (int64_t)seg * seg_len;
  const int64_t tend = tbeg + seg_len < T ? tbeg + seg_len : T;
  // a thread's rows of a tile are `rs` elements apart (backwards in memory for a reversed scan) and its first row
  // moves by a whole tile per iteration: no multiplication and no 64-bit compare inside the loop
  const int64_t rs = reverse ? -D : D;
  const int64_t row0 = tbeg + rl * CS_RPT;
  const int64_t off0 = n * T * D + c + (reverse ? (T - 1 - row0) : row0) * D;
  const TI* ps = src + off0;
  const TI* ps2 = sub ? sub + off0 : nullptr;
  TO* po = dst + off0;
  const int64_t step = (int64_t)CS_RPT * C4_RL * rs;
  // rows of this thread that lie inside the segment, for the tile being fetched / stored (<= 0: none)
  auto rows_in = [&](int64_t t0) -> int {
    const int64_t left = tend - (t0 + rl * CS_RPT);
    return !cvalid ? 0 : left >= CS_RPT ? CS_RPT : left < 0 ? 0 : (int)left;
  };
  auto fetch = [&](int nr, float4 (&y)[CS_RPT]) {
#pragma unroll
    for (int r = 0; r < CS_RPT; ++r) {
      y[r] = r < nr ? ld4_f(ps + r * rs) : ident;
      if (ps2 && r < nr) {
        const float4 z = ld4_f(ps2 + r * rs);
        y[r].x -= z.x; y[r].y -= z.y; y[r].z -= z.z; y[r].w -= z.w;
      }
    }
    ps += step;
    if (ps2) ps2 += step;
  };
  float4 xn[CS_RPT];
  fetch(rows_in(tbeg), xn);
  if (!TOTALS) {
    if (rl == C4_RL - 1) car[0][tx] = carry;
  }
  int par = 0;
  for (int64_t t0 = tbeg; t0 < tend; t0 += CS_RPT * C4_RL, par ^= 1) {
    float4 x[CS_RPT];
#pragma unroll
    for (int r = 0; r < CS_RPT; ++r) x[r] = xn[r];
    const int nr = rows_in(t0);
    if (t0 + CS_RPT * C4_RL < tend) fetch(rows_in(t0 + CS_RPT * C4_RL), xn);
#pragma unroll
    for (int r = 1; r < CS_RPT; ++r) x[r] = op4<OP>(x[r - 1], x[r]);
    if (TOTALS) {
      carry = op4<OP>(carry, x[CS_RPT - 1]);    // commutative rules only, as in the scalar form
      continue;
    }
    tot[par][rl][tx] = x[CS_RPT - 1];
    __syncthreads();
    // the carry into this tile (left by the last row lane at the end of the tile before) combined with the row
    // lanes before this one: the trip count is the same for the whole warp
    float4 off = car[par][tx];
    for (int r2 = 0; r2 < rl; ++r2) off = op4<OP>(off, tot[par][r2][tx]);
    if (rl == C4_RL - 1) car[par ^ 1][tx] = op4<OP>(off, x[CS_RPT - 1]);
#pragma unroll
    for (int r = 0; r < CS_RPT; ++r)
      if (r < nr) st4_f(po + r * rs, op4<OP>(off, x[r]));
    po += step;
  }
  if (TOTALS) {
    tot[0][rl][tx] = carry;
    __syncthreads();
    if (rl == 0 && cvalid) {
      float4 total = ident;
#pragma unroll
      for (int r2 = 0; r2 < C4_RL; ++r2) total = op4<OP>(total, tot[0][r2][tx]);
      *reinterpret_cast<float4*>(totals + (n * nseg + seg) * D + c) = total;
    }
  }
}

// ---------------------------------------------------------------------------------------
// The float32 scan of wide rows as a TMA pipeline.  What limits the kernels above on a long axis is how many bytes
// a thread block can keep in flight with ordinary loads; here a 64-row x 128-column tile travels as ONE tensor copy
// (cp.async.bulk.tensor over a 3-d map (column, row, n): rows past the end of the axis and columns past D are
// zero-filled on the way in and skipped on the way out) into a ring of NST shared-memory stages, the threads scan
// a landed tile out of shared memory, write the result into one of two staging tiles, and a tensor store takes it
// back.  Up to NST tiles (32 KB each) are in flight per block at no register cost.  (One bulk copy per ROW was
// measured first: 128 copy instructions per tile made the kernel twice as slow as the load/store one.)
//   thread 0       issues the copy of tile i + NST once tile i has been read
//   thread 32      issues the store of tile i and waits for the store of tile i - 2 to have read its stage
//   all 8 warps    thread = four columns x eight consecutive scan positions; row lanes combine as in the kernel above
// A reversed scan walks the tiles from the end of the axis; its tiles are laid out so that every one but the FIRST
// in scan order starts on a multiple of 64 rows from the end (no store ever starts at a negative row), and a
// thread's scan position p sits in stage row nr - 1 - p.
// Every mbarrier wait is bounded; a block whose wait expires stops, waits (bounded) for the copies it still has
// in flight and counts itself in g_scan_wait_timeouts.
// ---------------------------------------------------------------------------------------
namespace {
using namespace tc;
__device__ unsigned int g_scan_wait_timeouts = 0;
constexpr int BK_RL = 8;                       // row lanes
constexpr int BK_ROWS = CS_RPT * BK_RL;        // rows of a tile (64)
constexpr int BK_NST = 4;                      // input stages
constexpr int BK_TILE = BK_ROWS * 128 * 4;     // bytes of a tile (32 KB)
constexpr int BK_SMEM = (BK_NST + 2) * BK_TILE + 1024;

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int PENDING> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(PENDING) : "memory");
}
template <int PENDING> __device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" :: "n"(PENDING) : "memory");
}

struct ScanMaps { CUtensorMap in, out; };

template <typename OP, bool MULTI>
__global__ void __launch_bounds__(32 * BK_RL, 1) cumsum_tma_kernel(const __grid_constant__ ScanMaps maps, const float* __restrict__ init,
                                                                   int64_t N, int64_t T, int64_t D, int reverse) {
  extern __shared__ uint8_t bk_raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)bk_raw + 1023) & ~(uintptr_t)1023);
  __shared__ float4 tot[2][BK_RL][32];
  __shared__ float4 car[2][32];
  __shared__ uint64_t full[BK_NST];
  const int tx = threadIdx.x, rl = threadIdx.y, tid = rl * 32 + tx;
  // Work items are (row n, block of 128 columns); a block takes items blockIdx.x, + gridDim.x, ... and streams their
  // tiles back to back through the same ring, so that short axes (a chunk of 128 positions is two tiles) do not pay
  // a block start-up each.
  const int64_t gy = (D + 127) / 128, items = N * gy;
  // MULTI == false is the same kernel for grids with one item per block: the walk over items folds away
  const int64_t my_items = MULTI ? (items - blockIdx.x + gridDim.x - 1) / gridDim.x : 1;
  // tiles of an item in scan order: forward tile i starts at row 64 i; reversed, tile 0 holds the last `rem` rows of
  // the axis and tile i >= 1 the 64 rows before those of tile i - 1
  const int rem = (int)(T % BK_ROWS ? T % BK_ROWS : BK_ROWS);
  const int64_t ntiles = (T + BK_ROWS - 1) / BK_ROWS, total = my_items * ntiles;
  const int Ti = (int)T;
  auto rows_of = [&](int i) {
    if (reverse) return i == 0 ? rem : BK_ROWS;
    const int left = Ti - i * BK_ROWS;
    return left < BK_ROWS ? left : BK_ROWS;
  };
  auto start_of = [&](int i) { return reverse ? Ti - rem - i * BK_ROWS : i * BK_ROWS; };
  const uint32_t in0 = smem_u32(sm), out0 = in0 + BK_NST * BK_TILE, full0 = smem_u32(full);
  const float4 ident = make_float4(OP::id(), OP::id(), OP::id(), OP::id());

  if (tid == 0) {
    for (int s2 = 0; s2 < BK_NST; ++s2) mbar_init(full0 + 8 * s2, 1);
    mbar_fence_init();
  }
  __syncthreads();
  static_assert((BK_NST & (BK_NST - 1)) == 0, "the ring index is kept with a mask");
  // the producer's own walk over (item, tile), NST tiles ahead of the consumers'; all walks keep their place with
  // counters (no division per tile)
  int64_t p_item = blockIdx.x, p_g = 0;
  int p_i = 0, p_n = (int)(p_item / gy), p_c0 = (int)(p_item % gy) * 128;
  auto issue_load = [&]() {                   // one thread
    const uint32_t sidx = (uint32_t)p_g & (BK_NST - 1), bar = full0 + 8 * sidx;
    mbar_arrive_expect_tx(bar, BK_TILE);      // the box counts in full, zero-filled parts included
    tma_load_3d(in0 + sidx * BK_TILE, &maps.in, p_c0, start_of(p_i), p_n, bar);
    ++p_g;
    ++p_i;
    if (MULTI && p_i == (int)ntiles) {
      p_i = 0; p_item += gridDim.x;
      p_n = (int)(p_item / gy); p_c0 = (int)(p_item % gy) * 128;
    }
  };
  if (tid == 0)
    for (int a = 0; a < BK_NST && p_g < total; ++a) issue_load();
  auto init_of = [&](int nn, int cc) {
    const int64_t c = (int64_t)cc + tx * 4;
    return (init != nullptr && c < D) ? ld4_f(init + (int64_t)nn * D + c) : ident;
  };
  int64_t item = blockIdx.x, g = 0;
  int i = 0, n = (int)(item / gy), c0 = (int)(item % gy) * 128;
  if (rl == BK_RL - 1 && total > 0) car[0][tx] = init_of(n, c0);
  bool ok = true;
  int par = 0, st = 0;
  uint32_t phase = 0;
  for (; g < total; ++g, par ^= 1) {
    const bool cvalid = (int64_t)c0 + tx * 4 < D;
    ok = mbar_wait(full0 + 8 * st, phase);       // on expiry the tile is garbage: voted on below
    const int nrt = rows_of(i);
    const int nr = nrt - rl * CS_RPT;                 // this thread's scan positions inside the tile (<= 0: none)
    // scan position p = 8 rl + r of the tile sits in stage row p (forward) or nrt - 1 - p (reversed)
    const int row0 = reverse ? nrt - 1 - rl * CS_RPT : rl * CS_RPT, rstep = reverse ? -32 : 32;
    const float4* in = reinterpret_cast<const float4*>(sm + st * BK_TILE) + row0 * 32 + tx;
    float4 x[CS_RPT];
#pragma unroll
    for (int r = 0; r < CS_RPT; ++r) x[r] = (cvalid && r < nr) ? in[r * rstep] : ident;
#pragma unroll
    for (int r = 1; r < CS_RPT; ++r) x[r] = op4<OP>(x[r - 1], x[r]);
    tot[par][rl][tx] = x[CS_RPT - 1];
    // the staging tile that this tile is about to write was last read by the store of two tiles ago: all but the
    // newest store group must have read their stage
    if (tid == 32) bulk_wait_read<1>();
    // stage st has been read by everyone and the totals are visible; the same barrier takes the vote on the waits,
    // so that the whole block leaves together if any thread's wait expired
    if (!__syncthreads_and(ok)) { ok = false; break; }
    if (tid == 0 && p_g < total) issue_load();
    float4 off = car[par][tx];
    for (int r2 = 0; r2 < rl; ++r2) off = op4<OP>(off, tot[par][r2][tx]);
    const bool last_tile = MULTI && i + 1 == (int)ntiles;
    int n2 = n, c2 = c0;
    if (last_tile) { const int64_t nx = item + gridDim.x; n2 = (int)(nx / gy); c2 = (int)(nx % gy) * 128; }
    // the carry into the next tile: this item's running value, or the next item's initial value
    if (rl == BK_RL - 1)
      car[par ^ 1][tx] = !last_tile ? op4<OP>(off, x[CS_RPT - 1]) : item + gridDim.x < items ? init_of(n2, c2) : ident;
    float4* o = reinterpret_cast<float4*>(sm + (BK_NST + par) * BK_TILE) + row0 * 32 + tx;
#pragma unroll
    for (int r = 0; r < CS_RPT; ++r)
      if (r < nr) o[r * rstep] = op4<OP>(off, x[r]);
    fence_async_smem();                                // the staging tile is read by the async proxy
    __syncthreads();
    if (tid == 32) {
      tma_store_3d(&maps.out, c0, start_of(i), n, out0 + (uint32_t)par * BK_TILE);
      bulk_commit();
    }
    if (last_tile) { i = 0; item += gridDim.x; n = n2; c0 = c2; } else ++i;
    if (++st == BK_NST) { st = 0; phase ^= 1u; }
  }
  if (tid == 32) bulk_wait_all<0>();                    // the block's stores have completed before it leaves
  if (!ok) {
    // copies already requested land in this block's shared memory: give them their (bounded) time before leaving
    if (tid == 0)
      for (int64_t j = g; j < p_g; ++j) mbar_wait(full0 + 8 * ((uint32_t)j & (BK_NST - 1)), (uint32_t)((j / BK_NST) & 1));
    if (tid == 0) atomicAdd(&g_scan_wait_timeouts, 1u);
  }
}
}  // namespace

unsigned int scan_read_wait_timeouts() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_scan_wait_timeouts, sizeof(v));
  return v;
}

template <typename OP>
static int launch_cumsum_tma_op(cudaStream_t st, int64_t N, int64_t T, int64_t D, const float* src, const float* init, float* dst,
                                int reverse) {
  static SmemAttrOnce attr[2];
  GLA_TRY(attr[0].ensure(cumsum_tma_kernel<OP, false>, BK_SMEM));
  GLA_TRY(attr[1].ensure(cumsum_tma_kernel<OP, true>, BK_SMEM));
  ScanMaps maps;
  GLA_TRY(make_map_ntd_f32(&maps.in, src, N, T, D, BK_ROWS));
  GLA_TRY(make_map_ntd_f32(&maps.out, dst, N, T, D, BK_ROWS));
  // one block per SM (the ring takes most of its shared memory), fewer when there are fewer (row, column block) items
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t items = N * ((D + 127) / 128);
  dim3 block(32, BK_RL);
  if (items <= sms) cumsum_tma_kernel<OP, false><<<dim3((unsigned)items), block, BK_SMEM, st>>>(maps, init, N, T, D, reverse);
  else              cumsum_tma_kernel<OP, true><<<dim3((unsigned)sms), block, BK_SMEM, st>>>(maps, init, N, T, D, reverse);
  return GLA_OK;
}

// Column width of a block: the four-columns-per-thread kernel serves rows of at least 128 columns that are a
// multiple of four (and, checked at launch, 16-byte aligned pointers); the scalar kernel everything else.
static bool cumsum_wide(int64_t D) { return D >= 128 && D % 4 == 0; }

// Segments for a scan of N rows of length T: enough blocks to fill the device when N alone
// gives too few, but never segments shorter than 256 positions.
static int cumsum_segments(int64_t N, int64_t T, int64_t D) {
  const int64_t blocks = cumsum_wide(D) ? N * ((D + 127) / 128) : N * ((D + 31) / 32);
  const int64_t target = cumsum_wide(D) ? 2 * 148 : 4 * 148;
  const int64_t want = (target + blocks - 1) / blocks;
  int64_t nseg = want < 1 ? 1 : want;
  if (nseg > T / 256) nseg = T / 256;
  if (nseg < 1) nseg = 1;
  if (nseg > 64) nseg = 64;
  return (int)nseg;
}

size_t cumsum_scratch_bytes(int64_t N, int64_t T, int64_t D) {
  return (size_t)N * cumsum_segments(N, T, D) * D * sizeof(float);
}

template <typename TI, typename TO, typename OP>
static void cumsum_dispatch_op(cudaStream_t st, dim3 grid, dim3 block, const void* src, const void* sub,
                               const void* init, void* dst, int64_t T, int64_t D, int reverse, int nseg,
                               int64_t seg_len, float* totals) {
  if (block.y == C4_RL) {
    if (nseg > 1)
      cumsum_v4_kernel<TI, TO, true, OP><<<grid, block, 0, st>>>((const TI*)src, (const TI*)sub, (const TI*)init, (TO*)dst, T,
                                                                  D, reverse, nseg, seg_len, totals);
    cumsum_v4_kernel<TI, TO, false, OP><<<grid, block, 0, st>>>((const TI*)src, (const TI*)sub, (const TI*)init, (TO*)dst, T,
                                                                 D, reverse, nseg, seg_len, nseg > 1 ? totals : nullptr);
    return;
  }
  if (nseg > 1)
    cumsum_kernel<TI, TO, true, OP><<<grid, block, 0, st>>>((const TI*)src, (const TI*)sub, (const TI*)init, (TO*)dst, T, D,
                                                             reverse, nseg, seg_len, totals);
  cumsum_kernel<TI, TO, false, OP><<<grid, block, 0, st>>>((const TI*)src, (const TI*)sub, (const TI*)init, (TO*)dst, T, D,
                                                            reverse, nseg, seg_len, nseg > 1 ? totals : nullptr);
}
template <typename TI, typename TO>
static void cumsum_dispatch(cudaStream_t st, dim3 grid, dim3 block, const void* src, const void* sub,
                            const void* init, void* dst, int64_t T, int64_t D, int reverse, int nseg,
                            int64_t seg_len, float* totals, int op = GLA_SCAN_ADD) {
  switch (op) {
    case GLA_SCAN_MUL: cumsum_dispatch_op<TI, TO, OpMul>(st, grid, block, src, sub, init, dst, T, D, reverse, nseg, seg_len, totals); break;
    case GLA_SCAN_MAX: cumsum_dispatch_op<TI, TO, OpMax>(st, grid, block, src, sub, init, dst, T, D, reverse, nseg, seg_len, totals); break;
    case GLA_SCAN_MIN: cumsum_dispatch_op<TI, TO, OpMin>(st, grid, block, src, sub, init, dst, T, D, reverse, nseg, seg_len, totals); break;
    case GLA_SCAN_LOGADDEXP: cumsum_dispatch_op<TI, TO, OpLogAddExp>(st, grid, block, src, sub, init, dst, T, D, reverse, nseg, seg_len, totals); break;
    default: cumsum_dispatch_op<TI, TO, OpAdd>(st, grid, block, src, sub, init, dst, T, D, reverse, nseg, seg_len, totals); break;
  }
}

int launch_cumsum(cudaStream_t st, int64_t N, int64_t T, int64_t D, const void* src, const void* init,
                  void* dst, int reverse, int in_bf16, int out_bf16, const void* sub, float* scratch, int op) {
  if (N <= 0 || T <= 0 || D <= 0) return GLA_ERR_BAD_DIMS;
  if (op < GLA_SCAN_ADD || op > GLA_SCAN_LOGADDEXP || (sub != nullptr && op != GLA_SCAN_ADD)) return GLA_ERR_UNSUPPORTED;
  // 16-byte accesses need every row start on that boundary in each array: D % 4 == 0 makes the row pitch a
  // multiple of 16 bytes (8 for bf16), so the base pointers decide
  auto aligned = [](const void* p, int is_bf16) { return p == nullptr || ((uintptr_t)p % (is_bf16 ? 8 : 16)) == 0; };
  const bool wide = cumsum_wide(D) && aligned(src, in_bf16) && aligned(sub, in_bf16) && aligned(init, in_bf16) &&
                    aligned(dst, out_bf16) && aligned(scratch, 0);
  // float32 in and out, no second source, one pass: the bulk-copy pipeline
  if (wide && !in_bf16 && !out_bf16 && sub == nullptr && scratch == nullptr && T >= 2 * BK_ROWS) {
    if ((D + 127) / 128 > 65535 || N > 2147483647LL) return GLA_ERR_TOO_LARGE;
    ProfScope ps("cumsum_kernel", st);
    int rc;
    switch (op) {
      case GLA_SCAN_MUL: rc = launch_cumsum_tma_op<OpMul>(st, N, T, D, (const float*)src, (const float*)init, (float*)dst, reverse); break;
      case GLA_SCAN_MAX: rc = launch_cumsum_tma_op<OpMax>(st, N, T, D, (const float*)src, (const float*)init, (float*)dst, reverse); break;
      case GLA_SCAN_MIN: rc = launch_cumsum_tma_op<OpMin>(st, N, T, D, (const float*)src, (const float*)init, (float*)dst, reverse); break;
      case GLA_SCAN_LOGADDEXP: rc = launch_cumsum_tma_op<OpLogAddExp>(st, N, T, D, (const float*)src, (const float*)init, (float*)dst, reverse); break;
      default: rc = launch_cumsum_tma_op<OpAdd>(st, N, T, D, (const float*)src, (const float*)init, (float*)dst, reverse); break;
    }
    if (rc != GLA_OK) return rc;
    GLA_CHECK_LAUNCH();
    return GLA_OK;
  }
  const int64_t gy = wide ? (D + 127) / 128 : (D + 31) / 32;
  // without scratch for the segment sums the scan runs in one pass, one block per row and column group
  const int nseg = scratch ? cumsum_segments(N, T, D) : 1;
  const int64_t tile = CS_RPT * C4_RL;      // rows of the wide kernel's tile, a multiple of the scalar kernel's
  static_assert((CS_RPT * C4_RL) % (CS_RPT * CS_RL) == 0, "segment lengths must be whole tiles of both kernels");
  int64_t seg_len = (T + nseg - 1) / nseg;
  seg_len = (seg_len + tile - 1) / tile * tile;
  if (gy > 65535 || N * nseg > 2147483647LL) return GLA_ERR_TOO_LARGE;
  dim3 grid((unsigned)(N * nseg), (unsigned)gy), block(32, wide ? C4_RL : CS_RL);
  ProfScope ps("cumsum_kernel", st);
  if (!in_bf16 && !out_bf16)
    cumsum_dispatch<float, float>(st, grid, block, src, sub, init, dst, T, D, reverse, nseg, seg_len, scratch, op);
  else if (!in_bf16 && out_bf16)
    cumsum_dispatch<float, bf16>(st, grid, block, src, sub, init, dst, T, D, reverse, nseg, seg_len, scratch, op);
  else if (in_bf16 && !out_bf16)
    cumsum_dispatch<bf16, float>(st, grid, block, src, sub, init, dst, T, D, reverse, nseg, seg_len, scratch, op);
  else
    cumsum_dispatch<bf16, bf16>(st, grid, block, src, sub, init, dst, T, D, reverse, nseg, seg_len, scratch, op);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

// ---------------------------------------------------------------------------------------
// rnn_scan: sequential over T, parallel over the elements of the state.  A thread owns FOUR consecutive value
// columns of one key row (one 16- or 8-byte access per step instead of four scalar ones, and one exp() of the
// gate per step for the four), and keeps the loads of the next UNR steps in flight while it combines the
// current ones: the recurrence is a chain, so what the kernel can overlap is the memory latency of later steps.
// The scalar form below serves value widths that are not multiples of four.
// ---------------------------------------------------------------------------------------
template <typename TKV, bool RUNS>
__global__ void __launch_bounds__(128) rnn_scan_vec4_kernel(int64_t T, int64_t K, int64_t V, int64_t nblk,
                                                            const float* __restrict__ g, const TKV* __restrict__ kv,
                                                            const float* __restrict__ ig, const TKV* __restrict__ ikv,
                                                            float* __restrict__ out_log, TKV* __restrict__ out_state,
                                                            int reverse, int last_only, int nseg, int64_t L) {
  constexpr int UNR = 4;
  // nseg > 1: the axis is cut into runs of L scan positions that separate blocks scan, every run but the first from
  // the identity; rnn_carry_kernel / rnn_fix_kernel below then put the runs together (long axes with few rows)
  // (RUNS == false is the plain scan: the run arithmetic folds away)
  const int64_t prob2 = blockIdx.x / nblk, prob = RUNS ? prob2 / nseg : prob2, seg = RUNS ? prob2 % nseg : 0;
  const int64_t e4 = (blockIdx.x % nblk) * 128 + threadIdx.x;      // group of four value columns
  const int64_t KV = K * V, V4 = V / 4;
  if (e4 >= K * V4) return;
  const int64_t kk = e4 / V4, e = e4 * 4;
  const bool writes_log = (e4 % V4) == 0;
  float A = (ig && seg == 0) ? ig[prob * K + kk] : 0.f;
  float4 b = (ikv && seg == 0) ? ld4_f(ikv + prob * KV + e) : make_float4(0.f, 0.f, 0.f, 0.f);
  const float* gp = g + prob * T * K + kk;
  const TKV* xp = kv + prob * T * KV + e;
  TKV* op = out_state + prob * T * KV + e;
  float* lp = out_log + prob * T * K + kk;
  const int64_t s_beg = RUNS ? seg * L : 0;
  const int64_t Tfull = T;
  if (RUNS) T = Tfull - s_beg < L ? Tfull - s_beg : L;             // scan positions of this run (T below: the run's)
  auto tix = [&](int64_t s) { return reverse ? (Tfull - 1 - (s_beg + s)) : s_beg + s; };
  float gn[UNR];
  float4 xn[UNR];
#pragma unroll
  for (int u = 0; u < UNR; ++u) {
    const int64_t t = tix(u < T ? u : T - 1);
    gn[u] = gp[t * K];
    xn[u] = ld4_f(xp + t * KV);
  }
  for (int64_t s0 = 0; s0 < T; s0 += UNR) {
    float gc[UNR];
    float4 xc[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) { gc[u] = gn[u]; xc[u] = xn[u]; }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {           // the next group's loads, issued before this group is combined
      const int64_t sn = s0 + UNR + u;
      const int64_t t = tix(sn < T ? sn : T - 1);
      gn[u] = gp[t * K];
      xn[u] = ld4_f(xp + t * KV);
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int64_t sc = s0 + u;
      if (sc < T) {
        const float f = expf(gc[u]);
        b.x = fmaf(f, b.x, xc[u].x); b.y = fmaf(f, b.y, xc[u].y);
        b.z = fmaf(f, b.z, xc[u].z); b.w = fmaf(f, b.w, xc[u].w);
        A += gc[u];
        if (!last_only || sc == T - 1) {
          const int64_t t = tix(sc);
          st4_f(op + t * KV, b);
          if (writes_log) lp[t * K] = A;
        }
      }
    }
  }
}

// The runs of a segmented scan put together.  carry (one thread per four value columns, sequential over the runs):
// the true pair at the end of run s - 1, C_s = (CL_s, CS_s), from the runs' local last rows
//   C_1 = local last row of run 0 (which started from the caller's initial pair),
//   CL_{s+1} = CL_s + l_s,   CS_{s+1} = exp(l_s) CS_s + x_s        (l_s, x_s: local last row of run s),
// into wsL (batch, nseg, K) and wsS (batch, nseg, K, V), float32.
template <typename TKV>
__global__ void __launch_bounds__(128) rnn_carry_kernel(int64_t T, int64_t K, int64_t V, int64_t nblk, int nseg, int64_t L,
                                                        const float* __restrict__ out_log, const TKV* __restrict__ out_state,
                                                        float* __restrict__ wsL, float* __restrict__ wsS, int reverse) {
  const int64_t prob = blockIdx.x / nblk;
  const int64_t e4 = (blockIdx.x % nblk) * 128 + threadIdx.x;
  const int64_t KV = K * V, V4 = V / 4;
  if (e4 >= K * V4) return;
  const int64_t kk = e4 / V4, e = e4 * 4;
  const bool writes_log = (e4 % V4) == 0;
  float CL = 0.f;
  float4 CS = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sg = 0; sg < nseg; ++sg) {
    if (sg > 0) {
      if (writes_log) wsL[(prob * nseg + sg) * K + kk] = CL;
      *reinterpret_cast<float4*>(wsS + (prob * nseg + sg) * KV + e) = CS;
    }
    const int64_t last = (sg + 1) * L < T ? (sg + 1) * L - 1 : T - 1;      // scan position of the run's last row
    const int64_t row = reverse ? T - 1 - last : last;
    const float l = out_log[(prob * T + row) * K + kk];
    const float4 x = ld4_f(out_state + (prob * T + row) * KV + e);
    const float f = expf(l);
    CS = make_float4(fmaf(f, CS.x, x.x), fmaf(f, CS.y, x.y), fmaf(f, CS.z, x.z), fmaf(f, CS.w, x.w));
    CL += l;
  }
}
// fix (one thread per row and four value columns, rows of the runs after the first): state = exp(local log) C_S + local
// state.  The logs are corrected by rnn_fix_log_kernel afterwards (this kernel reads the local ones).
template <typename TKV>
__global__ void __launch_bounds__(256) rnn_fix_kernel(int64_t batch, int64_t T, int64_t K, int64_t V, int nseg, int64_t L,
                                                      const float* __restrict__ out_log, TKV* __restrict__ out_state,
                                                      const float* __restrict__ wsS, int reverse) {
  const int64_t KV4 = K * (V / 4), rows = T - L;
  const int64_t id = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (id >= batch * rows * KV4) return;
  const int64_t e4 = id % KV4, pos = L + (id / KV4) % rows, prob = id / KV4 / rows;
  const int64_t kk = e4 / (V / 4), e = e4 * 4, sg = pos / L;
  const int64_t row = reverse ? T - 1 - pos : pos;
  const float f = expf(out_log[(prob * T + row) * K + kk]);
  const float4 c = *reinterpret_cast<const float4*>(wsS + (prob * nseg + sg) * K * V + e);
  TKV* p = out_state + (prob * T + row) * K * V + e;
  const float4 x = ld4_f(p);
  st4_f(p, make_float4(fmaf(f, c.x, x.x), fmaf(f, c.y, x.y), fmaf(f, c.z, x.z), fmaf(f, c.w, x.w)));
}
__global__ void __launch_bounds__(256) rnn_fix_log_kernel(int64_t batch, int64_t T, int64_t K, int nseg, int64_t L,
                                                          float* __restrict__ out_log, const float* __restrict__ wsL,
                                                          int reverse) {
  const int64_t rows = T - L;
  const int64_t id = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (id >= batch * rows * K) return;
  const int64_t kk = id % K, pos = L + (id / K) % rows, prob = id / K / rows;
  const int64_t row = reverse ? T - 1 - pos : pos;
  out_log[(prob * T + row) * K + kk] += wsL[(prob * nseg + pos / L) * K + kk];
}

template <typename TKV>
__global__ void __launch_bounds__(256) rnn_scan_kernel(int64_t T, int64_t K, int64_t V, int64_t nblk,
                                                       const float* __restrict__ g, const TKV* __restrict__ kv,
                                                       const float* __restrict__ ig, const TKV* __restrict__ ikv,
                                                       float* __restrict__ out_log, TKV* __restrict__ out_state,
                                                       int reverse, int last_only) {
  const int64_t prob = blockIdx.x / nblk;
  const int64_t e = (blockIdx.x % nblk) * 256 + threadIdx.x;
  const int64_t KV = K * V;
  if (e >= KV) return;
  const int64_t kk = e / V, vv = e % V;
  float A = ig ? ig[prob * K + kk] : 0.f;
  float b = ikv ? ld_f(ikv, prob * KV + e) : 0.f;
  const float* gp = g + prob * T * K + kk;
  const TKV* xp = kv + prob * T * KV + e;
  TKV* op = out_state + prob * T * KV + e;
  float* lp = out_log + prob * T * K + kk;
#pragma unroll 4
  for (int64_t s = 0; s < T; ++s) {
    const int64_t t = reverse ? (T - 1 - s) : s;
    const float gt = gp[t * K];
    b = expf(gt) * b + ld_f(xp, t * KV);
    A += gt;
    if (!last_only || s == T - 1) {
      st_f(op, t * KV, b);
      if (vv == 0) lp[t * K] = A;
    }
  }
}

// Runs for a long axis with few rows: enough blocks for the device, runs of at least 128 positions.
static void rnn_scan_runs(int64_t batch, int64_t T, int64_t K, int64_t V, int* nseg, int64_t* L) {
  *nseg = 1; *L = T;
  if (V % 4 != 0 || T < 512) return;
  const int64_t blocks = batch * ((K * (V / 4) + 127) / 128);
  if (blocks >= 2 * 148) return;
  int64_t want = (4 * 148 + blocks - 1) / blocks;
  if (want > T / 128) want = T / 128;
  if (want < 2) return;
  *L = (T + want - 1) / want;
  *nseg = (int)((T + *L - 1) / *L);
}
size_t rnn_scan_ws_bytes(int64_t batch, int64_t T, int64_t K, int64_t V) {
  int nseg; int64_t L;
  rnn_scan_runs(batch, T, K, V, &nseg, &L);
  return nseg > 1 ? (size_t)(batch * nseg * (K + K * V)) * sizeof(float) + 16 : 0;
}

int launch_rnn_scan(cudaStream_t st, int64_t batch, int64_t T, int64_t K, int64_t V, const float* g,
                    const void* kv, const float* ig, const void* ikv, float* out_log, void* out_state,
                    int reverse, int last_only, int kv_bf16, float* ws, size_t ws_bytes) {
  ProfScope ps("rnn_scan_kernel", st);
  const bool al = (((uintptr_t)kv | (uintptr_t)out_state | (uintptr_t)ikv) & 15) == 0;
  if (V % 4 == 0 && al) {
    int64_t nblk = (K * (V / 4) + 127) / 128;
    int nseg = 1; int64_t L = T;
    if (ws != nullptr && !last_only && ((uintptr_t)ws & 15) == 0) {
      rnn_scan_runs(batch, T, K, V, &nseg, &L);
      if (ws_bytes < (size_t)(batch * nseg * (K + K * V)) * sizeof(float) + 16) { nseg = 1; L = T; }
    }
    if (nblk * batch * nseg > 2147483647LL) return GLA_ERR_TOO_LARGE;
    dim3 grid((unsigned)(nblk * batch * nseg)), block(128);
    if (kv_bf16 && nseg > 1)
      rnn_scan_vec4_kernel<bf16, true><<<grid, block, 0, st>>>(T, K, V, nblk, g, (const bf16*)kv, ig, (const bf16*)ikv,
                                                               out_log, (bf16*)out_state, reverse, last_only, nseg, L);
    else if (kv_bf16)
      rnn_scan_vec4_kernel<bf16, false><<<grid, block, 0, st>>>(T, K, V, nblk, g, (const bf16*)kv, ig, (const bf16*)ikv,
                                                                out_log, (bf16*)out_state, reverse, last_only, 1, T);
    else if (nseg > 1)
      rnn_scan_vec4_kernel<float, true><<<grid, block, 0, st>>>(T, K, V, nblk, g, (const float*)kv, ig, (const float*)ikv,
                                                                out_log, (float*)out_state, reverse, last_only, nseg, L);
    else
      rnn_scan_vec4_kernel<float, false><<<grid, block, 0, st>>>(T, K, V, nblk, g, (const float*)kv, ig, (const float*)ikv,
                                                                 out_log, (float*)out_state, reverse, last_only, 1, T);
    GLA_CHECK_LAUNCH();
    if (nseg > 1) {
      float* wsL = ws;
      float* wsS = ws + batch * nseg * K;      // batch * nseg * K floats: a multiple of 16 bytes when K % 4 == 0
      if ((batch * nseg * K) % 4 != 0) wsS += 4 - (batch * nseg * K) % 4;
      const int64_t nfix = batch * (T - L) * K * (V / 4), nlog = batch * (T - L) * K;
      if ((nfix + 255) / 256 > 2147483647LL) return GLA_ERR_TOO_LARGE;
      if (kv_bf16) {
        rnn_carry_kernel<bf16><<<(unsigned)(nblk * batch), 128, 0, st>>>(T, K, V, nblk, nseg, L, out_log, (const bf16*)out_state, wsL, wsS, reverse);
        rnn_fix_kernel<bf16><<<(unsigned)((nfix + 255) / 256), 256, 0, st>>>(batch, T, K, V, nseg, L, out_log, (bf16*)out_state, wsS, reverse);
      } else {
        rnn_carry_kernel<float><<<(unsigned)(nblk * batch), 128, 0, st>>>(T, K, V, nblk, nseg, L, out_log, (const float*)out_state, wsL, wsS, reverse);
        rnn_fix_kernel<float><<<(unsigned)((nfix + 255) / 256), 256, 0, st>>>(batch, T, K, V, nseg, L, out_log, (float*)out_state, wsS, reverse);
      }
      rnn_fix_log_kernel<<<(unsigned)((nlog + 255) / 256), 256, 0, st>>>(batch, T, K, nseg, L, out_log, wsL, reverse);
      GLA_CHECK_LAUNCH();
    }
    return GLA_OK;
  }
  int64_t nblk = (K * V + 255) / 256;
  if (nblk * batch > 2147483647LL) return GLA_ERR_TOO_LARGE;
  dim3 grid((unsigned)(nblk * batch)), block(256);
  if (kv_bf16)
    rnn_scan_kernel<bf16><<<grid, block, 0, st>>>(T, K, V, nblk, g, (const bf16*)kv, ig, (const bf16*)ikv,
                                                  out_log, (bf16*)out_state, reverse, last_only);
  else
    rnn_scan_kernel<float><<<grid, block, 0, st>>>(T, K, V, nblk, g, (const float*)kv, ig, (const float*)ikv,
                                                   out_log, (float*)out_state, reverse, last_only);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

// ---------------------------------------------------------------------------------------
// State scan over chunks (the D x D recurrence of the chunk algorithm, gla.py:711-723 and
// its mirror gla.py:759-771).  Four consecutive value-columns per thread; sequential over
// the N chunks; writes the state BEFORE each update ("exclusive") and the final state.
// ---------------------------------------------------------------------------------------
template <typename TX, typename TI, typename TB, typename TF>
__global__ void __launch_bounds__(256) state_scan_kernel(int64_t N, int64_t D, int64_t nblk,
                                                         const float* __restrict__ G, const TX* X,
                                                         const TI* __restrict__ init, TB* before,
                                                         TF* __restrict__ final_state, int reverse) {
  const int64_t bh = blockIdx.x / nblk;
  const int64_t e = ((blockIdx.x % nblk) * 256 + threadIdx.x) * 4;
  const int64_t DD = D * D;
  if (e >= DD) return;
  const int64_t dk = e / D;
  float s[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) s[i] = init ? ld_f(init, bh * DD + e + i) : 0.f;
  const float* gp = G + bh * N * D + dk;
  const TX* xp = X + bh * N * DD + e;
  TB* bp = before ? before + bh * N * DD + e : nullptr;
#pragma unroll 2
  for (int64_t i = 0; i < N; ++i) {
    const int64_t n = reverse ? (N - 1 - i) : i;
    const float f = expf(gp[n * D]);
    float x[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = ld_f(xp, n * DD + j);
    if (bp) {
#pragma unroll
      for (int j = 0; j < 4; ++j) st_f(bp, n * DD + j, s[j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j] = f * s[j] + x[j];
  }
  if (final_state) {
#pragma unroll
    for (int j = 0; j < 4; ++j) st_f(final_state, bh * DD + e + j, s[j]);
  }
}

template <typename TX, typename TI, typename TB>
static int state_scan_dispatch_final(cudaStream_t st, dim3 grid, int64_t N, int64_t D, int64_t nblk, const float* G,
                                     const void* X, const void* init, void* before, void* fin, int final_bf16,
                                     int reverse) {
  if (final_bf16)
    state_scan_kernel<TX, TI, TB, bf16><<<grid, 256, 0, st>>>(N, D, nblk, G, (const TX*)X, (const TI*)init,
                                                              (TB*)before, (bf16*)fin, reverse);
  else
    state_scan_kernel<TX, TI, TB, float><<<grid, 256, 0, st>>>(N, D, nblk, G, (const TX*)X, (const TI*)init,
                                                               (TB*)before, (float*)fin, reverse);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

int launch_state_scan(cudaStream_t st, int64_t BH, int64_t N, int64_t D, const float* G, const void* X,
                      int x_bf16, const void* init, int init_bf16, void* before, int before_bf16,
                      void* final_state, int final_bf16, int reverse) {
  if (x_bf16) return GLA_ERR_UNSUPPORTED;   // chunk products are always kept in float32
  int64_t nblk = (D * D / 4 + 255) / 256;
  dim3 grid((unsigned)(nblk * BH));
  ProfScope ps("state_scan_kernel", st);
  if (init_bf16) {
    if (before_bf16)
      return state_scan_dispatch_final<float, bf16, bf16>(st, grid, N, D, nblk, G, X, init, before, final_state, final_bf16, reverse);
    return state_scan_dispatch_final<float, bf16, float>(st, grid, N, D, nblk, G, X, init, before, final_state, final_bf16, reverse);
  }
  if (before_bf16)
    return state_scan_dispatch_final<float, float, bf16>(st, grid, N, D, nblk, G, X, init, before, final_state, final_bf16, reverse);
  return state_scan_dispatch_final<float, float, float>(st, grid, N, D, nblk, G, X, init, before, final_state, final_bf16, reverse);
}

// ---------------------------------------------------------------------------------------
// Cross-rank combine for sequence parallelism: an exclusive decayed scan over ranks of the
// per-rank (total log decay, local state) pairs, evaluated for one rank.
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) sp_combine_kernel(int64_t R, int64_t rank, int64_t BH, int64_t D,
                                                         const float* __restrict__ all_G,
                                                         const float* __restrict__ all_S,
                                                         const TI* __restrict__ init, TO* __restrict__ result,
                                                         int reverse) {
  const int64_t DD = D * D;
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= BH * DD) return;
  const int64_t bh = e / DD, dk = (e % DD) / D;
  float acc = init ? ld_f(init, e) : 0.f;
  if (!reverse) {
    for (int64_t s = 0; s < rank; ++s)
      acc = expf(all_G[(s * BH + bh) * D + dk]) * acc + all_S[s * BH * DD + e];
  } else {
    for (int64_t s = R - 1; s > rank; --s)
      acc = expf(all_G[(s * BH + bh) * D + dk]) * acc + all_S[s * BH * DD + e];
  }
  st_f(result, e, acc);
}

// Both results a rank needs from the gathered pairs in one launch: the state entering its slice (float32, for the
// correction of its stored states) and the state leaving the last slice in scan order (the whole sequence's
// hidden_final, or dhidden_init in the reverse direction).  The pairs may sit in one packed record per rank (what
// a single all-gather of [G | S] gives): gstride / sstride are the distances between ranks in floats.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) sp_combine2_kernel(int64_t R, int64_t rank, int64_t BH, int64_t D,
                                                          const float* __restrict__ all_G, int64_t gstride,
                                                          const float* __restrict__ all_S, int64_t sstride,
                                                          const TI* __restrict__ init, float* __restrict__ entering,
                                                          TO* __restrict__ total, int reverse) {
  const int64_t DD = D * D;
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= BH * DD) return;
  const int64_t bh = e / DD, dk = (e % DD) / D;
  float acc = init ? ld_f(init, e) : 0.f;
  for (int64_t i = 0; i < R; ++i) {
    const int64_t s = reverse ? R - 1 - i : i;
    if (s == rank && entering != nullptr) entering[e] = acc;
    acc = expf(all_G[s * gstride + bh * D + dk]) * acc + all_S[s * sstride + e];
  }
  if (total != nullptr) st_f(total, e, acc);
}

int launch_sp_combine2(cudaStream_t st, int64_t R, int64_t rank, int64_t BH, int64_t D, const float* all_G, int64_t gstride,
                       const float* all_S, int64_t sstride, const void* init, int init_bf16, float* entering, void* total,
                       int total_bf16, int reverse) {
  const int64_t n = BH * D * D;
  dim3 grid((unsigned)((n + 255) / 256));
  ProfScope ps("sp_combine_kernel", st);
  if (init_bf16 && total_bf16)
    sp_combine2_kernel<bf16, bf16><<<grid, 256, 0, st>>>(R, rank, BH, D, all_G, gstride, all_S, sstride, (const bf16*)init, entering, (bf16*)total, reverse);
  else if (init_bf16 && !total_bf16)
    sp_combine2_kernel<bf16, float><<<grid, 256, 0, st>>>(R, rank, BH, D, all_G, gstride, all_S, sstride, (const bf16*)init, entering, (float*)total, reverse);
  else if (!init_bf16 && total_bf16)
    sp_combine2_kernel<float, bf16><<<grid, 256, 0, st>>>(R, rank, BH, D, all_G, gstride, all_S, sstride, (const float*)init, entering, (bf16*)total, reverse);
  else
    sp_combine2_kernel<float, float><<<grid, 256, 0, st>>>(R, rank, BH, D, all_G, gstride, all_S, sstride, (const float*)init, entering, (float*)total, reverse);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

int launch_sp_combine(cudaStream_t st, int64_t R, int64_t rank, int64_t BH, int64_t D, const float* all_G,
                      const float* all_S, const void* init, int init_bf16, void* result, int result_bf16,
                      int reverse) {
  int64_t n = BH * D * D;
  dim3 grid((unsigned)((n + 255) / 256));
  ProfScope ps("sp_combine_kernel", st);
  if (init_bf16 && result_bf16)
    sp_combine_kernel<bf16, bf16><<<grid, 256, 0, st>>>(R, rank, BH, D, all_G, all_S, (const bf16*)init, (bf16*)result, reverse);
  else if (init_bf16 && !result_bf16)
    sp_combine_kernel<bf16, float><<<grid, 256, 0, st>>>(R, rank, BH, D, all_G, all_S, (const bf16*)init, (float*)result, reverse);
  else if (!init_bf16 && result_bf16)
    sp_combine_kernel<float, bf16><<<grid, 256, 0, st>>>(R, rank, BH, D, all_G, all_S, (const float*)init, (bf16*)result, reverse);
  else
    sp_combine_kernel<float, float><<<grid, 256, 0, st>>>(R, rank, BH, D, all_G, all_S, (const float*)init, (float*)result, reverse);
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

}  // namespace gla
