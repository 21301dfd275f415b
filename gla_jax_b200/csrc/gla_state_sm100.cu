// Chunk states of chunk_gla in ONE pass: kv products and the recurrence over chunks fused (sm_100a).
//
// Reference: gla.py:705-723 (k_hat^T v per chunk, then the scan S_n = e^{G_n} S_{n-1} + kv_n from
// hidden_init) and gla.py:748-766 (q_hat^T dO per chunk, then the reverse scan of the state
// gradient from dhidden_final).  The two-kernel form (a batched product that writes every chunk's
// float32 kv, then a scan that reads it back) moves 3 x 64 KB per chunk through HBM for what is a
// running sum.  Here the state never leaves the SM:
//
//   * the recurrence is independent per element of S[dk][dv] and its decay depends on dk only, so a
//     thread block owns one (batch, head) and a SLICE of 32 key features dk, and walks the chunks in
//     order with its 32 x 128 piece of S in float32 registers;
//   * per chunk it needs g and k (or q) for its 32 features only (24 KB) plus the whole v (or dO)
//     tile (32 KB); both arrive by TMA through rings (3 and 4 deep), three chunks ahead of use;
//   * per chunk: decay weights as running products of f = exp(g) <= 1 down the rows, k_hat^T stored
//     K-major, ONE tcgen05 product D[dv][dk] = sum_c v[c][dv] k_hat[c][dk] (M 128, N 32, K 128) into
//     one of two TMEM accumulators, then S_prev[n] = S (stored bf16), S = e^G S + D.
//
// The block is a pipeline of warp roles, each a step ahead of the next, so that a step costs the
// slowest role instead of their sum:
//   builders   2 groups x 8 warps; group (i & 1) writes k_hat^T of step i (thread = one feature, 16 rows)
//   issuer     1 warp: the eight MMAs of a step and their completion barrier
//   updaters   8 warps: own the state registers (thread = one dv row of TMEM, 16 features); read the
//              product, store S_prev, apply the decay
//   producer   1 warp: TMA loads into the rings as their stages come free
// Hand-offs: named barriers 3/4 (operand of an even/odd step written: builders arrive, issuer and
// producer wait), mbarriers for TMA arrival, MMA completion, accumulator release and the chunk's e^G.
// The issuer's serial path is kept to the eight MMAs: every wait it would need is taken by the builders
// before they arrive.
//
// MODE 0 walks chunks forward with k_hat = k prod_{t>r} f_t; MODE 1 walks them backward with
// q_hat = q prod_{t<=r} f_t and dO in place of v (the gradient recurrence is the same scan reversed).
// Parallelism is (batch x heads) x 4 blocks, each sequential over T/128 chunks: the caller picks
// this kernel when that beats the two-kernel form (few chunks per head relative to the SM count).
#include "gla_common.cuh"
#include "tc_ptx.cuh"
#include "tma_maps.cuh"
#include <cstdlib>

namespace gla {

using namespace tc;

namespace {

constexpr int SD = 128;          // head dim
constexpr int SC = 128;          // chunk length
constexpr int SL = 32;           // key features per block
constexpr int NBUILD = 512;      // 2 groups x 8 warps
constexpr int NUPD = 256;        // 8 warps
constexpr int STHREADS = NBUILD + NUPD + 64;     // + MMA issuer warp + TMA producer warp
constexpr int READY_COUNT = 256 + 64;            // one builder group + issuer + producer
constexpr int NY = 4, NGX = 3;   // ring depths

// Named barriers: 1/2 = inside builder group 0/1; 3/4 = operand of an even/odd step written.
__device__ __forceinline__ void bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int n) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory"); }

struct StSmem {
  static constexpr uint32_t Y = 0;                          // NY x 32 KB: v / dO tile, two SW128 halves of 128 rows x 64 cols
  static constexpr uint32_t GX = NY * 32768;                // NGX x (16 KB g slice [128][32] float + 8 KB k/q slice [128][32] bf16)
  static constexpr uint32_t GXS = 16384 + 8192;
  static constexpr uint32_t BOP = GX + NGX * GXS;           // 2 x 8 KB: k_hat^T, K-major, two 64-row K blocks (1024-aligned)
  static constexpr uint32_t TOT = BOP + 2 * 8192;           // [2 groups][2][8][32] float: gate products per 16 rows
  static constexpr uint32_t GSUM = TOT + 4 * 8 * SL * 4;    // [2 groups][2][8][32] float: gate sums per 16 rows
  static constexpr uint32_t EG = GSUM + 4 * 8 * SL * 4;     // [4][32] float: e^G of the chunk, by step & 3
  static constexpr uint32_t BAR = EG + 4 * SL * 4;          // fully[NY], fullgx[NGX], mma[2], accfree[2], egbar[4], yfree[NY], tmem slot
  static constexpr uint32_t END = BAR + 192;
};
static_assert(StSmem::BOP % 1024 == 0, "operand buffers need 1024-byte alignment");
constexpr size_t ST_SMEM = 1024 + StSmem::END;
static_assert(ST_SMEM <= 232448, "shared memory budget");

__device__ unsigned int g_state_wait_timeouts = 0;
__device__ unsigned int g_state_bad_offsets = 0;      // packed sequences whose offsets had to be clamped

struct StMaps { CUtensorMap g, x, y; };

template <int MODE>
__global__ void __launch_bounds__(STHREADS, 1)
tc_state_kernel(const __grid_constant__ StMaps maps, int64_t T, int64_t H, int R, int Nall, const int* __restrict__ cu,
                const bf16* __restrict__ init, bf16* __restrict__ states, bf16* __restrict__ fin, float* __restrict__ fin32,
                float* __restrict__ Gc, unsigned int* __restrict__ done, int nsegs) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* tot = reinterpret_cast<float*>(sm + StSmem::TOT);
  float* gsum = reinterpret_cast<float*>(sm + StSmem::GSUM);
  float* eG = reinterpret_cast<float*>(sm + StSmem::EG);
  uint64_t* fully = reinterpret_cast<uint64_t*>(sm + StSmem::BAR);
  uint64_t* fullgx = fully + NY;
  uint64_t* mma = fullgx + NGX;
  uint64_t* accfree = mma + 2;
  uint64_t* egbar = accfree + 2;
  uint64_t* yfree = egbar + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(yfree + NY);
  static_assert((NY + NGX + 2 + 2 + 4 + NY) * 8 + 8 <= 192, "barriers and the TMEM slot must fit the space reserved at StSmem::BAR");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slice = blockIdx.x & 3;
  // H counts VIRTUAL heads: a head of size 128 R is R x R independent (key block a, value block c) problems of size
  // 128, virtual head hh = (h R + a) R + c; in the (B, T, H_real R, 128) view of the arrays its key-side tensors are
  // head h R + a and its value-side tensors head h R + c.  R = 1: all three coincide.
  // Packed sequences (cu != null): the arrays hold ONE time axis (B = 1) with sequences laid end to end, cu[s] the
  // token offset of sequence s (a multiple of 128); blockIdx then ranges over (sequence, head, slice), the block
  // walks only its sequence's chunks, and init / fin are per (sequence, head).
  // Segments (nsegs > 1, dense batches only): the chunks of every (batch, head) are cut into nsegs runs of equal
  // length that are walked by separate blocks, each from a zero state except the first in walk order, which starts
  // from init; every run leaves its final state, unrounded, in fin32[(bh, segment)].  The recurrence is linear in
  // its starting state, so the caller corrects the stored states afterwards (seg_fix_states in the chunk file);
  // what this buys is nsegs times as many blocks for shapes with few heads and many chunks.
  const int seg = nsegs > 1 ? (int)((blockIdx.x >> 2) % nsegs) : 0;
  const int64_t bh = nsegs > 1 ? (blockIdx.x >> 2) / nsegs : blockIdx.x >> 2, hh = bh % H;
  const int64_t b = cu ? 0 : bh / H;
  // Offsets come from device memory nobody has validated: whatever they hold, this block only touches chunks
  // [base, base + N) inside [0, Nall).  Offsets that are not rising multiples of the chunk length inside the
  // array are clamped (the sequence is cut short or skipped) and counted in g_state_bad_offsets.
  int base = 0, N = Nall;
  if (cu) {
    const int lo = cu[bh / H], hi = cu[bh / H + 1];
    base = min(max(lo / SC, 0), Nall);
    N = min(max((hi - lo) / SC, 0), Nall - base);
    const bool bad = lo < 0 || hi < lo || lo % SC != 0 || hi % SC != 0 || hi / SC > Nall;
    if (bad && tid == 0 && slice == 0) atomicAdd(&g_state_bad_offsets, 1u);
  } else if (nsegs > 1) {
    const int Ns = (Nall + nsegs - 1) / nsegs;
    base = min(seg * Ns, Nall);
    N = min(Ns, Nall - base);
    if (seg != (MODE == 0 ? 0 : nsegs - 1)) init = nullptr;
    fin = nullptr;                                                // the caller combines the runs' final states
    fin32 += ((bh * nsegs + seg) - bh) * (int64_t)SD * SD;        // the element offsets below start at bh * SD * SD
  }
  const int64_t rowbase = cu ? hh * (int64_t)Nall + base : bh * (int64_t)Nall + base;   // row of chunk 0 in states / Gc
  const int64_t hk = (hh / (R * R)) * R + (hh % (R * R)) / R, hv = (hh / (R * R)) * R + hh % R;
  auto chunk_of = [&](int i) { return MODE == 0 ? i : N - 1 - i; };

  // `done` (optional): a counter in global memory that every block bumps once its states are written.  The
  // consumer kernel may then be launched as a programmatic dependent of this grid: it starts on the SMs this
  // grid leaves idle (4 x batch x heads blocks), does the part of its work that needs no state, and reads the
  // counter before it loads one.  Letting dependents go at once is safe: nothing here reads what they write.
  if (done != nullptr && tid == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tid == NBUILD + NUPD) {
    for (int s = 0; s < NY; ++s) mbar_init(smem_u32(fully + s), 1);
    for (int s = 0; s < NY; ++s) mbar_init(smem_u32(yfree + s), 1);
    for (int s = 0; s < NGX; ++s) mbar_init(smem_u32(fullgx + s), 1);
    mbar_init(smem_u32(mma + 0), 1);
    mbar_init(smem_u32(mma + 1), 1);
    mbar_init(smem_u32(accfree + 0), NUPD);
    mbar_init(smem_u32(accfree + 1), NUPD);
    for (int s = 0; s < 4; ++s) mbar_init(smem_u32(egbar + s), 32);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool ok = true;

  if (warp == (NBUILD + NUPD) / 32 + 1) {
    // ================= TMA producer warp =================
    const int z0 = (int)(b * T) + base * SC, yk = (int)hk, yv = (int)hv;
    const int zstep = MODE == 0 ? SC : -SC;
    const uint32_t sm_base = smem_u32(sm), fully0 = smem_u32(fully), fullgx0 = smem_u32(fullgx);
    auto load_y = [&](int z, int s) {
      const uint32_t dst = sm_base + StSmem::Y + s * 32768, fb = fully0 + 8 * s;
      mbar_arrive_expect_tx(fb, 32768);
      tma_load_3d(dst, &maps.y, 0, yv, z, fb);
      tma_load_3d(dst + 16384, &maps.y, 64, yv, z, fb);
    };
    auto load_gx = [&](int z, int s) {
      const uint32_t dst = sm_base + StSmem::GX + s * StSmem::GXS, fb = fullgx0 + 8 * s;
      mbar_arrive_expect_tx(fb, StSmem::GXS);
      tma_load_3d(dst, &maps.g, SL * slice, yk, z, fb);
      tma_load_3d(dst + 16384, &maps.x, SL * slice, yk, z, fb);
    };
    const int zfirst = z0 + chunk_of(0) * SC;
    if (lane == 0) {
      for (int i = 0; i < NGX && i < N; ++i) load_gx(zfirst + i * zstep, i);
      for (int i = 0; i < NY && i < N; ++i) load_y(zfirst + i * zstep, i);
    }
    int zgx = zfirst + NGX * zstep, sgx = 0;      // next g / k slice load: step j + NGX into ring stage j % NGX
    int zy = zfirst + NY * zstep, sy = 0;         // next tile load: step j - 1 + NY into ring stage (j - 1) % NY
    for (int j = 0; j < N; ++j) {
      const int g = j & 1;
      bar_sync(3 + g, READY_COUNT);          // operand of step j written: its g / k slices are consumed
      if (lane == 0) {
        if (j + NGX < N) load_gx(zgx, sgx);
        // the product of step j-1 has completed (or is about to): its tile stage takes step j-1+NY.  The wait is on
        // the STAGE's own barrier (the issuer commits every product to it as well): its next completion needs the
        // tile this thread is about to request, so the phase waited for cannot be overtaken.  (mma[g] also completes
        // for step j+1 without this thread's help; a parity wait on it that wakes late would miss a phase.)
        if (j >= 1 && j - 1 + NY < N) {
          if (ok) ok = mbar_wait(smem_u32(yfree + sy), (uint32_t)(((j - 1) / NY) & 1));
          load_y(zy, sy);
        }
      }
      zgx += zstep; sgx = sgx == NGX - 1 ? 0 : sgx + 1;
      if (j >= 1) { zy += zstep; sy = sy == NY - 1 ? 0 : sy + 1; }
      __syncwarp();
    }
    if (!ok && lane == 0) atomicAdd(&g_state_wait_timeouts, 1u);
  } else if (warp == (NBUILD + NUPD) / 32) {
    // ================= MMA issuer warp =================
    const uint32_t sm_base = smem_u32(sm);
    const uint64_t dB0 = desc_kmajor(sm_base + StSmem::BOP, 4096, 0), dB1 = desc_kmajor(sm_base + StSmem::BOP + 8192, 4096, 0);
    const uint64_t dY0 = desc_mnmajor(sm_base + StSmem::Y, 16384, 0);
    int ys = 0;                              // j % NY
    for (int j = 0; j < N; ++j) {
      const int g = j & 1;
      bar_sync(3 + g, READY_COUNT);          // operand of step j written
      if (lane == 0) {
        // No waits here: the builders held back their arrival until the v / dO tile of this step had landed
        // and the updaters had read accumulator g out, so this warp's serial path is the eight MMAs.
        tc_fence_after();
        constexpr uint32_t idesc = idesc_bf16(128, SL, 1, 0);
        const uint64_t a0 = desc_advance(dY0, (uint32_t)ys * 32768u), b0 = g ? dB1 : dB0;
        const uint32_t acc = tmem + SL * g;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)       // D[dv][dk] = sum_c y[c][dv] x_hat[c][dk]
          umma_bf16(acc, desc_advance(a0, ks * 2048), desc_advance(b0, (ks >> 2) * 4096 + (ks & 3) * 32), idesc, ks > 0);
        umma_commit(smem_u32(mma + g));
        umma_commit(smem_u32(yfree + ys));      // the tile stage of this step may be refilled
      }
      ys = ys == NY - 1 ? 0 : ys + 1;
      __syncwarp();
    }
    if (!ok && lane == 0) atomicAdd(&g_state_wait_timeouts, 1u);
  } else if (warp < NBUILD / 32) {
    // ================= builders: group g writes the operand of steps i = g, g+2, ... =================
    const int g = warp >> 3, w = warp & 7;           // thread: feature `lane` of the slice, rows 16 w + [0, 16)
    for (int i = g; i < N; i += 2) {
      const int s = i % NGX;
      // The product of step i-2 has completed: operand buffer g is free, and (through the accumulator
      // release the issuer waited for before step i-2) the updaters are done with the e^G slot of step i-4.
      if (i >= 2 && ok) ok = mbar_wait(smem_u32(mma + g), (uint32_t)(((i - 2) >> 1) & 1));
      float* tt = tot + (2 * g + ((i >> 1) & 1)) * 8 * SL;      // double-buffered: a warp a step ahead never
      float* gg = gsum + (2 * g + ((i >> 1) & 1)) * 8 * SL;     // overwrites what a slower warp still reads
      if (ok) ok = mbar_wait(smem_u32(fullgx + s), (uint32_t)((i / NGX) & 1));
      const float* gt = reinterpret_cast<const float*>(sm + StSmem::GX + s * StSmem::GXS);
      const unsigned short* xt = reinterpret_cast<const unsigned short*>(sm + StSmem::GX + s * StSmem::GXS + 16384);
      const int r0 = 16 * w;
      float f[16];
      uint32_t xr[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        f[j] = gt[(r0 + j) * SL + lane];
        xr[j] = xt[(r0 + j) * SL + lane];
      }
      // The product of the 16 gates first (as the exponential of their sum), so that the groups can exchange
      // totals early and the running products below start from the cross-group factor.
      float gs = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) gs += f[j];
      tt[w * SL + lane] = __expf(gs);
      if (MODE == 0) gg[w * SL + lane] = gs;
      bar_sync(1 + g, 256);
      float tw[8];
#pragma unroll
      for (int w2 = 0; w2 < 8; ++w2) tw[w2] = tt[w2 * SL + lane];
      float run = 1.f;
#pragma unroll
      for (int w2 = 0; w2 < 8; ++w2) {
        const bool use = (MODE == 0) ? (w2 > w) : (w2 < w);
        run *= use ? tw[w2] : 1.f;
      }
      if (w == (MODE == 0 ? 7 : 0)) {           // chunk totals of the slice's features
        float e = 1.f, sg = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 8; ++w2) { e *= tw[w2]; if (MODE == 0) sg += gg[w2 * SL + lane]; }
        eG[(i & 3) * SL + lane] = e;
        mbar_arrive(smem_u32(egbar + (i & 3)));       // release: the updaters acquire it before reading e^G
        if (MODE == 0 && Gc != nullptr) Gc[(rowbase + chunk_of(i)) * SD + SL * slice + lane] = sg;
      }
      // weights by running product from the cross-group factor, applied on the fly
      float v[16];
      if (MODE == 0) {
#pragma unroll
        for (int j = 15; j >= 0; --j) { v[j] = __uint_as_float(xr[j] << 16) * run; run *= __expf(f[j]); }   // exclusive suffix
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) { run *= __expf(f[j]); v[j] = __uint_as_float(xr[j] << 16) * run; }    // inclusive prefix
      }
      uint32_t pk[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
      // row = feature (the N index); 64 chunk rows per 128-byte line; this thread's 16 rows = two 16-byte pieces
      uint8_t* bop = sm + StSmem::BOP + g * 8192 + (w >> 2) * 4096;
      *reinterpret_cast<uint4*>(bop + sw128_chunk(lane, 2 * (w & 3))) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      *reinterpret_cast<uint4*>(bop + sw128_chunk(lane, 2 * (w & 3) + 1)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      fence_async_smem();
      // on behalf of the issuer (these have long completed as a rule): accumulator g read out by the updaters
      // (step i-2), and the v / dO tile of step i landed.  The issuer goes once ALL warps of the group have arrived,
      // so one warp checking each condition before its own arrival is enough; even a completed mbarrier costs a
      // wait some 300 cycles, and the builders' serial path is what paces the kernel (measured with clock stamps).
      if (w == 0 && i >= 2 && ok) ok = mbar_wait(smem_u32(accfree + g), (uint32_t)(((i - 2) >> 1) & 1));
      if (w == 1 && ok) ok = mbar_wait(smem_u32(fully + (i % NY)), (uint32_t)((i / NY) & 1));
      bar_arrive(3 + g, READY_COUNT);
    }
    if (!ok && lane == 0) atomicAdd(&g_state_wait_timeouts, 1u);
  } else {
    // ================= updaters: the state registers =================
    // TMEM lane = dv; this thread's 16 columns = key features 16 cg + [0, 16) of the slice
    const int e8 = warp - NBUILD / 32;
    const int q4 = e8 & 3, cg = e8 >> 2;            // (warp % 4) == q4: the TMEM lanes this warp may read
    const int dv = 32 * q4 + lane;
    const int64_t el0 = ((bh * SD) + SL * slice + 16 * cg) * SD + dv;     // element (bh, dk0, dv); dk stride SD
    float S[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) S[j] = init ? __bfloat162float(init[el0 + (int64_t)j * SD]) : 0.f;
    for (int i = 0; i < N; ++i) {
      const int g = i & 1;
      if (ok) ok = mbar_wait(smem_u32(egbar + (i & 3)), (uint32_t)((i >> 2) & 1));     // e^G of step i written
      float e[16];
#pragma unroll
      for (int j4 = 0; j4 < 4; ++j4) {          // 16 consecutive floats, 64-byte aligned: four 16-byte loads
        const float4 t = *reinterpret_cast<const float4*>(eG + (i & 3) * SL + 16 * cg + 4 * j4);
        e[4 * j4] = t.x; e[4 * j4 + 1] = t.y; e[4 * j4 + 2] = t.z; e[4 * j4 + 3] = t.w;
      }
      if (ok) ok = mbar_wait(smem_u32(mma + g), (uint32_t)((i >> 1) & 1));
      tc_fence_after();
      uint32_t r[16];
      tmem_ld16(tmem + ((uint32_t)(q4 * 32) << 16) + SL * g + 16 * cg, r);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(accfree + g));    // accumulator g may be overwritten by step i + 2
      bf16* so = states + (rowbase + chunk_of(i)) * SD * SD + (el0 - bh * SD * SD);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        so[(int64_t)j * SD] = __float2bfloat16_rn(S[j]);
        S[j] = fmaf(e[j], S[j], __uint_as_float(r[j]));
      }
    }
    if (fin != nullptr) {
#pragma unroll
      for (int j = 0; j < 16; ++j) fin[el0 + (int64_t)j * SD] = __float2bfloat16_rn(S[j]);
    }
    if (fin32 != nullptr) {          // the unrounded state, for the exchange between sequence-parallel ranks
#pragma unroll
      for (int j = 0; j < 16; ++j) fin32[el0 + (int64_t)j * SD] = S[j];
    }
    if (!ok && lane == 0) atomicAdd(&g_state_wait_timeouts, 1u);
  }
  tc_fence_before();
  __syncthreads();
  if (done != nullptr && tid == 0) {       // the block's stores are ordered before the bump (barrier, then a device-scope fence)
    __threadfence();
    atomicAdd(done, 1u);
  }
  if (warp == 1) tmem_dealloc(tmem, 64);
}

}  // namespace

unsigned int tc_state_read_wait_timeouts() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_state_wait_timeouts, sizeof(v));
  return v;
}
unsigned int tc_state_read_bad_offsets() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_state_bad_offsets, sizeof(v));
  return v;
}

// Whether the one-pass kernel is expected to beat the product + scan pair for this shape.
// Its time is (waves of (B*H*4) blocks over the SMs) x N sequential steps; the pair's time grows with
// the total number of chunks.  Step and per-chunk costs measured on B200; the caller's option bits
// GLA_OPT_STATE_ONE_PASS / GLA_OPT_STATE_TWO_KERNELS override the estimate.
static int sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    sms[dev] = n;
  }
  return sms[dev];
}
bool tc_state_fused_preferred(int64_t BH, int64_t N, int opts) {
  if (opts & GLA_OPT_STATE_ONE_PASS) return true;
  if (opts & GLA_OPT_STATE_TWO_KERNELS) return false;
  const int sms = sm_count();
  if (tc_state_segments(BH, N, opts) > 1) return true;          // runs make the one-pass form the better one
  const double waves = (double)((4 * BH + sms - 1) / sms);
  const double t_fused = waves * (double)N * 1.0 + 8.0;          // us
  const double t_pair = (double)(BH * N) * 0.1 + 10.0;           // us
  return t_fused < t_pair;
}

// How many runs to cut every head's chunks into for the one-pass kernel (1: none).  A run costs its chunks in
// sequence, the grid costs its waves over the SMs, and cutting adds a correction pass over the stored states
// (read + write, 64 KB per chunk-head) plus three small launches; runs shorter than four chunks are not worth it.
// The option bit GLA_OPT_STATE_SEGMENTS forces runs (four, or two below 16 chunks, none below 8) for any shape.
int tc_state_segments(int64_t BH, int64_t N, int opts) {
  // the runs must all be non-empty: with ns chunks per run, ceil(N / ns) runs cover the axis
  auto whole_runs = [&](int64_t c) { const int64_t ns = (N + c - 1) / c; return (int)((N + ns - 1) / ns); };
  if (opts & GLA_OPT_STATE_TWO_KERNELS) return 1;
  if (opts & GLA_OPT_STATE_SEGMENTS) return N >= 16 ? whole_runs(4) : N >= 8 ? 2 : 1;    // at most N / 4 runs
  if (opts & GLA_OPT_STATE_ONE_PASS) return 1;
  const int sms = sm_count();
  auto cost = [&](int64_t nsegs) {
    const int64_t waves = (4 * BH * nsegs + sms - 1) / sms, ns = (N + nsegs - 1) / nsegs;
    double t = (double)waves * ((double)ns * 1.25 + 3.0) + 8.0;       // a block: its steps plus start-up
    // correction pass over the stored states, three small launches, the sequential walks over a run's chunks and over
    // the runs (whose final states, 64 KB per head and run, are written, read and turned into corrections)
    if (nsegs > 1) t += (double)(BH * N) * 0.015 + 30.0 + (double)ns * 0.2 + (double)nsegs * ((double)BH * 0.03 + 0.5);
    return t;
  };
  int64_t best = 1;
  double tb = cost(1);
  for (int64_t c = 2; c <= N / 4 && c <= 512; ++c) {
    const double t = cost(c);
    if (t < tb) { tb = t; best = c; }
  }
  best = whole_runs(best);
  return cost(best) < 0.8 * cost(1) ? (int)best : 1;
}

// H counts virtual heads of size 128 (real heads x R x R for head size 128 R; init/states/fin are laid out per
// virtual head as 128 x 128 tiles).
// mode 0: states[n] = state before chunk n (from init), fin = state after the last chunk, Gc = chunk gate sums.
// mode 1: states[n] = gradient state after chunk n (from init = dhidden_final), fin = dhidden_init.
int tc_state_fused(cudaStream_t st, int mode, int64_t B, int64_t T, int64_t H, int R, const float* g, const void* x,
                   const void* y, const void* init, void* states, void* fin, float* Gc, int64_t nseq, const int* cu,
                   unsigned int* done, unsigned int* done_target, float* fin32, int nsegs) {
  if (nsegs < 1 || (nsegs > 1 && (cu != nullptr || fin32 == nullptr || done != nullptr || nsegs > T / SC))) return GLA_ERR_UNSUPPORTED;
  // packed sequences: B == 1, cu (device, nseq + 1 token offsets) non-null, init / fin are (nseq, H, 128, 128)
  const int64_t N = T / SC, BH = (cu ? nseq : B) * H;          // H: virtual heads (real heads x R x R)
  const int64_t HK = H / R;                      // heads of the (B, T, HK, 128) view of the arrays
  StMaps maps;
  GLA_TRY(make_map_bthd(&maps.g, g, 1, B, T, HK, SL, 0));
  GLA_TRY(make_map_bthd(&maps.x, x, 0, B, T, HK, SL, 0));
  GLA_TRY(make_map_bthd(&maps.y, y, 0, B, T, HK, 64, 1));
  auto kern = mode == 0 ? tc_state_kernel<0> : tc_state_kernel<1>;
  static SmemAttrOnce attr[2];
  GLA_TRY(attr[mode != 0].ensure(kern, ST_SMEM));
  cudaError_t e;
  if (done != nullptr) {
    e = cudaMemsetAsync(done, 0, sizeof(unsigned int), st);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (done_target) *done_target = (unsigned int)(BH * 4);
  }
  {
    ProfScope ps(mode == 0 ? "tc_state_kernel" : "tc_dstate_scan_kernel", st);
    if (BH * 4 * nsegs > 2147483647LL) return GLA_ERR_TOO_LARGE;
    kern<<<(unsigned)(BH * 4 * nsegs), STHREADS, ST_SMEM, st>>>(maps, T, H, R, (int)N, cu, (const bf16*)init, (bf16*)states,
                                                                (bf16*)fin, fin32, Gc, done, nsegs);
  }
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

}  // namespace gla
