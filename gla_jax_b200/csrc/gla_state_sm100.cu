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
//     tile (32 KB); all of it arrives by TMA through a 3-stage ring, two chunks ahead of use;
//   * per chunk: decay weights as running products of f = exp(g) <= 1 down the rows, k_hat^T stored
//     K-major, ONE tcgen05 product D[dv][dk] = sum_c v[c][dv] k_hat[c][dk] (M 128, N 32, K 128) into
//     one of two TMEM accumulators, then S_prev[n] = S (stored bf16), S = e^G S + D;
//   * the product of chunk n+1 is built and issued before the state update of chunk n is done, so
//     the tensor core, the TMA engine and the update overlap.
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
constexpr int SWORKERS = 512;    // 16 warps: operand build and state update
constexpr int STHREADS = SWORKERS + 32;   // + 1 warp: TMA producer and MMA issuer
constexpr int NSTAGE = 3;

// Named barriers: 1 = among the worker warps; 2 = workers arrive (operand written), issuer waits.
__device__ __forceinline__ void bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int n) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory"); }

struct StSmem {
  static constexpr uint32_t Y = 0;                       // v / dO tile: two SW128 halves of 128 rows x 64 cols
  static constexpr uint32_t G = 2 * 16384;               // g slice  [128][32] float
  static constexpr uint32_t X = G + 16384;               // k / q slice [128][32] bf16
  static constexpr uint32_t STAGE = X + 8192;            // 56 KB, a multiple of 1024
  static constexpr uint32_t BOP = NSTAGE * STAGE;        // 2 x 8 KB: k_hat^T, K-major, two 64-row K blocks
  static constexpr uint32_t TOT = BOP + 2 * 8192;        // [2][16][32] float: gate products per 8 rows
  static constexpr uint32_t GSUM = TOT + 2 * 16 * SL * 4;  // [2][16][32] float: gate sums per 8 rows
  static constexpr uint32_t EG = GSUM + 2 * 16 * SL * 4;   // [2][32] float: e^G of the chunk
  static constexpr uint32_t BAR = EG + 2 * SL * 4;       // full[3], mma[2], tmem slot
  static constexpr uint32_t END = BAR + 64;
};
constexpr size_t ST_SMEM = 1024 + StSmem::END;

__device__ unsigned int g_state_wait_timeouts = 0;

struct StMaps { CUtensorMap g, x, y; };
#ifdef ST_TRACE
__device__ long long g_st_trace[4][16];
#define ST_STAMP(k) do { if (blockIdx.x == 40 && i == 10 && lane == 0 && (warp == 0 || warp == 7 || warp == 15)) g_st_trace[warp == 0 ? 0 : warp == 7 ? 1 : 2][k] = clock64(); } while (0)
#define ST_STAMP_I(k) do { if (blockIdx.x == 40 && j == 10 && lane == 0) g_st_trace[3][k] = clock64(); } while (0)
#else
#define ST_STAMP(k)
#define ST_STAMP_I(k)
#endif

template <int MODE>
__global__ void __launch_bounds__(STHREADS, 1)
tc_state_kernel(const __grid_constant__ StMaps maps, int64_t T, int64_t H, int N, const bf16* __restrict__ init,
                bf16* __restrict__ states, bf16* __restrict__ fin, float* __restrict__ Gc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* tot = reinterpret_cast<float*>(sm + StSmem::TOT);
  float* gsum = reinterpret_cast<float*>(sm + StSmem::GSUM);
  float* eG = reinterpret_cast<float*>(sm + StSmem::EG);
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + StSmem::BAR);
  uint64_t* mma = full + NSTAGE;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slice = blockIdx.x & 3;
  const int64_t bh = blockIdx.x >> 2, b = bh / H, h = bh % H;

  auto chunk_of = [&](int i) { return MODE == 0 ? i : N - 1 - i; };
  const int z0 = (int)(b * T), y = (int)h;
  const uint32_t sm_base = smem_u32(sm), full_base = smem_u32(full);
  auto issue_loads = [&](int i) {           // one thread: chunk of step i into ring stage i % NSTAGE
    const int sidx = i % NSTAGE;
    const uint32_t st = sm_base + sidx * StSmem::STAGE, fb = full_base + sidx * 8;
    const int z = z0 + chunk_of(i) * SC;
    mbar_arrive_expect_tx(fb, StSmem::STAGE);
    tma_load_3d(st + StSmem::Y, &maps.y, 0, y, z, fb);
    tma_load_3d(st + StSmem::Y + 16384, &maps.y, 64, y, z, fb);
    tma_load_3d(st + StSmem::G, &maps.g, SL * slice, y, z, fb);
    tma_load_3d(st + StSmem::X, &maps.x, SL * slice, y, z, fb);
  };

  if (tid == SWORKERS) {
    for (int s = 0; s < NSTAGE; ++s) mbar_init(smem_u32(full + s), 1);
    mbar_init(smem_u32(mma + 0), 1);
    mbar_init(smem_u32(mma + 1), 1);
    mbar_fence_init();
    for (int i = 0; i < NSTAGE && i < N; ++i) issue_loads(i);
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

  if (warp == SWORKERS / 32) {
    // ---- issuer warp: product of step j as soon as its operand is written ------------------------------
    // descriptors of the two operands at K slice 0, per ring stage / operand buffer; later slices by desc_advance
    uint64_t dY[NSTAGE], dB[2];
#pragma unroll
    for (int s = 0; s < NSTAGE; ++s) dY[s] = desc_mnmajor(smem_u32(sm + s * StSmem::STAGE + StSmem::Y), 16384, 0);
    dB[0] = desc_kmajor(smem_u32(sm + StSmem::BOP), 4096, 0);
    dB[1] = desc_kmajor(smem_u32(sm + StSmem::BOP + 8192), 4096, 0);
    int stage = 0;
    for (int j = 0; j < N; ++j) {
      ST_STAMP_I(0);
      bar_sync(2, STHREADS);
      ST_STAMP_I(1);
      if (lane == 0) {
        tc_fence_after();
        constexpr uint32_t idesc = idesc_bf16(128, SL, 1, 0);
        const uint64_t a0 = stage == 0 ? dY[0] : stage == 1 ? dY[1] : dY[2];
        const uint64_t b0 = (j & 1) ? dB[1] : dB[0];
        const uint32_t acc = tmem + SL * (j & 1);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)      // D[dv][dk] = sum_c y[c][dv] x_hat[c][dk]
          umma_bf16(acc, desc_advance(a0, ks * 2048), desc_advance(b0, (ks >> 2) * 4096 + (ks & 3) * 32), idesc, ks > 0);
        umma_commit(smem_u32(mma + (j & 1)));
        // When this product has completed its ring stage is free: refill it at once with the loads of
        // step j + NSTAGE, so that they have almost NSTAGE steps to land.
        if (j + NSTAGE < N) {
          if (ok) ok = mbar_wait(smem_u32(mma + (j & 1)), (uint32_t)((j >> 1) & 1));
          issue_loads(j + NSTAGE);
        }
      }
      stage = stage == NSTAGE - 1 ? 0 : stage + 1;
      __syncwarp();
    }
    if (!ok && lane == 0) atomicAdd(&g_state_wait_timeouts, 1u);
  } else {
    // ---- worker warps ---------------------------------------------------------------------------------------
    // state registers: TMEM lane = dv, this thread's 8 columns = key features 8 cg + [0, 8) of the slice
    const int q4 = warp & 3, cg = warp >> 2;
    const int dv = 32 * q4 + lane;
    const int64_t el0 = ((bh * SD) + SL * slice + 8 * cg) * SD + dv;     // element (bh, dk0, dv); dk stride SD
    float S[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) S[j] = init ? __bfloat162float(init[el0 + (int64_t)j * SD]) : 0.f;

    // Build k_hat^T (or q_hat^T) of step i into operand buffer i & 1 and hand it to the issuer.
    auto build = [&](int i) {
      const int s = i % NSTAGE;
      ST_STAMP(0);
      if (ok) ok = mbar_wait(smem_u32(full + s), (uint32_t)((i / NSTAGE) & 1));
      ST_STAMP(1);
      const float* gt = reinterpret_cast<const float*>(sm + s * StSmem::STAGE + StSmem::G);
      const unsigned short* xt = reinterpret_cast<const unsigned short*>(sm + s * StSmem::STAGE + StSmem::X);
      float* tt = tot + (i & 1) * 16 * SL;
      float* gg = gsum + (i & 1) * 16 * SL;
      const int r0 = 8 * warp;                 // this thread: feature `lane` of the slice, rows r0 + [0, 8)
      float f[8];
      uint32_t xr[8];
      float gs = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[j] = gt[(r0 + j) * SL + lane];
        xr[j] = xt[(r0 + j) * SL + lane];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { gs += f[j]; f[j] = __expf(f[j]); }
      float run = 1.f;
      if (MODE == 0) {
#pragma unroll
        for (int j = 7; j >= 0; --j) { const float t = f[j]; f[j] = run; run *= t; }      // exclusive suffix
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) { run *= f[j]; f[j] = run; }                          // inclusive prefix
      }
      tt[warp * SL + lane] = run;
      if (MODE == 0) gg[warp * SL + lane] = gs;
      ST_STAMP(2);
      bar_sync(1, SWORKERS);
      ST_STAMP(3);
      float tw[16];
#pragma unroll
      for (int w2 = 0; w2 < 16; ++w2) tw[w2] = tt[w2 * SL + lane];
      float cross = 1.f;
#pragma unroll
      for (int w2 = 0; w2 < 16; ++w2) {
        const bool use = (MODE == 0) ? (w2 > warp) : (w2 < warp);
        cross *= use ? tw[w2] : 1.f;
      }
      if (warp == (MODE == 0 ? 15 : 0)) {       // chunk totals of the slice's features
        float e = 1.f, sg = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 16; ++w2) { e *= tw[w2]; if (MODE == 0) sg += gg[w2 * SL + lane]; }
        eG[(i & 1) * SL + lane] = e;
        if (MODE == 0 && Gc != nullptr) Gc[(bh * N + chunk_of(i)) * SD + SL * slice + lane] = sg;
      }
      uint4 pk;
      pk.x = pack_bf16x2(__uint_as_float(xr[0] << 16) * (f[0] * cross), __uint_as_float(xr[1] << 16) * (f[1] * cross));
      pk.y = pack_bf16x2(__uint_as_float(xr[2] << 16) * (f[2] * cross), __uint_as_float(xr[3] << 16) * (f[3] * cross));
      pk.z = pack_bf16x2(__uint_as_float(xr[4] << 16) * (f[4] * cross), __uint_as_float(xr[5] << 16) * (f[5] * cross));
      pk.w = pack_bf16x2(__uint_as_float(xr[6] << 16) * (f[6] * cross), __uint_as_float(xr[7] << 16) * (f[7] * cross));
      // row = feature (the N index), 64 chunk rows per 128-byte line, this thread's 8 rows = one 16-byte piece
      uint8_t* bop = sm + StSmem::BOP + (i & 1) * 8192 + (warp >> 3) * 4096;
      *reinterpret_cast<uint4*>(bop + sw128_chunk(lane, warp & 7)) = pk;
      ST_STAMP(4);
      fence_async_smem();
      tc_fence_before();
      bar_arrive(2, STHREADS);
      ST_STAMP(5);
    };

    if (N > 0) build(0);
    for (int i = 0; i < N; ++i) {
      if (i + 1 < N) build(i + 1);
      else bar_sync(1, SWORKERS);          // the totals written while building step i are visible to all
      // state update of step i
      ST_STAMP(6);
      if (ok) ok = mbar_wait(smem_u32(mma + (i & 1)), (uint32_t)((i >> 1) & 1));
      ST_STAMP(7);
      tc_fence_after();
      uint32_t r[8];
      tmem_ld8(tmem + ((uint32_t)(q4 * 32) << 16) + SL * (i & 1) + 8 * cg, r);
      tmem_ld_wait();
      tc_fence_before();
      ST_STAMP(8);
      bf16* so = states + (int64_t)(bh * N + chunk_of(i)) * SD * SD + (el0 - bh * SD * SD);
      const float* e = eG + (i & 1) * SL + 8 * cg;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        so[(int64_t)j * SD] = __float2bfloat16_rn(S[j]);
        S[j] = fmaf(e[j], S[j], __uint_as_float(r[j]));
      }
      ST_STAMP(9);
    }
    if (fin != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) fin[el0 + (int64_t)j * SD] = __float2bfloat16_rn(S[j]);
    }
    if (!ok && lane == 0) atomicAdd(&g_state_wait_timeouts, 1u);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 64);
}

}  // namespace

#ifdef ST_TRACE
void tc_state_read_trace(long long* o) { cudaMemcpyFromSymbol(o, g_st_trace, sizeof(g_st_trace)); }
#endif
unsigned int tc_state_read_wait_timeouts() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_state_wait_timeouts, sizeof(v));
  return v;
}

// Whether the one-pass kernel is expected to beat the product + scan pair for this shape.
// Its time is (waves of (B*H*4) blocks over the SMs) x N sequential steps; the pair's time grows with
// the total number of chunks.  Step and per-chunk costs measured on B200; GLA_B200_STATE_FUSED=0/1
// overrides the estimate.
bool tc_state_fused_preferred(int64_t BH, int64_t N) {
  static int forced = -2;
  if (forced == -2) { const char* e = getenv("GLA_B200_STATE_FUSED"); forced = e ? (e[0] == '0' ? 0 : 1) : -1; }
  if (forced >= 0) return forced == 1;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const double waves = (double)((4 * BH + sms - 1) / sms);
  const double t_fused = waves * (double)N * 1.0 + 5.0;          // us
  const double t_pair = (double)(BH * N) * 0.1 + 10.0;           // us
  return t_fused < t_pair;
}

// mode 0: states[n] = state before chunk n (from init), fin = state after the last chunk, Gc = chunk gate sums.
// mode 1: states[n] = gradient state after chunk n (from init = dhidden_final), fin = dhidden_init.
int tc_state_fused(cudaStream_t st, int mode, int64_t B, int64_t T, int64_t H, const float* g, const void* x,
                   const void* y, const void* init, void* states, void* fin, float* Gc) {
  const int64_t N = T / SC, BH = B * H;
  StMaps maps;
  GLA_TRY(make_map_bthd(&maps.g, g, 1, B, T, H, SL, 0));
  GLA_TRY(make_map_bthd(&maps.x, x, 0, B, T, H, SL, 0));
  GLA_TRY(make_map_bthd(&maps.y, y, 0, B, T, H, 64, 1));
  auto kern = mode == 0 ? tc_state_kernel<0> : tc_state_kernel<1>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ST_SMEM);
  if (e != cudaSuccess) return record_cuda_error(e);
  {
    ProfScope ps(mode == 0 ? "tc_state_kernel" : "tc_dstate_scan_kernel", st);
    kern<<<(unsigned)(BH * 4), STHREADS, ST_SMEM, st>>>(maps, T, H, (int)N, (const bf16*)init, (bf16*)states, (bf16*)fin, Gc);
  }
  GLA_CHECK_LAUNCH();
  return GLA_OK;
}

}  // namespace gla
