// Thin inline-PTX wrappers for the sm_100a tensor-core path: tcgen05.mma with shared-memory
// operand descriptors, tensor memory (TMEM) allocation and loads, mbarriers, proxy fences.
//
// Shared-memory operand format used everywhere in this library ("SW128 tile"):
//   R rows x 64 bf16 (128 bytes per row), tile base 1024-byte aligned; the 16-byte chunk c of
//   row r is stored at chunk position (c ^ (r & 7)).  This is the 128-byte-swizzle canonical
//   layout of tcgen05 (and what a TMA box of 64 x R elements with SWIZZLE_128B produces).
//   The same tile serves as a K-major operand (rows = M/N index, the 64 columns run along K)
//   or as an MN-major operand (rows = K index, the 64 columns run along M/N); only the
//   descriptor strides and the major bits of the instruction descriptor differ.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace gla {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// byte offset of element (r, c), c in [0, 64), inside one SW128 tile
__device__ __forceinline__ uint32_t sw128_off(int r, int c) {
  return (uint32_t)(r * 128 + ((((c >> 3) ^ (r & 7)) << 4) | ((c & 7) << 1)));
}
// byte offset of the 16-byte chunk ch (0..7) of row r
__device__ __forceinline__ uint32_t sw128_chunk(int r, int ch) { return (uint32_t)(r * 128 + ((ch ^ (r & 7)) << 4)); }

// ---- descriptors -----------------------------------------------------------------------
// 64-bit shared-memory matrix descriptor: start address, leading/stride byte offsets (all in
// units of 16 bytes), descriptor version 1 (Blackwell), 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// K-major operand: rows = M/N index; k-step ks covers K = [16 ks, 16 ks + 16).  The operand is a
// row of K-blocks (tiles of 64 columns), tile_stride bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, uint32_t tile_stride, int ks) {
  return smem_desc(base + (uint32_t)(ks >> 2) * tile_stride + (uint32_t)(ks & 3) * 32u, 16u, 1024u);
}
// MN-major operand: rows = K index (128 bytes each); M/N blocks of 64 are tile_stride bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, uint32_t tile_stride, int ks) {
  return smem_desc(base + (uint32_t)ks * 2048u, tile_stride, 1024u);
}
// A descriptor whose start address is `bytes` further on (bytes a multiple of 16, the sum staying below the
// 256 KB the 14-bit field covers): only the low word changes, so stepping through the K slices of an
// operand costs one 32-bit add per MMA instead of rebuilding the descriptor.
__device__ __forceinline__ uint64_t desc_advance(uint64_t d, uint32_t bytes) {
  uint32_t lo = (uint32_t)d + (bytes >> 4), hi = (uint32_t)(d >> 32);
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
// 32-bit instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// 32-byte global store (sm_100: 256-bit vector stores); p must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&r)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               :: "l"(p), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}

// ---- L2 prefetch --------------------------------------------------------------------------
// Asks the memory system to bring [p, p + bytes) into L2 (p and bytes multiples of 16); nothing waits on it.
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// ---- MMA issue / completion -------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on an mbarrier when all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Make generic-proxy shared-memory writes visible to the async proxy (tcgen05.mma operand reads).
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- mbarrier -----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// Bounded wait: returns false if the phase did not complete within the iteration limit, so a
// kernel can never spin forever on a completion that is not coming.  The suspend-time hint lets the
// hardware park the thread until the phase completes instead of re-issuing the test every few cycles:
// spinning waiters would otherwise take issue slots from the warps doing the work.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < (1 << 18); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(10000u) : "memory");
    if (ok) return true;
  }
  return false;
}

// Plain arrival (counts one towards the barrier's expected arrivals).
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

// Arrive on the barrier and add `bytes` to its pending transaction count (one thread).
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}

// ---- TMA (bulk tensor copies global -> shared, completion on an mbarrier) ------------------
// The innermost coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const void* tmap, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      :: "r"(smem_dst), "l"((uint64_t)tmap), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      :: "r"(smem_dst), "l"((uint64_t)tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}
// The same box as tma_load_3d would copy, requested into L2 only (no shared-memory destination, no barrier).
__device__ __forceinline__ void tma_prefetch_l2_3d(const void* tmap, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
               :: "l"((uint64_t)tmap), "r"(x), "r"(y), "r"(z) : "memory");
}
// Bulk tensor store shared -> global of one box (bulk-group completion); never start one at a negative coordinate.
__device__ __forceinline__ void tma_store_3d(const void* tmap, int x, int y, int z, uint32_t smem_src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
               :: "l"((uint64_t)tmap), "r"(x), "r"(y), "r"(z), "r"(smem_src) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" :: "l"((uint64_t)tmap) : "memory");
}

// ---- tensor memory ------------------------------------------------------------------------
// Executed by one full warp.  ncols: power of two >= 32.  The base address lands in *dst (smem).
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Each thread of the warp reads N consecutive 32-bit columns of ITS lane (lane = 32*(warp%4) +
// laneid; taddr's lane field must be the warp's quadrant base).
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(h);
}

}  // namespace tc
// Device-scope acquire load (flag written by another grid with a fence + atomic), and the fence that orders
// such generic-proxy observations before this thread's later TMA (async proxy) reads of global memory.
__device__ __forceinline__ uint32_t ld_acquire_u32(const unsigned int* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

}  // namespace gla
