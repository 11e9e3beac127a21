// Thin wrappers over the sm_100a PTX this backend uses: mbarrier, bulk/tensor async copies
// (TMA), tcgen05 (tensor memory + 5th-gen tensor-core MMA).  Every wait is bounded: after a
// fixed number of polls it reports failure to the caller instead of spinning forever, so a
// protocol bug can never leave the GPU hung.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace ekptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Poll limit of one wait.  Each poll may itself suspend for a hardware-defined short time;
// with the back-off below the total is of the order of a second, far beyond any legitimate
// wait inside these kernels and short enough to keep the context responsive.
constexpr uint32_t kWaitPolls = 1u << 22;

// Returns false if the barrier did not flip within the limit or another thread of the CTA
// raised `*abort_flag` (shared memory) meanwhile.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < kWaitPolls; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it >= 32) {
      __nanosleep(it < 4096 ? 20 : 200);
      if ((it & 255u) == 0 && *abort_flag) return false;
    }
  }
  *abort_flag = 1;
  return false;
}

// ---- async copies (TMA) -----------------------------------------------------------------
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Same with an L2 eviction-priority hint (weights are streamed once: evict_first).
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// 2-D tiled tensor copy global -> shared.  x (innermost coordinate) times the element size
// must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int32_t x, int32_t y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// all state spaces: orders generic-proxy accesses (global memory included) with later TMA accesses
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// ---- tcgen05: tensor memory --------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// mbarrier arrives once when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// 32 lanes x 32 bit, 32 consecutive columns: thread i of the warp writes r[0..31] to lane
// (lane base of the warp)+i, columns taddr.col .. +31.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::
          "r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ---- tensor-memory loads that are complete when they return ---------------------------------
// tcgen05.ld delivers its destination registers asynchronously: until tcgen05.wait::ld they must be
// neither read nor reused.  The compiler does not know that - to it the registers are defined as
// soon as the asm statement ends, so under register pressure it may spill them (storing values
// that have not arrived yet) and hand the physical registers to something else, which the late
// delivery then overwrites: wrong data at best, a wild address and a launch failure at worst.
// Keeping the loads and the wait in ONE asm statement closes that window.
// Columns [c, c+8) of two accumulators for this thread's lane, complete on return.
__device__ __forceinline__ void tmem_ld8x2_wait(uint32_t ta, uint32_t tb, uint32_t* a, uint32_t* b) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%16];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%8,%9,%10,%11,%12,%13,%14,%15}, [%17];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]),
        "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7])
      : "r"(ta), "r"(tb)
      : "memory");
}
// Columns [c, c+32) of two accumulators for this thread's lane, complete on return.
__device__ __forceinline__ void tmem_ld32x2_wait(uint32_t ta, uint32_t tb, uint32_t* a, uint32_t* b) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]), "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31]),
        "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]), "=r"(b[16]), "=r"(b[17]), "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]), "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]), "=r"(b[30]), "=r"(b[31])
      : "r"(ta), "r"(tb)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16_wait(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// ---- tcgen05: MMA ------------------------------------------------------------------------
// Shared-memory operand descriptor, K-major tile whose rows are 128 bytes (64 x 16-bit) with
// the 128-byte swizzle that a TMA load with SWIZZLE_128B produces.  8-row groups are 1024 B
// apart.  The tile base must be 1024-byte aligned; `byte_off` (< 128, multiple of 32)
// advances along K inside the swizzle atom.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address  [0,14)
  d |= static_cast<uint64_t>(1) << 16;                       // leading byte offset (unused) [16,30)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;               // stride byte offset [32,46)
  d |= static_cast<uint64_t>(1) << 46;                       // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                       // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, M = 128, given N.
__device__ __forceinline__ uint32_t umma_idesc_bf16(uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem]   (one thread issues)
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The MMAs of one weight tile in a single statement: the issuing thread's instruction stream is
// latency-bound (one thread, no other warps to hide behind on its scheduler slot), so the
// predicate set-up is shared and descriptors arrive precomputed.  D (+)= A[tmem + 8j] * B[desc_j];
// only the first product may overwrite D (`accumulate_first` = 0).
__device__ __forceinline__ void umma_ts_x8(uint32_t d, uint32_t a, const uint64_t* b, uint32_t idesc,
                                           uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t"
      "setp.ne.b32 p0, %19, 0;\n\t"
      "setp.ne.b32 p1, %18, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %9, %18, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], %10, %18, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%3], %11, %18, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %12, %18, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%5], %13, %18, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%6], %14, %18, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%7], %15, %18, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%8], %16, %18, p1;\n\t}" ::"r"(d),
      "r"(a), "r"(a + 8), "r"(a + 16), "r"(a + 24), "r"(a + 32), "r"(a + 40), "r"(a + 48), "r"(a + 56),
      "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]), "l"(b[7]),
      "r"(0), "r"(idesc), "r"(accumulate_first)
      : "memory");
}
__device__ __forceinline__ void umma_ts_x4(uint32_t d, uint32_t a, const uint64_t* b, uint32_t idesc,
                                           uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t"
      "setp.ne.b32 p0, %10, 0;\n\t"
      "setp.ne.b32 p1, %9, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %5, %9, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], %6, %9, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%3], %7, %9, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %8, %9, p1;\n\t}" ::"r"(d),
      "r"(a), "r"(a + 8), "r"(a + 16), "r"(a + 24), "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "r"(idesc),
      "r"(accumulate_first)
      : "memory");
}

// Four K steps with both operands in shared memory.
__device__ __forceinline__ void umma_ss_x4(uint32_t d, const uint64_t* a, const uint64_t* b, uint32_t idesc,
                                           uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t"
      "setp.ne.b32 p0, %10, 0;\n\t"
      "setp.ne.b32 p1, %9, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %5, %9, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %2, %6, %9, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %7, %9, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %8, %9, p1;\n\t}" ::"r"(d),
      "l"(a[0]), "l"(a[1]), "l"(a[2]), "l"(a[3]), "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "r"(idesc),
      "r"(accumulate_first)
      : "memory");
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

}  // namespace ekptx
