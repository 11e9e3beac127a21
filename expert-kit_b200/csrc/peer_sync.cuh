// Step-number flags between the ranks of an expert-parallel group: stored into the consumer's flag
// words with a system-scope release after the data, polled locally with system-scope acquires.
// Every wait is bounded.  Shared by the peer-memory kernels (ep_peer.cu) and by the kernels that
// take a wait or a signal along instead of a launch of its own (router_tc.cu, combine.cu).
#pragma once
#include "ek_internal.h"

namespace ek {

constexpr uint32_t kPeerPollLimit = 1u << 20;   // polls with a ~100 ns back-off: about a second

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits until flag >= want; false after the poll limit.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want) {
  for (uint32_t i = 0; i < kPeerPollLimit; ++i) {
    if (ld_acquire_sys(flag) >= want) return true;
    if (i > 64) __nanosleep(100);
  }
  return false;
}

// Lane r of the calling warp waits for rank r's step number; the warp agrees on the outcome and one
// lane records a timeout.  All 32 lanes must call.
__device__ __forceinline__ bool warp_wait_ranks(const PeerWait& w, DevStatus* st, int lane) {
  bool ok = true;
  if (lane < w.world) ok = wait_flag(w.flags + lane, w.step_no);
  const unsigned bad = __ballot_sync(0xffffffffu, !ok);
  if (bad && lane == 0 && atomicCAS(&st->code, DEV_OK, DEV_TIMEOUT) == DEV_OK) {
    st->where = w.where;
    st->aux0 = __ffs(bad) - 1;
    st->aux1 = (int)w.step_no;
  }
  return bad == 0;
}

// After the CTA's own results are written: the CTA that finishes last publishes the step number to
// every rank.  All threads of the CTA must call; `n_ctas` is the size of the grid.
__device__ __forceinline__ void cta_signal_when_last(const PeerSignal& g, unsigned n_ctas) {
  __shared__ int s_sig_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(g.ticket, 1u);
    s_sig_last = t == n_ctas - 1;
    if (s_sig_last) *g.ticket = 0;                // launches on one stream do not overlap
  }
  __syncthreads();
  if (s_sig_last && (int)threadIdx.x < g.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(g.flags.p[threadIdx.x]) + g.slot, g.step_no);
  }
}

}  // namespace ek
