// Expert parallelism over peer memory: token dispatch and the combine of the partial sums as this
// library's own kernels over NVLink, instead of an all-gather and a reduce-scatter.
//
// The reference moves rows between controller and workers by gRPC, one request per distinct expert
// (ek-computation/src/controller/executor.rs:141-226).  Here one process per GPU maps every peer's
// buffers (CUDA IPC, set up by the host) and
//   push    : each rank stores its tokens straight into every rank's gathered-token buffer,
//   finish  : each rank LOADS the fp32 partial sums of its own tokens from every rank's buffer, adds
//             them in rank order (deterministic), adds the shared expert and rounds -- the
//             reduce-scatter and the final combine are one kernel.
// Ranks synchronise through monotonically increasing step numbers stored into the consumer's flag
// words (release at system scope after the data) and polled locally (acquire at system scope).
// Plain loads and stores only: no TMA on peer memory, no multimem.  Every wait is bounded.
#include "ek_internal.h"
#include "peer_sync.cuh"

namespace ek {

namespace {

constexpr int kMaxRanks = EK_EP_MAX_RANKS;

// grid (world, slices): CTA (dst, s) copies its share of this rank's rows into rank dst's buffer;
// the last CTA of a destination publishes the step number there.
__global__ void __launch_bounds__(256) ep_push_kernel(const __nv_bfloat16* __restrict__ x, int32_t T, int32_t H,
                                                      PeerPtrs xall, PeerPtrs flags, int32_t rank, uint32_t step_no,
                                                      size_t dst_elem_off, uint32_t* __restrict__ counters) {
  pdl_wait();
  pdl_trigger();
  const int dst = blockIdx.x, slices = gridDim.y;
  const int per = (T + slices - 1) / slices;
  const int r_lo = blockIdx.y * per, r_hi = min(T, r_lo + per);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(xall.p[dst]) + dst_elem_off;
  const int nv = H / 8;
  for (int r = r_lo; r < r_hi; ++r) {
    const uint4* s = reinterpret_cast<const uint4*>(x + (size_t)r * H);
    uint4* d = reinterpret_cast<uint4*>(out + (size_t)r * H);
    for (int v = threadIdx.x; v < nv; v += blockDim.x) d[v] = s[v];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t done = atomicAdd(&counters[dst], 1u);
    if (done == (uint32_t)slices - 1) {
      counters[dst] = 0;                 // ready for the next step (launches on one stream do not overlap)
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(flags.p[dst]) + rank, step_no);
    }
  }
}

// One warp: lane r waits for rank r's step number in this rank's own flag words (for passes whose
// first kernel cannot take the wait along).
__global__ void ep_wait_kernel(PeerWait w, DevStatus* st) {
  pdl_wait();
  pdl_trigger();
  warp_wait_ranks(w, st, threadIdx.x);
}

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// grid (T_local, H slices): y[t] = bf16( sum over ranks r = 0..world-1 of partial_r[t0 + t] ) + shared[t].
// The partial rows are read from the peers' memory with plain vector loads.
__global__ void __launch_bounds__(256) ep_pull_finish_kernel(PeerPtrs partial, size_t src_elem_off, int32_t world,
                                                             const uint32_t* __restrict__ my_flags, uint32_t step_no,
                                                             const __nv_bfloat16* __restrict__ shared, int32_t n_shared,
                                                             int32_t T, int32_t H, __nv_bfloat16* __restrict__ y,
                                                             DevStatus* st) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < world && !wait_flag(my_flags + threadIdx.x, step_no)) {
    s_ok = 0;
    if (atomicCAS(&st->code, DEV_OK, DEV_TIMEOUT) == DEV_OK) {
      st->where = 510;
      st->aux0 = threadIdx.x;
      st->aux1 = (int)step_no;
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const int t = blockIdx.x;
  const int nv = H / 8, per = (nv + gridDim.y - 1) / gridDim.y;
  const int v_lo = blockIdx.y * per, v_hi = min(nv, v_lo + per);
  for (int v = v_lo + threadIdx.x; v < v_hi; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // the loads of eight ranks are in flight together: one NVLink round trip for a box of eight
    for (int r0 = 0; r0 < world; r0 += 8) {
      float4 a[8], b[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (r0 + i < world) {
          const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(partial.p[r0 + i]) +
                                                              src_elem_off + (size_t)t * H + (size_t)v * 8);
          a[i] = __ldcv(src);
          b[i] = __ldcv(src + 1);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (r0 + i < world) {
          acc[0] += a[i].x; acc[1] += a[i].y; acc[2] += a[i].z; acc[3] += a[i].w;
          acc[4] += b[i].x; acc[5] += b[i].y; acc[6] += b[i].z; acc[7] += b[i].w;
        }
      }
    }
    if (n_shared > 0) {
      // the routed sum is a bf16 tensor before the shared expert's bf16 output is added
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = round_bf16(acc[j]);
      float sh[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) sh[j] = 0.f;
      for (int q = 0; q < n_shared; ++q) {
        const uint4 raw = *reinterpret_cast<const uint4*>(shared + ((size_t)q * T + t) * H + (size_t)v * 8);
        const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(pp[i]);
          sh[2 * i] += f.x;
          sh[2 * i + 1] += f.y;
        }
      }
      if (n_shared > 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) sh[j] = round_bf16(sh[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += sh[j];
    }
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) op[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(y + (size_t)t * H + (size_t)v * 8) = o;
  }
}

PeerPtrs ptrs_of(void* const* p, int n) {
  PeerPtrs o;
  for (int i = 0; i < kMaxRanks; ++i) o.p[i] = i < n ? p[i] : nullptr;
  return o;
}

}  // namespace

int launch_ep_push(const __nv_bfloat16* x, int32_t T, int32_t H, void* const* xall, void* const* flags, int32_t world,
                   int32_t rank, uint32_t step_no, size_t dst_elem_off, uint32_t* counters, cudaStream_t s) {
  int slices = T < 16 ? T : 16;
  if (slices < 1) slices = 1;
  launch_pdl(ep_push_kernel, dim3(world, slices), dim3(256), 0, s, x, T, H, ptrs_of(xall, world), ptrs_of(flags, world), rank,
             step_no, dst_elem_off, counters);
  return 1;
}

int launch_ep_wait(const uint32_t* flags, int32_t world, uint32_t step_no, DevStatus* st, int32_t where, cudaStream_t s) {
  PeerWait w;
  w.flags = flags; w.world = world; w.step_no = step_no; w.where = where;
  launch_pdl(ep_wait_kernel, dim3(1), dim3(32), 0, s, w, st);
  return 1;
}

int launch_ep_pull_finish(void* const* partial, size_t src_elem_off, int32_t world, const uint32_t* my_flags,
                          uint32_t step_no, const __nv_bfloat16* shared, int32_t n_shared, int32_t T, int32_t H,
                          __nv_bfloat16* y, DevStatus* st, cudaStream_t s) {
  if (T < 1) return 0;
  int parts = (296 + T - 1) / T;
  const int most = (H / 8 + 255) / 256;
  if (parts > most) parts = most;
  if (parts < 1) parts = 1;
  launch_pdl(ep_pull_finish_kernel, dim3(T, parts), dim3(256), 0, s, ptrs_of(partial, world), src_elem_off, world, my_flags,
             step_no, shared, n_shared, T, H, y, st);
  return 1;
}

}  // namespace ek
