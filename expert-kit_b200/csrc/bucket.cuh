// Device routines shared by the bucketing kernels (permute.cu) and the fused front kernel for small
// batches (front_small.cu).
#pragma once
#include "ek_internal.h"

namespace ek {

// eight bf16 -> eight f16 (round to nearest, saturating at +-65504)
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(v & 0xFFFF0000u)), "f"(__uint_as_float(v << 16)));
  return r;
}
__device__ __forceinline__ uint4 bf16x8_to_f16x8(uint4 v) {
  v.x = bf16x2_to_f16x2(v.x); v.y = bf16x2_to_f16x2(v.y); v.z = bf16x2_to_f16x2(v.z); v.w = bf16x2_to_f16x2(v.w);
  return v;
}

// Chunk descriptors: every expert this rank serves has its row range cut into pieces of `chunk_rows`,
// followed by the virtual shared experts (all T tokens each).  One CTA of NT threads.
// `s_counts` / `s_offsets`: the histogram and the offsets in shared memory when the calling CTA made
// them itself (the fused front kernel); null: read from global memory at L2.
template <int NT>
__device__ __forceinline__ void build_worklist(const WorklistParams& p, const int* s_counts = nullptr,
                                               const int* s_offsets = nullptr) {
  static_assert(NT % 32 == 0 && NT <= 1024, "whole warps");
  __shared__ int s_scan[64];
  __shared__ int s_total;
  const int tid = threadIdx.x;
  const int n_local = p.e_hi - p.e_lo;
  if (p.counts_copy)
    for (int e = tid; e < p.E; e += NT) p.counts_copy[e] = s_counts ? s_counts[e] : __ldcg(&p.counts[e]);
  // experts this rank serves: its window (slot = e - e_lo), or, with an owner table, every expert
  // the table gives to this rank (slot from the layer's slot table: own experts and replicas)
  const int first = p.owners ? 0 : p.e_lo, last = p.owners ? p.E : p.e_hi;
  int running = 0;
  // shared virtual experts: their registration flags are fetched now, alongside the loads of the loop below
  const int per_shared = (p.T + p.chunk_rows - 1) / p.chunk_rows;
  int shared_registered = 1;
  if (tid < p.n_shared * per_shared && tid % per_shared == 0) shared_registered = p.registered[n_local + tid / per_shared];
  for (int e0 = first; e0 < last; e0 += NT) {
    const int e = e0 + tid;
    int cnt = 0, nch = 0, slot = -1;
    if (e < last && (!p.owners || p.owners[e] == p.rank)) {
      cnt = s_counts ? s_counts[e] : __ldcg(&p.counts[e]);   // the histogram is built with atomics: read it at L2
      slot = p.slot_of ? p.slot_of[e] : e - p.e_lo;
      nch = (cnt + p.chunk_rows - 1) / p.chunk_rows;
      if (cnt > 0 && (slot < 0 || !p.registered[slot])) {
        if (atomicCAS(&p.status->code, DEV_OK, DEV_MISSING_EXPERT) == DEV_OK) {
          p.status->where = 2;
          p.status->aux0 = e;
        }
        nch = 0;
      }
    }
    // inclusive scan of the chunk counts: shuffles inside a warp, then the warps' totals
    int inc = nch;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc, o);
      if ((tid & 31) >= o) inc += v;
    }
    if ((tid & 31) == 31) s_scan[tid >> 5] = inc;
    __syncthreads();
    if (tid < 32) {
      int w = tid < NT / 32 ? s_scan[tid] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, w, o);
        if (tid >= o) w += v;
      }
      s_scan[32 + tid] = w;                      // inclusive totals of warps 0..tid
    }
    __syncthreads();
    const int before = (tid >> 5) > 0 ? s_scan[32 + (tid >> 5) - 1] : 0;
    int first_chunk = running + before + inc - nch;
    if (tid == NT - 1) s_total = before + inc;
    if (nch > 0) {
      const int off = s_offsets ? s_offsets[e] : __ldcg(&p.offsets[e]);   // may have been written by another CTA of this kernel
      for (int c = 0; c < nch; ++c) {
        if (first_chunk + c >= p.max_chunks) break;
        ChunkDesc d;
        d.slot = slot;
        d.out_row = off + c * p.chunk_rows;
        d.in_row = p.same_row ? 0 : d.out_row;
        d.n_rows = min(p.chunk_rows, cnt - c * p.chunk_rows) | (nch > 1 ? kChunkMulti : 0);
        p.chunks[first_chunk + c] = d;
      }
    }
    __syncthreads();
    running += s_total;
    __syncthreads();
  }
  // shared virtual experts
  for (int i = tid; i < p.n_shared * per_shared; i += NT) {
    const int j = i / per_shared, c = i % per_shared;
    if (running + i >= p.max_chunks) break;
    ChunkDesc d;
    d.slot = n_local + j;
    d.in_row = p.same_row ? 0 : p.Tk + c * p.chunk_rows;
    d.out_row = p.Tk + j * p.T + c * p.chunk_rows;
    d.n_rows = min(p.chunk_rows, p.T - c * p.chunk_rows) | (per_shared > 1 ? kChunkMulti : 0);
    p.chunks[running + i] = d;
    if (c == 0 && !(i == tid ? shared_registered : p.registered[d.slot])) {
      if (atomicCAS(&p.status->code, DEV_OK, DEV_MISSING_EXPERT) == DEV_OK) {
        p.status->where = 3;
        p.status->aux0 = -1 - j;
      }
    }
  }
  // (the list is read by later kernels only: the end of this kernel publishes it, no fence needed here)
  __syncthreads();
  if (tid == 0) {
    int total = running + p.n_shared * per_shared;
    if (total > p.max_chunks) {
      if (atomicCAS(&p.status->code, DEV_OK, DEV_BOUNDS) == DEV_OK) {
        p.status->where = 4;
        p.status->aux0 = total;
      }
      total = p.max_chunks;
    }
    // a missing expert cancels the GEMMs altogether
    *p.n_chunks = (*reinterpret_cast<volatile int32_t*>(&p.status->code) == DEV_OK) ? total : 0;
  }
}

}  // namespace ek
