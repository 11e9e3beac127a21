// Everything in front of the grouped GEMMs in ONE launch, for small batches (T <= 8, E <= 256,
// router weight exactly representable in bf16): router logits, scoring and group-limited top-k,
// per-expert histogram, offsets, permutation, chunk work list and - when the rows are few - the row
// gather.  At these sizes the five kernels it replaces (tensor-core router, select, permute, work
// list, gather) cost more in launches and hand-overs than in work: a one-token pass of the
// DeepSeek-V3-shape layer spent 36 of its 106 us in them.
//
// Semantics are those of the separate kernels: frontend routing (expertkit_torch/models/
// qwen3_moe.py:161-169; the DeepSeek-V3 router called at deepseek_v3/model.py:142) and the
// controller's bucketing (ek-computation/src/controller/executor.rs:283-299,112-133).
//
// Phase 1 (grid = K slices of 512 elements x blocks of 32 experts, about 112 CTAs at H = 7168,
// E = 256): a warp owns one expert, its lanes two 16-byte vectors of the slice each (coalesced 1 KiB
// row segments, the weights stay in registers over all tokens); a butterfly adds the lanes and the
// fp32 partial logit goes to partial[slice][T][E].
// Phase 2 (the CTA that finishes last, found with a ticket counter): all threads add the partials in
// slice order (deterministic); one warp per token routes it with the same routine as the stand-alone
// select kernel; then the CTA scans the histogram, ranks the assignments (stable: rows of an expert
// in ascending token order), writes the work list and, if asked, gathers the rows.
#include "bucket.cuh"
#include "ek_internal.h"
#include "route_select.cuh"

namespace ek {

namespace {

constexpr int kThreads = 1024;
constexpr int kMaxT = 8;         // tokens (one warp each in phase 2); beyond that the separate kernels are as fast
constexpr int kMaxE = 256;       // experts
constexpr int kMaxTk = 1024;     // assignments (T * k)
constexpr int kSlice = 512;      // K elements per CTA of phase 1: two 16-byte vectors per lane
constexpr int kTokBatch = 4;     // tokens in flight per warp (independent loads and butterflies)

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(q[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__global__ void __launch_bounds__(kThreads, 1) front_small_kernel(const __grid_constant__ FrontParams p) {
  extern __shared__ float smem[];
  __shared__ int s_last;
  const RouteParams& r = p.route;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = r.T, E = r.E, H = r.H;
  pdl_wait();
  pdl_trigger();

  // ---- phase 1: partial logits of (K slice blockIdx.x, experts blockIdx.y * 32 + warp) -----------
  {
    const int e = blockIdx.y * 32 + warp;
    const int ka = blockIdx.x * kSlice + lane * 8, kb = ka + kSlice / 2;   // H is a multiple of 8
    if (e < E) {
      const __nv_bfloat16* wrow = reinterpret_cast<const __nv_bfloat16*>(r.wg) + (size_t)e * H;
      float w[16];
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
      unpack8(ka < H ? __ldg(reinterpret_cast<const uint4*>(wrow + ka)) : zero, w);
      unpack8(kb < H ? __ldg(reinterpret_cast<const uint4*>(wrow + kb)) : zero, w + 8);
      float* out = p.partial + (size_t)blockIdx.x * T * E + e;
      for (int t0 = 0; t0 < T; t0 += kTokBatch) {
        uint4 xa[kTokBatch], xb[kTokBatch];
#pragma unroll
        for (int tt = 0; tt < kTokBatch; ++tt) {
          const __nv_bfloat16* xr = r.x + (size_t)min(t0 + tt, T - 1) * H;
          xa[tt] = ka < H ? *reinterpret_cast<const uint4*>(xr + ka) : zero;
          xb[tt] = kb < H ? *reinterpret_cast<const uint4*>(xr + kb) : zero;
        }
        float acc[kTokBatch];
#pragma unroll
        for (int tt = 0; tt < kTokBatch; ++tt) {
          float f[16];
          unpack8(xa[tt], f);
          unpack8(xb[tt], f + 8);
          float a = 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) a = fmaf(f[j], w[j], a);
          acc[tt] = a;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
          for (int tt = 0; tt < kTokBatch; ++tt) acc[tt] += __shfl_xor_sync(0xffffffffu, acc[tt], o);
        }
        float mine = acc[0];
#pragma unroll
        for (int tt = 1; tt < kTokBatch; ++tt) mine = lane == tt ? acc[tt] : mine;
        if (lane < kTokBatch && t0 + lane < T) out[(size_t)(t0 + lane) * E] = mine;
      }
    }
  }
  // ---- who is last? ---------------------------------------------------------------------------
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned ticket = atomicAdd(p.ticket, 1u);
    s_last = ticket == gridDim.x * gridDim.y - 1;
    if (s_last) *p.ticket = 0;                          // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  // ---- phase 2: logits = partial sums in slice order; then routing, one warp per token ---------
  // Everything the CTA makes and uses again stays in shared memory (logits, ids, weights, histogram,
  // offsets, permutation): the chain of steps below would otherwise pay a round trip to L2 at every
  // hand-over.  The results go to global memory on the side, for the kernels behind and the caller.
  __shared__ float s_logits[kMaxT * kMaxE];
  __shared__ float s_w[kMaxTk];
  __shared__ int s_ids[kMaxTk];
  __shared__ int s_perm[kMaxTk];
  __shared__ int s_hist[kMaxE];                         // the histogram over all experts
  __shared__ int s_cnt[kMaxE];                          // ... of the experts this rank serves (0 elsewhere)
  __shared__ int s_off[kMaxE + 1];
  const int Tk = T * r.k;
  {
    const int n_slices = (int)gridDim.x;
    for (int e = tid; e < E; e += kThreads) s_hist[e] = 0;
    for (int o = tid; o < T * E; o += kThreads) {
      float v = 0.f;
      for (int c0 = 0; c0 < n_slices; c0 += 16) {
        float tmp[16];
#pragma unroll
        for (int a = 0; a < 16; ++a) tmp[a] = c0 + a < n_slices ? __ldcg(p.partial + (size_t)(c0 + a) * T * E + o) : 0.f;
#pragma unroll
        for (int a = 0; a < 16; ++a) v += tmp[a];
      }
      // the softmax router's linear layer runs in bf16 in the reference
      v = r.scoring == EK_SCORE_SOFTMAX ? __bfloat162float(__float2bfloat16_rn(v)) : v;
      s_logits[o] = v;
      r.logits[o] = v;
    }
    __syncthreads();
    float* sc = smem + (size_t)warp * (2 * kMaxE + 64);
    if (warp < T) {
      RouteParams rs = r;                               // the same routine as the stand-alone select kernel, on shared memory
      rs.logits = s_logits;
      rs.ids = s_ids;
      rs.weights = s_w;
      rs.counts = s_hist;
      rs.partial = nullptr;                             // the logits are final
      select_token(rs, warp, lane, sc, sc + kMaxE, sc + 2 * kMaxE);
    }
  }
  __syncthreads();
  // ---- offsets: exclusive scan of the counts of the experts this rank serves -------------------
  const PermuteParams& pp = p.permute;
  auto is_local = [&](int j) { return pp.owners ? pp.owners[j] == pp.rank : (j >= pp.e_lo && j < pp.e_hi); };
  for (int i = tid; i < Tk; i += kThreads) {
    r.ids[i] = s_ids[i];
    r.weights[i] = s_w[i];
  }
  if (tid < E) {
    const int c = s_hist[tid];
    r.counts[tid] = c;
    s_cnt[tid] = is_local(tid) ? c : 0;
  }
  __syncthreads();
  if (warp == 0) {                                      // E <= 256: eight experts per lane
    int v[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane * 8 + j;
      v[j] = e < E ? s_cnt[e] : 0;
      sum += v[j];
    }
    int inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += u;
    }
    int run = inc - sum;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane * 8 + j;
      if (e < E) s_off[e] = run;
      run += v[j];
    }
    if (lane == 31) s_off[E] = inc;
  }
  __syncthreads();
  for (int e = tid; e <= E; e += kThreads) pp.offsets[e] = s_off[e];
  // ---- permutation: stable rank of every assignment inside its expert ---------------------------
  for (int i = tid; i < Tk; i += kThreads) {
    const int e = s_ids[i];
    if (is_local(e)) {
      int rank = 0;
      for (int j = 0; j < i; ++j) rank += s_ids[j] == e;
      const int pos = s_off[e] + rank;
      pp.perm[pos] = i;
      s_perm[pos] = i;
      pp.inv[i] = pos;
    } else {
      pp.inv[i] = -1;
    }
  }
  __syncthreads();
  // ---- chunk work list -----------------------------------------------------------------------------
  build_worklist<kThreads>(p.worklist, s_hist, s_off);
  // ---- row gather (only when the host asked for it: a handful of rows) --------------------------------
  if (p.gather_rows) {
    __syncthreads();
    const int n_routed = s_off[E];
    // one token: its row is gathered once, to row 0, and every chunk of the work list reads it there
    const int rows = p.worklist.same_row ? 1 : Tk + p.shared_T;
    const int nv = H / 8;
    // a thread owns a 16-byte column of the rows; four rows in flight (the loads are what this step costs)
    for (int v = tid; v < nv; v += kThreads) {
      for (int row0 = 0; row0 < rows; row0 += 4) {
        uint4 val[4];
        bool ok[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int row = row0 + u;
          ok[u] = row < rows && (p.worklist.same_row || row >= Tk || row < n_routed);
          const int src = !ok[u] || p.worklist.same_row ? 0 : row < Tk ? s_perm[row] / r.k : p.shared_t0 + row - Tk;
          if (ok[u]) val[u] = reinterpret_cast<const uint4*>(r.x + (size_t)src * H)[v];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (ok[u])
            reinterpret_cast<uint4*>(p.xp + (size_t)(row0 + u) * H)[v] = p.to_f16 ? bf16x8_to_f16x8(val[u]) : val[u];
      }
    }
  }
}

}  // namespace

// K slice per CTA of phase 1
int front_small_slice(int) { return kSlice; }

bool front_small_supported(int T, int E, int k, int H) {
  // the partial-sum buffer holds 148 * 128 * E floats: (H / 512) * T * E stays far below that
  return T >= 1 && T <= kMaxT && E >= 1 && E <= kMaxE && T * k <= 1024 && H % 8 == 0 && H <= kSlice * 256;
}

int launch_front_small(const FrontParams& p, cudaStream_t s) {
  const int n_slices = (p.route.H + kSlice - 1) / kSlice;
  const int n_eblocks = (p.route.E + 31) / 32;
  const size_t smem = (size_t)kMaxT * (2 * kMaxE + 64) * sizeof(float);   // phase 2: one warp per token
  cudaFuncSetAttribute(front_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_pdl(front_small_kernel, dim3(n_slices, n_eblocks), dim3(kThreads), smem, s, p);
  return 1;
}

}  // namespace ek
