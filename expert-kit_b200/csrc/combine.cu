// Weighted unpermute-combine and the plain unpermute.
//
// combine: y[t] = sum_k w[t,k] * out[t,k] (+ shared(x)[t]) -- the frontend's step after the
// expert outputs return (expertkit_torch/models/deepseek_v3/model.py:96-104,152;
// expertkit_torch/models/qwen3_moe.py:102-104).
// unpermute: out[t,s,:] = row of (t,s) -- NaiveExecutor's scatter + two-level stack
// (ek-computation/src/controller/executor.rs:203-251).
#include "ek_internal.h"
#include "peer_sync.cuh"

namespace ek {

namespace {

constexpr int kMaxK = 32;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// Rows of the k slots of one 8-element vector, loaded BATCH at a time before the ordered sum: the
// loads are independent, the additions are not.  Small batches of tokens want all eight loads in
// flight per thread (few CTAs, latency-bound); large ones run with four (two measured 20 % slower
// at 4096 tokens).
template <int BATCH>
__device__ __forceinline__ void weighted_rows(const CombineParams& p, const int* s_row, const float* s_w, int v,
                                              float* acc) {
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  for (int s0 = 0; s0 < p.k; s0 += BATCH) {
    uint4 raw[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int row = s0 + i < p.k ? s_row[s0 + i] : -1;
      raw[i] = row >= 0 ? *reinterpret_cast<const uint4*>(p.obuf + (size_t)row * p.H + v * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      if (s0 + i >= p.k || s_row[s0 + i] < 0) continue;
      float f[8];
      unpack8(raw[i], f);
      const float w = s_w[s0 + i];
      if (p.bf16_products) {
        // routing weights were rounded to bf16 upstream; products are bf16 tensors
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], round_bf16(__fmul_rn(w, f[j])));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(w, f[j]));
      }
    }
  }
}

// One CTA per (token, slice of H): 128-bit loads of the k expert rows, fp32 accumulation in slot
// order.  gridDim.y slices keep small batches from running on a handful of SMs.
template <int BATCH>
__global__ void __launch_bounds__(256) combine_kernel(CombineParams p) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_row[kMaxK];
  __shared__ float s_w[kMaxK];
  const int t = blockIdx.x;
  if (threadIdx.x < p.k) {
    s_row[threadIdx.x] = p.inv[(size_t)t * p.k + threadIdx.x];
    s_w[threadIdx.x] = p.weights[(size_t)t * p.k + threadIdx.x];
  }
  __syncthreads();
  const int nv = p.H / 8, per = (nv + gridDim.y - 1) / gridDim.y;
  const int v_lo = blockIdx.y * per, v_hi = min(nv, v_lo + per);
  for (int v = v_lo + threadIdx.x; v < v_hi; v += blockDim.x) {
    float acc[8];
    weighted_rows<BATCH>(p, s_row, s_w, v, acc);
    if (p.n_shared > 0) {
      // the routed sum is a bf16 tensor before the shared expert's bf16 output is added
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = round_bf16(acc[j]);
      float sh[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) sh[j] = 0.f;
      for (int q = 0; q < p.n_shared; ++q) {
        float f[8];
        const __nv_bfloat16* sh_rows = p.shared ? p.shared : p.obuf + (size_t)p.Tk * p.H;
        unpack8(*reinterpret_cast<const uint4*>(sh_rows + ((size_t)q * p.T + t) * p.H + v * 8), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) sh[j] += f[j];
      }
      if (p.n_shared > 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) sh[j] = round_bf16(sh[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += sh[j];
    }
    *reinterpret_cast<uint4*>(p.y + (size_t)t * p.H + v * 8) = pack8(acc);
  }
}

__global__ void __launch_bounds__(128) unpermute_kernel(const __nv_bfloat16* __restrict__ obuf,
                                                        const int32_t* __restrict__ inv,
                                                        __nv_bfloat16* __restrict__ out, int32_t H) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x;  // token*k + slot
  const int row = inv[i];
  uint4* d = reinterpret_cast<uint4*>(out + (size_t)i * H);
  if (row < 0) {
    for (int v = threadIdx.x; v < H / 8; v += blockDim.x) d[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* s = reinterpret_cast<const uint4*>(obuf + (size_t)row * H);
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) d[v] = s[v];
}

template <int BATCH>
__global__ void __launch_bounds__(256) combine_partial_kernel(CombineParams p, float* __restrict__ partial,
                                                              const __grid_constant__ PeerSignal sig) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_row[kMaxK];
  __shared__ float s_w[kMaxK];
  const int t = blockIdx.x;
  if (threadIdx.x < p.k) {
    s_row[threadIdx.x] = p.inv[(size_t)t * p.k + threadIdx.x];
    s_w[threadIdx.x] = p.weights[(size_t)t * p.k + threadIdx.x];
  }
  __syncthreads();
  const int nv = p.H / 8, per = (nv + gridDim.y - 1) / gridDim.y;
  const int v_lo = blockIdx.y * per, v_hi = min(nv, v_lo + per);
  for (int v = v_lo + threadIdx.x; v < v_hi; v += blockDim.x) {
    float acc[8];
    weighted_rows<BATCH>(p, s_row, s_w, v, acc);
    float4* d = reinterpret_cast<float4*>(partial + (size_t)t * p.H + v * 8);
    d[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    d[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  if (sig.world > 0) cta_signal_when_last(sig, gridDim.x * gridDim.y);
}

__global__ void __launch_bounds__(256) combine_finish_kernel(const float* __restrict__ reduced,
                                                             const __nv_bfloat16* __restrict__ shared,
                                                             int32_t n_shared, int32_t T, int32_t H,
                                                             __nv_bfloat16* __restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int nv = H / 8, per = (nv + gridDim.y - 1) / gridDim.y;
  const int v_lo = blockIdx.y * per, v_hi = min(nv, v_lo + per);
  for (int v = v_lo + threadIdx.x; v < v_hi; v += blockDim.x) {
    const float4* r = reinterpret_cast<const float4*>(reduced + (size_t)t * H + v * 8);
    const float4 a = r[0], b = r[1];
    float acc[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    if (n_shared > 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = round_bf16(acc[j]);
      float sh[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) sh[j] = 0.f;
      for (int q = 0; q < n_shared; ++q) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(shared + ((size_t)q * T + t) * H + v * 8), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) sh[j] += f[j];
      }
      if (n_shared > 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) sh[j] = round_bf16(sh[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += sh[j];
    }
    *reinterpret_cast<uint4*>(y + (size_t)t * H + v * 8) = pack8(acc);
  }
}

// One CTA per (segment, row-in-segment): rows move between arrival order and expert order.
__global__ void __launch_bounds__(128) segment_copy_kernel(const __nv_bfloat16* __restrict__ src,
                                                           __nv_bfloat16* __restrict__ dst,
                                                           const RowSegment* __restrict__ segs, int32_t H) {
  const RowSegment sg = segs[blockIdx.y];
  const int i = blockIdx.x;
  if (i >= sg.n) return;
  const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)(sg.src + i) * H);
  uint4* d = reinterpret_cast<uint4*>(dst + (size_t)(sg.dst + i) * H);
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) d[v] = s[v];
}

}  // namespace

int launch_segment_copy(const __nv_bfloat16* src, __nv_bfloat16* dst, const RowSegment* segs, int32_t n_segs,
                        int32_t max_rows_per_seg, int32_t H, cudaStream_t s) {
  if (n_segs <= 0 || max_rows_per_seg <= 0) return 0;
  dim3 grid(max_rows_per_seg, n_segs);
  segment_copy_kernel<<<grid, 128, 0, s>>>(src, dst, segs, H);
  return 1;
}

// H slices per token: enough CTAs for two per SM, at least 256 threads' worth of vectors each
static int h_slices(int T, int H) {
  int parts = (296 + T - 1) / T;
  const int most = (H / 8 + 255) / 256;
  if (parts > most) parts = most;
  return parts < 1 ? 1 : parts;
}

int launch_combine_partial(const CombineParams& p, float* partial, const PeerSignal* sig, cudaStream_t s) {
  const PeerSignal g = sig ? *sig : PeerSignal();
  if (p.T > 0) {
    if (p.T < 1024) launch_pdl(combine_partial_kernel<8>, dim3(p.T, h_slices(p.T, p.H)), dim3(256), 0, s, p, partial, g);
    else launch_pdl(combine_partial_kernel<4>, dim3(p.T, 1), dim3(256), 0, s, p, partial, g);
  }
  return p.T > 0 ? 1 : 0;
}
int launch_combine_finish(const float* reduced, const __nv_bfloat16* shared, int32_t n_shared, int32_t T,
                          int32_t H, __nv_bfloat16* y, cudaStream_t s) {
  if (T > 0) launch_pdl(combine_finish_kernel, dim3(T, h_slices(T, H)), dim3(256), 0, s, reduced, shared, n_shared, T, H, y);
  return T > 0 ? 1 : 0;
}

int launch_combine(const CombineParams& p, cudaStream_t s) {
  if (p.T > 0) {
    if (p.T < 1024) launch_pdl(combine_kernel<8>, dim3(p.T, h_slices(p.T, p.H)), dim3(256), 0, s, p);
    else launch_pdl(combine_kernel<4>, dim3(p.T, 1), dim3(256), 0, s, p);
  }
  return p.T > 0 ? 1 : 0;
}

int launch_unpermute(const __nv_bfloat16* obuf, const int32_t* inv, __nv_bfloat16* out, int32_t T,
                     int32_t k, int32_t H, cudaStream_t s) {
  if (T * k > 0) launch_pdl(unpermute_kernel, dim3(T * k), dim3(128), 0, s, obuf, inv, out, H);
  return T * k > 0 ? 1 : 0;
}

}  // namespace ek
