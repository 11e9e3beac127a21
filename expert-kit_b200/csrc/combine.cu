// Weighted unpermute-combine and the plain unpermute.
//
// combine: y[t] = sum_k w[t,k] * out[t,k] (+ shared(x)[t]) -- the frontend's step after the
// expert outputs return (expertkit_torch/models/deepseek_v3/model.py:96-104,152;
// expertkit_torch/models/qwen3_moe.py:102-104).
// unpermute: out[t,s,:] = row of (t,s) -- NaiveExecutor's scatter + two-level stack
// (ek-computation/src/controller/executor.rs:203-251).
#include "ek_internal.h"

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

// One CTA per token, 128-bit loads of the k expert rows, fp32 accumulation in slot order.
__global__ void __launch_bounds__(256) combine_kernel(CombineParams p) {
  __shared__ int s_row[kMaxK];
  __shared__ float s_w[kMaxK];
  const int t = blockIdx.x;
  if (threadIdx.x < p.k) {
    s_row[threadIdx.x] = p.inv[(size_t)t * p.k + threadIdx.x];
    s_w[threadIdx.x] = p.weights[(size_t)t * p.k + threadIdx.x];
  }
  __syncthreads();
  for (int v = threadIdx.x; v < p.H / 8; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < p.k; ++s) {
      const int row = s_row[s];
      if (row < 0) continue;
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(p.obuf + (size_t)row * p.H + v * 8), f);
      const float w = s_w[s];
      if (p.bf16_products) {
        // routing weights were rounded to bf16 upstream; products are bf16 tensors
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], round_bf16(__fmul_rn(w, f[j])));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(w, f[j]));
      }
    }
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

__global__ void __launch_bounds__(256) combine_partial_kernel(CombineParams p, float* __restrict__ partial) {
  __shared__ int s_row[kMaxK];
  __shared__ float s_w[kMaxK];
  const int t = blockIdx.x;
  if (threadIdx.x < p.k) {
    s_row[threadIdx.x] = p.inv[(size_t)t * p.k + threadIdx.x];
    s_w[threadIdx.x] = p.weights[(size_t)t * p.k + threadIdx.x];
  }
  __syncthreads();
  for (int v = threadIdx.x; v < p.H / 8; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < p.k; ++s) {
      const int row = s_row[s];
      if (row < 0) continue;
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(p.obuf + (size_t)row * p.H + v * 8), f);
      const float w = s_w[s];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        acc[j] = __fadd_rn(acc[j], p.bf16_products ? round_bf16(__fmul_rn(w, f[j])) : __fmul_rn(w, f[j]));
    }
    float4* d = reinterpret_cast<float4*>(partial + (size_t)t * p.H + v * 8);
    d[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    d[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

__global__ void __launch_bounds__(256) combine_finish_kernel(const float* __restrict__ reduced,
                                                             const __nv_bfloat16* __restrict__ shared,
                                                             int32_t n_shared, int32_t T, int32_t H,
                                                             __nv_bfloat16* __restrict__ y) {
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
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

int launch_combine_partial(const CombineParams& p, float* partial, cudaStream_t s) {
  if (p.T > 0) combine_partial_kernel<<<p.T, 256, 0, s>>>(p, partial);
  return p.T > 0 ? 1 : 0;
}
int launch_combine_finish(const float* reduced, const __nv_bfloat16* shared, int32_t n_shared, int32_t T,
                          int32_t H, __nv_bfloat16* y, cudaStream_t s) {
  if (T > 0) combine_finish_kernel<<<T, 256, 0, s>>>(reduced, shared, n_shared, T, H, y);
  return T > 0 ? 1 : 0;
}

int launch_combine(const CombineParams& p, cudaStream_t s) {
  if (p.T > 0) combine_kernel<<<p.T, 256, 0, s>>>(p);
  return p.T > 0 ? 1 : 0;
}

int launch_unpermute(const __nv_bfloat16* obuf, const int32_t* inv, __nv_bfloat16* out, int32_t T,
                     int32_t k, int32_t H, cudaStream_t s) {
  if (T * k > 0) unpermute_kernel<<<T * k, 128, 0, s>>>(obuf, inv, out, H);
  return T * k > 0 ? 1 : 0;
}

}  // namespace ek
