// Router: logits = x . Wg^T, scoring (softmax or sigmoid with group-limited selection),
// canonical top-k and the per-expert histogram.
//
// Replaces the frontend routing of expertkit_torch/models/qwen3_moe.py:161-169 and of the
// DeepSeek-V3 router called at expertkit_torch/models/deepseek_v3/model.py:142.
#include "ek_internal.h"
#include "route_select.cuh"

namespace ek {

namespace {

constexpr int kTokTile = 8;     // tokens per CTA
constexpr int kExpTile = 32;    // experts per CTA (4 per warp)
constexpr int kHChunk = 2048;   // activations staged per pass (bf16, 32 KiB)

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// logits[t,e] = sum_h x[t,h] * wg[e,h], fp32 accumulation of exact bf16 x bf16 (or bf16 x
// fp32) products.  For softmax scoring the reference evaluates the linear layer in bf16, so
// the result is rounded to bf16 (and stored widened).
template <bool WG_F32>
__global__ void __launch_bounds__(256) router_logits_kernel(RouteParams p) {
  pdl_wait();
  pdl_trigger();
  __shared__ __align__(16) __nv_bfloat16 xs[kTokTile][kHChunk];
  const int t0 = blockIdx.x * kTokTile;
  const int e0 = blockIdx.y * kExpTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float acc[4][kTokTile];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int t = 0; t < kTokTile; ++t) acc[i][t] = 0.f;

  for (int h0 = 0; h0 < p.H; h0 += kHChunk) {
    const int hc = min(kHChunk, p.H - h0);
    __syncthreads();
    // stage activations (16-byte vectors; H is a multiple of 8)
    for (int i = threadIdx.x; i < kTokTile * (hc / 8); i += blockDim.x) {
      int t = i / (hc / 8), v = i % (hc / 8);
      uint4 val = make_uint4(0, 0, 0, 0);
      if (t0 + t < p.T)
        val = *reinterpret_cast<const uint4*>(p.x + (size_t)(t0 + t) * p.H + h0 + v * 8);
      *reinterpret_cast<uint4*>(&xs[t][v * 8]) = val;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = e0 + warp * 4 + i;
      if (e >= p.E) continue;
      for (int v = lane; v < hc / 8; v += 32) {
        float w[8];
        if (WG_F32) {
          const float4* src = reinterpret_cast<const float4*>(
              reinterpret_cast<const float*>(p.wg) + (size_t)e * p.H + h0 + v * 8);
          float4 a = src[0], b = src[1];
          w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
          w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        } else {
          uint4 raw = *reinterpret_cast<const uint4*>(
              reinterpret_cast<const __nv_bfloat16*>(p.wg) + (size_t)e * p.H + h0 + v * 8);
          unpack8(raw, w);
        }
#pragma unroll
        for (int t = 0; t < kTokTile; ++t) {
          float xf[8];
          unpack8(*reinterpret_cast<const uint4*>(&xs[t][v * 8]), xf);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][t] = fmaf(xf[j], w[j], acc[i][t]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = e0 + warp * 4 + i;
#pragma unroll
    for (int t = 0; t < kTokTile; ++t) {
      float v = acc[i][t];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && e < p.E && t0 + t < p.T) {
        if (p.scoring == EK_SCORE_SOFTMAX) v = __bfloat162float(__float2bfloat16_rn(v));
        p.logits[(size_t)(t0 + t) * p.E + e] = v;
      }
    }
  }
}

constexpr int kMaxExperts = 1024;
constexpr int kSelWarps = 4;

// One warp per token.
__global__ void __launch_bounds__(kSelWarps * 32) route_select_kernel(RouteParams p) {
  pdl_wait();
  pdl_trigger();
  __shared__ float s_score[kSelWarps][kMaxExperts];   // unbiased scores (weights come from these)
  __shared__ float s_choice[kSelWarps][kMaxExperts];  // biased / masked scores used for selection
  __shared__ float s_group[kSelWarps][64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kSelWarps + warp;
  if (t >= p.T) return;
  select_token(p, t, lane, s_score[warp], s_choice[warp], s_group[warp]);
}

__global__ void histogram_kernel(const int32_t* ids, int32_t n, int32_t E, int32_t* counts,
                                 DevStatus* st) {
  pdl_wait();
  pdl_trigger();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int e = ids[i];
  if (e < 0 || e >= E) {
    if (atomicCAS(&st->code, DEV_OK, DEV_BOUNDS) == DEV_OK) {
      st->where = 1;
      st->aux0 = i;
      st->aux1 = e;
    }
    return;
  }
  atomicAdd(&counts[e], 1);
}

}  // namespace

int launch_router_logits(const RouteParams& p, cudaStream_t s) {
  dim3 grid((p.T + kTokTile - 1) / kTokTile, (p.E + kExpTile - 1) / kExpTile);
  if (p.wg_f32)
    launch_pdl(router_logits_kernel<true>, grid, dim3(256), 0, s, p);
  else
    launch_pdl(router_logits_kernel<false>, grid, dim3(256), 0, s, p);
  return 1;
}

int launch_route_select(const RouteParams& p, cudaStream_t s, bool counts_cleared) {
  if (!counts_cleared) cudaMemsetAsync(p.counts, 0, sizeof(int32_t) * p.E, s);
  launch_pdl(route_select_kernel, dim3((p.T + kSelWarps - 1) / kSelWarps), dim3(kSelWarps * 32), 0, s, p);
  return 1;
}

int launch_histogram(const int32_t* ids, int32_t n, int32_t E, int32_t* counts, DevStatus* st,
                     cudaStream_t s) {
  cudaMemsetAsync(counts, 0, sizeof(int32_t) * E, s);
  if (n > 0) launch_pdl(histogram_kernel, dim3((n + 255) / 256), dim3(256), 0, s, ids, n, E, counts, st);
  return n > 0 ? 1 : 0;
}

}  // namespace ek
