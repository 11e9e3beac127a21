// CUDA-core evaluation of the grouped SwiGLU FFN over the tiled weight layout.
//
// It computes the same function as the tensor-core kernels in ffn_tc.cu from the same device
// buffers, with one thread per weight row and the reference's own dequantisation formula
// (bf16_rne(float(w) * scale), ek-computation/src/ffn/expert_torch.rs:24-53).  The tests use it
// as a second, independent evaluation at sizes the CPU checker cannot reach; it is not a
// performance path.
#include <cuda_fp8.h>

#include "ek_internal.h"

namespace ek {

namespace {

constexpr int kRows = 16;  // activation rows per CTA (== chunk_rows of the work list)

template <int QUANT>
__device__ __forceinline__ void decode16(const uint4& raw, float scale, float* out) {
  if (QUANT == EK_QUANT_BF16) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __bfloat1622float2(p[i]);
      out[2 * i] = t.x;
      out[2 * i + 1] = t.y;
    }
  } else {
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float v;
      if (QUANT == EK_QUANT_FP8_BLOCK128) {
        __nv_fp8_e4m3 q;
        q.__x = b[i];
        v = static_cast<float>(q);
      } else {
        v = static_cast<float>(static_cast<int>(b[i]) - 128);   // tiles keep int8 codes in offset binary
      }
      out[i] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(v, scale)));
    }
  }
}

// One tile row of this thread times the staged activations.
template <int QUANT>
__device__ __forceinline__ void row_times_x(const uint8_t* tile, int r, float scale,
                                            const float (*xs)[128], float* acc) {
  constexpr int EPC = QUANT == EK_QUANT_BF16 ? 8 : 16;  // elements per 16-byte chunk
#pragma unroll 1
  for (int j = 0; j < kChunksPerRow; ++j) {
    const uint4 raw = *reinterpret_cast<const uint4*>(tile + (size_t)(j * kTileRows + r) * 16);
    float w[16];
    decode16<QUANT>(raw, scale, w);
#pragma unroll
    for (int e = 0; e < EPC; ++e) {
      const float wv = w[e];
#pragma unroll
      for (int t = 0; t < kRows; ++t) acc[t] = fmaf(xs[t][j * EPC + e], wv, acc[t]);
    }
  }
}

template <int QUANT>
__global__ void __launch_bounds__(128) simt_gateup_kernel(FfnParams p) {
  __shared__ float xs[kRows][128];
  const int c = blockIdx.x;
  if (c >= *p.n_chunks) return;
  ChunkDesc cd = p.chunks[c];
  cd.n_rows &= kChunkRowsMask;
  const int it = blockIdx.y, r = threadIdx.x;
  const int TK = QUANT == EK_QUANT_BF16 ? 64 : 128;
  float ag[kRows], au[kRows];
#pragma unroll
  for (int t = 0; t < kRows; ++t) ag[t] = au[t] = 0.f;
  const size_t tile0 = ((size_t)cd.slot * p.d.it + it) * p.d.kt_gu * 2;
  for (int kt = 0; kt < p.d.kt_gu; ++kt) {
    __syncthreads();
    for (int i = threadIdx.x; i < kRows * TK; i += blockDim.x) {
      const int t = i / TK, col = kt * TK + i % TK;
      float v = 0.f;
      if (t < cd.n_rows && col < p.d.H) v = __bfloat162float(p.xp[(size_t)(cd.in_row + t) * p.d.H + col]);
      xs[t][i % TK] = v;
    }
    __syncthreads();
    const uint8_t* tg = p.w.gu_tiles + (tile0 + (size_t)kt * 2) * kTileBytes;
    float sg = 1.f, su = 1.f;
    if (QUANT != EK_QUANT_BF16) {
      sg = p.w.gu_scale[(tile0 + (size_t)kt * 2)];
      su = p.w.gu_scale[(tile0 + (size_t)kt * 2) + 1];
    }
    row_times_x<QUANT>(tg, r, sg, xs, ag);
    row_times_x<QUANT>(tg + kTileBytes, r, su, xs, au);
  }
  const int o = it * kTileRows + r;
#pragma unroll
  for (int t = 0; t < kRows; ++t) {
    if (t < cd.n_rows) {
      const float g = ag[t], u = au[t];
      const float h = u * (g / (1.f + expf(-g)));
      p.hbuf[(size_t)(cd.out_row + t) * p.d.Ip + o] = __float2bfloat16_rn(h);
    }
  }
}

template <int QUANT>
__global__ void __launch_bounds__(128) simt_down_kernel(FfnParams p) {
  __shared__ float xs[kRows][128];
  const int c = blockIdx.x;
  if (c >= *p.n_chunks) return;
  ChunkDesc cd = p.chunks[c];
  cd.n_rows &= kChunkRowsMask;
  const int ht = blockIdx.y, r = threadIdx.x;
  const int TK = QUANT == EK_QUANT_BF16 ? 64 : 128;
  float acc[kRows];
#pragma unroll
  for (int t = 0; t < kRows; ++t) acc[t] = 0.f;
  // tile (ht, kt) of the pair-interleaved down layout
  const size_t tile0 = ((size_t)cd.slot * p.d.hp + (ht >> 1)) * p.d.kt_dn * 2 + (ht & 1);
  for (int kt = 0; kt < p.d.kt_dn; ++kt) {
    __syncthreads();
    for (int i = threadIdx.x; i < kRows * TK; i += blockDim.x) {
      const int t = i / TK, col = kt * TK + i % TK;
      float v = 0.f;
      if (t < cd.n_rows && col < p.d.Ip) v = __bfloat162float(p.hbuf[(size_t)(cd.out_row + t) * p.d.Ip + col]);
      xs[t][i % TK] = v;
    }
    __syncthreads();
    const uint8_t* tw = p.w.dn_tiles + (tile0 + (size_t)kt * 2) * kTileBytes;
    float s = 1.f;
    if (QUANT != EK_QUANT_BF16) s = p.w.dn_scale[tile0 + (size_t)kt * 2];
    row_times_x<QUANT>(tw, r, s, xs, acc);
  }
  const int hcol = ht * kTileRows + r;
  if (hcol < p.d.H) {
#pragma unroll
    for (int t = 0; t < kRows; ++t)
      if (t < cd.n_rows) p.obuf[(size_t)(cd.out_row + t) * p.d.H + hcol] = __float2bfloat16_rn(acc[t]);
  }
}

}  // namespace

int launch_ffn_simt(const FfnParams& p, int which, cudaStream_t s) {
  if (p.max_chunks <= 0) return 0;
  // blocks beyond the device-side chunk count leave at once
  dim3 g(p.max_chunks, which == 0 ? p.d.it : p.d.ht);
#define EK_SIMT_LAUNCH(Q)                                     \
  do {                                                        \
    if (which == 0) simt_gateup_kernel<Q><<<g, 128, 0, s>>>(p); \
    else simt_down_kernel<Q><<<g, 128, 0, s>>>(p);            \
  } while (0)
  switch (p.d.quant) {
    case EK_QUANT_BF16: EK_SIMT_LAUNCH(EK_QUANT_BF16); break;
    case EK_QUANT_FP8_BLOCK128: EK_SIMT_LAUNCH(EK_QUANT_FP8_BLOCK128); break;
    default: EK_SIMT_LAUNCH(EK_QUANT_INT8_BLOCK128); break;
  }
#undef EK_SIMT_LAUNCH
  return 1;
}

}  // namespace ek
