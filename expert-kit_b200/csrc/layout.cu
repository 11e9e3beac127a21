// Registration-time layout kernels: re-tile row-major expert weights into the 16 KiB tiles
// the GEMM kernels stream (int8 codes are kept in offset binary, b ^ 0x80, which saves the GEMM's
// converters an instruction per weight pair), re-order the block scales to match, and the stand-alone block
// dequantisation (w8a16_activate, ek-computation/src/ffn/expert_torch.rs:24-53).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "ek_internal.h"

namespace ek {

namespace {

// One CTA per tile; thread handles 4 of the tile's 1024 16-byte chunks.
__global__ void __launch_bounds__(256) retile_kernel(RetileParams p) {
  const int rt = blockIdx.y, kt = blockIdx.x;
  uint8_t* tile = p.rt_pairs ? p.dst + ((int64_t)((rt >> 1) * p.n_kt + kt) * 2 + (rt & 1)) * kTileBytes
                             : p.dst + (int64_t)rt * p.rt_stride + (int64_t)kt * p.kt_stride;
  const uint8_t* src = reinterpret_cast<const uint8_t*>(p.src);
  const int64_t row_bytes = (int64_t)p.cols * p.esz;
  const bool vec_ok = (row_bytes % 16 == 0) && (((int64_t)p.col0 * p.esz) % 16 == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.src) & 15) == 0);
  for (int c = threadIdx.x; c < kTileRows * kChunksPerRow; c += blockDim.x) {
    const int j = c / kTileRows, r = c % kTileRows;   // chunk j of row r
    const int lr = rt * kTileRows + r;                // row inside the window
    const int64_t lcb = (int64_t)kt * 128 + j * 16;   // byte column inside the window
    const int64_t win_bytes = (int64_t)p.n_cols * p.esz;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (lr < p.n_rows && lcb < win_bytes) {
      const uint8_t* s = src + (int64_t)(p.row0 + lr) * row_bytes + (int64_t)p.col0 * p.esz + lcb;
      if (vec_ok && lcb + 16 <= win_bytes) {
        v = *reinterpret_cast<const uint4*>(s);
      } else {
        uint8_t tmp[16];
#pragma unroll
        for (int b = 0; b < 16; ++b) tmp[b] = (lcb + b < win_bytes) ? s[b] : 0;
        v = *reinterpret_cast<uint4*>(tmp);
      }
    }
    v.x ^= p.xor_mask; v.y ^= p.xor_mask; v.z ^= p.xor_mask; v.w ^= p.xor_mask;   // padding zeros become code 0 too
    *reinterpret_cast<uint4*>(tile + (size_t)(j * kTileRows + r) * 16) = v;
  }
}

__global__ void scale_retile_kernel(ScaleRetileParams p) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= p.n_rt * p.n_kt) return;
  const int rt = i / p.n_kt, kt = i % p.n_kt;
  const int sr = p.rb0 + rt, scol = p.kb0 + kt;
  float v = 0.f;
  if (sr < p.src_rows && scol < p.src_cols) v = p.src[(size_t)sr * p.src_cols + scol];
  if (p.rt_pairs) p.dst[((size_t)(rt >> 1) * p.n_kt + kt) * 2 + (rt & 1)] = v;
  else p.dst[(size_t)i * p.stride + p.lane] = v;
}

// out[0] = 2^c with max|scale| * 2^c in (2^-5, 2^-4]: the power of two that keeps the scaled
// activation operand of the GEMM (x * block scale * 2^c) in the middle of the f16 range.
__global__ void __launch_bounds__(256) scale_pow_kernel(const float* a, int64_t na, const float* b, int64_t nb, float* out) {
  __shared__ float s_max[256];
  float m = 0.f;
  for (int64_t i = threadIdx.x; i < na; i += 256) m = fmaxf(m, fabsf(a[i]));
  for (int64_t i = threadIdx.x; i < nb; i += 256) m = fmaxf(m, fabsf(b[i]));
  s_max[threadIdx.x] = m;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) s_max[threadIdx.x] = fmaxf(s_max[threadIdx.x], s_max[threadIdx.x + o]);
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float mx = s_max[0];
    float pw = 1.f;
    if (mx > 0.f && isfinite(mx)) {
      int e;
      frexpf(mx, &e);                 // mx = f * 2^e, f in [0.5, 1)
      pw = ldexpf(1.f, -e - 4);       // mx * pw in [2^-5, 2^-4)
    }
    out[0] = pw;
  }
}

__global__ void fill_f32_kernel(float* dst, float v, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = v;
}

__global__ void f16_to_bf16_kernel(const __half* src, __nv_bfloat16* dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2bfloat16_rn(__half2float(src[i]));
}

// out[i,j] = bf16_rne(float(w[i,j]) * scale[i/128, j/128])
template <int WDT>
__global__ void dequant_kernel(const uint8_t* w, const float* scale, int rows, int cols,
                               __nv_bfloat16* out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)rows * cols) return;
  const int r = (int)(i / cols), c = (int)(i % cols);
  const float s = scale[(size_t)(r / 128) * ((cols + 127) / 128) + c / 128];
  float v;
  if (WDT == EK_F8_E4M3) {
    __nv_fp8_e4m3 q;
    q.__x = w[i];
    v = static_cast<float>(q);
  } else {
    v = static_cast<float>(static_cast<int8_t>(w[i]));
  }
  out[i] = __float2bfloat16_rn(__fmul_rn(v, s));
}

}  // namespace

int launch_retile(const RetileParams& p, cudaStream_t s) {
  dim3 grid(p.n_kt, p.n_rt);
  retile_kernel<<<grid, 256, 0, s>>>(p);
  return 1;
}
int launch_scale_retile(const ScaleRetileParams& p, cudaStream_t s) {
  const int n = p.n_rt * p.n_kt;
  scale_retile_kernel<<<(n + 255) / 256, 256, 0, s>>>(p);
  return 1;
}
int launch_scale_pow(const float* a, int64_t na, const float* b, int64_t nb, float* out, cudaStream_t s) {
  scale_pow_kernel<<<1, 256, 0, s>>>(a, na, b, nb, out);
  return 1;
}
int launch_fill_f32(float* dst, float v, int64_t n, cudaStream_t s) {
  fill_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(dst, v, n);
  return 1;
}
int launch_f16_to_bf16(const void* src, __nv_bfloat16* dst, int64_t n, cudaStream_t s) {
  f16_to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(reinterpret_cast<const __half*>(src), dst, n);
  return 1;
}
int launch_dequant(const void* w, int32_t w_dtype, const float* scale, int32_t rows, int32_t cols,
                   __nv_bfloat16* out, cudaStream_t s) {
  const int64_t n = (int64_t)rows * cols;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (w_dtype == EK_F8_E4M3)
    dequant_kernel<EK_F8_E4M3><<<blocks, 256, 0, s>>>(reinterpret_cast<const uint8_t*>(w), scale, rows, cols, out);
  else
    dequant_kernel<EK_I8><<<blocks, 256, 0, s>>>(reinterpret_cast<const uint8_t*>(w), scale, rows, cols, out);
  return 1;
}

}  // namespace ek
