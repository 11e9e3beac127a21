// Router logits on the tensor cores: partial[ks][t][e] = sum over the ks-th K range of
// x[t,:] * Wg[e,:], bf16 operands, fp32 accumulation in tensor memory.  Split along K so that a
// handful of token tiles still fill the GPU; the select kernel adds the partial sums in a fixed
// order (deterministic, no atomics).
//
// Replaces `self.gate(hidden_states)` (expertkit_torch/models/qwen3_moe.py:161) and the linear
// layer of the DeepSeek-V3 router called at expertkit_torch/models/deepseek_v3/model.py:142 for
// router weights that are exactly representable in bf16 (products of bf16 values are exact in
// fp32, so only the summation order differs from an fp32 evaluation).
#include "ek_internal.h"
#include "peer_sync.cuh"
#include "ptx.cuh"

namespace ek {

namespace {

using namespace ekptx;

constexpr int kStages = 4;
constexpr int kTokTile = 128;
constexpr int kAtomBytesA = kTokTile * 128;   // 128 token rows x 64 bf16

__global__ void __launch_bounds__(192, 1) router_tc_kernel(const __grid_constant__ RouterTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages], bar_empty[kStages], bar_acc;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t b_bytes = (uint32_t)p.E * 128;
  const uint32_t stage_bytes = kAtomBytesA + b_bytes;
  volatile int* abortp = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(&bar_full[i]), 1);
      mbar_init(smem_u32(&bar_empty[i]), 1);
    }
    mbar_init(smem_u32(&bar_acc), 1);
    mbar_init_fence();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&s_tmem), p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  pdl_wait();
  pdl_trigger();
  if (p.zero_counts && blockIdx.x == 0 && blockIdx.y == 0)
    for (int i = tid; i < p.E; i += blockDim.x) p.zero_counts[i] = 0;
  const int m0 = blockIdx.x * kTokTile;
  const int a_lo = blockIdx.y * p.atoms_per_split;
  const int a_hi = min(a_lo + p.atoms_per_split, p.n_atoms);
  const int n_it = a_hi - a_lo;

  if (p.wait.flags) {
    // the activations are stored by the peers: every rank's step number first (one warp, a lane per
    // rank), then the TMA reads (async proxy) are ordered behind the acquiring loads (generic proxy)
    if (warp == 4) {
      if (!warp_wait_ranks(p.wait, p.status, lane) && lane == 0) *abortp = 1;
      fence_proxy_async_all();
    }
    __syncthreads();
  }
  const bool go = *abortp == 0;
  if (warp == 4) {
    if (lane == 0 && go) {
      for (int i = 0; i < n_it; ++i) {
        const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
        if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abortp)) break;
        const uint32_t full = smem_u32(&bar_full[s]);
        const uint32_t dst = base + s * stage_bytes;
        mbar_arrive_expect_tx(full, stage_bytes);
        tma_load_2d(dst, &p.x_map, (a_lo + i) * 64, m0, full);
        tma_load_2d(dst + kAtomBytesA, &p.w_map, (a_lo + i) * 64, 0, full);
      }
      // copies in flight land before the CTA leaves
      const int lo = n_it > kStages ? n_it - kStages : 0;
      for (int i = lo; i < n_it; ++i)
        for (uint32_t poll = 0; poll < (1u << 20); ++poll) {
          if (mbar_try_wait(smem_u32(&bar_full[i % kStages]), (i / kStages) & 1u)) break;
          __nanosleep(64);
        }
    }
  } else if (warp == 5) {
    if (lane == 0 && go) {
      const uint32_t idesc = umma_idesc_bf16(p.E);
      bool ok = true;
      for (int i = 0; i < n_it; ++i) {
        const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
        if (!mbar_wait(smem_u32(&bar_full[s]), ph, abortp)) { ok = false; break; }
        tc_fence_after();
        const uint64_t a0 = umma_desc_sw128(base + s * stage_bytes);
        const uint64_t b0 = umma_desc_sw128(base + s * stage_bytes + kAtomBytesA);
        uint64_t ad[4], bd[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { ad[j] = a0 + j * 2; bd[j] = b0 + j * 2; }
        umma_ss_x4(tmem, ad, bd, idesc, i > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_empty[s]));
      }
      if (ok) tc_commit(smem_u32(&bar_acc));
      if (!ok && atomicCAS(&p.status->code, DEV_OK, DEV_TIMEOUT) == DEV_OK) p.status->where = 400;
    }
  } else {
    // epilogue: thread = token row, 16 experts per tcgen05.ld
    if (n_it > 0 && go) {
      if (mbar_wait(smem_u32(&bar_acc), 0, abortp)) {
        tc_fence_after();
        const int t = m0 + warp * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        float* dst = p.partial + ((size_t)blockIdx.y * p.T + t) * p.E;
        for (int c = 0; c < p.E; c += 16) {
          uint32_t v[16];
          tmem_ld16_wait(lane_base + c, v);
          if (t < p.T) {
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              *reinterpret_cast<float4*>(dst + c + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                    __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
          }
        }
      } else if (atomicCAS(&p.status->code, DEV_OK, DEV_TIMEOUT) == DEV_OK) {
        p.status->where = 401;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, p.tmem_cols);
  }
}

__global__ void f32_to_bf16_check_kernel(const float* src, __nv_bfloat16* dst, int64_t n, int32_t* inexact) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = src[i];
  const __nv_bfloat16 b = __float2bfloat16_rn(v);
  dst[i] = b;
  if (__bfloat162float(b) != v) atomicOr(inexact, 1);
}

}  // namespace

bool router_tc_supported(int E, int H) { return E >= 16 && E <= 256 && E % 16 == 0 && H % 8 == 0; }

// Chooses the K split: enough CTAs to cover the GPU, at least one 64-element atom each.
void router_tc_plan(int T, int H, int n_sm, int* n_splits, int* atoms_per_split) {
  const int n_atoms = (H + 63) / 64;
  const int m_tiles = (T + kTokTile - 1) / kTokTile;
  int ks = n_sm / m_tiles;
  if (ks > 16) ks = 16;   // the select kernel adds the partial sums serially: keep that chain short
  if (ks < 1) ks = 1;
  if (ks > n_atoms) ks = n_atoms;
  const int per = (n_atoms + ks - 1) / ks;
  *atoms_per_split = per;
  *n_splits = (n_atoms + per - 1) / per;
}

int launch_router_tc(const RouterTcParams& p, cudaStream_t s) {
  const int smem = kStages * (kAtomBytesA + p.E * 128) + 1024;
  cudaFuncSetAttribute(router_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  dim3 grid((p.T + kTokTile - 1) / kTokTile, p.n_splits);
  launch_pdl(router_tc_kernel, grid, dim3(192), (size_t)smem, s, p);
  return 1;
}

int launch_f32_to_bf16_check(const float* src, __nv_bfloat16* dst, int64_t n, int32_t* inexact, cudaStream_t s) {
  f32_to_bf16_check_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, dst, n, inexact);
  return 1;
}

}  // namespace ek
