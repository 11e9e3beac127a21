// Per-token routing shared by the stand-alone select kernel (route.cu) and the fused front kernel
// for small batches (front_small.cu): split-K partial logits are added in split order, then
// softmax or sigmoid (+ correction bias) scoring, group-limited selection, canonical top-k
// (descending score, ties -> lower index), renormalisation and the histogram.
//
// Replaces the frontend routing of expertkit_torch/models/qwen3_moe.py:161-169 and of the
// DeepSeek-V3 router called at expertkit_torch/models/deepseek_v3/model.py:142.
#pragma once
#include "ek_internal.h"

namespace ek {

// (value, index) argmax over the warp with the canonical tie rule: larger value first, then lower
// index.  Two warp reductions instead of a butterfly of shuffles: the maximum of the values mapped to
// unsigned integers that order like the floats (no NaN reaches this point; -0 is folded into +0 so
// that equal floats map to equal integers), then the lowest index among the lanes that hold it.
// Every lane returns the winner.
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
  const uint32_t b = __float_as_uint(v + 0.0f);
  const uint32_t key = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  const uint32_t best = __reduce_max_sync(0xffffffffu, key);
  idx = (int)__reduce_min_sync(0xffffffffu, key == best ? (uint32_t)idx : 0xffffffffu);
  v = __uint_as_float((best & 0x80000000u) ? (best & 0x7fffffffu) : ~best);
}

// One warp routes token t.  `sc`, `ch`: per-warp scratch of E floats each (unbiased scores, scores used
// for the selection); `gs`: 64 floats (group scores).
__device__ __forceinline__ void select_token(const RouteParams& p, int t, int lane, float* sc, float* ch, float* gs) {
  float* lg = p.logits + (size_t)t * p.E;
  const int E = p.E;
  if (p.partial) {
    // add the split-K partial sums in split order; the softmax path works on bf16 logits like the
    // reference's bf16 linear layer.  Eight experts per lane and eight splits per round: 64
    // independent loads in flight (the loads are what this step costs: a round trip to L2 each round).
    for (int e0 = lane; e0 < E; e0 += 256) {
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k0 = 0; k0 < p.n_partials; k0 += 8) {
        float tmp[8][8];
#pragma unroll
        for (int a = 0; a < 8; ++a)
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int e = e0 + 32 * j;
            tmp[a][j] = (k0 + a < p.n_partials && e < E) ? __ldcg(&p.partial[((size_t)(k0 + a) * p.T + t) * E + e]) : 0.f;
          }
#pragma unroll
        for (int a = 0; a < 8; ++a)
          if (k0 + a < p.n_partials) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] += tmp[a][j];
          }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = e0 + 32 * j;
        if (e < E) lg[e] = p.scoring == EK_SCORE_SOFTMAX ? __bfloat162float(__float2bfloat16_rn(v[j])) : v[j];
      }
    }
    __syncwarp();
  }

  if (p.scoring == EK_SCORE_SOFTMAX) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, lg[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      float ex = expf(lg[e] - m);
      sc[e] = ex;
      sum += ex;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    for (int e = lane; e < E; e += 32) {
      float pr = sc[e] / sum;
      sc[e] = pr;
      ch[e] = pr;
    }
  } else {
    // the correction bias comes from global memory: eight loads in flight, not one per round behind
    // the stores of the round before
    for (int e0 = lane; e0 < E; e0 += 256) {
      float b[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) b[j] = (p.bias && e0 + 32 * j < E) ? __ldg(&p.bias[e0 + 32 * j]) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = e0 + 32 * j;
        if (e < E) {
          float s = 1.f / (1.f + expf(-lg[e]));
          sc[e] = s;
          ch[e] = p.bias ? s + b[j] : s;
        }
      }
    }
  }
  __syncwarp();

  if (p.n_group > 1) {
    const int per = E / p.n_group;
    const int lpg = 32 / p.n_group;          // lanes per group, when the groups divide the warp
    if (p.n_group <= 32 && lpg * p.n_group == 32 && per % lpg == 0) {
      // all lanes at work: a group's members are split over `lpg` neighbouring lanes, each keeps its
      // two largest, a butterfly inside the group merges them (the sum of the two largest does not
      // depend on the order they were found in)
      const int g = lane / lpg, sub = lane % lpg;
      float a = -INFINITY, b = -INFINITY;
      for (int j = sub; j < per; j += lpg) {
        const float v = ch[g * per + j];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      for (int o = lpg >> 1; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, a, o), ob = __shfl_xor_sync(0xffffffffu, b, o);
        if (oa > a) { b = fmaxf(a, ob); a = oa; } else { b = fmaxf(b, oa); }
      }
      if (sub == 0) gs[g] = a + b;
    } else {
      for (int g = lane; g < p.n_group; g += 32) {
        float a = -INFINITY, b = -INFINITY;  // two largest
        for (int j = 0; j < per; ++j) {
          float v = ch[g * per + j];
          if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
        }
        gs[g] = a + b;
      }
    }
    __syncwarp();
    // keep the best topk_group groups (descending score, ties towards the lower group)
    unsigned long long keep = 0ull;
    for (int it = 0; it < p.topk_group; ++it) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < p.n_group; g += 32) {
        if ((keep >> g) & 1ull) continue;
        float v = gs[g];
        if (v > bv || (v == bv && g < bi)) { bv = v; bi = g; }
      }
      warp_argmax(bv, bi);
      keep |= 1ull << bi;
    }
    for (int e = lane; e < E; e += 32)
      if (!((keep >> (e / per)) & 1ull)) ch[e] = 0.0f;
    __syncwarp();
  }

  // top-k, canonical order
  unsigned taken = 0u;  // bit j: element lane + 32*j already selected
  float wsel = 0.f;     // lane i < k keeps the weight of the i-th pick
  int isel = -1;
  if (E <= 256) {
    // the lane's candidates stay in registers over the k rounds
    float mine[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) mine[j] = lane + 32 * j < E ? ch[lane + 32 * j] : -INFINITY;
    for (int it = 0; it < p.k; ++it) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = lane + 32 * j;
        if (e < E && !((taken >> j) & 1u) && (mine[j] > bv || (mine[j] == bv && e < bi))) { bv = mine[j]; bi = e; }
      }
      warp_argmax(bv, bi);
      if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
      if (lane == it) {
        isel = bi;
        wsel = sc[bi];
      }
    }
  } else {
    for (int it = 0; it < p.k; ++it) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int j = 0, e = lane; e < E; ++j, e += 32) {
        if ((taken >> j) & 1u) continue;
        float v = ch[e];
        if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
      }
      warp_argmax(bv, bi);
      if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
      if (lane == it) {
        isel = bi;
        wsel = sc[bi];
      }
    }
  }
  // renormalise: sequential sum in slot order (lane 0 .. k-1)
  float denom = 0.f;
  for (int i = 0; i < p.k; ++i) denom += __shfl_sync(0xffffffffu, wsel, i);
  if (lane < p.k) {
    float w = wsel;
    if (p.norm) w = (p.scoring == EK_SCORE_SOFTMAX) ? w / denom : w / (denom + 1e-20f);
    if (p.scoring != EK_SCORE_SOFTMAX) w *= p.scaling;
    if (p.bf16_weights) w = __bfloat162float(__float2bfloat16_rn(w));
    p.ids[(size_t)t * p.k + lane] = isel;
    p.weights[(size_t)t * p.k + lane] = w;
    atomicAdd(&p.counts[isel], 1);
  }
}

}  // namespace ek
