// Grouped SwiGLU expert FFN on the 5th-generation tensor cores (tcgen05 + tensor memory),
// fed by TMA, for sm_100a.  Replaces the three libtorch matmuls of TorchFFN::forward
// (ek-computation/src/ffn/expert_torch.rs:80-85) and the block dequantisation of
// w8a16_activate (expert_torch.rs:24-53) for ALL experts of a layer in two launches.
//
// Formulation ("weights as the M operand"): for one work item (chunk of <= NMAX activation
// rows of one expert, one pair of 128-row weight tiles)
//        D[128 weight rows, N rows of x] (+)= W_tile[128, K] * X_chunk[N, K]^T
// so the MMA always runs at M = 128 no matter how few tokens an expert received, and the
// weight stream - the thing that is HBM-bound at decode batch sizes - is read exactly once.
//
// Roles of the 640 threads of a CTA (one persistent CTA per SM):
//   2 producer threads : one bulk-copies the next 32 KiB of weight tiles (fp8 / int8 / bf16,
//                        already laid out for conflict-free reads) into the stage ring, the
//                        other TMA-loads the matching [N, K] activation tile (128-byte swizzle)
//   16 converter warps : two groups of 8 on alternating K steps.  Thread r reads weight row r
//                        of its tile from shared memory, turns it into the 16-bit A operand and
//                        stores it into tensor memory with tcgen05.st (the A operand never goes
//                        back through shared memory).  How the block scale is applied depends on
//                        the mode, see below.  The same warps run the epilogue.
//   2 MMA threads      : each issues tcgen05.mma for one of the two tiles of a stage (A from
//                        tensor memory, B from shared memory through a swizzled descriptor,
//                        fp32 accumulators in tensor memory): one thread's instruction stream
//                        between MMAs costs about as much as the MMAs take.
//
// Quantised weights (fp8 e4m3 / int8 with one fp32 scale per 128x128 block; K tile == scale block).
// The activations of these GEMMs are kept in f16 (the gather kernel and the gate/up epilogue write
// f16: exact for bf16 inputs inside the f16 range, saturating outside) and the weights are converted
// EXACTLY to f16 with no arithmetic: cvt.rn.f16x2.e4m3x2, or for int8 a magic-number subtraction - 2
// instructions per 4 weights.  kind::f16 needs both operands in the same 16-bit type (an f16 A with
// a bf16 B is an illegal instruction).  Where the block scale s goes depends on the chunk size:
//   scale-on-B  (chunks of <= 64 rows) the converters of the step rewrite the activation tile as
//               f16(x * s * 2^c) before the MMA reads it, one scaled copy per tile of the stage.  One
//               rounding per product term, to 11 bits, on the activation factor - where the
//               reference's bf16(w * s) * x rounds the weight factor to 8 bits.
//   scale-on-A  (128-row chunks: rewriting 128 activation rows per step costs more than scaling 128
//               weight rows) A = f16(w) * (s * 2^c') as a two-term packed f16 multiply, B = the f16
//               activations as TMA delivers them.
//   c, c' are powers of two per expert and GEMM, chosen at registration from the largest block
//   scale so that the scaled operand sits in the middle of the f16 range; the epilogue multiplies
//   the accumulators by 2^-c.
//   reference   (ek_set_precise_dequant) A = bf16_rne(float(w) * s), bf16 activations: the bit-exact
//               reference formula (expert_torch.rs:24-53), about 6 instructions per weight pair.
// bf16 weights pass through unconverted.
//
// Work decomposition: items are strided over the CTAs; the items left over after the last full
// wave are cut along K into equal parts over all CTAs ("stream-K tail").  The CTA holding the
// first part of a split item is its owner: the others leave fp32 partial accumulators in a
// scratch buffer and raise a flag, the owner adds them in part order (deterministic) before its
// epilogue and clears the flags.  A CTA computes the part it does not own FIRST and the part it
// owns LAST, so the owner practically never waits.
//
// Every wait (mbarrier or flag) is bounded; on a timeout the CTA records DEV_TIMEOUT in the
// status word, drains what it has in flight, frees its tensor memory and leaves.
#include <cuda_fp16.h>

#include <type_traits>

#include "ek_internal.h"
#include "ptx.cuh"

namespace ek {

namespace {

using namespace ekptx;

// Converter warps come in two groups of 8 (two warpgroups each: one per tile of the stage, one
// warp per tensor-memory lane quarter).  A group converts every other K step: two steps are in
// conversion at any time and each scheduler holds four converter warps whose dense phases overlap.
constexpr int kConvWarps = 16;
constexpr int kGroupWarps = 8;
constexpr int kGroups = kConvWarps / kGroupWarps;
static_assert(kGroups == 2, "the stage / A-slot protocol below is written for two converter groups");
constexpr int kMmaWarps = 2;
constexpr int kProdWarps = 2;                 // weight ring, activation ring: one warp each
constexpr int kFirstMmaWarp = kConvWarps + kProdWarps;
constexpr int kThreads = (kConvWarps + kProdWarps + kMmaWarps) * 32;
constexpr int kASlotCols = 64;   // tensor-memory columns per A staging slot (128 16-bit values along K)
constexpr int kTmemCols = 512;
constexpr int kMaxASlots = 6;
constexpr int kSmemLimit = 232448 - 4096;
constexpr int kMinPart = 8;      // K steps: smallest part of a split work item

enum { kModeRaw = 0, kModeScaleB2 = 1, kModeScaleAH = 2, kModeScaleA = 3 };

template <int QUANT, bool GATEUP, int NMAX, int MODE>
struct Cfg {
  static constexpr int TKE = QUANT == EK_QUANT_BF16 ? 64 : 128;   // K elements per tile
  // A stage holds two weight tiles of the same K step, one per converter warpgroup / MMA chain,
  // and the activation tile both multiply (two scaled copies of it in mode ScaleB2):
  //   gate/up : the gate and the up tile of intermediate-row tile rt
  //   down    : the tiles of hidden-row tiles 2*rp and 2*rp+1
  static constexpr int W_BYTES = 2 * kTileBytes;
  static constexpr int X_ATOMS = TKE / 64;                        // 64-element swizzle atoms along K
  static constexpr int X_BYTES = NMAX * X_ATOMS * 128;
  static constexpr int X_COPIES = MODE == kModeScaleB2 ? 2 : 1;
  static constexpr int STAGE_BYTES = W_BYTES + X_COPIES * X_BYTES;
  static constexpr int STAGES_RAW = kSmemLimit / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int MMAS = TKE / 16;                           // MMA instructions per tile
  static constexpr int NCH = 8;                                   // 16-byte chunks per thread (its tile row)
  static constexpr int WPC = QUANT == EK_QUANT_BF16 ? 4 : 8;      // 32-bit A words per chunk
  static constexpr int NW = NCH * WPC;
  static constexpr bool SCALE_B = MODE == kModeScaleB2;
  static constexpr bool F16 = MODE == kModeScaleB2 || MODE == kModeScaleAH;   // both MMA operands f16, h written as f16
  // tensor memory: two accumulators of NMAX columns (one per chain) - twice that in the 32-row
  // variant, where consecutive work items alternate between two accumulator sets so that the
  // epilogue of an item can be put off behind the first conversions of the next one - and the rest
  // is a ring of A staging slots (an even number, shared by the two chains): 6 slots for the decode
  // variants, 4 at NMAX = 128
  static constexpr int ACC_BUFS = NMAX <= 32 ? 2 : 1;
  static constexpr int A_BASE = ACC_BUFS * 2 * NMAX;
  static constexpr int A_SLOTS_RAW = ((kTmemCols - A_BASE) / kASlotCols) & ~1;
  static constexpr int A_SLOTS = A_SLOTS_RAW > kMaxASlots ? kMaxASlots : A_SLOTS_RAW;
  static constexpr int A_PER = A_SLOTS / 2;                       // slots per chain
  static_assert(A_SLOTS >= 4, "need at least two A slots per chain");
  // a converter reaches step it + STAGES only after its chain completed step it + STAGES - A_PER >= it,
  // i.e. after the ready barrier of step it has flipped: arrivals of two laps never mix; the same
  // inequality makes the converters' parity waits exact (see the converter loop)
  static_assert(A_PER <= STAGES, "A slots per chain must not exceed the stage count");
  static_assert(STAGE_BYTES % 1024 == 0, "stage must keep 1024-byte alignment");
  static_assert(STAGES >= 2, "not enough shared memory for a pipeline");
  static_assert(QUANT != EK_QUANT_BF16 || MODE == kModeRaw, "bf16 weights are not converted");
};

__device__ __forceinline__ void report(DevStatus* st, int code, int where, int a0, int a1) {
  if (atomicCAS(&st->code, DEV_OK, code) == DEV_OK) {
    st->where = where;
    st->aux0 = a0;
    st->aux1 = a1;
  }
}

// ---- work decomposition ----------------------------------------------------------------------
// The same sequence of units is walked by every role of a CTA.
struct Unit {
  int item, kt0, kt1;
};
__device__ __forceinline__ ChunkDesc load_chunk(const ChunkDesc* c) {   // from L2: see the weight producer
  static_assert(sizeof(ChunkDesc) == 16, "one 16-byte load");
  const int4 v = __ldcg(reinterpret_cast<const int4*>(c));
  ChunkDesc d;
  d.slot = v.x; d.in_row = v.y; d.out_row = v.z; d.n_rows = v.w;
  return d;
}

struct Sched {
  int KT, n_full, tail_hi, next_item, g, L;
  __device__ __forceinline__ Sched(int total, int KT_, int split_k) {
    KT = KT_;
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    n_full = split_k ? (total / G) * G : total;
    int tk = (total - n_full) * KT;              // K steps of the left-over items (< G * KT)
    L = (tk + G - 1) / G;
    if (L < kMinPart) L = kMinPart;
    if (L * 10 > KT * 9) {   // cutting would shorten the tail by less than a tenth: not worth the partial sums
      n_full = total;
      L = KT;
      tk = 0;
    }
    const int lo = min(c * L, tk);
    tail_hi = min(lo + L, tk);
    next_item = c;
    g = lo;
  }
  __device__ __forceinline__ bool next(Unit& u) {
    if (next_item < n_full) {
      u.item = next_item; u.kt0 = 0; u.kt1 = KT;
      next_item += (int)gridDim.x;
      return true;
    }
    if (g < tail_hi) {
      u.item = n_full + g / KT;
      u.kt0 = g % KT;
      u.kt1 = min(KT, u.kt0 + (tail_hi - g));
      g += u.kt1 - u.kt0;
      return true;
    }
    return false;
  }
  // CTAs after this one that hold the remaining parts of an item this CTA owns up to kt1
  __device__ __forceinline__ int followers(const Unit& u) const { return (KT - u.kt1 + L - 1) / L; }
};

// ---- conversion of a weight row into packed 16-bit A words --------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t fma_f16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// two e4m3 bytes -> two f16, exact (every e4m3 value, subnormals included, is an f16 value)
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(static_cast<unsigned short>(two_bytes)));
  return r;
}
// four int8 codes in offset binary (u = b ^ 0x80 = b + 128, as the tiles keep them) -> four f16, exact:
// 0x6400 | u is the f16 value 1024 + u; subtract 1152
__device__ __forceinline__ void s8x4_to_f16(uint32_t w, uint32_t* out) {
  out[0] = sub_f16x2(__byte_perm(w, 0x64646464u, 0x4140), 0x64806480u);
  out[1] = sub_f16x2(__byte_perm(w, 0x64646464u, 0x4342), 0x64806480u);
}
__device__ __forceinline__ float2 f16x2_to_float2(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

// One 32-bit word of four quantised weights -> two A words.
//   kModeScaleA  : bf16_rne(float(w) * scale), the reference formula (expert_torch.rs:24-53)
//   kModeScaleAH : f16(w) * (s_hi + s_lo), packed f16
//   kModeScaleB2 : f16(w) exactly
template <int QUANT, int MODE>
__device__ __forceinline__ void cvt_word(uint32_t w, float scale, uint32_t s_hi, uint32_t s_lo, uint32_t* out) {
  if (MODE == kModeScaleA) {
    if (QUANT == EK_QUANT_FP8_BLOCK128) {
      const float2 a = f16x2_to_float2(e4m3x2_to_f16x2(w & 0xFFFFu)), b = f16x2_to_float2(e4m3x2_to_f16x2(w >> 16));
      out[0] = pack_bf16(__fmul_rn(a.x, scale), __fmul_rn(a.y, scale));
      out[1] = pack_bf16(__fmul_rn(b.x, scale), __fmul_rn(b.y, scale));
    } else {
      const float f0 = static_cast<float>(static_cast<int>(w & 0xff) - 128);           // offset binary
      const float f1 = static_cast<float>(static_cast<int>((w >> 8) & 0xff) - 128);
      const float f2 = static_cast<float>(static_cast<int>((w >> 16) & 0xff) - 128);
      const float f3 = static_cast<float>(static_cast<int>(w >> 24) - 128);
      out[0] = pack_bf16(__fmul_rn(f0, scale), __fmul_rn(f1, scale));
      out[1] = pack_bf16(__fmul_rn(f2, scale), __fmul_rn(f3, scale));
    }
  } else {
    if (QUANT == EK_QUANT_FP8_BLOCK128) {
      out[0] = e4m3x2_to_f16x2(w & 0xFFFFu);
      out[1] = e4m3x2_to_f16x2(w >> 16);
    } else {
      s8x4_to_f16(w, out);
    }
    if (MODE == kModeScaleAH) {
      out[0] = fma_f16x2(out[0], s_hi, mul_f16x2(out[0], s_lo));
      out[1] = fma_f16x2(out[1], s_hi, mul_f16x2(out[1], s_lo));
    }
  }
}

// a factor split into two packed f16 terms (hi + lo): a two-instruction packed multiply then keeps
// 22 significant bits of the factor
__device__ __forceinline__ void split_f16x2(float v, uint32_t& hi2, uint32_t& lo2) {
  const __half hi = __float2half_rn(v);
  const __half2 h2 = __halves2half2(hi, hi);
  const __half2 l2 = __float2half2_rn(v - __half2float(hi));
  hi2 = *reinterpret_cast<const uint32_t*>(&h2);
  lo2 = *reinterpret_cast<const uint32_t*>(&l2);
}
// eight f16 activations times the split factor
__device__ __forceinline__ uint4 scale_f16x8(const uint4& x, uint32_t hi2, uint32_t lo2) {
  uint4 o;
  o.x = fma_f16x2(x.x, hi2, mul_f16x2(x.x, lo2));
  o.y = fma_f16x2(x.y, hi2, mul_f16x2(x.y, lo2));
  o.z = fma_f16x2(x.z, hi2, mul_f16x2(x.z, lo2));
  o.w = fma_f16x2(x.w, hi2, mul_f16x2(x.w, lo2));
  return o;
}

__device__ __forceinline__ int pick_n(int rows, int nmax) {
  int n = rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : 128;
  return n > nmax ? nmax : n;
}
__device__ __forceinline__ int map_index(int n) { return n == 16 ? 0 : n == 32 ? 1 : n == 64 ? 2 : 3; }

// Instruction descriptor: D fp32, A and B both f16 or both bf16, both K-major, M = 128.
__device__ __forceinline__ uint32_t idesc_for(uint32_t n, bool f16) {
  return (1u << 4) | (f16 ? 0u : ((1u << 7) | (1u << 10))) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int W>
__device__ __forceinline__ void tmem_ld_pair_wait(uint32_t ta, uint32_t tb, uint32_t* a, uint32_t* b) {
  if constexpr (W == 32) tmem_ld32x2_wait(ta, tb, a, b);
  else tmem_ld8x2_wait(ta, tb, a, b);
}

// A finished work item whose epilogue is still to run.
struct Pending {
  ChunkDesc cd;
  int rt, N, item, kt0, kt1, n_follow;
  float out_pow;
  uint32_t n;            // index of the item in this CTA's sequence
};

// The epilogue of a finished work item: tensor memory -> (partial sums of split items) -> SwiGLU or
// plain rounding -> global memory.  In the variants with two accumulator sets it runs behind the
// warp's first conversion step of the NEXT item (or behind the last item): the converters - the unit
// that sets the pace of this kernel - then do not sit out the latency of the item's last MMAs, and
// the MMA chains go straight on into the other accumulator set.  Not inlined: the converters' K loop
// stays small.
template <int QUANT, bool GATEUP, int NMAX, int MODE>
__device__ __noinline__ bool run_epilogue(const FfnParams& p, const Pending& e, uint32_t tmem, uint64_t* bar_accfull,
                                          uint64_t* bar_accempty, volatile int* abortp) {
  using C = Cfg<QUANT, GATEUP, NMAX, MODE>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q = warp & 3;
  const int r = q * 32 + lane;
  const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
    const uint32_t ab = C::ACC_BUFS == 2 ? (e.n & 1u) : 0u;
    const uint32_t ause = C::ACC_BUFS == 2 ? (e.n >> 1) : e.n;
    if (!mbar_wait(smem_u32(&bar_accfull[ab]), ause & 1u, abortp)) {
      report(p.status, DEV_TIMEOUT, 302, e.item, 0);
      return false;
    }
    const ChunkDesc& cd = e.cd;
    const int rt = e.rt, N = e.N;
    const float out_pow = e.out_pow;
    const uint32_t acc_base = lane_base + ab * (2 * NMAX);
    tc_fence_after();
    // a split item: parts that do not start at K step 0 leave their accumulators in the scratch
    // buffer; the part that does adds them, in part order, before the epilogue proper
    const bool part_write = e.kt0 > 0;
    const int n_follow = e.n_follow;
    float* const sk_mine = p.sk_buf + (size_t)blockIdx.x * (2 * NMAX * 128);
    if (n_follow > 0) {
      int got = 1;
      if (lane == 0) {
        for (int j = 1; j <= n_follow && got; ++j) {
          const uint32_t* f = p.sk_flags + ((size_t)blockIdx.x + j) * 32 + warp;
          got = 0;
          for (uint32_t poll = 0; poll < (1u << 21); ++poll) {
            if (ld_acquire_gpu(f) != 0u) { got = 1; break; }
            if (poll > 64) __nanosleep(100);
            if ((poll & 1023u) == 1023u && *abortp) break;
          }
        }
      }
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) {
        if (lane == 0) {
          report(p.status, DEV_TIMEOUT, 304, e.item, e.kt1);
          *abortp = 1;
        }
        return false;
      }
    }
    // gate/up: this thread owns intermediate feature rt*128 + r (gate in accumulator 0, up in 1);
    // down: hidden features (2*rt)*128 + r (accumulator 0) and (2*rt+1)*128 + r (accumulator 1)
    const int feat = (GATEUP ? rt : 2 * rt) * kTileRows + r;
    // Row pointers advance by a constant stride; full column blocks take a branch-free path.
    const size_t ostride = GATEUP ? (size_t)p.d.Ip : (size_t)p.d.H;
    __nv_bfloat16* obase = (GATEUP ? p.hbuf : p.obuf) + (size_t)cd.out_row * ostride + feat;
    const bool f0 = GATEUP || feat < p.d.H, f1 = !GATEUP && feat + kTileRows < p.d.H;
    auto emit = [&](__nv_bfloat16* o, float gv, float uv) {
      if (C::F16) {
        gv *= out_pow;
        uv *= out_pow;
      }
      if (GATEUP) {
        const float h = uv * __fdividef(gv, 1.f + __expf(-gv));
        if (C::F16) {   // the down GEMM of these modes takes f16 activations
          const __half hh = __float2half_rn(fminf(fmaxf(h, -65504.f), 65504.f));
          *reinterpret_cast<__half*>(o) = hh;
        } else {
          *o = __float2bfloat16_rn(h);
        }
      } else {
        if (f0) *o = __float2bfloat16_rn(gv);
        if (f1) o[kTileRows] = __float2bfloat16_rn(uv);
      }
    };
    auto columns = [&](auto wtag) {
      constexpr int W = decltype(wtag)::value;
      for (int cb = warp >> 2; cb < N / W; cb += kConvWarps / 4) {
        const int c0 = cb * W;
        if (c0 >= cd.n_rows) break;
        uint32_t g[W], uu[W];
        tmem_ld_pair_wait<W>(acc_base + c0, acc_base + NMAX + c0, g, uu);
        if (part_write) {
          float* d = sk_mine + (size_t)c0 * 128 + r;
#pragma unroll
          for (int i = 0; i < W; ++i)
            if (c0 + i < cd.n_rows) {
              d[(size_t)i * 128] = __uint_as_float(g[i]);
              d[(size_t)(NMAX + i) * 128] = __uint_as_float(uu[i]);
            }
          continue;
        }
        for (int j = 1; j <= n_follow; ++j) {
          const float* sp = p.sk_buf + ((size_t)blockIdx.x + j) * (2 * NMAX * 128) + (size_t)c0 * 128 + r;
#pragma unroll
          for (int i = 0; i < W; ++i)
            if (c0 + i < cd.n_rows) {
              g[i] = __float_as_uint(__uint_as_float(g[i]) + __ldcg(sp + (size_t)i * 128));
              uu[i] = __float_as_uint(__uint_as_float(uu[i]) + __ldcg(sp + (size_t)(NMAX + i) * 128));
            }
        }
        __nv_bfloat16* o = obase + (size_t)c0 * ostride;
        if (c0 + W <= cd.n_rows) {
#pragma unroll
          for (int i = 0; i < W; ++i, o += ostride) emit(o, __uint_as_float(g[i]), __uint_as_float(uu[i]));
        } else {
#pragma unroll
          for (int i = 0; i < W; ++i, o += ostride)
            if (c0 + i < cd.n_rows) emit(o, __uint_as_float(g[i]), __uint_as_float(uu[i]));
        }
      }
    };
    if (NMAX >= 64 && N >= 64) columns(std::integral_constant<int, 32>());   // 32 columns per tensor-memory round trip
    else columns(std::integral_constant<int, 8>());
    if (part_write) {
      __threadfence();
      __syncwarp();
      if (lane == 0) st_release_gpu(p.sk_flags + (size_t)blockIdx.x * 32 + warp, 1u);
    } else if (n_follow > 0) {
      __syncwarp();
      if (lane == 0)
        for (int j = 1; j <= n_follow; ++j) p.sk_flags[((size_t)blockIdx.x + j) * 32 + warp] = 0u;   // consumed
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bar_accempty[ab]));
    return true;
}

template <int QUANT, bool GATEUP, int NMAX, int MODE>
__global__ void __launch_bounds__(kThreads, 1) ffn_tc_kernel(const __grid_constant__ FfnParams p) {
  using C = Cfg<QUANT, GATEUP, NMAX, MODE>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_wfull[8], bar_wempty[8], bar_xfull[8], bar_ready[8], bar_done[kMmaWarps][8];
  __shared__ __align__(8) uint64_t bar_accfull[2], bar_accempty[2], bar_drain[kMmaWarps];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ Pending s_pend[kConvWarps];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t stage0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const stage0_ptr = smem_raw + (stage0 - smem_u32(smem_raw));
  volatile int* abortp = &s_abort;

  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < C::STAGES; ++i) {
      mbar_init(smem_u32(&bar_wfull[i]), 1);               // weight tiles of the stage have landed
      mbar_init(smem_u32(&bar_wempty[i]), kGroupWarps);    // the step's converter group has read the weight tiles
      mbar_init(smem_u32(&bar_xfull[i]), 1);               // scale-on-B: the raw activation tile has landed
      // both A tiles of the step are in tensor memory (one arrival per converter warp) and the
      // activation tile is in place: landed (the producer's expect_tx arrival + the copy's bytes)
      // or, scale-on-B, rewritten by those same converter warps
      mbar_init(smem_u32(&bar_ready[i]), C::SCALE_B ? kGroupWarps : kGroupWarps + 1);
      for (int c = 0; c < kMmaWarps; ++c) mbar_init(smem_u32(&bar_done[c][i]), 1);   // chain c's MMAs of the step are complete
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bar_accfull[i]), kMmaWarps);     // both chains' MMAs of a work item are complete
      mbar_init(smem_u32(&bar_accempty[i]), kConvWarps);   // every converter warp has read the item's accumulators
    }
    for (int i = 0; i < kMmaWarps; ++i) mbar_init(smem_u32(&bar_drain[i]), 1);
    mbar_init_fence();
  }
  if (warp == kFirstMmaWarp) {
    tmem_alloc(smem_u32(&s_tmem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  // barriers and tensor memory are this CTA's own; everything below reads what earlier kernels wrote.
  // One thread may go ahead (`weights_ahead`): the weight producer, when the kernel launched in front
  // of this one does not write the work list - gate/up in front of a down GEMM, the row gather in
  // front of gate/up.  The list was then complete before that kernel began, and registered weights
  // do not change during a pass: the stages fill with weight tiles while the last CTAs of the
  // kernel in front are still at work.  The producer reads the work list past L1 (a line kept from an
  // earlier pass must not be used).
  const bool ahead = p.weights_ahead && warp == kConvWarps;
  if (!ahead) pdl_wait();
  pdl_trigger();
  const int n_chunks = __ldcg(p.n_chunks);
  const int n_rt = GATEUP ? p.d.it : p.d.hp;       // work items per chunk
  const int KT = GATEUP ? p.d.kt_gu : p.d.kt_dn;   // K tiles of the GEMM = pipeline stages per work item
  const int total = n_chunks * n_rt;

  if (warp < kFirstMmaWarp && warp >= kConvWarps) {
    // =============================== producers =============================================
    // Two threads in two warps, two independent rings over the same stages: one refills the weight
    // tiles of a stage as soon as the converters have read them, the other the activation tile once
    // both MMA chains are done with the stage.  The weights (the long-latency HBM stream) thereby
    // start their next trip a whole MMA phase earlier than the activations.
    if (lane == 0) {
      const bool weights = warp == kConvWarps;
      const CUtensorMap* maps = GATEUP ? p.x_maps : p.h_maps;
      const uint64_t stream_once = policy_evict_first();   // weights read exactly once per pass
      uint64_t* bar_full = weights ? bar_wfull : (C::SCALE_B ? bar_xfull : bar_ready);
      uint32_t it = 0;
      bool ok = true;
      Sched sched(total, KT, p.split_k);
      Unit u;
      while (ok && sched.next(u)) {
        ChunkDesc cd = load_chunk(p.chunks + u.item / n_rt);
        // weights that the neighbouring items read again stay in L2; the rest is streamed through
        const bool reread = (cd.n_rows & kChunkMulti) != 0;
        cd.n_rows &= kChunkRowsMask;
        const int rt = u.item % n_rt;
        const int N = pick_n(cd.n_rows, NMAX);
        const CUtensorMap* map = maps + map_index(N);
        const uint8_t* wsrc =
            GATEUP ? p.w.gu_tiles + ((size_t)cd.slot * p.d.it + rt) * (size_t)p.d.kt_gu * C::W_BYTES
                   : p.w.dn_tiles + ((size_t)cd.slot * p.d.hp + rt) * (size_t)p.d.kt_dn * C::W_BYTES;
        const int brow = GATEUP ? cd.in_row : cd.out_row;
        for (int kt = u.kt0; kt < u.kt1; ++kt, ++it) {
          const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1u;
          // a fresh barrier passes a wait on parity 1: the first lap over the ring does not block
          bool free_ok;
          if (weights) {
            free_ok = mbar_wait(smem_u32(&bar_wempty[s]), ph ^ 1u, abortp);
          } else {
            free_ok = mbar_wait(smem_u32(&bar_done[0][s]), ph ^ 1u, abortp) &&
                      mbar_wait(smem_u32(&bar_done[1][s]), ph ^ 1u, abortp);
          }
          if (!free_ok) {
            report(p.status, DEV_TIMEOUT, weights ? 100 : 101, u.item, kt);
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t dst = stage0 + s * C::STAGE_BYTES;
          if (weights) {
            mbar_arrive_expect_tx(full, C::W_BYTES);
            // one 32 KiB bulk copy per stage (tiled TMA or smaller pieces measured no faster)
            if (reread) bulk_g2s(dst, wsrc + (size_t)kt * C::W_BYTES, C::W_BYTES, full);
            else bulk_g2s_hint(dst, wsrc + (size_t)kt * C::W_BYTES, C::W_BYTES, full, stream_once);
          } else {
            mbar_arrive_expect_tx(full, C::X_ATOMS * N * 128);
#pragma unroll
            for (int a = 0; a < C::X_ATOMS; ++a)
              tma_load_2d(dst + C::W_BYTES + a * N * 128, map, kt * C::TKE + a * 64, brow, full);
          }
        }
      }
      // never leave with copies in flight: wait (bounded) for every stage armed in the last lap
      const uint32_t lo = it > (uint32_t)C::STAGES ? it - C::STAGES : 0;
      for (uint32_t i = lo; i < it; ++i) {
        const uint32_t bar = smem_u32(&bar_full[i % C::STAGES]);
        for (uint32_t poll = 0; poll < (1u << 20); ++poll) {
          if (mbar_try_wait(bar, (i / C::STAGES) & 1u)) break;
          __nanosleep(64);
        }
      }
    }
  } else if (warp >= kFirstMmaWarp) {
    // =============================== MMA issuers ===========================================
    // Two issuing threads in two warps ("chains"), each with its own accumulator.  Each chain does
    // one wait and one commit per K step and nothing else.
    //   gate/up : chain 0 issues the gate tile, chain 1 the up tile of every K step
    //   down    : chain c issues hidden-row tile 2*rp + c
    if (lane == 0) {
      const uint32_t chain = warp - kFirstMmaWarp;
      uint32_t it = 0, units_done = 0, s = 0, ph = 0, ai = 0;
      bool ok = true;
      // descriptor of stage 0's activation tile (this chain's copy); stages are a constant number of
      // 16-byte units apart
      const uint64_t b_base =
          umma_desc_sw128(stage0 + C::W_BYTES + (C::SCALE_B ? chain * C::X_BYTES : 0));
      Sched sched(total, KT, p.split_k);
      Unit u;
      while (ok && sched.next(u)) {
        const ChunkDesc cd = p.chunks[u.item / n_rt];
        const int N = pick_n(cd.n_rows & kChunkRowsMask, NMAX);
        const uint32_t idesc = idesc_for(N, C::F16);
        const uint32_t atom_step = (uint32_t)(N * 128) >> 4;   // descriptor units between 64-element K atoms
        // accumulator set of this item and how often it has been used before
        const uint32_t ab = C::ACC_BUFS == 2 ? (units_done & 1u) : 0u;
        const uint32_t ause = C::ACC_BUFS == 2 ? (units_done >> 1) : units_done;
        const uint32_t d_tmem = tmem + ab * (2 * NMAX) + chain * NMAX;
        if (!mbar_wait(smem_u32(&bar_accempty[ab]), (ause & 1u) ^ 1u, abortp)) {
          report(p.status, DEV_TIMEOUT, 200, u.item, 0);
          ok = false;
          break;
        }
        tc_fence_after();
        for (int kt = u.kt0; kt < u.kt1; ++kt, ++it) {
          const uint32_t cs = s, cph = ph;
          if (++s == (uint32_t)C::STAGES) { s = 0; ph ^= 1u; }
          const uint32_t a_tmem = tmem + C::A_BASE + (ai * 2 + chain) * kASlotCols;
          if (++ai == (uint32_t)C::A_PER) ai = 0;
          // B descriptors of the stage's activation tile: one per 16-element K step
          const uint64_t b0 = b_base + (uint64_t)(cs * (uint32_t)(C::STAGE_BYTES >> 4));
          uint64_t bd[C::MMAS];
#pragma unroll
          for (int j = 0; j < C::MMAS; ++j) bd[j] = b0 + (uint64_t)((j / 4) * atom_step + (j % 4) * 2);
          // both A tiles stored and the activation tile in place
          if (!mbar_wait(smem_u32(&bar_ready[cs]), cph, abortp)) {
            report(p.status, DEV_TIMEOUT, 201, u.item, kt);
            ok = false;
            break;
          }
          tc_fence_after();
          if (C::MMAS == 8) umma_ts_x8(d_tmem, a_tmem, bd, idesc, kt > u.kt0 ? 1u : 0u);
          else umma_ts_x4(d_tmem, a_tmem, bd, idesc, kt > u.kt0 ? 1u : 0u);
          tc_commit(smem_u32(&bar_done[chain][cs]));
        }
        if (ok) tc_commit(smem_u32(&bar_accfull[ab]));
        ++units_done;
      }
      // drain: every MMA issued by this thread has completed before tensor memory is freed
      tc_commit(smem_u32(&bar_drain[chain]));
      for (uint32_t poll = 0; poll < (1u << 20); ++poll) {
        if (mbar_try_wait(smem_u32(&bar_drain[chain]), 0)) break;
        __nanosleep(64);
      }
    }
  } else {
    // =============================== converters + epilogue =================================
    // warp -> (group, tile of the stage, lane quarter of tensor memory)
    const int grp = warp / kGroupWarps, wg = (warp % kGroupWarps) >> 2, q = warp & 3;
    const int r = q * 32 + lane;
    const int gt = (warp % kGroupWarps) * 32 + lane;     // thread index inside the group (activation rescale)
    const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
    uint32_t it_base = 0, units_done = 0;
    bool ok = true;
    // this warp's copy of the finished item that still waits for its epilogue (see run_epilogue)
    Pending* const pend = &s_pend[warp];
    bool has_pend = false;
    Sched sched(total, KT, p.split_k);
    Unit u;
    while (ok && sched.next(u)) {
      ChunkDesc cd = p.chunks[u.item / n_rt];
      cd.n_rows &= kChunkRowsMask;
      const int rt = u.item % n_rt;
      const int N = pick_n(cd.n_rows, NMAX);
      // block scales of the two tiles of a stage: [K step][tile] in both GEMMs
      const float2* sc2 = nullptr;
      if (QUANT != EK_QUANT_BF16) {
        sc2 = reinterpret_cast<const float2*>(
            GATEUP ? p.w.gu_scale + ((size_t)cd.slot * p.d.it + rt) * (size_t)p.d.kt_gu * 2
                   : p.w.dn_scale + ((size_t)cd.slot * p.d.hp + rt) * (size_t)p.d.kt_dn * 2);
      }
      // power of two that keeps the scaled operand in the middle of the f16 range (scale-on-B: the
      // largest block scale times 2^c lies in [2^-5, 2^-4); scale-on-A: 2^9 higher, since the weight
      // codes reach 448); the epilogue takes it out again
      float op_pow = 1.f, out_pow = 1.f;
      if (C::F16) {
        op_pow = __ldg((GATEUP ? p.w.gu_pow : p.w.dn_pow) + cd.slot) * (MODE == kModeScaleAH ? 512.f : 1.f);
        out_pow = 1.f / op_pow;                  // exact: a power of two
      }
      // this group's steps of the unit: those whose ring index is congruent to the group
      const uint32_t it0 = it_base;
      int kt = u.kt0 + (int)((grp + kGroups - it0 % kGroups) % kGroups);
      float2 scale_next = make_float2(1.f, 1.f);
      if (QUANT != EK_QUANT_BF16 && kt < u.kt1) scale_next = __ldg(sc2 + kt);
      for (; kt < u.kt1; kt += kGroups) {
        const uint32_t it = it0 + (uint32_t)(kt - u.kt0);
        const float2 scale = scale_next;
        if (QUANT != EK_QUANT_BF16 && kt + kGroups < u.kt1) scale_next = __ldg(sc2 + kt + kGroups);
        const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1u;
        // A slot of this step: free once this warpgroup's chain has completed step it - A_PER.
        // This wait comes FIRST.  A group sees a stage only on every other lap when the stage count
        // is odd, and a parity wait cannot tell "lap L has completed" from "lap L-2 has completed":
        // it is exact only if lap L-1 is known to be over.  MMA completion of step it - A_PER (in
        // order, so of every earlier step too) says exactly that for the stage's weight and
        // activation barriers, because A_PER <= STAGES.  Waiting for the weights first let a fast
        // converter pass on the stale lap, release the stage a lap early and make the producer arm
        // a barrier whose previous transaction was still pending - an mbarrier fault.
        const uint32_t a = (it % C::A_PER) * 2 + wg;
        if (it >= (uint32_t)C::A_PER) {
          const uint32_t j = it - C::A_PER;
          if (!mbar_wait(smem_u32(&bar_done[wg][j % C::STAGES]), (j / C::STAGES) & 1u, abortp)) {
            report(p.status, DEV_TIMEOUT, 301, u.item, kt);
            ok = false;
            break;
          }
        }
        if (!mbar_wait(smem_u32(&bar_wfull[s]), ph, abortp)) {
          report(p.status, DEV_TIMEOUT, 300, u.item, kt);
          ok = false;
          break;
        }
        uint8_t* const stage_ptr = stage0_ptr + (size_t)s * C::STAGE_BYTES;
        const uint8_t* tile = stage_ptr + wg * kTileBytes;
        uint4 raw[C::NCH];
#pragma unroll
        for (int j = 0; j < C::NCH; ++j)
          raw[j] = *reinterpret_cast<const uint4*>(tile + (size_t)(j * kTileRows + r) * 16);
        // how this tile's block scale is applied (see the file header)
        const float my_scale = wg == 0 ? scale.x : scale.y;
        uint32_t a_hi = 0, a_lo = 0;
        if (MODE == kModeScaleAH) split_f16x2(my_scale * op_pow, a_hi, a_lo);
        uint32_t aw[C::NW];
        if (MODE == kModeRaw) {
#pragma unroll
          for (int j = 0; j < C::NCH; ++j) {
            aw[4 * j] = raw[j].x; aw[4 * j + 1] = raw[j].y; aw[4 * j + 2] = raw[j].z; aw[4 * j + 3] = raw[j].w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < C::NCH; ++j) {
            cvt_word<QUANT, MODE>(raw[j].x, my_scale, a_hi, a_lo, aw + (j * 8 + 0) % C::NW);
            cvt_word<QUANT, MODE>(raw[j].y, my_scale, a_hi, a_lo, aw + (j * 8 + 2) % C::NW);
            cvt_word<QUANT, MODE>(raw[j].z, my_scale, a_hi, a_lo, aw + (j * 8 + 4) % C::NW);
            cvt_word<QUANT, MODE>(raw[j].w, my_scale, a_hi, a_lo, aw + (j * 8 + 6) % C::NW);
          }
        }
        const uint32_t col0 = C::A_BASE + a * kASlotCols;
        tc_fence_after();
        if (C::NW >= 32) {
#pragma unroll
          for (int w0 = 0; w0 < C::NW; w0 += 32) tmem_st32(lane_base + col0 + w0, aw + w0);
        } else {
          tmem_st16(lane_base + col0, aw);
        }
        if (C::SCALE_B) {
          // the weights are in registers / on their way to tensor memory: the producer may refill
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_wempty[s]));
          // rewrite the activation tile of the step as bf16(x * block scale) while the stores fly
          if (!mbar_wait(smem_u32(&bar_xfull[s]), ph, abortp)) {
            report(p.status, DEV_TIMEOUT, 303, u.item, kt);
            ok = false;
            break;
          }
          uint32_t h0, l0, h1, l1;
          split_f16x2(scale.x * op_pow, h0, l0);
          split_f16x2(scale.y * op_pow, h1, l1);
          uint4* xt = reinterpret_cast<uint4*>(stage_ptr + C::W_BYTES);
          const int nvec = N * C::X_ATOMS * 8;           // 16-byte vectors of the [N, TKE] tile
          for (int v = gt; v < nvec; v += kGroupWarps * 32) {
            const uint4 x = xt[v];
            xt[v] = scale_f16x8(x, h0, l0);
            xt[v + C::X_BYTES / 16] = scale_f16x8(x, h1, l1);
          }
          fence_proxy_async();                           // generic-proxy writes -> tensor-core reads
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bar_ready[s]));
          if (!C::SCALE_B) mbar_arrive(smem_u32(&bar_wempty[s]));
        }
        // this warp's first step of the item is on its way: now the epilogue of the item before it
        if (C::ACC_BUFS == 2 && has_pend) {
          has_pend = false;
          if (!run_epilogue<QUANT, GATEUP, NMAX, MODE>(p, *pend, tmem, bar_accfull, bar_accempty, abortp)) {
            ok = false;
            break;
          }
        }
      }
      it_base += (uint32_t)(u.kt1 - u.kt0);
      if (!ok) break;
      // the unit had no step for this group: the item before it is still waiting for its epilogue
      if (has_pend) {
        has_pend = false;
        if (!run_epilogue<QUANT, GATEUP, NMAX, MODE>(p, *pend, tmem, bar_accfull, bar_accempty, abortp)) { ok = false; break; }
      }
      __syncwarp();
      if (lane == 0) {
        Pending cur;
        cur.cd = cd; cur.rt = rt; cur.N = N; cur.item = u.item; cur.kt0 = u.kt0; cur.kt1 = u.kt1;
        cur.n_follow = (u.kt0 == 0 && u.kt1 < KT) ? sched.followers(u) : 0;
        cur.out_pow = out_pow;
        cur.n = units_done;
        *pend = cur;
      }
      __syncwarp();
      if (C::ACC_BUFS == 2) {   // with a single accumulator set the MMAs could not go on anyway: deferring measured slower
        has_pend = true;       // read the accumulators behind the first step of the next item (two or three steps measured the same)
      } else if (!run_epilogue<QUANT, GATEUP, NMAX, MODE>(p, *pend, tmem, bar_accfull, bar_accempty, abortp)) {
        ok = false;
        break;
      }
      ++units_done;
    }
    if (ok && has_pend) run_epilogue<QUANT, GATEUP, NMAX, MODE>(p, *pend, tmem, bar_accfull, bar_accempty, abortp);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kFirstMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <int QUANT, bool GATEUP, int NMAX, int MODE>
int launch_one(const FfnParams& p, cudaStream_t s) {
  using C = Cfg<QUANT, GATEUP, NMAX, MODE>;
  const int smem = C::STAGES * C::STAGE_BYTES + 1024;
  cudaFuncSetAttribute(ffn_tc_kernel<QUANT, GATEUP, NMAX, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  launch_pdl(ffn_tc_kernel<QUANT, GATEUP, NMAX, MODE>, dim3(p.n_sm), dim3(kThreads), (size_t)smem, s, p);
  return 1;
}

template <int QUANT, int MODE_DECODE, int MODE_PREFILL>
int launch_quant(const FfnParams& p, int nmax, int which, cudaStream_t s) {
  if (nmax <= 32)
    return which == 0 ? launch_one<QUANT, true, 32, MODE_DECODE>(p, s) : launch_one<QUANT, false, 32, MODE_DECODE>(p, s);
  if (nmax <= 64)   // (scale-on-A measured no faster than scale-on-B at this chunk size)
    return which == 0 ? launch_one<QUANT, true, 64, MODE_DECODE>(p, s) : launch_one<QUANT, false, 64, MODE_DECODE>(p, s);
  return which == 0 ? launch_one<QUANT, true, 128, MODE_PREFILL>(p, s) : launch_one<QUANT, false, 128, MODE_PREFILL>(p, s);
}

}  // namespace

size_t ffn_tc_scratch_floats(int n_sm) { return (size_t)n_sm * 2 * 128 * 128; }

bool ffn_tc_f16_activations(int quant, int precise) { return quant != EK_QUANT_BF16 && !precise; }

int launch_ffn_tc(const FfnParams& p, int nmax, int which, cudaStream_t s) {
  switch (p.d.quant) {
    case EK_QUANT_BF16: return launch_quant<EK_QUANT_BF16, kModeRaw, kModeRaw>(p, nmax, which, s);
    case EK_QUANT_FP8_BLOCK128:
      return p.precise ? launch_quant<EK_QUANT_FP8_BLOCK128, kModeScaleA, kModeScaleA>(p, nmax, which, s)
                       : launch_quant<EK_QUANT_FP8_BLOCK128, kModeScaleB2, kModeScaleAH>(p, nmax, which, s);
    default:
      return p.precise ? launch_quant<EK_QUANT_INT8_BLOCK128, kModeScaleA, kModeScaleA>(p, nmax, which, s)
                       : launch_quant<EK_QUANT_INT8_BLOCK128, kModeScaleB2, kModeScaleAH>(p, nmax, which, s);
  }
}

}  // namespace ek
