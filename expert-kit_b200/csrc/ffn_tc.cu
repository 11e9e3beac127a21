// Grouped SwiGLU expert FFN on the 5th-generation tensor cores (tcgen05 + tensor memory),
// fed by TMA, for sm_100a.  Replaces the three libtorch matmuls of TorchFFN::forward
// (ek-computation/src/ffn/expert_torch.rs:80-85) and the block dequantisation of
// w8a16_activate (expert_torch.rs:24-53) for ALL experts of a layer in two launches.
//
// Formulation ("weights as the M operand"): for one work item (chunk of <= NMAX activation
// rows of one expert, one tile of 128 weight rows)
//        D[128 weight rows, N rows of x] (+)= W_tile[128, K] * X_chunk[N, K]^T
// so the MMA always runs at M = 128 no matter how few tokens an expert received, and the
// weight stream - the thing that is HBM-bound at decode batch sizes - is read exactly once.
//
//   producer warp   : bulk-copies the next 16 KiB weight tile(s) (fp8 / int8 / bf16, already
//                     laid out for conflict-free reads) and TMA-loads the matching [N, K]
//                     activation tile (128-byte swizzle) into a ring of shared-memory stages
//   converter warps : thread r reads weight row r of the tile from shared memory, dequantises
//                     it to bf16 (block scale applied in fp32, one rounding - the reference
//                     formula) and stores it into tensor memory with tcgen05.st as the A operand
//   MMA warp        : one thread issues tcgen05.mma (A from tensor memory, B from shared
//                     memory through a swizzled descriptor, fp32 accumulators in tensor memory)
//   epilogue        : the converter warps read the accumulators with tcgen05.ld; gate/up mode
//                     applies silu(gate) * up in fp32 and writes h (bf16); down mode writes
//                     the expert output rows (bf16)
//
// Every mbarrier wait is bounded (see ptx.cuh); on a timeout the CTA records DEV_TIMEOUT in
// the status word, drains what it has in flight and leaves, so a protocol error can never
// hang the device.
#include "ek_internal.h"
#include "ptx.cuh"

namespace ek {

namespace {

using namespace ekptx;

// Converter warps come in groups of 8 (two warpgroups: one per tile of the stage, one warp per
// tensor-memory lane quarter).  Group g converts the K steps kt = g, g + kGroups, ...: with two
// groups, two steps are in conversion at any time and each scheduler holds four converter warps
// instead of two, whose conversion phases (bound by the half-rate integer pipe and by dependent
// issue) overlap instead of taking turns.  Splitting a tile row between two warps instead doubled
// the per-warp barrier work and measured 4-9 % slower.
#ifndef EK_CONV_WARPS
#define EK_CONV_WARPS 16
#endif
constexpr int kConvWarps = EK_CONV_WARPS;
constexpr int kGroupWarps = 8;
constexpr int kGroups = kConvWarps / kGroupWarps;
static_assert(kConvWarps % kGroupWarps == 0 && kGroups >= 1 && kGroups <= 2,
              "converter warps come in one or two groups of 8 (three groups faulted at launch and are not supported)");
constexpr int kMmaWarps = 2;
constexpr int kProdWarps = 2;                 // weight ring, activation ring: one warp each
constexpr int kFirstMmaWarp = kConvWarps + kProdWarps;
#ifdef EK_TC_PROFILE
constexpr int kObserverWarps = 1;   // watches the weight barriers: true issue -> landed time
#else
constexpr int kObserverWarps = 0;
#endif
constexpr int kThreads = (kConvWarps + kProdWarps + kMmaWarps + kObserverWarps) * 32;
constexpr int kASlotCols = 64;   // tensor-memory columns per A staging slot (128 bf16 along K)
constexpr int kTmemCols = 512;
#ifndef EK_MAX_A_SLOTS
#define EK_MAX_A_SLOTS 6
#endif
constexpr int kMaxASlots = EK_MAX_A_SLOTS;
constexpr int kSmemLimit = 232448 - 4096;

template <int QUANT, bool GATEUP, int NMAX>
struct Cfg {
  static constexpr int TKE = QUANT == EK_QUANT_BF16 ? 64 : 128;   // K elements per tile
  // A stage holds two weight tiles of the same K step, one per converter warpgroup / MMA chain,
  // and the one activation tile both multiply:
  //   gate/up : the gate and the up tile of intermediate-row tile rt
  //   down    : the tiles of hidden-row tiles 2*rp and 2*rp+1
  static constexpr int W_BYTES = 2 * kTileBytes;
  static constexpr int X_ATOMS = TKE / 64;                        // 64-element swizzle atoms along K
  static constexpr int X_BYTES = NMAX * X_ATOMS * 128;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int STAGES_RAW = kSmemLimit / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int MMAS = TKE / 16;                           // MMA instructions per tile
  static constexpr int NCH = 8;                                   // 16-byte chunks per thread (its tile row)
  static constexpr int WPC = QUANT == EK_QUANT_BF16 ? 4 : 8;      // 32-bit A words per chunk
  static constexpr int NW = NCH * WPC;
  // tensor memory: two accumulators of NMAX columns, the rest is a ring of A staging slots (an
  // even number, shared by the two chains): 6 slots for the decode variants, 4 at NMAX = 128
  static constexpr int A_BASE = 2 * NMAX;
  static constexpr int A_SLOTS_RAW = ((kTmemCols - A_BASE) / kASlotCols) & ~1;
  static constexpr int A_SLOTS = A_SLOTS_RAW > kMaxASlots ? kMaxASlots : A_SLOTS_RAW;
  static constexpr int A_PER = A_SLOTS / 2;                       // slots per chain
  static_assert(A_SLOTS >= 4, "need at least two A slots per chain");
  // a converter reaches step it + STAGES only after its chain completed step it + STAGES - A_PER >= it,
  // i.e. after the ready barrier of step it has flipped: arrivals of two laps never mix
  static_assert(A_PER <= STAGES_RAW, "A slots per chain must not exceed the stage count");
  static_assert(STAGE_BYTES % 1024 == 0, "stage must keep 1024-byte alignment");
  static_assert(STAGES >= 2, "not enough shared memory for a pipeline");
};



// Optional per-role cycle accounting (build with -DEK_TC_PROFILE): where each role's time goes.
#ifdef EK_TC_PROFILE
#define PROF_DECL long long pt_[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long pc_ = clock64();
#define PROF_LAP(i) { long long n_ = clock64(); pt_[i] += n_ - pc_; pc_ = n_; }
#define PROF_DUMP(role) \
  if (p.prof) for (int i_ = 0; i_ < 6; ++i_) atomicAdd((unsigned long long*)&p.prof[(role) * 8 + i_], (unsigned long long)pt_[i_]);
#define TRACE(itv, ev) \
  if (GATEUP && blockIdx.x == 7 && p.prof && (itv) >= 300u && (itv) < 300u + kTraceSteps) \
    p.prof[32 + ((itv) - 300u) * kTraceEvents + (ev)] = clock64();
#else
#define PROF_DECL
#define PROF_LAP(i)
#define PROF_DUMP(role)
#define TRACE(itv, ev)
#endif

__device__ __forceinline__ void report(DevStatus* st, int code, int where, int a0, int a1) {
  if (atomicCAS(&st->code, DEV_OK, code) == DEV_OK) {
    st->where = where;
    st->aux0 = a0;
    st->aux1 = a1;
  }
}

// ---- dequantisation of one 16-byte chunk into packed bf16 pairs ---------------------------
// fp8 e4m3 payloads are stored pair-interleaved (see layout.cu): for two K-consecutive
// weights a, b the stored bytes are
//     p = [sa . . . . ea3 ea2 ea1] | [. eb0 mb2 mb1 mb0 . . .]
//     q = [sb . . . . eb3 eb2 eb1] | [. ea0 ma2 ma1 ma0 . . .]
// so that with w1 = w << 1 one byte permute and one AND yield, per 16-bit lane,
//     [s 0000 eeee mmm 0000]  =  bf16 bits of  value * 2^-120   (exact, subnormals included).
// One shift per four weights, one permute + one AND per two: 1.25 integer ops per weight
// instead of 4 for plain e4m3 bytes - the integer pipe is what bounds this kernel otherwise.
//
// The block scale is then applied either
//   fast   : packed, with the scale split into two bf16 terms s = hi + lo (hi = bf16(s * 2^120),
//            lo = bf16(s * 2^120 - hi)):  out = fma(y, hi, y * lo)  - two bf16x2 ops per two
//            weights, 16 significant bits of the scale, one final rounding; differs from the
//            reference formula only where the product lies within 2^-17 of a rounding boundary, or
//   precise: in fp32, one rounding to bf16 - bit-exact bf16_rne(float(w) * scale), the reference
//            formula (ek-computation/src/ffn/expert_torch.rs:24-53).
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
template <bool PRECISE>
__device__ __forceinline__ void cvt_fp8_word(uint32_t w, float scale, uint32_t s_hi, uint32_t s_lo, uint32_t* out) {
  const uint32_t w1 = w << 1;
  const uint32_t y0 = __byte_perm(w, w1, 0x1405) & 0x87F087F0u;
  const uint32_t y1 = __byte_perm(w, w1, 0x3627) & 0x87F087F0u;
  if (PRECISE) {
    const float k = 0x1p120f;
    out[0] = pack_bf16(__fmul_rn(__fmul_rn(__uint_as_float(y0 << 16), k), scale),
                       __fmul_rn(__fmul_rn(__uint_as_float(y0 & 0xFFFF0000u), k), scale));
    out[1] = pack_bf16(__fmul_rn(__fmul_rn(__uint_as_float(y1 << 16), k), scale),
                       __fmul_rn(__fmul_rn(__uint_as_float(y1 & 0xFFFF0000u), k), scale));
  } else {
    out[0] = fma_bf16x2(y0, s_hi, mul_bf16x2(y0, s_lo));
    out[1] = fma_bf16x2(y1, s_hi, mul_bf16x2(y1, s_lo));
  }
}
__device__ __forceinline__ void cvt_int8_word(uint32_t w, float scale, uint32_t* out) {
  float f0 = static_cast<float>(static_cast<int>(static_cast<int8_t>(w & 0xff)));
  float f1 = static_cast<float>(static_cast<int>(static_cast<int8_t>((w >> 8) & 0xff)));
  float f2 = static_cast<float>(static_cast<int>(static_cast<int8_t>((w >> 16) & 0xff)));
  float f3 = static_cast<float>(static_cast<int>(static_cast<int8_t>((w >> 24) & 0xff)));
  out[0] = pack_bf16(__fmul_rn(f0, scale), __fmul_rn(f1, scale));
  out[1] = pack_bf16(__fmul_rn(f2, scale), __fmul_rn(f3, scale));
}
template <int QUANT, bool PRECISE>
__device__ __forceinline__ void cvt_chunk(const uint4& raw, float scale, uint32_t s_hi, uint32_t s_lo, uint32_t* out) {
  if (QUANT == EK_QUANT_BF16) {
    out[0] = raw.x; out[1] = raw.y; out[2] = raw.z; out[3] = raw.w;
  } else if (QUANT == EK_QUANT_FP8_BLOCK128) {
    cvt_fp8_word<PRECISE>(raw.x, scale, s_hi, s_lo, out + 0);
    cvt_fp8_word<PRECISE>(raw.y, scale, s_hi, s_lo, out + 2);
    cvt_fp8_word<PRECISE>(raw.z, scale, s_hi, s_lo, out + 4);
    cvt_fp8_word<PRECISE>(raw.w, scale, s_hi, s_lo, out + 6);
  } else {
    cvt_int8_word(raw.x, scale, out + 0);
    cvt_int8_word(raw.y, scale, out + 2);
    cvt_int8_word(raw.z, scale, out + 4);
    cvt_int8_word(raw.w, scale, out + 6);
  }
}

__device__ __forceinline__ int pick_n(int rows, int nmax) {
  int n = rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : 128;
  return n > nmax ? nmax : n;
}
__device__ __forceinline__ int map_index(int n) { return n == 16 ? 0 : n == 32 ? 1 : n == 64 ? 2 : 3; }

template <int QUANT, bool GATEUP, int NMAX, bool PRECISE>
__global__ void __launch_bounds__(kThreads, 1) ffn_tc_kernel(const __grid_constant__ FfnParams p) {
  using C = Cfg<QUANT, GATEUP, NMAX>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_wfull[8], bar_wempty[8], bar_ready[8], bar_done[kMmaWarps][8];
  __shared__ __align__(8) uint64_t bar_accfull, bar_accempty, bar_drain[kMmaWarps];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
#ifdef EK_TC_PROFILE
  __shared__ long long s_issue[8];   // when the weight copy of each stage was issued
#endif

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t stage0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile int* abortp = &s_abort;

  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < C::STAGES; ++i) {
      mbar_init(smem_u32(&bar_wfull[i]), 1);               // weight tiles of the stage have landed
      mbar_init(smem_u32(&bar_wempty[i]), kGroupWarps);    // the step's converter group has read the weight tiles
      // both A tiles of the step are in tensor memory (one arrival per converter warp) and the
      // activation tile has landed (the producer's expect_tx arrival + the copy's bytes)
      mbar_init(smem_u32(&bar_ready[i]), kGroupWarps + 1);
      for (int c = 0; c < kMmaWarps; ++c) mbar_init(smem_u32(&bar_done[c][i]), 1);   // chain c's MMAs of the step are complete
    }
    mbar_init(smem_u32(&bar_accfull), kMmaWarps);
    mbar_init(smem_u32(&bar_accempty), kConvWarps);
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

  // barriers and tensor memory are this CTA's own; everything below reads what earlier kernels wrote
  pdl_wait();
  pdl_trigger();
  const int n_chunks = *p.n_chunks;
  const int n_rt = GATEUP ? p.d.it : p.d.hp;   // work items per chunk
  const int KT = GATEUP ? p.d.kt_gu : p.d.kt_dn;   // K tiles of the GEMM = pipeline stages per work item
  const int total = n_chunks * n_rt;

  if (warp < kFirstMmaWarp && warp >= kConvWarps) {
    // =============================== producers =============================================
    // Two threads in two warps, two independent rings over the same stages: one refills the weight
    // tiles of a stage as soon as the converters have read them, the other the activation tile once
    // both MMA chains are done with the stage.  The weights (the long-latency HBM stream) thereby
    // start their next trip a whole MMA phase earlier than the activations.  The activation copy
    // signals the stage's `ready` barrier, the one the MMA threads wait on.
    if (lane == 0) {
      const bool weights = warp == kConvWarps;
      const CUtensorMap* maps = GATEUP ? p.x_maps : p.h_maps;
      const uint64_t stream_once = policy_evict_first();   // weights read exactly once per pass
      uint64_t* bar_full = weights ? bar_wfull : bar_ready;
      uint32_t it = 0;
      bool ok = true;
      PROF_DECL
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        ChunkDesc cd = p.chunks[item / n_rt];
        // weights that the neighbouring items read again stay in L2; the rest is streamed through
        const bool reread = (cd.n_rows & kChunkMulti) != 0;
        cd.n_rows &= kChunkRowsMask;
        const int rt = item % n_rt;
        const int N = pick_n(cd.n_rows, NMAX);
        const CUtensorMap* map = maps + map_index(N);
        const uint8_t* wsrc =
            GATEUP ? p.w.gu_tiles + ((size_t)cd.slot * p.d.it + rt) * (size_t)p.d.kt_gu * C::W_BYTES
                   : p.w.dn_tiles + ((size_t)cd.slot * p.d.hp + rt) * (size_t)p.d.kt_dn * C::W_BYTES;
        const int brow = GATEUP ? cd.in_row : cd.out_row;
        for (int kt = 0; kt < KT; ++kt, ++it) {
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
            report(p.status, DEV_TIMEOUT, weights ? 100 : 101, item, kt);
            ok = false;
            break;
          }
          PROF_LAP(0)
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t dst = stage0 + s * C::STAGE_BYTES;
          if (weights) {
#ifdef EK_TC_PROFILE
            s_issue[s] = clock64();
#endif
            TRACE(it, 0)
            mbar_arrive_expect_tx(full, C::W_BYTES);
            // one 32 KiB bulk copy per stage (tiled TMA or smaller pieces measured no faster)
            if (reread) bulk_g2s(dst, wsrc + (size_t)kt * C::W_BYTES, C::W_BYTES, full);
            else bulk_g2s_hint(dst, wsrc + (size_t)kt * C::W_BYTES, C::W_BYTES, full, stream_once);
            TRACE(it, 1)
          } else {
            TRACE(it, 19)
            mbar_arrive_expect_tx(full, C::X_ATOMS * N * 128);
#pragma unroll
            for (int a = 0; a < C::X_ATOMS; ++a)
              tma_load_2d(dst + C::W_BYTES + a * N * 128, map, kt * C::TKE + a * 64, brow, full);
          }
          PROF_LAP(1)
        }
      }
      if (weights) { PROF_DUMP(0) }
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
#ifdef EK_TC_PROFILE
  } else if (warp >= kFirstMmaWarp + kMmaWarps) {
    if (lane == 0 && p.prof) {
      uint32_t it = 0;
      unsigned long long sum = 0, n = 0, mx = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        for (int kt = 0; kt < KT; ++kt, ++it) {
          const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bar_wfull[s]), ph, abortp)) { ok = false; break; }
          const unsigned long long lat = (unsigned long long)(clock64() - s_issue[s]);
          TRACE(it, 2)
          sum += lat; ++n;
          if (lat > mx) mx = lat;
        }
      }
      atomicAdd((unsigned long long*)&p.prof[30], sum);
      atomicAdd((unsigned long long*)&p.prof[31], n);
      atomicMax((unsigned long long*)&p.prof[29], mx);
    }
#endif
  } else if (warp >= kFirstMmaWarp) {
    // =============================== MMA issuers ===========================================
    // Two issuing threads in two warps ("chains"), each with its own accumulator: the instruction
    // stream of one thread between MMAs (barrier waits, descriptors, commits) costs about as much
    // time as the MMAs take, so a single issuer leaves the tensor pipe idle half of the time.  For
    // the same reason each chain does one wait and one commit per K step and nothing else.
    //   gate/up : chain 0 issues the gate tile, chain 1 the up tile of every K step
    //   down    : chain c issues hidden-row tile 2*rp + c
    if (lane == 0) {
      const uint32_t chain = warp - kFirstMmaWarp;
      uint32_t it = 0, items_done = 0, s = 0, ph = 0, ai = 0;
      bool ok = true;
      PROF_DECL
      const uint32_t d_tmem = tmem + chain * NMAX;
      // descriptor of stage 0's activation tile; stages are a constant number of 16-byte units apart
      const uint64_t b_base = umma_desc_sw128(stage0 + C::W_BYTES);
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x, ++items_done) {
        const ChunkDesc cd = p.chunks[item / n_rt];
        const int N = pick_n(cd.n_rows & kChunkRowsMask, NMAX);
        const uint32_t idesc = umma_idesc_bf16(N);
        const uint32_t atom_step = (uint32_t)(N * 128) >> 4;   // descriptor units between 64-element K atoms
        if (!mbar_wait(smem_u32(&bar_accempty), (items_done & 1u) ^ 1u, abortp)) {
          report(p.status, DEV_TIMEOUT, 200, item, 0);
          ok = false;
          break;
        }
        tc_fence_after();
        PROF_LAP(0)
        for (int kt = 0; kt < KT; ++kt, ++it) {
          const uint32_t cs = s, cph = ph;
          if (++s == (uint32_t)C::STAGES) { s = 0; ph ^= 1u; }
          const uint32_t a_tmem = tmem + C::A_BASE + (ai * 2 + chain) * kASlotCols;
          if (++ai == (uint32_t)C::A_PER) ai = 0;
          // B descriptors of the stage's activation tile: one per 16-element K step
          const uint64_t b0 = b_base + (uint64_t)(cs * (uint32_t)(C::STAGE_BYTES >> 4));
          uint64_t bd[C::MMAS];
#pragma unroll
          for (int j = 0; j < C::MMAS; ++j) bd[j] = b0 + (uint64_t)((j / 4) * atom_step + (j % 4) * 2);
          PROF_LAP(1)
          if (chain == 0) { TRACE(it, 21) }
          // both A tiles stored and the activation tile landed
          if (!mbar_wait(smem_u32(&bar_ready[cs]), cph, abortp)) {
            report(p.status, DEV_TIMEOUT, 201, item, kt);
            ok = false;
            break;
          }
          tc_fence_after();
          PROF_LAP(2)
          TRACE(it, 12 + 4 * chain)
          if (C::MMAS == 8) umma_ts_x8(d_tmem, a_tmem, bd, idesc, kt > 0 ? 1u : 0u);
          else umma_ts_x4(d_tmem, a_tmem, bd, idesc, kt > 0 ? 1u : 0u);
          PROF_LAP(3)
          TRACE(it, 13 + 4 * chain)
          tc_commit(smem_u32(&bar_done[chain][cs]));
          PROF_LAP(4)
          TRACE(it, 14 + 4 * chain)
        }
        if (ok) tc_commit(smem_u32(&bar_accfull));
      }
      if (chain == 0) { PROF_DUMP(1) }
      // drain: every MMA issued by this thread has completed before tensor memory is freed
      tc_commit(smem_u32(&bar_drain[chain]));
      for (uint32_t poll = 0; poll < (1u << 20); ++poll) {
        if (mbar_try_wait(smem_u32(&bar_drain[chain]), 0)) break;
        __nanosleep(64);
      }
    }
  } else {
    // =============================== converters + epilogue =================================
    // warp -> (tile of the stage, K part of the tile row, lane quarter of tensor memory)
    const int grp = warp / kGroupWarps, wg = (warp % kGroupWarps) >> 2, q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
    uint32_t it_base = 0, items_done = 0;
    bool ok = true;
    PROF_DECL
    for (int item = blockIdx.x; item < total && ok; item += gridDim.x, ++items_done) {
      ChunkDesc cd = p.chunks[item / n_rt];
      cd.n_rows &= kChunkRowsMask;
      const int rt = item % n_rt;
      const int N = pick_n(cd.n_rows, NMAX);
      // block scale of this warpgroup's tile: [K step][warpgroup] in both modes
      const float* sc = nullptr;
      if (QUANT != EK_QUANT_BF16) {
        sc = GATEUP ? p.w.gu_scale + ((size_t)cd.slot * p.d.it + rt) * (size_t)p.d.kt_gu * 2 + wg
                    : p.w.dn_scale + ((size_t)cd.slot * p.d.hp + rt) * (size_t)p.d.kt_dn * 2 + wg;
      }
      float scale_next = 1.f;
      if (QUANT != EK_QUANT_BF16 && grp < KT) scale_next = __ldg(sc + (size_t)grp * 2);
      const uint32_t it0 = it_base;   // global index of the item's first K step (the same in every role)
      for (int kt = grp; kt < KT; kt += kGroups) {
        const uint32_t it = it0 + kt;
        const float scale = scale_next;
        if (QUANT != EK_QUANT_BF16 && kt + kGroups < KT) scale_next = __ldg(sc + (size_t)(kt + kGroups) * 2);
        const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1u;
        if (!mbar_wait(smem_u32(&bar_wfull[s]), ph, abortp)) {
          report(p.status, DEV_TIMEOUT, 300, item, kt);
          ok = false;
          break;
        }
        PROF_LAP(0)
        if (q == 0 && lane == 0) { TRACE(it, 3 + 4 * wg) }
        // A slot of this step: free once this warpgroup's chain has completed step it - A_PER
        const uint32_t a = (it % C::A_PER) * 2 + wg;
        if (it >= (uint32_t)C::A_PER) {
          const uint32_t j = it - C::A_PER;
          if (!mbar_wait(smem_u32(&bar_done[wg][j % C::STAGES]), (j / C::STAGES) & 1u, abortp)) {
            report(p.status, DEV_TIMEOUT, 301, item, kt);
            ok = false;
            break;
          }
        }
        PROF_LAP(1)
        if (q == 0 && lane == 0) { TRACE(it, 4 + 4 * wg) }
        const uint8_t* tile = smem_raw + (stage0 - smem_u32(smem_raw)) + s * C::STAGE_BYTES + wg * kTileBytes;
        uint4 raw[C::NCH];
#pragma unroll
        for (int j = 0; j < C::NCH; ++j)
          raw[j] = *reinterpret_cast<const uint4*>(tile + (size_t)(j * kTileRows + r) * 16);
        uint32_t aw[C::NW];
        uint32_t s_hi = 0, s_lo = 0;
        if (QUANT == EK_QUANT_FP8_BLOCK128 && !PRECISE) {
          const float sk = scale * 0x1p120f;
          const __nv_bfloat16 hi = __float2bfloat16_rn(sk);
          const __nv_bfloat162 h2 = __halves2bfloat162(hi, hi);
          const __nv_bfloat162 l2 = __float2bfloat162_rn(sk - __bfloat162float(hi));
          s_hi = *reinterpret_cast<const uint32_t*>(&h2);
          s_lo = *reinterpret_cast<const uint32_t*>(&l2);
        }
#pragma unroll
        for (int j = 0; j < C::NCH; ++j) cvt_chunk<QUANT, PRECISE>(raw[j], scale, s_hi, s_lo, aw + j * C::WPC);
        const uint32_t col0 = C::A_BASE + a * kASlotCols;
        tc_fence_after();
        if (C::NW >= 32) {
#pragma unroll
          for (int w0 = 0; w0 < C::NW; w0 += 32) tmem_st32(lane_base + col0 + w0, aw + w0);
        } else {
          tmem_st16(lane_base + col0, aw);
        }
        PROF_LAP(2)
        if (q == 0 && lane == 0) { TRACE(it, 5 + 4 * wg) }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bar_ready[s]));
          mbar_arrive(smem_u32(&bar_wempty[s]));
        }
        PROF_LAP(3)
        if (q == 0 && lane == 0) { TRACE(it, 6 + 4 * wg) }
      }
      it_base += (uint32_t)KT;
      if (!ok) break;
      // ---- epilogue ----
      if (!mbar_wait(smem_u32(&bar_accfull), items_done & 1u, abortp)) {
        report(p.status, DEV_TIMEOUT, 302, item, 0);
        ok = false;
        break;
      }
      tc_fence_after();
      PROF_LAP(4)
      // gate/up: this thread owns intermediate feature rt*128 + r (gate in accumulator 0, up in 1);
      // down: hidden features (2*rt)*128 + r (accumulator 0) and (2*rt+1)*128 + r (accumulator 1)
      const int feat = (GATEUP ? rt : 2 * rt) * kTileRows + r;
      // Row pointers advance by a constant stride; full column blocks take a branch-free path.
      const size_t ostride = GATEUP ? (size_t)p.d.Ip : (size_t)p.d.H;
      __nv_bfloat16* obase = (GATEUP ? p.hbuf : p.obuf) + (size_t)cd.out_row * ostride + feat;
      const bool f0 = GATEUP || feat < p.d.H, f1 = !GATEUP && feat + kTileRows < p.d.H;
      auto emit = [&](__nv_bfloat16* o, float gv, float uv) {
        if (GATEUP) {
          *o = __float2bfloat16_rn(uv * __fdividef(gv, 1.f + __expf(-gv)));
        } else {
          if (f0) *o = __float2bfloat16_rn(gv);
          if (f1) o[kTileRows] = __float2bfloat16_rn(uv);
        }
      };
      if (NMAX >= 64 && N >= 64) {
        // wide tiles: 32 columns of both accumulators per tensor-memory round trip
        for (int cb = warp >> 2; cb < N / 32; cb += kConvWarps / 4) {
          const int c0 = cb * 32;
          if (c0 >= cd.n_rows) break;
          uint32_t g[32], u[32];
          tmem_ld32(lane_base + c0, g);
          tmem_ld32(lane_base + NMAX + c0, u);
          tc_wait_ld();
          __nv_bfloat16* o = obase + (size_t)c0 * ostride;
          if (c0 + 32 <= cd.n_rows) {
#pragma unroll
            for (int i = 0; i < 32; ++i, o += ostride) emit(o, __uint_as_float(g[i]), __uint_as_float(u[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i, o += ostride)
              if (c0 + i < cd.n_rows) emit(o, __uint_as_float(g[i]), __uint_as_float(u[i]));
          }
        }
      } else {
        for (int cb = warp >> 2; cb < N / 8; cb += kConvWarps / 4) {
          const int c0 = cb * 8;
          if (c0 >= cd.n_rows) break;
          uint32_t g[8], u[8];
          tmem_ld8(lane_base + c0, g);
          tmem_ld8(lane_base + NMAX + c0, u);
          tc_wait_ld();
          __nv_bfloat16* o = obase + (size_t)c0 * ostride;
#pragma unroll
          for (int i = 0; i < 8; ++i, o += ostride)
            if (c0 + i < cd.n_rows) emit(o, __uint_as_float(g[i]), __uint_as_float(u[i]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_accempty));
      PROF_LAP(5)
    }
    if (lane == 0 && (warp == 0 || warp == 4)) { PROF_DUMP(2 + wg) }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kFirstMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <int QUANT, bool GATEUP, int NMAX, bool PRECISE>
int launch_one(const FfnParams& p, cudaStream_t s) {
  using C = Cfg<QUANT, GATEUP, NMAX>;
  const int smem = C::STAGES * C::STAGE_BYTES + 1024;
  cudaFuncSetAttribute(ffn_tc_kernel<QUANT, GATEUP, NMAX, PRECISE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  launch_pdl(ffn_tc_kernel<QUANT, GATEUP, NMAX, PRECISE>, dim3(p.n_sm), dim3(kThreads), (size_t)smem, s, p);
  return 1;
}

template <int QUANT, bool PRECISE>
int launch_quant(const FfnParams& p, int nmax, int which, cudaStream_t s) {
  if (nmax <= 32)
    return which == 0 ? launch_one<QUANT, true, 32, PRECISE>(p, s) : launch_one<QUANT, false, 32, PRECISE>(p, s);
  if (nmax <= 64)
    return which == 0 ? launch_one<QUANT, true, 64, PRECISE>(p, s) : launch_one<QUANT, false, 64, PRECISE>(p, s);
  return which == 0 ? launch_one<QUANT, true, 128, PRECISE>(p, s) : launch_one<QUANT, false, 128, PRECISE>(p, s);
}

}  // namespace

int launch_ffn_tc(const FfnParams& p, int nmax, int which, cudaStream_t s) {
  switch (p.d.quant) {
    case EK_QUANT_BF16: return launch_quant<EK_QUANT_BF16, true>(p, nmax, which, s);
    case EK_QUANT_FP8_BLOCK128:
      return p.precise ? launch_quant<EK_QUANT_FP8_BLOCK128, true>(p, nmax, which, s)
                       : launch_quant<EK_QUANT_FP8_BLOCK128, false>(p, nmax, which, s);
    default: return launch_quant<EK_QUANT_INT8_BLOCK128, true>(p, nmax, which, s);
  }
}

}  // namespace ek
