// Internal declarations shared by the host side (backend.cu) and the kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/ek_b200.h"

#ifdef __CUDACC__
#include <cstdlib>
#include <utility>
// Programmatic dependent launch: the kernels of one layer pass are launched back to back with this
// attribute, each begins with pdl_wait() (returns when every earlier kernel of the stream has
// completed and its writes are visible) and then lets its successor start launching, so that the
// launch latency and the prologue of kernel n+1 overlap the tail of kernel n.  Nothing produced by
// an earlier kernel may be touched before pdl_wait().
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // EK_B200_NO_PDL=1: plain stream order (griddepcontrol.* are no-ops then); for diagnosis
  static const bool pdl = !(getenv("EK_B200_NO_PDL") && getenv("EK_B200_NO_PDL")[0] == '1');
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}
#endif

namespace ek {

// ---- weight tile geometry ----------------------------------------------------------------
// Expert weights live in HBM as 16 KiB tiles of 128 weight rows x 128 bytes of K
// (128 fp8/int8 elements or 64 bf16 elements).  Inside a tile the 16-byte chunk j of row r
// sits at byte (j*128 + r)*16, so that thread r of a converter warpgroup reads its own row
// with conflict-free 16-byte shared-memory loads after a plain bulk copy of the tile.
// Tiles of one (expert, row tile) are contiguous along K in exactly the order the kernel's
// K loop consumes them (gate and up tiles of the same K step adjacent), so every CTA streams
// one contiguous HBM range.
constexpr int kTileRows = 128;
constexpr int kTileBytes = 16384;
constexpr int kChunksPerRow = 8;  // 16-byte chunks per tile row

__host__ __device__ inline int tile_k_elems(int quant) { return quant == EK_QUANT_BF16 ? 64 : 128; }
__host__ __device__ inline int elem_bytes(int quant) { return quant == EK_QUANT_BF16 ? 2 : 1; }
__host__ __device__ inline int round_up(int a, int b) { return (a + b - 1) / b * b; }

// One contiguous run of rows that all go through the same expert slot.
struct ChunkDesc {
  int32_t slot;      // expert slot in the layer slab
  int32_t in_row;    // first row in the permuted activation buffer (GEMM B operand)
  int32_t out_row;   // first row in the output buffer
  int32_t n_rows;    // valid rows (1..chunk size) in the low 16 bits; bit 16: the expert's rows span
                     // several chunks, i.e. its weights are read again by the neighbouring items
};
constexpr int32_t kChunkRowsMask = 0xFFFF;
constexpr int32_t kChunkMulti = 1 << 16;

// Device-side error word: {code, where}.  Kernels only ever write non-zero values.
struct DevStatus {
  int32_t code;
  int32_t where;
  int32_t aux0;
  int32_t aux1;
};
enum { DEV_OK = 0, DEV_TIMEOUT = 1, DEV_MISSING_EXPERT = 2, DEV_BOUNDS = 3 };

// Layer slab (device pointers).
struct LayerWeights {
  const uint8_t* gu_tiles;   // [slot][it][kt][gate|up][16 KiB]
  const uint8_t* dn_tiles;   // [slot][hp][kt][row tile 2hp | 2hp+1][16 KiB]
  const float* gu_scale;     // [slot][it][kt][2]   (quantised only; K tile == 128-wide scale block)
  const float* dn_scale;     // [slot][hp][kt][2]
  const float* gu_pow;       // [slot] power of two applied to the scaled activations of the gate/up GEMM
  const float* dn_pow;       // [slot] same for the down GEMM (quantised only)
  const int32_t* registered; // [slots] 1 when the slot holds weights
  int32_t n_slots;
};

struct Dims {
  int32_t H, I;          // logical sizes
  int32_t Hp, Ip;        // padded to multiples of 128
  int32_t quant;
  int32_t kt_gu;         // K tiles of the gate/up GEMM  = Hp / tile_k
  int32_t kt_dn;         // K tiles of the down GEMM     = Ip / tile_k
  int32_t it;            // row tiles of gate/up         = Ip / 128
  int32_t ht;            // row tiles of down            = Hp / 128
  int32_t hp;            // row-tile pairs of down       = ceil(ht / 2)
};

// ---- kernel launchers (each returns the number of kernels it launched) ---------------------
struct RouteParams {
  const __nv_bfloat16* x;      // [T,H]
  const void* wg;              // [E,H] bf16 or f32
  int32_t wg_f32;
  const float* bias;           // [E] or null
  float* logits;               // [T,E]
  const float* partial;        // [n_partials][T,E] split-K partial logits, or null: logits are final
  int32_t n_partials;
  int32_t* ids;                // [T,k]
  float* weights;              // [T,k]
  int32_t* counts;             // [E] (zeroed by the launcher)
  int32_t T, H, E, k;
  int32_t scoring, n_group, topk_group, norm;
  float scaling;
  int32_t bf16_weights;        // round routing weights to bf16 (Qwen3 combine)
};
int launch_router_logits(const RouteParams& p, cudaStream_t s);

// Expert-parallel step flags handed to a kernel instead of a launch of their own (peer_sync.cuh).
struct PeerPtrs {
  void* p[EK_EP_MAX_RANKS];
};
struct PeerWait {            // wait until every rank's flag word has reached step_no
  const uint32_t* flags = nullptr;   // this rank's own flag words, one per rank; null: no wait
  int32_t world = 0;
  uint32_t step_no = 0;
  int32_t where = 0;         // recorded in the device status on a timeout
};
struct PeerSignal {          // publish step_no into word `slot` of every rank's flags
  PeerPtrs flags;
  int32_t world = 0;         // 0: no signal
  int32_t slot = 0;
  uint32_t step_no = 0;
  uint32_t* ticket = nullptr;   // zeroed counter that finds the last CTA
};

// Tensor-core router (router_tc.cu): split-K partial logits, summed by route_select.
struct RouterTcParams {
  CUtensorMap x_map;        // activations [T,H] bf16, box {64, 128}, 128-byte swizzle
  CUtensorMap w_map;        // router weight [E,H] bf16, box {64, E}
  float* partial;           // [n_splits][T][E]
  int32_t* zero_counts = nullptr;   // [E] histogram cleared here for the select kernel that follows (may be null)
  DevStatus* status;
  int32_t T, H, E;
  int32_t n_atoms;          // ceil(H / 64)
  int32_t n_splits, atoms_per_split;
  int32_t tmem_cols;        // power of two >= max(32, E)
  PeerWait wait;            // expert parallel: x is written by the peers; wait for them first
};
bool router_tc_supported(int E, int H);
void router_tc_plan(int T, int H, int n_sm, int* n_splits, int* atoms_per_split);
int launch_router_tc(const RouterTcParams& p, cudaStream_t s);
int launch_f32_to_bf16_check(const float* src, __nv_bfloat16* dst, int64_t n, int32_t* inexact, cudaStream_t s);
// `counts_cleared`: the router kernel launched just before already zeroed p.counts
int launch_route_select(const RouteParams& p, cudaStream_t s, bool counts_cleared = false);
int launch_histogram(const int32_t* ids, int32_t n, int32_t E, int32_t* counts, DevStatus* st,
                     cudaStream_t s);

struct PermuteParams {
  const int32_t* ids;     // [T*k]
  const int32_t* counts;  // [E]
  int32_t* offsets;       // [E+1]
  int32_t* perm;          // [T*k]
  int32_t* inv;           // [T*k]
  int32_t T, k, E;
  // expert-parallel window: experts [e_lo, e_hi) are local; rows of other experts are left out
  int32_t e_lo, e_hi;
  // per-pass owner table [E] -> rank (replicated experts): when set it replaces the window rule
  const int32_t* owners = nullptr;
  int32_t rank = 0;
};
int launch_permute(const PermuteParams& p, cudaStream_t s);

struct WorklistParams {
  const int32_t* counts;     // [E]
  const int32_t* offsets;    // [E+1]
  const int32_t* registered; // [slots]
  ChunkDesc* chunks;         // out
  int32_t* n_chunks;         // out (single int)
  int32_t* counts_copy = nullptr;   // out [E]: copy of counts kept per layer for the activation metric (may be null)
  int32_t E, e_lo, e_hi;     // local expert window; slot = e - e_lo
  const int32_t* owners = nullptr;   // [E] -> rank; replaces the window rule when set
  const int32_t* slot_of = nullptr;  // [E] slot of every expert this rank holds (-1: none); needed with `owners`
  int32_t rank = 0;
  int32_t chunk_rows;        // rows per chunk
  int32_t n_shared, T;       // shared virtual experts: slot = (e_hi-e_lo)+j, in_row = Tk, out_row = Tk+j*T
  int32_t Tk;
  int32_t max_chunks;
  DevStatus* status;
  int32_t same_row = 0;      // a batch of one token: every chunk reads activation row 0 (the one row that is gathered)
};
// permutation and work list in one launch (the CTA that finishes last builds the list); `ticket`: a zeroed counter
struct PermuteWorklistParams {
  PermuteParams permute;
  WorklistParams worklist;
  uint32_t* ticket = nullptr;
  int32_t with_worklist = 0;
};
int launch_permute_worklist(const PermuteParams& p, const WorklistParams& w, uint32_t* ticket, cudaStream_t s);

// Router + bucketing + work list (+ gather of a handful of rows) in one launch for small batches
// (front_small.cu).  `route.wg` must be the bf16 router weight; `route.partial` is unused, the
// kernel keeps its K-slice partial logits in `partial` ([slices][T][E]).
struct FrontParams {
  RouteParams route;
  PermuteParams permute;
  WorklistParams worklist;
  float* partial;
  uint32_t* ticket;          // zero between launches
  __nv_bfloat16* xp;         // gathered rows (when gather_rows)
  int32_t gather_rows;       // 1: also gather; rows [0,Tk) routed, [Tk, Tk+shared_T) tokens from shared_t0
  int32_t shared_t0, shared_T;
  int32_t to_f16;
  int32_t slice;             // K elements per CTA of the logits phase: front_small_slice(H)
};
bool front_small_supported(int T, int E, int k, int H);
int front_small_slice(int H);
int launch_front_small(const FrontParams& p, cudaStream_t s);

// rows [0,Tk): xp[r] = x[perm[r]/k]; rows [Tk, Tk+T) = x (only when with_shared)
// `n_routed` (device) = number of permuted rows that exist on this rank (offsets[E]).
// The shared expert's rows are tokens [shared_t0, shared_t0 + shared_T) of x (shared_T = 0: none).
// `to_f16`: write the rows as f16 (round to nearest, saturating), the activation type of the
// quantised GEMM modes.
int launch_gather(const __nv_bfloat16* x, const int32_t* perm, const int32_t* n_routed,
                  __nv_bfloat16* xp, int32_t T, int32_t k, int32_t H, int32_t shared_t0, int32_t shared_T,
                  bool to_f16, cudaStream_t s);
// rows[0 .. n_rows) of a [*, H] bf16 buffer -> f16 in place (same size)
int launch_rows_to_f16(__nv_bfloat16* rows, int64_t n_rows, int32_t H, cudaStream_t s);

struct FfnParams {
  Dims d;
  LayerWeights w;
  const ChunkDesc* chunks;
  const int32_t* n_chunks;
  const __nv_bfloat16* xp;   // [rows, H]
  __nv_bfloat16* hbuf;       // [rows, Ip]
  __nv_bfloat16* obuf;       // [rows, H]
  int32_t rows_cap;
  int32_t max_chunks;        // capacity of `chunks`
  DevStatus* status;
  int32_t chunk_rows;
  // TMA descriptors (tcgen05 path): index 0..3 <-> box rows 16,32,64,128
  const CUtensorMap* x_maps;   // device array[4]
  const CUtensorMap* h_maps;   // device array[4]
  int32_t n_sm;
  int32_t precise;           // quantised weights: bf16_rne(float(w) * scale) as the A operand (bit-exact reference dequantisation)
  int32_t split_k;           // cut the work items left over after the last full wave along K over all CTAs
  int32_t weights_ahead;     // the weight producer does not wait for the kernel launched in front of this one: allowed
                             // only if that kernel does not write the work list
  float* sk_buf;             // [n_sm][2][128][128] fp32 partial accumulators of split items
  uint32_t* sk_flags;        // [n_sm][32] one word per (CTA, warp): partial written; zero between launches
};
size_t ffn_tc_scratch_floats(int n_sm);
// true: the tensor-core GEMMs of this configuration take (and, gate/up, produce) f16 activations
bool ffn_tc_f16_activations(int quant, int precise);
// Straightforward CUDA-core evaluation of the same tiled weights; used by the tests as an
// independent check of the tensor-core path at sizes the CPU oracle cannot reach.
// `which`: 0 = gate/up + SwiGLU (xp -> hbuf), 1 = down projection (hbuf -> obuf).
int launch_ffn_simt(const FfnParams& p, int which, cudaStream_t s);
// tcgen05 / TMEM / TMA grouped GEMMs.
int launch_ffn_tc(const FfnParams& p, int nmax, int which, cudaStream_t s);

struct CombineParams {
  const __nv_bfloat16* obuf;   // [rows, H]
  const int32_t* inv;          // [T*k]  row of (token,slot); <0 = not local (skipped)
  const float* weights;        // [T,k]
  __nv_bfloat16* y;            // [T,H]
  int32_t T, k, H;
  int32_t n_shared, Tk;        // shared rows at shared[(j*T + t)]
  int32_t bf16_products;
  const __nv_bfloat16* shared; // [n_shared*T, H]; null: obuf + Tk*H
};
int launch_combine(const CombineParams& p, cudaStream_t s);
// Expert-parallel partial sums: partial[t,:] = sum over the slots whose expert is local of
// w[t,k] * out[t,k,:] in fp32 (no shared expert, no rounding); and the finish after the
// cross-rank sum: y[i,:] = bf16(reduced[i,:]) + shared rows.
// `sig` (may be null): the CTA that finishes last tells every rank that the partial sums are complete.
int launch_combine_partial(const CombineParams& p, float* partial, const PeerSignal* sig, cudaStream_t s);
int launch_combine_finish(const float* reduced, const __nv_bfloat16* shared, int32_t n_shared, int32_t T,
                          int32_t H, __nv_bfloat16* y, cudaStream_t s);
// out[t,s,:] = obuf[inv[t*k+s]]
int launch_unpermute(const __nv_bfloat16* obuf, const int32_t* inv, __nv_bfloat16* out, int32_t T,
                     int32_t k, int32_t H, cudaStream_t s);

// Row-segment copies for the expert-parallel regroup: dst[seg.dst + i] = src[seg.src + i], i < seg.n
struct RowSegment {
  int32_t src, dst, n, pad;
};
int launch_ep_push(const __nv_bfloat16* x, int32_t T, int32_t H, void* const* xall, void* const* flags, int32_t world,
                   int32_t rank, uint32_t step_no, size_t dst_elem_off, uint32_t* counters, cudaStream_t s);
int launch_ep_wait(const uint32_t* flags, int32_t world, uint32_t step_no, DevStatus* st, int32_t where, cudaStream_t s);
int launch_ep_pull_finish(void* const* partial, size_t src_elem_off, int32_t world, const uint32_t* my_flags,
                          uint32_t step_no, const __nv_bfloat16* shared, int32_t n_shared, int32_t T, int32_t H,
                          __nv_bfloat16* y, DevStatus* st, cudaStream_t s);
int launch_segment_copy(const __nv_bfloat16* src, __nv_bfloat16* dst, const RowSegment* segs, int32_t n_segs,
                        int32_t max_rows_per_seg, int32_t H, cudaStream_t s);

// Registration-time layout kernels.
struct RetileParams {
  const void* src;        // [rows, cols] row-major, element size 1 or 2
  int32_t rows, cols;     // logical matrix
  int32_t row0, n_rows;   // source row window written as tiles (virtual shared experts)
  int32_t col0, n_cols;   // source column window
  int32_t esz;            // 1 or 2
  int32_t rt_pairs;         // 1: row tiles 2j and 2j+1 are stored next to each other per K tile:
                            //    tile(rt,kt) at dst + (((rt>>1)*n_kt + kt)*2 + (rt&1)) * 16 KiB
  uint8_t* dst;           // first tile of (row tile 0, k tile 0)
  int64_t rt_stride;      // bytes between consecutive row tiles
  int64_t kt_stride;      // bytes between consecutive K tiles
  int32_t n_rt, n_kt;     // tiles to write (padding tiles are zero-filled)
  uint32_t xor_mask = 0;  // applied to every 32-bit word written: 0x80808080 turns int8 codes into offset binary
};
int launch_retile(const RetileParams& p, cudaStream_t s);
struct ScaleRetileParams {
  const float* src;       // [ceil(rows/128), ceil(cols/128)]
  int32_t src_cols;
  int32_t rb0, kb0;       // window origin in blocks
  int32_t n_rt, n_kt;
  float* dst;             // dst[(rt*n_kt + kt)*stride + lane]
  int32_t stride, lane;
  int32_t src_rows;
  int32_t rt_pairs;       // 1: dst[(((rt>>1)*n_kt + kt)*2 + (rt&1))]
};
int launch_scale_retile(const ScaleRetileParams& p, cudaStream_t s);
int launch_scale_pow(const float* a, int64_t na, const float* b, int64_t nb, float* out, cudaStream_t s);
int launch_fill_f32(float* dst, float v, int64_t n, cudaStream_t s);
int launch_dequant(const void* w, int32_t w_dtype, const float* scale, int32_t rows, int32_t cols,
                   __nv_bfloat16* out, cudaStream_t s);
int launch_f16_to_bf16(const void* src, __nv_bfloat16* dst, int64_t n, cudaStream_t s);

}  // namespace ek
