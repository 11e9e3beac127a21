/*
 * ek_b200.h -- C ABI of the B200 (sm_100a) expert-worker compute backend for Expert Kit.
 *
 * This is the only boundary between the Expert Kit worker (Rust, `ek-computation`) or the
 * Python integration packages and the CUDA code.  Plain pointers and sizes only.  Every
 * entry point names the reference interface it stands in for (paths are relative to the
 * expert-kit repository root).
 *
 * Conventions
 *   - Every function returns an ek_status_t; nothing throws or aborts across the boundary.
 *     (The reference panics on malformed requests: ek-computation/src/worker/core.rs:52-56;
 *     here those become EK_INVALID_INPUT.)
 *   - `x`, `y`, `out` buffers may be HOST or DEVICE pointers; the library looks at the
 *     pointer attributes and stages host buffers through its own pinned/device workspace.
 *   - Weights are copied (and re-tiled) at registration; the caller's bytes may be freed as
 *     soon as the call returns (the reference aliases them instead:
 *     ek-computation/src/backend/torch/mod.rs:119-130).  Device-resident weights are read on
 *     the library's own load stream, which waits for no other stream: the work that produced
 *     them must be complete when the registration call is made.
 *   - All workspace is sized from `max_tokens` at create time; forward calls allocate nothing.
 *   - A backend may be used from many host threads; forward calls on one backend share one
 *     workspace and run one after the other on the backend's stream, except that worker-level
 *     calls (ek_expert_forward, ek_worker_forward_wire) that arrive together are served as one
 *     grouped launch; registration/eviction may run concurrently.
 */
#ifndef EK_B200_H_
#define EK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes; the first group mirrors EKError (ek-base/src/error.rs:13-72). */
typedef enum ek_status {
  EK_OK = 0,
  EK_EXPERT_NOT_FOUND = 1,        /* EKError::ExpertNotFound        error.rs:26-27 */
  EK_EXPERT_WEIGHT_NOT_FOUND = 2, /* EKError::ExpertWeightNotFound  error.rs:29-30 */
  EK_INVALID_INPUT = 3,           /* EKError::InvalidInput          error.rs:50-51 */
  EK_SAFETENSOR = 4,              /* EKError::SafeTensorError       error.rs:14-15 */
  EK_NOT_FOUND = 5,               /* EKError::NotFound              error.rs:32-33 */
  EK_CUDA = 16,                   /* a CUDA runtime/driver call failed */
  EK_TIMEOUT = 17,                /* a bounded device-side wait ran out; context stays usable */
  EK_BOUNDS = 18,                 /* device-side index check failed (debug builds) */
  EK_NO_MEMORY = 19,
  EK_UNSUPPORTED = 20
} ek_status_t;

/* Element types; mirrors DType (ek-computation/src/backend/mod.rs:6-15) and the safetensors
 * dtype strings the weight server emits. */
typedef enum ek_dtype {
  EK_BF16 = 0,    /* "BF16" */
  EK_F32 = 1,     /* "F32"  */
  EK_F8_E4M3 = 2, /* "F8_E4M3" */
  EK_I8 = 3,      /* "I8" */
  EK_I32 = 4,     /* "I32" */
  EK_F16 = 5,     /* "F16" (accepted for weights, converted to bf16 at registration) */
  EK_U8 = 6,
  EK_I64 = 7
} ek_dtype_t;

/* A named tensor view: what `safetensors::tensor::TensorView` carries
 * (ek-computation/src/backend/mod.rs:22-29, torch/mod.rs:137-153). */
typedef struct ek_tensor_view {
  const char* name;     /* e.g. "model.layers.3.mlp.experts.17.up_proj.weight" */
  int32_t dtype;        /* ek_dtype_t */
  int32_t ndim;
  int64_t shape[4];
  const void* data;     /* host or device, row-major, contiguous */
} ek_tensor_view_t;

enum { EK_SCORE_SOFTMAX = 0, EK_SCORE_SIGMOID = 1 };
enum { EK_QUANT_BF16 = 0, EK_QUANT_FP8_BLOCK128 = 1, EK_QUANT_INT8_BLOCK128 = 2 };

/* Layer/instance configuration.  Stands in for EKInstance{hidden, intermediate, backend}
 * (ek-computation/src/x.rs:27-43, filled from `inference.*`, ek-base/src/config.rs:26-31) plus
 * the routing hyper-parameters the Python frontends read from the HF model config
 * (expertkit_torch/models/qwen3_moe.py:61-63; deepseek_v3/model.py:56). */
typedef struct ek_config {
  int32_t hidden;            /* H */
  int32_t intermediate;      /* I of a routed expert */
  int32_t n_experts;         /* routed experts per layer (global count) */
  int32_t top_k;
  int32_t scoring;           /* EK_SCORE_* */
  int32_t n_group;           /* 1 = no group limit */
  int32_t topk_group;
  int32_t norm_topk_prob;    /* renormalise the selected weights */
  float routed_scaling;      /* multiplied into the weights after renormalisation */
  int32_t n_shared_experts;  /* shared expert intermediate = intermediate * n_shared_experts */
  int32_t bf16_combine;      /* 1: routing weights rounded to bf16, bf16 products (Qwen3 path) */
  int32_t quant;             /* EK_QUANT_* : storage form of expert weights */
  int32_t max_tokens;        /* largest T of one forward call; sizes the workspace */
  int32_t max_layers;        /* number of distinct layer indices that may hold experts */
  int32_t device;            /* CUDA device ordinal */
  int32_t ep_rank;           /* expert-parallel rank of this process */
  int32_t ep_size;           /* number of expert-parallel ranks; experts e with
                                e / (n_experts/ep_size) == ep_rank are local */
  int32_t replica_slots;     /* extra expert slots per layer for experts OUTSIDE this rank's window
                                (replicas of hot experts); 0 = none */
  char model_name[64];       /* prefix of expert ids: "<model_name>/l<layer>-e<expert>" */
} ek_config_t;

typedef struct ek_backend ek_backend_t;

/* ---- lifetime ------------------------------------------------------------------------- */

/* ExpertBackend::build's environment (ek-computation/src/ffn/mod.rs:22-35) + the global
 * ExpertDB (ek-computation/src/worker/manager.rs:32-44). */
int32_t ek_backend_create(const ek_config_t* cfg, ek_backend_t** out);
void ek_backend_destroy(ek_backend_t* be);

/* Why the last ek_backend_create on this thread's process failed (no handle exists yet). */
const char* ek_create_error(void);
/* Message of the last failure on this backend (handle-local, valid until the next call). */
const char* ek_last_error(const ek_backend_t* be);
const char* ek_status_name(int32_t status);

/* ---- expert registry: ExpertDB (ek-computation/src/worker/manager.rs:13-23) ------------- */

/* ExpertDB::insert after ExpertBackend::build -> ExpertWeight::from_safetensor
 * (ek-computation/src/worker/x.rs:13-34, ffn/meta.rs:57-75).  `id` is
 * ExpertKey::as_object_key, "model/l{L}-e{E}" (ek-db/src/safetensor/mod.rs:57-91); a shared
 * expert uses "model/l{L}-shared".  Tensors are picked by the reference's suffix rule:
 * "w1.weight"|"up_proj.weight", "w2.weight"|"down_proj.weight", "w3.weight"|"gate_proj.weight",
 * first match wins (torch/mod.rs:137-153); quantised payloads additionally take
 * "<weight name>_scale_inv" (F32, [ceil(rows/128), ceil(cols/128)];
 * ek-db/src/safetensor/transformer.rs:258-270). */
int32_t ek_expert_register(ek_backend_t* be, const char* id,
                           const ek_tensor_view_t* tensors, int32_t n_tensors);

/* Same, from the serialised bundle the weight server returns for GET /expert/{m}/{l}/{e}
 * (ek-db/src/safetensor/transformer.rs:282-296; SafeTensorDB::load, mod.rs:136-173). */
int32_t ek_expert_register_safetensors(ek_backend_t* be, const char* id,
                                       const void* blob, size_t blob_len);

/* The expert as this library keeps it in HBM (16 KiB tiles, int8 codes in offset binary, re-ordered
 * scales and the per-expert powers of two), for a cache next to the raw bundle in the weight server's file cache
 * (ek-db/src/safetensor/mod.rs:144-171): a restart registers the blob with plain copies and skips
 * decoding and re-tiling.  The blob is only valid for the same quant/hidden/intermediate and for
 * EK_TILE_LAYOUT_VERSION; anything else is refused (EK_UNSUPPORTED / EK_INVALID_INPUT) and the
 * caller falls back to the bundle.  *needed receives the blob size; EK_INVALID_INPUT when `cap`
 * is too small. */
#define EK_TILE_LAYOUT_VERSION 5
int32_t ek_expert_export_tiles(ek_backend_t* be, const char* id, void* blob, size_t cap, size_t* needed);
int32_t ek_expert_register_tiles(ek_backend_t* be, const char* id, const void* blob, size_t blob_len);

/* ExpertDB::mark_loading (manager.rs:60-70): *fresh = 1 when this call claimed the id. */
int32_t ek_expert_mark_loading(ek_backend_t* be, const char* id, int32_t* fresh);
/* ExpertDB::remove (manager.rs:71-74; caller: worker/state.rs:157-165).  Removing an unknown id
 * is not an error, as in the reference.  Device memory of the slot is reused by later
 * registrations once forwards in flight have drained. */
int32_t ek_expert_evict(ek_backend_t* be, const char* id);
/* ExpertDB::has / loaded / loading / keys (manager.rs:46-58,86-88). */
int32_t ek_expert_has(const ek_backend_t* be, const char* id);
int32_t ek_expert_loaded(const ek_backend_t* be);
int32_t ek_expert_loading(const ek_backend_t* be);
/* Writes the ids in ascending string order (BTreeMap order), '\n'-separated, NUL-terminated;
 * returns EK_INVALID_INPUT and sets *needed when `cap` is too small. */
int32_t ek_expert_keys(const ek_backend_t* be, char* buf, size_t cap, size_t* needed);

/* Router weight of one layer: `gate.weight` [E,H] (BF16 or F32) and, for sigmoid scoring, the
 * optional `e_score_correction_bias` [E] F32 (expertkit_torch/models/qwen3_moe.py:65;
 * deepseek_v3/model.py:56).  Needed only by ek_moe_forward_fused. */
int32_t ek_router_register(ek_backend_t* be, int32_t layer, const void* weight, int32_t weight_dtype,
                           const float* bias /* may be NULL */);

/* ---- forward -------------------------------------------------------------------------- */

/* Worker level: EKInstanceGate::forward -> ExpertBackend::forward -> TorchFFN::forward
 * (ek-computation/src/worker/core.rs:47-74, ffn/mod.rs:39-52, ffn/expert_torch.rs:80-101):
 * y[n,H] = down( up(x) * silu(gate(x)) ) for one registered expert, bf16 in, bf16 out. */
int32_t ek_expert_forward(ek_backend_t* be, const char* id, const void* x_bf16, int32_t n,
                          void* y_bf16);

/* Controller level: NaiveExecutor submit/exec/output
 * (ek-computation/src/controller/executor.rs:85-110,135-262,283-299): `ids[T,k]` names one local
 * expert per (token, slot); `out[T,k,H]` receives the UNWEIGHTED bf16 expert outputs in the
 * request's slot order -- the payload of ForwardResp (ek-proto/ek/worker/v1/expert.proto:14-17). */
int32_t ek_moe_forward(ek_backend_t* be, int32_t layer, const void* x_bf16, int32_t T,
                       const int32_t* ids, int32_t k, void* out_bf16);

/* Optional outputs of the fused call; any pointer may be NULL.  All are written in the
 * canonical order "descending score, ties towards the lower expert index". */
typedef struct ek_route_debug {
  float* logits;      /* [T,E]  fp32 (softmax scoring: the bf16-rounded logits, widened) */
  int32_t* ids;       /* [T,k]  */
  float* weights;     /* [T,k]  fp32 (bf16_combine: the bf16-rounded weights, widened) */
  int32_t* counts;    /* [E]    rows per expert */
  int32_t* offsets;   /* [E+1]  exclusive prefix sum of counts */
  int32_t* perm;      /* [T*k]  perm[offsets[e]+r] = token*k+slot of expert e's r-th row */
} ek_route_debug_t;

/* Frontend + controller + worker in one call: router (qwen3_moe.py:161-169 or the
 * DeepSeek-V3 router called at deepseek_v3/model.py:142), bucketing (executor.rs:283-299),
 * expert FFNs (expert_torch.rs:80-85), weighted combine (model.py:96-104, qwen3_moe.py:102-104)
 * and shared expert (model.py:152):  y[T,H] = shared(x) + sum_k w[t,k] * expert_{ids[t,k]}(x[t]). */
int32_t ek_moe_forward_fused(ek_backend_t* be, int32_t layer, const void* x_bf16, int32_t T,
                             void* y_bf16, const ek_route_debug_t* debug /* may be NULL */);

/* Frontend routing alone on caller-supplied logits [T,E] fp32 (same canonical order). */
int32_t ek_route_from_logits(ek_backend_t* be, const float* logits, int32_t T,
                             const float* bias /* may be NULL */, int32_t* ids, float* weights,
                             int32_t* counts, int32_t* offsets, int32_t* perm);

/* Weighted combine alone: y[T,H] = sum_k w[t,k]*out[t,k,:] (+ shared[T,H] if non-NULL), the
 * frontend's step after ForwardResp (model.py:96-104,152; qwen3_moe.py:102-104). */
int32_t ek_combine(ek_backend_t* be, const void* out_bf16, const float* weights, int32_t T,
                   int32_t k, const void* shared_bf16 /* may be NULL */, void* y_bf16);

/* w8a16_activate (ek-computation/src/ffn/expert_torch.rs:24-53):
 * out_bf16[i,j] = bf16_rne(float(w[i,j]) * scale[i/128, j/128]); rows, cols multiples of 128. */
int32_t ek_w8a16_activate(ek_backend_t* be, const void* w, int32_t w_dtype, const float* scale,
                          int32_t rows, int32_t cols, void* out_bf16);

/* Wire level: the worker's handling of one ForwardReq (worker/core.rs:47-74): `req_tensor` is
 * the safetensors blob holding the single key "data" ([n,H] BF16); `expert_id` is
 * sequences[0].experts[0]; the reply blob (key "data", [n,H] BF16) is written to `resp`.
 * *resp_len receives the needed size; EK_INVALID_INPUT if `resp_cap` is too small. */
int32_t ek_worker_forward_wire(ek_backend_t* be, const char* expert_id, const void* req_tensor,
                               size_t req_len, void* resp, size_t resp_cap, size_t* resp_len);

/* ---- expert parallel over peer memory ----------------------------------------------------
 * The gather scheme with this library's own kernels over NVLink instead of an all-gather and a
 * reduce-scatter.  One process per GPU.  Each rank allocates three buffers
 *   xall     gathered tokens   [2][world*T][H] bf16   (written by every rank)
 *   partial  partial sums      [2][world*T][H] fp32   (written by the owner, read by all)
 *   flags    flag words        [2*EK_EP_MAX_RANKS] u32
 * with ek_ep_peer_alloc, which returns their CUDA IPC handles; the host exchanges the handles (any
 * transport) and every rank opens every other rank's with ek_ep_peer_open.  `step` counts the layer
 * passes of the group (the same value on every rank, increasing by one from 0 after alloc); buffers
 * are used alternately by step parity.  push / partial / finish are asynchronous on the backend's
 * stream and must be called by every rank in the same order.  Device-side waits for a peer are
 * bounded: a rank that never arrives surfaces as EK_TIMEOUT at the next ek_sync, the context stays
 * usable.  ek_ep_peer_close unmaps the peers' buffers; call it on every rank, then synchronise the
 * ranks, before a rank destroys its backend (which frees its own buffers).  No reference
 * counterpart: the reference moves rows by gRPC (ek-computation/src/controller/executor.rs:141-226). */
#define EK_EP_MAX_RANKS 16
#define EK_IPC_HANDLE_BYTES 64
int32_t ek_ep_peer_alloc(ek_backend_t* be, int32_t tokens_per_rank, uint8_t* handles /* out [3*EK_IPC_HANDLE_BYTES] */);
int32_t ek_ep_peer_open(ek_backend_t* be, int32_t rank, const uint8_t* handles /* that rank's [3*EK_IPC_HANDLE_BYTES] */);
int32_t ek_ep_peer_close(ek_backend_t* be);
/* Stores this rank's tokens x[T,H] into every rank's xall and publishes the step there. */
int32_t ek_ep_peer_push(ek_backend_t* be, const void* x_dev, int32_t T, uint32_t step);
/* Waits for every rank's tokens, then routes the gathered batch, runs this rank's experts and leaves
 * the fp32 partial sums in this rank's `partial`; publishes the step to every rank. */
int32_t ek_ep_peer_partial(ek_backend_t* be, int32_t layer, int32_t T, uint32_t step);
/* Waits for every rank's partial sums, loads this rank's token slice from all of them, adds in rank
 * order, adds the shared expert, rounds: y[T,H] bf16. */
int32_t ek_ep_peer_finish(ek_backend_t* be, int32_t layer, int32_t T, uint32_t step, void* y_dev);

/* ---- observability -------------------------------------------------------------------- */

/* Rows per expert seen by the last fused/controller-level call on `layer`: the quantity the
 * worker exports as `worker_expert_activation` (ek-computation/src/metrics.rs:22-71). */
int32_t ek_expert_counts(ek_backend_t* be, int32_t layer, int32_t* counts /* [n_experts] */);

/* Expert ids [T,k] and routing weights [T,k] that the last routing pass of this backend produced
 * (fused, expert-parallel partial or route stage), for checks against the frontend's own routing
 * (expertkit_torch/models/qwen3_moe.py:161-169; deepseek_v3/model.py:142).  Either pointer may be
 * NULL; host or device.  Synchronises the backend's stream. */
int32_t ek_last_routing(ek_backend_t* be, int32_t T, int32_t* ids, float* weights);

enum { EK_STAGE_ROUTE = 0, EK_STAGE_PERMUTE = 1, EK_STAGE_GATEUP = 2, EK_STAGE_DOWN = 3,
       EK_STAGE_COMBINE = 4, EK_STAGE_COUNT = 5 };
/* Device time (ms, CUDA events on the backend's stream) of each stage when stage timing is
 * enabled: the mean over the layer passes issued since the previous ek_sync (the newest 64 of
 * them), so that a back-to-back run can be profiled without a host synchronisation per pass;
 * the analogue of PerfTimer (ek-base/src/utils.rs:4-45). */
int32_t ek_stage_timing_enable(ek_backend_t* be, int32_t on);
int32_t ek_stage_times(ek_backend_t* be, float* ms /* [EK_STAGE_COUNT] */);

/* Number of kernels this library launched on the backend since creation. */
int64_t ek_kernel_launches(const ek_backend_t* be);

/* Worker-level calls (`ek_expert_forward`, `ek_worker_forward_wire`) issued from several threads at
 * once are served together: whoever holds the forward lock runs every request queued so far as one
 * grouped launch per layer, the way the reference's 48 runtime threads each enter
 * EKInstanceGate::forward (ek-computation/src/worker/core.rs:47-74) but share one GPU here.
 * `calls` = requests served so far, `batches` = grouped passes that served them. */
int32_t ek_worker_batch_stats(ek_backend_t* be, int64_t* calls, int64_t* batches);

/* FP8 / INT8 block scales inside the grouped GEMM.  0 (default): the weight codes are converted
 * exactly to f16 and both MMA operands are f16 (the activations of these GEMMs are kept in f16 from
 * the row gather on); the block scale, times a per-expert power of two that the epilogue takes out
 * again, is applied to the activation tile (chunks of <= 64 rows) or to the weight operand (128-row
 * chunks) with one rounding to 11 bits per element, where the reference's bf16(w * s) rounds to 8.
 * 1: bf16 operands with A = bf16_rne(float(w) * s), bit-exact w8a16_activate
 * (ek-computation/src/ffn/expert_torch.rs:24-53), at roughly a third of the weight-streaming rate.
 * ek_w8a16_activate itself is always exact. */
int32_t ek_set_precise_dequant(ek_backend_t* be, int32_t on);

/* Test hook: 0 = tensor-core kernels (default), 1 = the CUDA-core evaluation of the same
 * tiled weights that the tests use as a second opinion at large sizes.  Not a tuning knob. */
int32_t ek_debug_set_ffn_impl(ek_backend_t* be, int32_t impl);

/* ---- device-resident fast path (no host staging, used by the Python integration, the
 *      benchmark and expert-parallel drivers; stream is a cudaStream_t or NULL) ----------- */
/* All later work of this backend runs on `cuda_stream` (NULL = CUDA's default stream);
 * (void*)-1 returns to the backend's own non-blocking stream. */
int32_t ek_set_stream(ek_backend_t* be, void* cuda_stream);
/* Same as ek_moe_forward_fused with device pointers, asynchronous on the backend stream. */
int32_t ek_moe_forward_fused_async(ek_backend_t* be, int32_t layer, const void* x_dev, int32_t T,
                                   void* y_dev);
int32_t ek_sync(ek_backend_t* be);

/* ---- expert-parallel stages ------------------------------------------------------------------
 * The reference shards experts over worker processes and moves rows by one gRPC per expert
 * (ek-computation/src/controller/executor.rs:141-226).  Here expert e of a layer lives on rank
 * e / (n_experts / ep_size) of one multi-GPU box and rows move by all-to-all over NVLink, which
 * the caller performs between these three stages (see ek_b200/ep.py).  All pointers are device
 * pointers; all work is asynchronous on the backend stream (ek_set_stream / ek_sync).
 *
 * 1. ek_ep_route: route this rank's tokens over ALL experts and gather their rows in global expert
 *    order into send_rows_dev[T*k, H] (rows of one destination rank are contiguous).
 *    counts_dev[n_experts] receives the rows per expert.
 * 2. ek_ep_ffn: rows_dev holds what arrived, ordered by (source rank, local expert);
 *    counts_src_host[ep_size][n_experts/ep_size] (HOST) gives the row count of each such segment.
 *    Runs this rank's experts on them, and the shared expert on the local tokens x_dev[T,H];
 *    out_rows_dev receives the expert outputs in the same arrival order.
 * 3. ek_ep_combine: returned_rows_dev[T*k, H] are the outputs sent back by the owners, in the
 *    order of stage 1's send rows; y_dev[T,H] = sum_k w*out + shared(x). */
int32_t ek_ep_route(ek_backend_t* be, int32_t layer, const void* x_dev, int32_t T, void* send_rows_dev,
                    int32_t* counts_dev);
int32_t ek_ep_ffn(ek_backend_t* be, int32_t layer, const void* rows_dev, const int32_t* counts_src_host,
                  const void* x_dev, int32_t T, void* out_rows_dev);
int32_t ek_ep_combine(ek_backend_t* be, int32_t layer, const void* returned_rows_dev, int32_t T, void* y_dev);

/* Expert parallelism for decode-sized batches, without data-dependent exchange sizes or host
 * synchronisation: the caller all-gathers the tokens of all ranks into x_all_dev[T_all,H];
 * ek_ep_partial routes all of them, runs THIS rank's experts on the rows routed to them (and the
 * shared expert on the rank's own slice [t0, t0+T_local)) and writes fp32 partial sums
 * partial_dev[T_all,H]; the caller sums the partials over the ranks (reduce-scatter) and
 * ek_ep_finish turns its slice into y_dev[T_local,H] = bf16(sum) + shared(x).  Same exchange the
 * reference performs with gRPC fan-out/fan-in (executor.rs:141-226), as two collectives. */
int32_t ek_ep_partial(ek_backend_t* be, int32_t layer, const void* x_all_dev, int32_t T_all, int32_t t0,
                      int32_t T_local, float* partial_dev);
int32_t ek_ep_finish(ek_backend_t* be, int32_t layer, const float* reduced_dev, int32_t T_local, void* y_dev);

/* Replicated experts.  The reference may hold an expert on several workers and sends each request
 * for it to one of them, chosen at random (ExpertRegistryImpl::select_random,
 * ek-computation/src/controller/registry.rs:49-72; the histogram that tells which experts are hot is
 * ek_expert_counts).  Here a rank created with `replica_slots` > 0 may register experts outside its
 * window (ek_expert_register / ek_expert_register_tiles take any expert index then; ek_expert_evict
 * frees the slot), and ek_ep_set_owners names, for the following passes on `layer`, the ONE rank that
 * serves each expert: owners[n_experts] (host), every rank passing the same table; a rank must hold
 * what the table gives it (EK_EXPERT_NOT_FOUND otherwise).  NULL returns to the window rule.  Applies
 * to the schemes in which every rank routes the gathered batch (ek_ep_partial, ek_ep_peer_partial). */
int32_t ek_ep_set_owners(ek_backend_t* be, int32_t layer, const int32_t* owners /* [n_experts] or NULL */);

/* ---- allocation-free bucketing ------------------------------------------------------------
 * No counterpart in the reference.  Some callers are not allowed to allocate device memory (a
 * worker whose memory is one pre-carved pool, a plugin running inside another runtime's step);
 * this entry point needs no backend handle and calls no allocator: it buckets caller-supplied
 * assignments with the library's own kernels, using a scratch array that is built into the
 * library image (EK_NOALLOC_MAX_ASSIGNMENTS ints plus a status word per GPU, held until exit).
 *
 *   ids_dev[T*k] (device, values in [0,n_experts))  ->  counts_dev[n_experts],
 *   offsets_dev[n_experts+1], perm_dev[T*k]  (device), same definition as ek_route_debug_t.
 *
 * Runs on `cuda_stream` of the CURRENT device.  EVERY call ends by copying the device status word
 * back and synchronising that stream, so it returns only after the kernels have completed and it
 * must never be issued on a stream that is being captured.  The first call on a device also
 * resolves the scratch address.  T*k beyond EK_NOALLOC_MAX_ASSIGNMENTS is refused with
 * EK_INVALID_INPUT; `errbuf` (may be NULL) receives a message.  Calls share the scratch: do not
 * overlap two of them on one GPU. */
#define EK_NOALLOC_MAX_ASSIGNMENTS 65536
int32_t ek_bucket_noalloc(const int32_t* ids_dev, int32_t T, int32_t k, int32_t n_experts,
                          int32_t* counts_dev, int32_t* offsets_dev, int32_t* perm_dev,
                          void* cuda_stream, char* errbuf, size_t errcap);

#ifdef __cplusplus
}
#endif
#endif /* EK_B200_H_ */
