// Host side of the C ABI: expert registry (the worker's ExpertDB), weight loader that re-tiles
// bundles into the device layout, workspace, and the forward entry points that chain the
// kernels on one stream.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <thread>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <set>
#include <shared_mutex>
#include <string>
#include <vector>

#include "ek_internal.h"
#include "safetensors.hpp"

using namespace ek;

namespace {

struct Layer {
  uint8_t* gu = nullptr;
  uint8_t* dn = nullptr;
  float* gu_scale = nullptr;
  float* dn_scale = nullptr;
  float* pow2 = nullptr;             // [2][n_slots]: gate/up and down activation powers of two (quantised only)
  int32_t* registered = nullptr;     // device flags [n_slots]
  std::vector<char> host_registered;
  void* router_w = nullptr;
  int router_f32 = 0;
  __nv_bfloat16* router_bf16 = nullptr;   // bf16 view of the router weight for the tensor-core router
  bool router_bf16_owned = false;
  bool router_tc = false;
  CUtensorMap router_map;
  float* router_bias = nullptr;
  int32_t* last_counts = nullptr;    // device [E]
  bool have_counts = false;
  // replicas: slot of every expert this rank holds (own window and replica slots), -1 otherwise
  int32_t* slot_of = nullptr;        // device [E]
  std::vector<int32_t> host_slot_of;
  std::vector<int32_t> replica_expert;   // [replica_slots] expert held by each replica slot, -1 = free
  int32_t* owners = nullptr;         // device [E]: per-pass owner table (valid while has_owners)
  bool has_owners = false;
};

struct ExpertRef {
  int layer;
  int slot;
};

}  // namespace

// Buffers of the peer-memory expert-parallel scheme: this rank's own allocations and every other
// rank's, mapped through CUDA IPC.
struct PeerTable {
  int T_cap = 0;
  void* own[3] = {nullptr, nullptr, nullptr};
  void* xall[EK_EP_MAX_RANKS] = {};
  void* partial[EK_EP_MAX_RANKS] = {};
  void* flags[EK_EP_MAX_RANKS] = {};
  bool opened[EK_EP_MAX_RANKS] = {};
};

// One worker-level call waiting to be served (lives on its caller's stack).
struct ExpertReq {
  const char* id = nullptr;
  const void* x = nullptr;
  void* y = nullptr;
  int n = 0;
  int row0 = 0;
  int rc = EK_OK;
  std::atomic<bool> done{false};   // set (release) by whoever served the request, after rc
};

// One of a few independent loader lanes: registrations from several threads run side by side, each
// with its own stream, device staging and pinned bounce buffer (the reference loads up to 64 experts
// concurrently, ek-computation/src/worker/state.rs:178-197).
struct LoadLane {
  cudaStream_t stream = nullptr;
  cudaEvent_t ev = nullptr;
  void* stage[3] = {nullptr, nullptr, nullptr};
  size_t stage_cap[3] = {0, 0, 0};
  float* stage_scale[3] = {nullptr, nullptr, nullptr};
  size_t stage_scale_cap[3] = {0, 0, 0};
  void* stage_cvt = nullptr;
  size_t stage_cvt_cap = 0;
  uint8_t* bounce = nullptr;           // pinned host memory: pageable sources are copied here by the calling thread
  size_t bounce_cap = 0;
  bool busy = false;
};
constexpr int kLoadLanes = 8;

struct ek_backend {
  ek_config_t cfg;
  Dims d;
  int n_local = 0, e_lo = 0, e_hi = 0, n_slots = 0;
  int n_sm = 148;
  int rows_cap = 0, max_chunks = 0;
  cudaStream_t stream = nullptr;       // forward stream (owned unless replaced by ek_set_stream)
  cudaStream_t own_stream = nullptr;
  cudaStream_t load_stream = nullptr;
  cudaEvent_t fwd_done = nullptr;
  // stage timers: one set of events per layer pass, for up to kTimingRing passes between two reads
  static constexpr int kTimingRing = 64;
  cudaEvent_t ev[kTimingRing][EK_STAGE_COUNT + 1] = {};
  int ev_pass = 0;                     // passes recorded since the last read
  bool timing = false;
  float stage_ms[EK_STAGE_COUNT] = {};
  int ffn_impl = 0;                    // 0 tensor cores, 1 CUDA-core checker
  int ep_rows = 0, ep_T = 0;           // rows / tokens of the last ek_ep_ffn
  cudaEvent_t ep_upload_done = nullptr;
  bool ep_uploaded = false;
  int32_t* h_ep_count = nullptr;       // pinned
  int precise = 0;                     // fp8 block scales in fp32 inside the GEMM

  // workspace
  __nv_bfloat16 *x_dev = nullptr, *y_dev = nullptr, *xp = nullptr, *hbuf = nullptr, *obuf = nullptr;
  __nv_bfloat16* tk_dev = nullptr;     // [T,k,H] staging of the controller-level call (lazy)
  size_t tk_cap = 0;
  float *logits = nullptr, *weights = nullptr, *bias_scratch = nullptr, *partial = nullptr;
  void* encode_fn = nullptr;           // cuTensorMapEncodeTiled
  int32_t* flag_dev = nullptr;
  int32_t *ids = nullptr, *counts = nullptr, *offsets = nullptr, *perm = nullptr, *inv = nullptr;
  ChunkDesc* chunks = nullptr;
  int32_t* n_chunks = nullptr;
  DevStatus* status = nullptr;
  uint32_t* front_ticket = nullptr;    // last-CTA tickets: [0] fused small-batch front kernel, [1] expert-parallel signal, [2] permute + work list
  int front_small = 1;                 // use that kernel when the batch qualifies
  float* sk_buf = nullptr;             // partial accumulators of K-split work items
  uint32_t* sk_flags = nullptr;
  int split_k = 1;
  int weights_ahead = 1;
  DevStatus* h_status = nullptr;       // pinned
  ChunkDesc* h_chunks = nullptr;       // pinned, worker-level call
  int h_chunks_cap = 0;
  RowSegment* segs = nullptr;          // device, expert-parallel regroup
  RowSegment* h_segs = nullptr;        // pinned
  int segs_cap = 0;
  CUtensorMap* maps = nullptr;         // device: x_maps[4], h_maps[4]
  void* h_x = nullptr;                 // pinned staging
  void* h_y = nullptr;
  size_t h_cap = 0;
  void* h_tk = nullptr;
  size_t h_tk_cap = 0;
  // loader staging
  void* stage[3] = {nullptr, nullptr, nullptr};
  size_t stage_cap[3] = {0, 0, 0};
  float* stage_scale[3] = {nullptr, nullptr, nullptr};
  size_t stage_scale_cap[3] = {0, 0, 0};
  void* stage_cvt = nullptr;
  size_t stage_cvt_cap = 0;

  std::map<int, Layer> layers;
  std::map<std::string, ExpertRef> experts;   // BTreeMap<String, Arc<ExpertBackend>>
  std::set<std::string> loading;
  mutable std::shared_mutex reg_mu;           // the worker's RwLock around ExpertDB
  uint32_t* ep_counters = nullptr;            // per-destination CTA counters of the peer push kernel
  PeerTable peers;                            // expert parallel over peer memory
  std::mutex fwd_mu;                          // forwards share one workspace
  std::mutex pend_mu;                         // queue of worker-level requests waiting for a grouped launch
  std::vector<ExpertReq*> pending;
  std::condition_variable pend_cv;            // signalled after every grouped pass
  int last_batch = 1;                         // requests served by the previous pass
  int64_t batched_calls = 0, batched_launches = 0;   // worker-level calls served / grouped launches used (under fwd_mu)
  std::mutex load_mu;                         // loads other than ek_expert_register share one set of staging buffers
  LoadLane lanes[kLoadLanes];                 // ek_expert_register: one lane per registration in flight
  std::mutex lane_mu;
  std::condition_variable lane_cv;
  std::set<std::string> lane_ids;             // ids being registered right now (one registration per id at a time)
  mutable std::mutex err_mu;
  mutable std::string err;
  std::atomic<int64_t> launches{0};
};

namespace {

int fail(const ek_backend* be, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (be) {
    std::lock_guard<std::mutex> g(be->err_mu);
    be->err = buf;
  }
  return code;
}

#define CK(call)                                                                              \
  do {                                                                                        \
    cudaError_t e__ = (call);                                                                 \
    if (e__ != cudaSuccess)                                                                   \
      return fail(be, EK_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
  } while (0)

bool is_device_ptr(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

bool is_pinned_host(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeHost;
}

bool ends_with(const std::string& s, const char* suf) {
  size_t n = strlen(suf);
  return s.size() >= n && memcmp(s.data() + s.size() - n, suf, n) == 0;
}

// "model/l{L}-e{E}" (ExpertKey::from_expert_id, ek-db/src/safetensor/mod.rs:57-73) or
// "model/l{L}-shared".  Returns false on a malformed id.
bool parse_id(const std::string& id, std::string& model, int& layer, int& expert, bool& shared) {
  size_t p = id.rfind("/l");
  if (p == std::string::npos) return false;
  model = id.substr(0, p);
  std::string rest = id.substr(p + 2);
  size_t q = rest.find('-');
  if (q == std::string::npos || q == 0) return false;
  for (size_t i = 0; i < q; ++i)
    if (rest[i] < '0' || rest[i] > '9') return false;
  layer = atoi(rest.substr(0, q).c_str());
  std::string tail = rest.substr(q + 1);
  if (tail == "shared") {
    shared = true;
    expert = -1;
    return true;
  }
  shared = false;
  if (tail.size() < 2 || tail[0] != 'e') return false;
  for (size_t i = 1; i < tail.size(); ++i)
    if (tail[i] < '0' || tail[i] > '9') return false;
  expert = atoi(tail.c_str() + 1);
  return true;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

int make_maps(ek_backend* be) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  if (!fn || qres != cudaDriverEntryPointSuccess)
    return fail(be, EK_CUDA, "cuTensorMapEncodeTiled not available from the driver");
  EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(fn);
  be->encode_fn = fn;
  CUtensorMap host[8];
  const int rows_box[4] = {16, 32, 64, 128};
  for (int which = 0; which < 2; ++which) {
    void* base = which == 0 ? (void*)be->xp : (void*)be->hbuf;
    const uint64_t inner = which == 0 ? (uint64_t)be->d.H : (uint64_t)be->d.Ip;
    for (int i = 0; i < 4; ++i) {
      cuuint64_t gdim[2] = {inner, (cuuint64_t)be->rows_cap};
      cuuint64_t gstride[1] = {inner * 2};
      cuuint32_t box[2] = {64, (cuuint32_t)rows_box[i]};
      cuuint32_t estr[2] = {1, 1};
      CUresult r = encode(&host[which * 4 + i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, gdim, gstride, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return fail(be, EK_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    }
  }
  CK(cudaMemcpy(be->maps, host, sizeof host, cudaMemcpyHostToDevice));
  return EK_OK;
}

// 2-D bf16 tensor map [rows, inner] with a {64, box_rows} box and the 128-byte swizzle.
bool encode_2d(ek_backend* be, CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint32_t box_rows) {
  if (!be->encode_fn || (reinterpret_cast<uintptr_t>(base) & 15) || (inner * 2) % 16) return false;
  EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(be->encode_fn);
  cuuint64_t gdim[2] = {inner, rows};
  cuuint64_t gstride[1] = {inner * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int ensure_layer(ek_backend* be, int layer, Layer** out) {
  auto it = be->layers.find(layer);
  if (it != be->layers.end()) {
    *out = &it->second;
    return EK_OK;
  }
  if ((int)be->layers.size() >= be->cfg.max_layers)
    return fail(be, EK_INVALID_INPUT, "layer %d exceeds max_layers=%d", layer, be->cfg.max_layers);
  Layer L;
  const Dims& d = be->d;
  const size_t gu_bytes = (size_t)be->n_slots * d.it * d.kt_gu * 2 * kTileBytes;
  const size_t dn_bytes = (size_t)be->n_slots * d.hp * d.kt_dn * 2 * kTileBytes;
  CK(cudaMalloc(&L.gu, gu_bytes));
  CK(cudaMalloc(&L.dn, dn_bytes));
  if (d.quant != EK_QUANT_BF16) {
    CK(cudaMalloc(&L.gu_scale, (size_t)be->n_slots * d.it * d.kt_gu * 2 * sizeof(float)));
    CK(cudaMalloc(&L.dn_scale, (size_t)be->n_slots * d.hp * d.kt_dn * 2 * sizeof(float)));
    CK(cudaMalloc(&L.pow2, (size_t)be->n_slots * 2 * sizeof(float)));
    be->launches += launch_fill_f32(L.pow2, 1.f, (int64_t)be->n_slots * 2, be->load_stream);
  }
  // clear on the load stream and wait: the backend's streams are non-blocking, so a memset on the
  // default stream could land after a later flag update
  CK(cudaMalloc(&L.registered, sizeof(int32_t) * be->n_slots));
  CK(cudaMemsetAsync(L.registered, 0, sizeof(int32_t) * be->n_slots, be->load_stream));
  CK(cudaMalloc(&L.last_counts, sizeof(int32_t) * be->cfg.n_experts));
  CK(cudaMemsetAsync(L.last_counts, 0, sizeof(int32_t) * be->cfg.n_experts, be->load_stream));
  L.host_slot_of.assign(be->cfg.n_experts, -1);
  for (int e = be->e_lo; e < be->e_hi; ++e) L.host_slot_of[e] = e - be->e_lo;
  L.replica_expert.assign(be->cfg.replica_slots, -1);
  CK(cudaMalloc(&L.slot_of, sizeof(int32_t) * be->cfg.n_experts));
  CK(cudaMalloc(&L.owners, sizeof(int32_t) * be->cfg.n_experts));
  CK(cudaMemcpyAsync(L.slot_of, L.host_slot_of.data(), sizeof(int32_t) * be->cfg.n_experts, cudaMemcpyHostToDevice,
                     be->load_stream));
  CK(cudaStreamSynchronize(be->load_stream));
  L.host_registered.assign(be->n_slots, 0);
  auto ins = be->layers.emplace(layer, L);
  *out = &ins.first->second;
  return EK_OK;
}

void free_layer(Layer& L) {
  cudaFree(L.gu);
  cudaFree(L.dn);
  cudaFree(L.gu_scale);
  cudaFree(L.dn_scale);
  cudaFree(L.pow2);
  cudaFree(L.registered);
  cudaFree(L.router_w);
  if (L.router_bf16_owned) cudaFree(L.router_bf16);
  cudaFree(L.router_bias);
  cudaFree(L.last_counts);
  cudaFree(L.slot_of);
  cudaFree(L.owners);
}

int grow(ek_backend* be, void** buf, size_t* cap, size_t need) {
  if (*cap >= need) return EK_OK;
  if (*buf) cudaFree(*buf);
  *buf = nullptr;
  *cap = 0;
  CK(cudaMalloc(buf, need));
  *cap = need;
  return EK_OK;
}

// Takes a free loader lane for `id`; waits while all lanes are busy or the same id is being registered.
struct LaneGuard {
  ek_backend* be;
  LoadLane* lane = nullptr;
  std::string id;
  LaneGuard(ek_backend* b, const std::string& i) : be(b), id(i) {
    std::unique_lock<std::mutex> lk(be->lane_mu);
    for (;;) {
      if (!be->lane_ids.count(id))
        for (auto& l : be->lanes)
          if (!l.busy) { lane = &l; break; }
      if (lane) break;
      be->lane_cv.wait(lk);
    }
    lane->busy = true;
    be->lane_ids.insert(id);
  }
  ~LaneGuard() {
    {
      std::lock_guard<std::mutex> lk(be->lane_mu);
      lane->busy = false;
      be->lane_ids.erase(id);
    }
    be->lane_cv.notify_all();
  }
  int ready() {   // stream, event (created on first use)
    if (!lane->stream) CK(cudaStreamCreateWithFlags(&lane->stream, cudaStreamNonBlocking));
    if (!lane->ev) CK(cudaEventCreateWithFlags(&lane->ev, cudaEventDisableTiming));
    return EK_OK;
  }
  // a host source goes through the pinned bounce buffer at byte offset *off (advanced)
  int upload(void* dst, const void* src, size_t bytes, size_t* off) {
    memcpy(lane->bounce + *off, src, bytes);
    CK(cudaMemcpyAsync(dst, lane->bounce + *off, bytes, cudaMemcpyHostToDevice, lane->stream));
    *off += (bytes + 255) & ~(size_t)255;
    return EK_OK;
  }
};

int grow_pinned(uint8_t** buf, size_t* cap, size_t need) {
  if (*cap >= need) return EK_OK;
  if (*buf) cudaFreeHost(*buf);
  *buf = nullptr;
  *cap = 0;
  if (cudaMallocHost(reinterpret_cast<void**>(buf), need) != cudaSuccess) return EK_NO_MEMORY;
  *cap = need;
  return EK_OK;
}

const ek_tensor_view_t* find_suffix(const ek_tensor_view_t* t, int n, const char* a, const char* b) {
  // first tensor (in bundle order) whose name ends with either suffix
  // (lookup_suffix, ek-computation/src/backend/torch/mod.rs:137-153)
  for (int i = 0; i < n; ++i) {
    std::string nm = t[i].name ? t[i].name : "";
    if (ends_with(nm, a) || ends_with(nm, b)) return &t[i];
  }
  return nullptr;
}
const ek_tensor_view_t* find_exact(const ek_tensor_view_t* t, int n, const std::string& name) {
  for (int i = 0; i < n; ++i)
    if (t[i].name && name == t[i].name) return &t[i];
  return nullptr;
}

// Clears the device and host flags of an expert's slot(s) (a shared expert occupies
// n_shared_experts virtual slots from its first one).  Forwards already queued keep reading the
// slot; the flags flip behind them on the forward stream and the call waits for that.  Caller
// holds reg_mu exclusively, so no forward is being enqueued meanwhile.
void unregister_slots(ek_backend* be, Layer& L, int slot0) {
  const bool shared = slot0 == be->n_local && be->cfg.n_shared_experts > 0;
  const int n = shared ? be->cfg.n_shared_experts : 1;
  static const int32_t zeros[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int v = 0; v < n; ++v) L.host_registered[slot0 + v] = 0;
  cudaMemcpyAsync(L.registered + slot0, zeros, sizeof(int32_t) * n, cudaMemcpyHostToDevice, be->stream);
  cudaStreamSynchronize(be->stream);
}

// Slot of a routed expert on this rank: its place in the window, the replica slot that holds it,
// or (allocate) a free replica slot.  -1: this rank cannot hold it.  Caller holds reg_mu exclusively
// when allocating.
int routed_slot(ek_backend* be, Layer& L, int expert, bool allocate) {
  if (expert >= be->e_lo && expert < be->e_hi) return expert - be->e_lo;
  const int base = be->n_local + be->cfg.n_shared_experts;
  int free_slot = -1;
  for (int i = 0; i < be->cfg.replica_slots; ++i) {
    if (L.replica_expert[i] == expert) return base + i;
    if (L.replica_expert[i] < 0 && free_slot < 0) free_slot = i;
  }
  if (!allocate || free_slot < 0) return -1;
  L.replica_expert[free_slot] = expert;
  return base + free_slot;
}

// Publishes (or withdraws, slot = -1) the slot of an expert outside the window on the device.
void publish_replica(ek_backend* be, Layer& L, int expert, int slot) {
  L.host_slot_of[expert] = slot;
  cudaMemcpyAsync(L.slot_of + expert, &L.host_slot_of[expert], sizeof(int32_t), cudaMemcpyHostToDevice, be->stream);
  cudaStreamSynchronize(be->stream);
}

FfnParams ffn_params(ek_backend* be, const Layer& L) {
  FfnParams p;
  p.d = be->d;
  p.w.gu_tiles = L.gu;
  p.w.dn_tiles = L.dn;
  p.w.gu_scale = L.gu_scale;
  p.w.dn_scale = L.dn_scale;
  p.w.gu_pow = L.pow2;
  p.w.dn_pow = L.pow2 ? L.pow2 + be->n_slots : nullptr;
  p.w.registered = L.registered;
  p.w.n_slots = be->n_slots;
  p.chunks = be->chunks;
  p.n_chunks = be->n_chunks;
  p.xp = be->xp;
  p.hbuf = be->hbuf;
  p.obuf = be->obuf;
  p.rows_cap = be->rows_cap;
  p.max_chunks = be->max_chunks;
  p.status = be->status;
  p.chunk_rows = 0;
  p.x_maps = be->maps;
  p.h_maps = be->maps + 4;
  p.n_sm = be->n_sm;
  p.precise = be->precise;
  p.split_k = be->split_k;
  p.weights_ahead = 0;
  p.sk_buf = be->sk_buf;
  p.sk_flags = be->sk_flags;
  return p;
}

// Activation type the GEMMs of the next pass expect in the permuted-row buffer: f16 for the
// quantised tensor-core modes, bf16 for bf16 weights, the reference-formula mode and the CUDA-core
// checker.
bool f16_rows(const ek_backend* be) {
  return be->ffn_impl == 0 && ffn_tc_f16_activations(be->cfg.quant, be->precise);
}

int pick_nmax(int rows, int n_segments) {
  const int avg = n_segments > 0 ? (rows + n_segments - 1) / n_segments : rows;
  // measured on the DeepSeek-V3-shape layer (Zipf-skewed load): 32-row chunks win up to 24 rows per
  // expert on average, 128-row chunks from 32 on; the 64-row variant only in between
  return avg <= 24 ? 32 : avg < 32 ? 64 : 128;
}

// Event i of the current pass; the last one closes the pass.
// EK_B200_DEBUG_SYNC=1: synchronise after every stage of a layer pass and name the stage a CUDA
// error surfaced behind (diagnosis only: it removes all overlap between kernels)
bool debug_sync_failed(ek_backend* be, const char* what) {
  static const bool on = getenv("EK_B200_DEBUG_SYNC") && getenv("EK_B200_DEBUG_SYNC")[0] == '1';
  if (!on) return false;
  const cudaError_t e = cudaStreamSynchronize(be->stream);
  if (e == cudaSuccess) return false;
  fail(be, EK_CUDA, "CUDA error behind stage '%s': %s", what, cudaGetErrorString(e));
  fprintf(stderr, "[ek_b200] CUDA error behind stage '%s': %s\n", what, cudaGetErrorString(e));
  return true;
}

void mark(ek_backend* be, int i) {
  if (!be->timing) return;
  cudaEventRecord(be->ev[be->ev_pass % ek_backend::kTimingRing][i], be->stream);
  if (i == EK_STAGE_COUNT) ++be->ev_pass;
}

// Mean stage times over the passes recorded since the last read (the newest kTimingRing of them).
int finish_timing(ek_backend* be) {
  if (!be->timing || be->ev_pass == 0) return EK_OK;
  const int R = ek_backend::kTimingRing;
  const int n = std::min(be->ev_pass, R);
  CK(cudaEventSynchronize(be->ev[(be->ev_pass - 1) % R][EK_STAGE_COUNT]));
  double sum[EK_STAGE_COUNT] = {};
  for (int p = be->ev_pass - n; p < be->ev_pass; ++p)
    for (int i = 0; i < EK_STAGE_COUNT; ++i) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, be->ev[p % R][i], be->ev[p % R][i + 1]);
      sum[i] += ms;
    }
  for (int i = 0; i < EK_STAGE_COUNT; ++i) be->stage_ms[i] = (float)(sum[i] / n);
  be->ev_pass = 0;
  return EK_OK;
}

// Runs gate/up (which = 0) or down (1) over the work list already on the device.  `list_older`: the
// kernel launched just before this one is not the one that wrote the work list (always true for down:
// gate/up is in front of it).
void run_ffn(ek_backend* be, const Layer& L, int nmax, int which, bool allow_split = true, bool list_older = false) {
  FfnParams p = ffn_params(be, L);
  if (!allow_split) p.split_k = 0;
  p.weights_ahead = be->weights_ahead && (which == 1 || list_older);
  if (be->ffn_impl == 1) {
    p.chunk_rows = 16;
    be->launches += launch_ffn_simt(p, which, be->stream);
  } else {
    p.chunk_rows = nmax;
    be->launches += launch_ffn_tc(p, nmax, which, be->stream);
  }
}

int check_status(ek_backend* be) {
  CK(cudaMemcpyAsync(be->h_status, be->status, sizeof(DevStatus), cudaMemcpyDeviceToHost, be->stream));
  CK(cudaStreamSynchronize(be->stream));
  const DevStatus st = *be->h_status;
  if (st.code == DEV_OK) return EK_OK;
  cudaMemsetAsync(be->status, 0, sizeof(DevStatus), be->stream);
  // a pass that gave up may have left split-item flags raised
  cudaMemsetAsync(be->sk_flags, 0, (size_t)be->n_sm * 32 * sizeof(uint32_t), be->stream);
  cudaMemsetAsync(be->front_ticket, 0, 4 * sizeof(uint32_t), be->stream);
  cudaStreamSynchronize(be->stream);
  switch (st.code) {
    case DEV_TIMEOUT:
      return fail(be, EK_TIMEOUT, "device-side wait ran out (where=%d item=%d k=%d)", st.where, st.aux0, st.aux1);
    case DEV_MISSING_EXPERT:
      if (st.aux0 < 0)
        return fail(be, EK_EXPERT_NOT_FOUND, "shared expert %d of the layer is not registered", -1 - st.aux0);
      return fail(be, EK_EXPERT_NOT_FOUND, "expert %d selected by routing is not registered", st.aux0);
    default:
      return fail(be, EK_BOUNDS, "device-side index check failed (where=%d a0=%d a1=%d)", st.where, st.aux0, st.aux1);
  }
}

// Stage timers, routing, bucketing, gather, FFN, combine on device buffers.  `x` is a device
// pointer to [T,H]; result in `y` (device [T,H]) or, for the controller-level call
// (given_ids != nullptr), in `out_tk` (device [T,k,H]).
// Expert-parallel variant of the fused call: the shared expert runs on the token slice
// [sh_t0, sh_t0 + sh_T) only and the routed (local) contributions are left as fp32 partial sums.
struct LayerOpts {
  int sh_t0 = 0;
  int sh_T = -1;            // -1: all T tokens
  float* partial = nullptr; // [T,H] fp32 instead of y
  PeerWait wait;            // expert parallel: x is complete once every rank's flag has reached a step number
  const PeerSignal* signal = nullptr;   // expert parallel: publish the step number once `partial` is complete
};

int run_layer(ek_backend* be, Layer& L, const __nv_bfloat16* x, int T, int k, const int32_t* given_ids_dev,
              __nv_bfloat16* y, __nv_bfloat16* out_tk, const LayerOpts& opt = LayerOpts()) {
  const ek_config_t& c = be->cfg;
  const int Tk = T * k;
  const bool fused = given_ids_dev == nullptr;
  const int n_shared = fused ? c.n_shared_experts : 0;
  const int sh_T = n_shared > 0 ? (opt.sh_T < 0 ? T : opt.sh_T) : 0;
  cudaStream_t s = be->stream;
  mark(be, 0);
  const int32_t* ids = given_ids_dev;
  RouteParams rp;
  rp.x = x;
  rp.wg = L.router_w;
  rp.wg_f32 = L.router_f32;
  rp.bias = L.router_bias;
  rp.logits = be->logits;
  rp.ids = be->ids;
  rp.weights = be->weights;
  rp.counts = be->counts;
  rp.T = T; rp.H = c.hidden; rp.E = c.n_experts; rp.k = k;
  rp.scoring = c.scoring; rp.n_group = c.n_group; rp.topk_group = c.topk_group;
  rp.norm = c.norm_topk_prob; rp.scaling = c.routed_scaling;
  rp.bf16_weights = c.bf16_combine;
  rp.partial = nullptr;
  rp.n_partials = 0;
  PermuteParams pp;
  pp.ids = fused ? be->ids : given_ids_dev; pp.counts = be->counts; pp.offsets = be->offsets; pp.perm = be->perm; pp.inv = be->inv;
  pp.T = T; pp.k = k; pp.E = c.n_experts; pp.e_lo = be->e_lo; pp.e_hi = be->e_hi;
  pp.owners = L.has_owners ? L.owners : nullptr; pp.rank = c.ep_rank;
  // expected rows per local expert: Tk / n_experts whatever the sharding
  const int nmax = pick_nmax((int)((int64_t)Tk * be->n_local / c.n_experts), be->n_local);
  WorklistParams wp;
  wp.counts = be->counts; wp.offsets = be->offsets; wp.registered = L.registered;
  wp.chunks = be->chunks; wp.n_chunks = be->n_chunks;
  wp.E = c.n_experts; wp.e_lo = be->e_lo; wp.e_hi = be->e_hi;
  wp.owners = pp.owners; wp.slot_of = L.slot_of; wp.rank = c.ep_rank;
  wp.chunk_rows = be->ffn_impl == 1 ? 16 : nmax;
  wp.n_shared = sh_T > 0 ? n_shared : 0; wp.T = sh_T; wp.Tk = Tk;
  wp.max_chunks = be->max_chunks;
  wp.status = be->status;
  wp.counts_copy = L.last_counts;   // the layer's activation metric, read back by ek_expert_counts
  // small batches: everything in front of the GEMMs in one launch
  const bool front = fused && be->front_small && L.router_bf16 && front_small_supported(T, c.n_experts, k, c.hidden);
  bool gathered = false;
  // a pending wait for the peers' tokens: taken along by the tensor-core router, else a launch of its own
  bool wait_pending = opt.wait.flags != nullptr;
  auto wait_now = [&]() {
    if (wait_pending) be->launches += launch_ep_wait(opt.wait.flags, opt.wait.world, opt.wait.step_no, be->status, opt.wait.where, s);
    wait_pending = false;
  };
  if (front) {
    wait_now();
    FrontParams fp;
    fp.route = rp;
    fp.route.wg = L.router_bf16;
    fp.route.wg_f32 = 0;
    fp.route.partial = nullptr;
    fp.route.n_partials = 0;
    fp.slice = front_small_slice(c.hidden);
    fp.permute = pp;
    fp.worklist = wp;
    fp.partial = be->partial;
    fp.ticket = be->front_ticket;
    fp.xp = be->xp;
    fp.gather_rows = Tk + sh_T <= 24 ? 1 : 0;
    // a batch of one token: all its rows are the same, one copy serves every expert
    fp.worklist.same_row = (T == 1 && fp.gather_rows && (sh_T == 0 || opt.sh_t0 == 0)) ? 1 : 0;
    fp.shared_t0 = opt.sh_t0; fp.shared_T = sh_T;
    fp.to_f16 = f16_rows(be) ? 1 : 0;
    be->launches += launch_front_small(fp, s);
    if (debug_sync_failed(be, "front (router + bucketing)")) return EK_CUDA;
    gathered = fp.gather_rows != 0;
    ids = be->ids;
    mark(be, 1);
  } else {
    if (fused) {
      bool tc_done = false;
      if (L.router_tc) {
        RouterTcParams tp;
        if (encode_2d(be, &tp.x_map, x, (uint64_t)c.hidden, (uint64_t)T, 128)) {
          tp.w_map = L.router_map;
          tp.partial = be->partial;
          tp.zero_counts = be->counts;
          tp.status = be->status;
          tp.T = T; tp.H = c.hidden; tp.E = c.n_experts;
          tp.n_atoms = (c.hidden + 63) / 64;
          router_tc_plan(T, c.hidden, be->n_sm, &tp.n_splits, &tp.atoms_per_split);
          tp.tmem_cols = 32;
          while (tp.tmem_cols < c.n_experts) tp.tmem_cols *= 2;
          if (wait_pending) tp.wait = opt.wait;
          wait_pending = false;
          be->launches += launch_router_tc(tp, s);
          rp.partial = be->partial;
          rp.n_partials = tp.n_splits;
          tc_done = true;
        }
      }
      wait_now();
      if (!tc_done) be->launches += launch_router_logits(rp, s);
      if (debug_sync_failed(be, "router logits")) return EK_CUDA;
      be->launches += launch_route_select(rp, s, tc_done);
      if (debug_sync_failed(be, "route select")) return EK_CUDA;
      ids = be->ids;
    } else {
      wait_now();
      // caller-supplied ids may be invalid: rows that no expert claims must read as "absent"
      cudaMemsetAsync(be->inv, 0xFF, sizeof(int32_t) * Tk, s);
      be->launches += launch_histogram(ids, Tk, c.n_experts, be->counts, be->status, s);
    }
    mark(be, 1);
    be->launches += launch_permute_worklist(pp, wp, be->front_ticket + 2, s);
    if (debug_sync_failed(be, "permute + work list")) return EK_CUDA;
  }
  if (!gathered) {
    be->launches += launch_gather(x, be->perm, be->offsets + c.n_experts, be->xp, T, k, c.hidden, opt.sh_t0, sh_T,
                                  f16_rows(be), s);
    if (debug_sync_failed(be, "gather")) return EK_CUDA;
  }
  L.have_counts = true;
  mark(be, 2);
  run_ffn(be, L, nmax, 0, true, /*list_older=*/!gathered);   // a gather launch of its own sits between the work list and gate/up
  if (debug_sync_failed(be, "gate/up GEMM")) return EK_CUDA;
  mark(be, 3);
  run_ffn(be, L, nmax, 1);
  if (debug_sync_failed(be, "down GEMM")) return EK_CUDA;
  mark(be, 4);
  if (fused && opt.partial) {
    CombineParams cp;
    cp.obuf = be->obuf; cp.inv = be->inv; cp.weights = be->weights; cp.y = nullptr;
    cp.T = T; cp.k = k; cp.H = c.hidden; cp.n_shared = 0; cp.Tk = Tk;
    cp.bf16_products = c.bf16_combine;
    cp.shared = nullptr;
    be->launches += launch_combine_partial(cp, opt.partial, opt.signal, s);
  } else if (fused) {
    CombineParams cp;
    cp.obuf = be->obuf; cp.inv = be->inv; cp.weights = be->weights; cp.y = y;
    cp.T = T; cp.k = k; cp.H = c.hidden; cp.n_shared = n_shared; cp.Tk = Tk;
    cp.bf16_products = c.bf16_combine;
    cp.shared = nullptr;
    be->launches += launch_combine(cp, s);
  } else {
    be->launches += launch_unpermute(be->obuf, be->inv, out_tk, T, k, c.hidden, s);
  }
  mark(be, 5);
  if (debug_sync_failed(be, "combine")) return EK_CUDA;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(be, EK_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
  return EK_OK;
}

}  // namespace

// =============================================================================================
// C ABI
// =============================================================================================
extern "C" {

const char* ek_status_name(int32_t s) {
  switch (s) {
    case EK_OK: return "EK_OK";
    case EK_EXPERT_NOT_FOUND: return "EK_EXPERT_NOT_FOUND";
    case EK_EXPERT_WEIGHT_NOT_FOUND: return "EK_EXPERT_WEIGHT_NOT_FOUND";
    case EK_INVALID_INPUT: return "EK_INVALID_INPUT";
    case EK_SAFETENSOR: return "EK_SAFETENSOR";
    case EK_NOT_FOUND: return "EK_NOT_FOUND";
    case EK_CUDA: return "EK_CUDA";
    case EK_TIMEOUT: return "EK_TIMEOUT";
    case EK_BOUNDS: return "EK_BOUNDS";
    case EK_NO_MEMORY: return "EK_NO_MEMORY";
    case EK_UNSUPPORTED: return "EK_UNSUPPORTED";
  }
  return "EK_UNKNOWN";
}

const char* ek_last_error(const ek_backend_t* be) {
  if (!be) return "";
  std::lock_guard<std::mutex> g(be->err_mu);
  static thread_local std::string copy;
  copy = be->err;
  return copy.c_str();
}

static std::string g_create_error;
const char* ek_create_error(void) { return g_create_error.c_str(); }

int32_t ek_backend_create(const ek_config_t* cfg, ek_backend_t** out) {
  if (!cfg || !out) return EK_INVALID_INPUT;
  *out = nullptr;
  const ek_config_t& c = *cfg;
  auto bad = [&](const char* m) {
    g_create_error = m;
    return (int32_t)EK_INVALID_INPUT;
  };
  if (c.hidden < 8 || c.hidden % 8) return bad("hidden must be a positive multiple of 8");
  if (c.intermediate < 8 || c.intermediate % 8) return bad("intermediate must be a positive multiple of 8");
  if (c.n_experts < 1 || c.n_experts > 1024) return bad("n_experts must be in [1,1024]");
  if (c.top_k < 1 || c.top_k > 32 || c.top_k > c.n_experts) return bad("top_k must be in [1,min(32,n_experts)]");
  if (c.n_group < 1 || c.n_group > 64 || c.n_experts % c.n_group) return bad("n_group must divide n_experts and be <= 64");
  if (c.topk_group < 1 || c.topk_group > c.n_group) return bad("topk_group must be in [1,n_group]");
  if (c.quant < 0 || c.quant > 2) return bad("unknown quant");
  if (c.max_tokens < 1) return bad("max_tokens must be positive");
  if (c.ep_size < 1 || c.ep_rank < 0 || c.ep_rank >= c.ep_size || c.n_experts % c.ep_size)
    return bad("ep_size must divide n_experts and ep_rank be in [0,ep_size)");
  if (c.n_shared_experts < 0 || c.n_shared_experts > 8) return bad("n_shared_experts must be in [0,8]");
  if (c.max_layers < 1) return bad("max_layers must be positive");
  if (c.replica_slots < 0 || c.replica_slots > c.n_experts) return bad("replica_slots must be in [0,n_experts]");
  // a quantised shared expert is cut into virtual experts at multiples of `intermediate`; the
  // 128x128 scale blocks only line up with those cuts when intermediate is a multiple of 128
  if (c.quant != EK_QUANT_BF16 && c.n_shared_experts > 1 && c.intermediate % 128) {
    g_create_error = "quantised weights with n_shared_experts > 1 need intermediate to be a multiple of 128";
    return EK_UNSUPPORTED;
  }

  ek_backend* be = new ek_backend();
  be->cfg = c;
  be->cfg.model_name[sizeof(be->cfg.model_name) - 1] = 0;
  auto cleanup_fail = [&](int code) {
    g_create_error = be->err;
    ek_backend_destroy(be);
    return (int32_t)code;
  };
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    g_create_error = "no CUDA device: this backend has no CPU path";
    delete be;
    return EK_CUDA;
  }
  if (cudaSetDevice(c.device) != cudaSuccess) {
    g_create_error = "cudaSetDevice failed";
    delete be;
    return EK_CUDA;
  }
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, c.device);
  if (prop.major != 10) {
    g_create_error = "this library is built for sm_100a (B200) only";
    delete be;
    return EK_UNSUPPORTED;
  }
  be->n_sm = prop.multiProcessorCount;
  Dims& d = be->d;
  d.H = c.hidden; d.I = c.intermediate;
  d.Hp = round_up(c.hidden, 128); d.Ip = round_up(c.intermediate, 128);
  d.quant = c.quant;
  const int tk = tile_k_elems(c.quant);
  d.kt_gu = d.Hp / tk; d.kt_dn = d.Ip / tk; d.it = d.Ip / 128; d.ht = d.Hp / 128; d.hp = (d.ht + 1) / 2;
  be->n_local = c.n_experts / c.ep_size;
  be->e_lo = c.ep_rank * be->n_local;
  be->e_hi = be->e_lo + be->n_local;
  be->n_slots = be->n_local + c.n_shared_experts + c.replica_slots;
  be->rows_cap = round_up(c.max_tokens * (c.top_k + c.n_shared_experts), 128) + 128;
  be->max_chunks = be->rows_cap / 16 + be->n_slots + c.n_shared_experts * (c.max_tokens / 16 + 1) + 8;

#define CKC(call)                                                                                  \
  do {                                                                                             \
    cudaError_t e__ = (call);                                                                      \
    if (e__ != cudaSuccess) {                                                                      \
      fail(be, EK_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__));                          \
      return cleanup_fail(e__ == cudaErrorMemoryAllocation ? EK_NO_MEMORY : EK_CUDA);              \
    }                                                                                              \
  } while (0)
  CKC(cudaStreamCreateWithFlags(&be->own_stream, cudaStreamNonBlocking));
  be->stream = be->own_stream;
  CKC(cudaStreamCreateWithFlags(&be->load_stream, cudaStreamNonBlocking));
  CKC(cudaEventCreateWithFlags(&be->fwd_done, cudaEventDisableTiming));
  CKC(cudaEventCreateWithFlags(&be->ep_upload_done, cudaEventDisableTiming));
  CKC(cudaMallocHost(&be->h_ep_count, 64));
  for (auto& pass : be->ev)
    for (auto& e : pass) CKC(cudaEventCreate(&e));
  const size_t T = c.max_tokens, H = c.hidden, E = c.n_experts, K = c.top_k;
  CKC(cudaMalloc(&be->x_dev, T * H * 2));
  CKC(cudaMalloc(&be->y_dev, T * H * 2));
  CKC(cudaMalloc(&be->xp, (size_t)be->rows_cap * H * 2));
  CKC(cudaMalloc(&be->hbuf, (size_t)be->rows_cap * d.Ip * 2));
  CKC(cudaMalloc(&be->obuf, (size_t)be->rows_cap * H * 2));
  CKC(cudaMemset(be->xp, 0, (size_t)be->rows_cap * H * 2));
  CKC(cudaMemset(be->hbuf, 0, (size_t)be->rows_cap * d.Ip * 2));
  CKC(cudaMalloc(&be->logits, T * E * 4));
  CKC(cudaMalloc(&be->weights, T * K * 4));
  CKC(cudaMalloc(&be->bias_scratch, E * 4));
  CKC(cudaMalloc(&be->partial, (size_t)be->n_sm * 128 * E * 4));
  CKC(cudaMalloc(&be->flag_dev, 4));
  CKC(cudaMalloc(&be->ids, T * K * 4));
  CKC(cudaMalloc(&be->counts, E * 4));
  CKC(cudaMalloc(&be->offsets, (E + 1) * 4));
  CKC(cudaMalloc(&be->perm, T * K * 4));
  CKC(cudaMalloc(&be->inv, T * K * 4));
  CKC(cudaMalloc(&be->chunks, sizeof(ChunkDesc) * be->max_chunks));
  CKC(cudaMalloc(&be->n_chunks, 4));
  CKC(cudaMalloc(&be->status, sizeof(DevStatus)));
  CKC(cudaMemset(be->status, 0, sizeof(DevStatus)));
  CKC(cudaMalloc(&be->ep_counters, EK_EP_MAX_RANKS * sizeof(uint32_t)));
  CKC(cudaMemset(be->ep_counters, 0, EK_EP_MAX_RANKS * sizeof(uint32_t)));
  CKC(cudaMalloc(&be->front_ticket, 4 * sizeof(uint32_t)));
  CKC(cudaMemset(be->front_ticket, 0, 4 * sizeof(uint32_t)));
  CKC(cudaMalloc(&be->sk_buf, ffn_tc_scratch_floats(be->n_sm) * sizeof(float)));
  CKC(cudaMalloc(&be->sk_flags, (size_t)be->n_sm * 32 * sizeof(uint32_t)));
  CKC(cudaMemset(be->sk_flags, 0, (size_t)be->n_sm * 32 * sizeof(uint32_t)));
  CKC(cudaMallocHost(&be->h_status, sizeof(DevStatus)));
  be->h_chunks_cap = std::max(1024, be->max_chunks);
  CKC(cudaMallocHost(&be->h_chunks, sizeof(ChunkDesc) * be->h_chunks_cap));
  be->segs_cap = c.ep_size * be->n_local;
  // forward (arrival -> expert order) and reverse lists side by side
  CKC(cudaMalloc(&be->segs, sizeof(RowSegment) * be->segs_cap * 2));
  CKC(cudaMallocHost(&be->h_segs, sizeof(RowSegment) * be->segs_cap * 2));
  CKC(cudaMalloc(&be->maps, sizeof(CUtensorMap) * 8));
  be->h_cap = T * H * 2;
  CKC(cudaMallocHost(&be->h_x, be->h_cap));
  CKC(cudaMallocHost(&be->h_y, be->h_cap));
#undef CKC
  int rc = make_maps(be);
  if (rc != EK_OK) return cleanup_fail(rc);
  // the memsets above ran on the default stream; the backend's own streams do not wait for it
  if (cudaDeviceSynchronize() != cudaSuccess) {
    fail(be, EK_CUDA, "device synchronisation failed after workspace set-up");
    return cleanup_fail(EK_CUDA);
  }
  // measurement switches (they take single kernels out of the pass to time what each is worth; the
  // results are the same either way): EK_B200_FRONT_SMALL=0, EK_B200_SPLIT_K=0, EK_B200_WEIGHTS_AHEAD=0
  const char* fs = getenv("EK_B200_FRONT_SMALL");
  if (fs && fs[0] == '0') be->front_small = 0;
  const char* sk = getenv("EK_B200_SPLIT_K");
  if (sk && sk[0] == '0') be->split_k = 0;
  const char* wa = getenv("EK_B200_WEIGHTS_AHEAD");
  if (wa && wa[0] == '0') be->weights_ahead = 0;
  *out = be;
  return EK_OK;
}

void ek_backend_destroy(ek_backend_t* be) {
  if (!be) return;
  cudaSetDevice(be->cfg.device);
  if (be->own_stream) cudaStreamSynchronize(be->own_stream);
  if (be->load_stream) cudaStreamSynchronize(be->load_stream);
  for (int r = 0; r < EK_EP_MAX_RANKS; ++r)
    if (be->peers.opened[r]) {
      cudaIpcCloseMemHandle(be->peers.xall[r]);
      cudaIpcCloseMemHandle(be->peers.partial[r]);
      cudaIpcCloseMemHandle(be->peers.flags[r]);
    }
  for (int i = 0; i < 3; ++i) cudaFree(be->peers.own[i]);
  for (auto& kv : be->layers) free_layer(kv.second);
  cudaFree(be->x_dev); cudaFree(be->y_dev); cudaFree(be->xp); cudaFree(be->hbuf); cudaFree(be->obuf);
  cudaFree(be->tk_dev);
  cudaFree(be->logits); cudaFree(be->weights); cudaFree(be->bias_scratch); cudaFree(be->partial); cudaFree(be->flag_dev); cudaFree(be->ids); cudaFree(be->counts);
  cudaFree(be->offsets); cudaFree(be->perm); cudaFree(be->inv); cudaFree(be->chunks);
  cudaFree(be->n_chunks); cudaFree(be->status); cudaFree(be->sk_buf); cudaFree(be->sk_flags); cudaFree(be->front_ticket); cudaFree(be->ep_counters); cudaFree(be->maps);
  cudaFreeHost(be->h_status); cudaFreeHost(be->h_chunks); cudaFreeHost(be->h_segs); cudaFree(be->segs); cudaFreeHost(be->h_x); cudaFreeHost(be->h_y);
  cudaFreeHost(be->h_tk);
  for (int i = 0; i < 3; ++i) { cudaFree(be->stage[i]); cudaFree(be->stage_scale[i]); }
  for (auto& l : be->lanes) {
    if (l.stream) { cudaStreamSynchronize(l.stream); cudaStreamDestroy(l.stream); }
    if (l.ev) cudaEventDestroy(l.ev);
    for (int i = 0; i < 3; ++i) { cudaFree(l.stage[i]); cudaFree(l.stage_scale[i]); }
    cudaFree(l.stage_cvt);
    if (l.bounce) cudaFreeHost(l.bounce);
  }
  cudaFree(be->stage_cvt);
  for (auto& pass : be->ev)
    for (auto& e : pass) if (e) cudaEventDestroy(e);
  if (be->fwd_done) cudaEventDestroy(be->fwd_done);
  if (be->ep_upload_done) cudaEventDestroy(be->ep_upload_done);
  cudaFreeHost(be->h_ep_count);
  if (be->own_stream) cudaStreamDestroy(be->own_stream);
  if (be->load_stream) cudaStreamDestroy(be->load_stream);
  delete be;
}

// ---- registry --------------------------------------------------------------------------------

int32_t ek_expert_mark_loading(ek_backend_t* be, const char* id, int32_t* fresh) {
  if (!be || !id) return EK_INVALID_INPUT;
  std::unique_lock<std::shared_mutex> g(be->reg_mu);
  bool was = be->loading.count(id) > 0;
  be->loading.insert(id);
  if (fresh) *fresh = was ? 0 : 1;
  return EK_OK;
}

int32_t ek_expert_has(const ek_backend_t* be, const char* id) {
  if (!be || !id) return 0;
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  return (be->loading.count(id) || be->experts.count(id)) ? 1 : 0;
}
int32_t ek_expert_loaded(const ek_backend_t* be) {
  if (!be) return 0;
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  return (int32_t)be->experts.size();
}
int32_t ek_expert_loading(const ek_backend_t* be) {
  if (!be) return 0;
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  return (int32_t)be->loading.size();
}
int32_t ek_expert_keys(const ek_backend_t* be, char* buf, size_t cap, size_t* needed) {
  if (!be) return EK_INVALID_INPUT;
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  std::string all;
  for (auto& kv : be->experts) {
    if (!all.empty()) all.push_back('\n');
    all += kv.first;
  }
  if (needed) *needed = all.size() + 1;
  if (!buf || cap < all.size() + 1) return EK_INVALID_INPUT;
  memcpy(buf, all.c_str(), all.size() + 1);
  return EK_OK;
}

int32_t ek_expert_evict(ek_backend_t* be, const char* id) {
  if (!be || !id) return EK_INVALID_INPUT;
  cudaSetDevice(be->cfg.device);
  std::unique_lock<std::shared_mutex> g(be->reg_mu);
  auto it = be->experts.find(id);
  if (it == be->experts.end()) return EK_OK;   // ExpertDB::remove ignores unknown ids
  Layer& L = be->layers[it->second.layer];
  unregister_slots(be, L, it->second.slot);
  const int ri = it->second.slot - be->n_local - be->cfg.n_shared_experts;
  if (ri >= 0) {   // a replica slot: withdraw it
    publish_replica(be, L, L.replica_expert[ri], -1);
    L.replica_expert[ri] = -1;
  }
  be->experts.erase(it);
  return EK_OK;
}

int32_t ek_expert_register(ek_backend_t* be, const char* id, const ek_tensor_view_t* t, int32_t n) {
  if (!be || !id || (!t && n > 0)) return EK_INVALID_INPUT;
  cudaSetDevice(be->cfg.device);
  const ek_config_t& c = be->cfg;
  const Dims& d = be->d;
  std::string model;
  int layer = 0, expert = 0;
  bool shared = false;
  if (!parse_id(id, model, layer, expert, shared)) return fail(be, EK_INVALID_INPUT, "invalid expert id: %s", id);
  if (c.model_name[0] && model != c.model_name)
    return fail(be, EK_INVALID_INPUT, "expert id %s does not belong to model %s", id, c.model_name);
  if (shared && c.n_shared_experts == 0) return fail(be, EK_INVALID_INPUT, "layer has no shared expert: %s", id);
  if (!shared && (expert < 0 || expert >= c.n_experts))
    return fail(be, EK_INVALID_INPUT, "expert %d outside [0,%d)", expert, c.n_experts);
  if (!shared && (expert < be->e_lo || expert >= be->e_hi) && c.replica_slots == 0)
    return fail(be, EK_INVALID_INPUT, "expert %d is not in this rank's range [%d,%d) and the backend has no replica slots",
                expert, be->e_lo, be->e_hi);

  // ExpertWeight::from_safetensor (ek-computation/src/ffn/meta.rs:57-75)
  const ek_tensor_view_t* up = find_suffix(t, n, "w1.weight", "up_proj.weight");
  if (!up) return fail(be, EK_EXPERT_WEIGHT_NOT_FOUND, "w1/up_w");
  const ek_tensor_view_t* down = find_suffix(t, n, "w2.weight", "down_proj.weight");
  if (!down) return fail(be, EK_EXPERT_WEIGHT_NOT_FOUND, "w2/down_w");
  const ek_tensor_view_t* gate = find_suffix(t, n, "w3.weight", "gate_proj.weight");
  if (!gate) return fail(be, EK_EXPERT_WEIGHT_NOT_FOUND, "w3/gate_w");
  const ek_tensor_view_t* w[3] = {gate, up, down};
  const int I_e = shared ? c.intermediate * c.n_shared_experts : c.intermediate;
  const int64_t want[3][2] = {{I_e, c.hidden}, {I_e, c.hidden}, {c.hidden, I_e}};
  const ek_tensor_view_t* sc[3] = {nullptr, nullptr, nullptr};
  for (int i = 0; i < 3; ++i) {
    if (w[i]->ndim != 2 || w[i]->shape[0] != want[i][0] || w[i]->shape[1] != want[i][1])
      return fail(be, EK_INVALID_INPUT, "%s has shape [%lld,%lld], expected [%lld,%lld]", w[i]->name,
                  (long long)w[i]->shape[0], (long long)(w[i]->ndim > 1 ? w[i]->shape[1] : 0),
                  (long long)want[i][0], (long long)want[i][1]);
    if (!w[i]->data) return fail(be, EK_INVALID_INPUT, "%s has no data", w[i]->name);
    if (c.quant == EK_QUANT_BF16) {
      if (w[i]->dtype != EK_BF16 && w[i]->dtype != EK_F16)
        return fail(be, EK_INVALID_INPUT, "%s: dtype %d not accepted by a bf16 backend", w[i]->name, w[i]->dtype);
    } else {
      const int wantdt = c.quant == EK_QUANT_FP8_BLOCK128 ? EK_F8_E4M3 : EK_I8;
      if (w[i]->dtype != wantdt)
        return fail(be, EK_INVALID_INPUT, "%s: dtype %d does not match the backend's quantisation", w[i]->name, w[i]->dtype);
      sc[i] = find_exact(t, n, std::string(w[i]->name) + "_scale_inv");
      if (!sc[i]) sc[i] = find_exact(t, n, std::string(w[i]->name) + "_scale");
      if (!sc[i]) return fail(be, EK_EXPERT_WEIGHT_NOT_FOUND, "%s_scale_inv", w[i]->name);
      const int64_t sr = (want[i][0] + 127) / 128, scn = (want[i][1] + 127) / 128;
      if (sc[i]->dtype != EK_F32 || sc[i]->ndim != 2 || sc[i]->shape[0] != sr || sc[i]->shape[1] != scn)
        return fail(be, EK_INVALID_INPUT, "%s must be F32 [%lld,%lld]", sc[i]->name, (long long)sr, (long long)scn);
      if (!sc[i]->data) return fail(be, EK_INVALID_INPUT, "%s has no data", sc[i]->name);
    }
  }

  LaneGuard lg(be, id);
  LoadLane* const lane = lg.lane;
  if (int rc = lg.ready()) return rc;
  Layer* L = nullptr;
  int slot_routed = -1;
  {
    std::unique_lock<std::shared_mutex> g(be->reg_mu);
    int rc = ensure_layer(be, layer, &L);
    if (rc != EK_OK) return rc;
    // replacing a live expert: take it out first, so that a forward enqueued while the new tiles
    // are being written reports EK_EXPERT_NOT_FOUND instead of reading half old, half new weights
    // (the reference swaps the Arc in one step, worker/manager.rs insert)
    auto live = be->experts.find(id);
    if (live != be->experts.end()) {
      unregister_slots(be, *L, live->second.slot);
      be->experts.erase(live);
    }
    if (!shared) {
      slot_routed = routed_slot(be, *L, expert, true);
      if (slot_routed < 0)
        return fail(be, EK_NO_MEMORY, "all %d replica slots of layer %d are taken", c.replica_slots, layer);
    }
  }
  cudaStream_t ls = lane->stream;
  // the slot may still be read by forwards queued before an eviction
  CK(cudaEventRecord(lane->ev, be->stream));
  CK(cudaStreamWaitEvent(ls, lane->ev, 0));

  const int esz = elem_bytes(c.quant);
  // host sources: the calling thread copies them into the lane's pinned buffer (threads do that side
  // by side), the DMA and the re-tiling kernels follow on the lane's stream
  size_t host_bytes = 0, host_off = 0;
  for (int i = 0; i < 3; ++i) {
    if (!is_device_ptr(w[i]->data))
      host_bytes += (((size_t)want[i][0] * want[i][1] * (w[i]->dtype == EK_F16 ? 2 : esz)) + 255) & ~(size_t)255;
    if (c.quant != EK_QUANT_BF16 && !is_device_ptr(sc[i]->data))
      host_bytes += (((size_t)sc[i]->shape[0] * sc[i]->shape[1] * 4) + 255) & ~(size_t)255;
  }
  if (host_bytes && grow_pinned(&lane->bounce, &lane->bounce_cap, host_bytes) != EK_OK)
    return fail(be, EK_NO_MEMORY, "no pinned host memory for the loader (%zu bytes)", host_bytes);
  const void* src[3];
  for (int i = 0; i < 3; ++i) {
    const size_t elems = (size_t)want[i][0] * want[i][1];
    const size_t in_bytes = elems * (w[i]->dtype == EK_F16 ? 2 : esz);
    const void* p = w[i]->data;
    if (!is_device_ptr(p)) {
      int rc = grow(be, &lane->stage[i], &lane->stage_cap[i], in_bytes);
      if (rc != EK_OK) return rc;
      rc = lg.upload(lane->stage[i], p, in_bytes, &host_off);
      if (rc != EK_OK) return rc;
      p = lane->stage[i];
    }
    if (w[i]->dtype == EK_F16) {
      int rc = grow(be, &lane->stage_cvt, &lane->stage_cvt_cap, elems * 2 * 3);
      if (rc != EK_OK) return rc;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(lane->stage_cvt) + (size_t)i * elems;
      be->launches += launch_f16_to_bf16(p, dst, (int64_t)elems, ls);
      p = dst;
    }
    src[i] = p;
  }
  const float* ssrc[3] = {nullptr, nullptr, nullptr};
  if (c.quant != EK_QUANT_BF16) {
    for (int i = 0; i < 3; ++i) {
      const size_t bytes = (size_t)sc[i]->shape[0] * sc[i]->shape[1] * 4;
      const void* p = sc[i]->data;
      if (!is_device_ptr(p)) {
        int rc = grow(be, (void**)&lane->stage_scale[i], &lane->stage_scale_cap[i], bytes);
        if (rc != EK_OK) return rc;
        rc = lg.upload(lane->stage_scale[i], p, bytes, &host_off);
        if (rc != EK_OK) return rc;
        p = lane->stage_scale[i];
      }
      ssrc[i] = reinterpret_cast<const float*>(p);
    }
  }

  const int n_virtual = shared ? c.n_shared_experts : 1;
  for (int v = 0; v < n_virtual; ++v) {
    const int slot = shared ? be->n_local + v : slot_routed;
    uint8_t* gu0 = L->gu + (size_t)slot * d.it * d.kt_gu * 2 * kTileBytes;
    uint8_t* dn0 = L->dn + (size_t)slot * d.hp * d.kt_dn * 2 * kTileBytes;
    for (int m = 0; m < 2; ++m) {   // 0 gate, 1 up
      RetileParams rp;
      rp.src = src[m]; rp.rows = I_e; rp.cols = c.hidden;
      rp.row0 = v * c.intermediate; rp.n_rows = c.intermediate;
      rp.col0 = 0; rp.n_cols = c.hidden;
      rp.esz = esz;
      rp.xor_mask = c.quant == EK_QUANT_INT8_BLOCK128 ? 0x80808080u : 0u;
      rp.dst = gu0 + (size_t)m * kTileBytes;
      rp.rt_stride = (int64_t)d.kt_gu * 2 * kTileBytes;
      rp.kt_stride = 2 * kTileBytes;
      rp.rt_pairs = 0;
      rp.n_rt = d.it; rp.n_kt = d.kt_gu;
      be->launches += launch_retile(rp, ls);
      if (c.quant != EK_QUANT_BF16) {
        ScaleRetileParams sp;
        sp.src = ssrc[m]; sp.src_cols = (int)sc[m]->shape[1]; sp.src_rows = (int)sc[m]->shape[0];
        sp.rb0 = v * c.intermediate / 128; sp.kb0 = 0;
        sp.n_rt = d.it; sp.n_kt = d.kt_gu;
        sp.dst = L->gu_scale + (size_t)slot * d.it * d.kt_gu * 2;
        sp.stride = 2; sp.lane = m; sp.rt_pairs = 0;
        be->launches += launch_scale_retile(sp, ls);
      }
    }
    RetileParams rp;
    rp.src = src[2]; rp.rows = c.hidden; rp.cols = I_e;
    rp.row0 = 0; rp.n_rows = c.hidden;
    rp.col0 = v * c.intermediate; rp.n_cols = c.intermediate;
    rp.esz = esz;
    rp.xor_mask = c.quant == EK_QUANT_INT8_BLOCK128 ? 0x80808080u : 0u;
    rp.dst = dn0;
    rp.rt_stride = 0; rp.kt_stride = 0;
    rp.rt_pairs = 1;                       // row tiles 2j, 2j+1 adjacent per K tile; an odd tail is zero-filled
    rp.n_rt = 2 * d.hp; rp.n_kt = d.kt_dn;
    be->launches += launch_retile(rp, ls);
    if (c.quant != EK_QUANT_BF16) {
      ScaleRetileParams sp;
      sp.src = ssrc[2]; sp.src_cols = (int)sc[2]->shape[1]; sp.src_rows = (int)sc[2]->shape[0];
      sp.rb0 = 0; sp.kb0 = v * c.intermediate / 128;
      sp.n_rt = 2 * d.hp; sp.n_kt = d.kt_dn;
      sp.dst = L->dn_scale + (size_t)slot * d.hp * d.kt_dn * 2;
      sp.stride = 1; sp.lane = 0; sp.rt_pairs = 1;
      be->launches += launch_scale_retile(sp, ls);
    }
    if (c.quant != EK_QUANT_BF16) {
      // one power of two per expert and GEMM, from the largest block scale of its matrices
      be->launches += launch_scale_pow(ssrc[0], (int64_t)sc[0]->shape[0] * sc[0]->shape[1], ssrc[1],
                                       (int64_t)sc[1]->shape[0] * sc[1]->shape[1], L->pow2 + slot, ls);
      be->launches += launch_scale_pow(ssrc[2], (int64_t)sc[2]->shape[0] * sc[2]->shape[1], nullptr, 0,
                                       L->pow2 + be->n_slots + slot, ls);
    }
    const int32_t one = 1;
    CK(cudaMemcpyAsync(L->registered + slot, &one, sizeof one, cudaMemcpyHostToDevice, ls));
  }
  CK(cudaStreamSynchronize(ls));
  CK(cudaGetLastError());
  {
    std::unique_lock<std::shared_mutex> g(be->reg_mu);
    for (int v = 0; v < n_virtual; ++v) L->host_registered[shared ? be->n_local + v : slot_routed] = 1;
    be->loading.erase(id);
    ExpertRef ref{layer, shared ? be->n_local : slot_routed};
    be->experts[id] = ref;
    if (!shared && (expert < be->e_lo || expert >= be->e_hi)) publish_replica(be, *L, expert, slot_routed);
  }
  return EK_OK;
}

// ---- device-ready form of an expert: export and direct registration -------------------------
// The weight server keeps fetched bundles in a file cache so a restarted worker does not hit the
// store again (ek-db/src/safetensor/mod.rs:144-171).  The same idea one step later: the tiles and
// scales exactly as this library keeps them in HBM, so that a restart (or a second GPU that owns
// the same expert) skips decoding, re-tiling and the fp8 byte re-encoding.
namespace {

struct TileBlobHeader {
  char magic[8];            // "EKTILES\0"
  uint32_t version;         // EK_TILE_LAYOUT_VERSION
  int32_t quant, hidden, intermediate, n_virtual;
  uint32_t reserved;
  uint64_t gu_bytes, dn_bytes, gu_scale_bytes, dn_scale_bytes;   // per virtual slot; quantised slots end with
                                                                 // two floats: the gate/up and down powers of two
};
constexpr size_t kBlobPowBytes = 2 * sizeof(float);
static_assert(sizeof(TileBlobHeader) == 64, "blob header is 64 bytes");

void tile_sizes(const ek_backend* be, TileBlobHeader* h) {
  const Dims& d = be->d;
  h->gu_bytes = (uint64_t)d.it * d.kt_gu * 2 * kTileBytes;
  h->dn_bytes = (uint64_t)d.hp * d.kt_dn * 2 * kTileBytes;
  const bool q = be->cfg.quant != EK_QUANT_BF16;
  h->gu_scale_bytes = q ? (uint64_t)d.it * d.kt_gu * 2 * 4 : 0;
  h->dn_scale_bytes = q ? (uint64_t)d.hp * d.kt_dn * 2 * 4 : 0;
}

int check_expert_id(ek_backend* be, const char* id, int* layer, int* expert, bool* shared) {
  const ek_config_t& c = be->cfg;
  std::string model;
  if (!parse_id(id, model, *layer, *expert, *shared)) return fail(be, EK_INVALID_INPUT, "invalid expert id: %s", id);
  if (c.model_name[0] && model != c.model_name)
    return fail(be, EK_INVALID_INPUT, "expert id %s does not belong to model %s", id, c.model_name);
  if (*shared && c.n_shared_experts == 0) return fail(be, EK_INVALID_INPUT, "layer has no shared expert: %s", id);
  if (!*shared && (*expert < 0 || *expert >= c.n_experts))
    return fail(be, EK_INVALID_INPUT, "expert %d outside [0,%d)", *expert, c.n_experts);
  if (!*shared && (*expert < be->e_lo || *expert >= be->e_hi) && c.replica_slots == 0)
    return fail(be, EK_INVALID_INPUT, "expert %d is not in this rank's range [%d,%d) and the backend has no replica slots",
                *expert, be->e_lo, be->e_hi);
  return EK_OK;
}

}  // namespace

int32_t ek_expert_export_tiles(ek_backend_t* be, const char* id, void* blob, size_t cap, size_t* needed) {
  if (!be || !id || !needed) return EK_INVALID_INPUT;
  cudaSetDevice(be->cfg.device);
  int layer, expert;
  bool shared;
  int rc = check_expert_id(be, id, &layer, &expert, &shared);
  if (rc != EK_OK) return rc;
  TileBlobHeader h;
  memset(&h, 0, sizeof h);
  memcpy(h.magic, "EKTILES", 8);
  h.version = EK_TILE_LAYOUT_VERSION;
  h.quant = be->cfg.quant; h.hidden = be->cfg.hidden; h.intermediate = be->cfg.intermediate;
  h.n_virtual = shared ? be->cfg.n_shared_experts : 1;
  tile_sizes(be, &h);
  const size_t per = h.gu_bytes + h.dn_bytes + h.gu_scale_bytes + h.dn_scale_bytes + (h.gu_scale_bytes ? kBlobPowBytes : 0);
  *needed = sizeof h + per * h.n_virtual;
  if (!blob || cap < *needed) return fail(be, EK_INVALID_INPUT, "tile blob needs %zu bytes", *needed);
  std::lock_guard<std::mutex> lg(be->load_mu);
  int slot0;
  Layer* L;
  {
    std::shared_lock<std::shared_mutex> g(be->reg_mu);
    auto it = be->experts.find(id);
    if (it == be->experts.end()) return fail(be, EK_EXPERT_NOT_FOUND, "%s", id);
    L = &be->layers[it->second.layer];
    slot0 = it->second.slot;
  }
  cudaStream_t ls = be->load_stream;
  uint8_t* o = reinterpret_cast<uint8_t*>(blob);
  memcpy(o, &h, sizeof h);
  o += sizeof h;
  for (int v = 0; v < h.n_virtual; ++v) {
    const int slot = slot0 + v;
    CK(cudaMemcpyAsync(o, L->gu + (size_t)slot * h.gu_bytes, h.gu_bytes, cudaMemcpyDeviceToHost, ls));
    o += h.gu_bytes;
    CK(cudaMemcpyAsync(o, L->dn + (size_t)slot * h.dn_bytes, h.dn_bytes, cudaMemcpyDeviceToHost, ls));
    o += h.dn_bytes;
    if (h.gu_scale_bytes) {
      CK(cudaMemcpyAsync(o, reinterpret_cast<const uint8_t*>(L->gu_scale) + (size_t)slot * h.gu_scale_bytes, h.gu_scale_bytes, cudaMemcpyDeviceToHost, ls));
      o += h.gu_scale_bytes;
      CK(cudaMemcpyAsync(o, reinterpret_cast<const uint8_t*>(L->dn_scale) + (size_t)slot * h.dn_scale_bytes, h.dn_scale_bytes, cudaMemcpyDeviceToHost, ls));
      o += h.dn_scale_bytes;
      CK(cudaMemcpyAsync(o, L->pow2 + slot, sizeof(float), cudaMemcpyDeviceToHost, ls));
      CK(cudaMemcpyAsync(o + sizeof(float), L->pow2 + be->n_slots + slot, sizeof(float), cudaMemcpyDeviceToHost, ls));
      o += kBlobPowBytes;
    }
  }
  CK(cudaStreamSynchronize(ls));
  return EK_OK;
}

int32_t ek_expert_register_tiles(ek_backend_t* be, const char* id, const void* blob, size_t len) {
  if (!be || !id || !blob) return EK_INVALID_INPUT;
  cudaSetDevice(be->cfg.device);
  int layer, expert;
  bool shared;
  int rc = check_expert_id(be, id, &layer, &expert, &shared);
  if (rc != EK_OK) return rc;
  TileBlobHeader h, want;
  if (len < sizeof h) return fail(be, EK_SAFETENSOR, "tile blob shorter than its header");
  memcpy(&h, blob, sizeof h);
  if (memcmp(h.magic, "EKTILES", 8) != 0) return fail(be, EK_SAFETENSOR, "not a tile blob");
  if (h.version != EK_TILE_LAYOUT_VERSION)
    return fail(be, EK_UNSUPPORTED, "tile blob has layout version %u, this library writes %d: register the bundle instead", h.version, EK_TILE_LAYOUT_VERSION);
  memset(&want, 0, sizeof want);
  tile_sizes(be, &want);
  const int n_virtual = shared ? be->cfg.n_shared_experts : 1;
  if (h.quant != be->cfg.quant || h.hidden != be->cfg.hidden || h.intermediate != be->cfg.intermediate ||
      h.n_virtual != n_virtual || h.gu_bytes != want.gu_bytes || h.dn_bytes != want.dn_bytes ||
      h.gu_scale_bytes != want.gu_scale_bytes || h.dn_scale_bytes != want.dn_scale_bytes)
    return fail(be, EK_INVALID_INPUT, "tile blob was written for another configuration (quant %d, H %d, I %d, %d slots)",
                h.quant, h.hidden, h.intermediate, h.n_virtual);
  const size_t per = h.gu_bytes + h.dn_bytes + h.gu_scale_bytes + h.dn_scale_bytes + (h.gu_scale_bytes ? kBlobPowBytes : 0);
  if (len != sizeof h + per * n_virtual) return fail(be, EK_SAFETENSOR, "tile blob has %zu bytes, expected %zu", len, sizeof h + per * n_virtual);

  std::lock_guard<std::mutex> lg(be->load_mu);
  Layer* L = nullptr;
  int slot_routed = -1;
  {
    std::unique_lock<std::shared_mutex> g(be->reg_mu);
    rc = ensure_layer(be, layer, &L);
    if (rc != EK_OK) return rc;
    auto live = be->experts.find(id);   // replacing a live expert: see ek_expert_register
    if (live != be->experts.end()) {
      unregister_slots(be, *L, live->second.slot);
      be->experts.erase(live);
    }
    if (!shared) {
      slot_routed = routed_slot(be, *L, expert, true);
      if (slot_routed < 0)
        return fail(be, EK_NO_MEMORY, "all %d replica slots of layer %d are taken", be->cfg.replica_slots, layer);
    }
  }
  cudaStream_t ls = be->load_stream;
  // the slot may still be read by forwards queued before an eviction
  CK(cudaEventRecord(be->fwd_done, be->stream));
  CK(cudaStreamWaitEvent(ls, be->fwd_done, 0));
  const uint8_t* in = reinterpret_cast<const uint8_t*>(blob) + sizeof h;
  for (int v = 0; v < n_virtual; ++v) {
    const int slot = shared ? be->n_local + v : slot_routed;
    CK(cudaMemcpyAsync(L->gu + (size_t)slot * h.gu_bytes, in, h.gu_bytes, cudaMemcpyHostToDevice, ls));
    in += h.gu_bytes;
    CK(cudaMemcpyAsync(L->dn + (size_t)slot * h.dn_bytes, in, h.dn_bytes, cudaMemcpyHostToDevice, ls));
    in += h.dn_bytes;
    if (h.gu_scale_bytes) {
      CK(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(L->gu_scale) + (size_t)slot * h.gu_scale_bytes, in, h.gu_scale_bytes, cudaMemcpyHostToDevice, ls));
      in += h.gu_scale_bytes;
      CK(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(L->dn_scale) + (size_t)slot * h.dn_scale_bytes, in, h.dn_scale_bytes, cudaMemcpyHostToDevice, ls));
      in += h.dn_scale_bytes;
      CK(cudaMemcpyAsync(L->pow2 + slot, in, sizeof(float), cudaMemcpyHostToDevice, ls));
      CK(cudaMemcpyAsync(L->pow2 + be->n_slots + slot, in + sizeof(float), sizeof(float), cudaMemcpyHostToDevice, ls));
      in += kBlobPowBytes;
    }
    const int32_t one = 1;
    CK(cudaMemcpyAsync(L->registered + slot, &one, sizeof one, cudaMemcpyHostToDevice, ls));
  }
  CK(cudaStreamSynchronize(ls));
  {
    std::unique_lock<std::shared_mutex> g(be->reg_mu);
    for (int v = 0; v < n_virtual; ++v) L->host_registered[shared ? be->n_local + v : slot_routed] = 1;
    be->loading.erase(id);
    ExpertRef ref{layer, shared ? be->n_local : slot_routed};
    be->experts[id] = ref;
    if (!shared && (expert < be->e_lo || expert >= be->e_hi)) publish_replica(be, *L, expert, slot_routed);
  }
  return EK_OK;
}

int32_t ek_expert_register_safetensors(ek_backend_t* be, const char* id, const void* blob, size_t len) {
  if (!be || !id || !blob) return EK_INVALID_INPUT;
  std::vector<ekst::Entry> ent;
  std::string err;
  if (!ekst::parse_blob(blob, len, ent, err)) return fail(be, EK_SAFETENSOR, "%s", err.c_str());
  // bundle order = order of data offsets (what SafeTensors::names()/tensors() iterate)
  std::sort(ent.begin(), ent.end(), [](const ekst::Entry& a, const ekst::Entry& b) { return a.begin < b.begin; });
  std::vector<ek_tensor_view_t> views(ent.size());
  for (size_t i = 0; i < ent.size(); ++i) {
    views[i].name = ent[i].name.c_str();
    views[i].dtype = ekst::dtype_from_string(ent[i].dtype);
    views[i].ndim = (int)std::min<size_t>(ent[i].shape.size(), 4);
    for (int j = 0; j < 4; ++j) views[i].shape[j] = j < (int)ent[i].shape.size() ? ent[i].shape[j] : 1;
    views[i].data = ent[i].data;
  }
  return ek_expert_register(be, id, views.data(), (int)views.size());
}

int32_t ek_router_register(ek_backend_t* be, int32_t layer, const void* weight, int32_t dt, const float* bias) {
  if (!be || !weight) return EK_INVALID_INPUT;
  if (dt != EK_BF16 && dt != EK_F32) return fail(be, EK_INVALID_INPUT, "router weight must be BF16 or F32");
  cudaSetDevice(be->cfg.device);
  std::lock_guard<std::mutex> lg(be->load_mu);
  std::unique_lock<std::shared_mutex> g(be->reg_mu);
  Layer* L = nullptr;
  int rc = ensure_layer(be, layer, &L);
  if (rc != EK_OK) return rc;
  CK(cudaStreamSynchronize(be->stream));
  const size_t bytes = (size_t)be->cfg.n_experts * be->cfg.hidden * (dt == EK_F32 ? 4 : 2);
  if (L->router_w) cudaFree(L->router_w);
  L->router_w = nullptr;
  CK(cudaMalloc(&L->router_w, bytes));
  CK(cudaMemcpy(L->router_w, weight, bytes, cudaMemcpyDefault));
  L->router_f32 = dt == EK_F32;
  // tensor-core router: needs the weight in bf16 without loss
  if (L->router_bf16_owned) cudaFree(L->router_bf16);
  L->router_bf16 = nullptr; L->router_bf16_owned = false; L->router_tc = false;
  if (router_tc_supported(be->cfg.n_experts, be->cfg.hidden)) {
    if (dt == EK_BF16) {
      L->router_bf16 = reinterpret_cast<__nv_bfloat16*>(L->router_w);
    } else {
      const int64_t n = (int64_t)be->cfg.n_experts * be->cfg.hidden;
      CK(cudaMalloc(&L->router_bf16, n * 2));
      L->router_bf16_owned = true;
      CK(cudaMemsetAsync(be->flag_dev, 0, 4, be->load_stream));
      be->launches += launch_f32_to_bf16_check(reinterpret_cast<const float*>(L->router_w), L->router_bf16, n,
                                              be->flag_dev, be->load_stream);
      int32_t inexact = 1;
      CK(cudaMemcpyAsync(&inexact, be->flag_dev, 4, cudaMemcpyDeviceToHost, be->load_stream));
      CK(cudaStreamSynchronize(be->load_stream));
      if (inexact) {   // fp32 weights that bf16 cannot hold: stay on the fp32 CUDA-core router
        cudaFree(L->router_bf16);
        L->router_bf16 = nullptr; L->router_bf16_owned = false;
      }
    }
    if (L->router_bf16)
      L->router_tc = encode_2d(be, &L->router_map, L->router_bf16, (uint64_t)be->cfg.hidden,
                               (uint64_t)be->cfg.n_experts, (uint32_t)be->cfg.n_experts);
  }
  if (L->router_bias) { cudaFree(L->router_bias); L->router_bias = nullptr; }
  if (bias) {
    CK(cudaMalloc(&L->router_bias, sizeof(float) * be->cfg.n_experts));
    CK(cudaMemcpy(L->router_bias, bias, sizeof(float) * be->cfg.n_experts, cudaMemcpyDefault));
  }
  // device-to-device copies above are asynchronous on the default stream, which the backend's
  // non-blocking streams do not wait for
  CK(cudaDeviceSynchronize());
  return EK_OK;
}

// ---- forward ---------------------------------------------------------------------------------

// ---- worker-level forward: concurrent single-expert calls are served as one grouped launch ----
//
// The reference worker runs one `forward` per RPC on up to 48 runtime threads
// (ek-computation/src/worker/core.rs:47-74, bin/worker.rs:5), each on its own expert.  A single
// expert occupies 16 of the 148 CTAs of the grouped GEMM, so here every caller queues its request
// and whoever gets the forward lock next serves everything queued so far in one launch per layer
// ("combining lock"); callers whose request was served by someone else just pick up the result.
namespace {

// One virtual-expert request served alone (shared experts with several virtual slots): the partial
// outputs are summed with the combine kernel.
int serve_shared(ek_backend* be, ExpertReq& r, const ExpertRef& ent) {
  const ek_config_t& c = be->cfg;
  const int n = r.n, n_virtual = c.n_shared_experts;
  if ((int64_t)n * n_virtual > be->rows_cap - 128) return fail(be, EK_INVALID_INPUT, "batch of %d rows exceeds the workspace", n);
  Layer& L = be->layers[ent.layer];
  const size_t H = c.hidden;
  cudaStream_t s = be->stream;
  CK(cudaMemcpyAsync(be->xp, r.x, (size_t)n * H * 2, cudaMemcpyDefault, s));
  if (f16_rows(be)) be->launches += launch_rows_to_f16(be->xp, n, c.hidden, s);
  const int nmax = n <= 32 ? 32 : n <= 64 ? 64 : 128;
  const int chunk_rows = be->ffn_impl == 1 ? 16 : nmax;
  const int per = (n + chunk_rows - 1) / chunk_rows;
  if (per * n_virtual > std::min(be->h_chunks_cap, be->max_chunks)) return fail(be, EK_INVALID_INPUT, "batch too large for a single-expert call");
  for (int v = 0; v < n_virtual; ++v)
    for (int cidx = 0; cidx < per; ++cidx) {
      ChunkDesc cd;
      cd.slot = ent.slot + v;
      cd.in_row = cidx * chunk_rows;
      cd.out_row = v * n + cidx * chunk_rows;
      cd.n_rows = std::min(chunk_rows, n - cidx * chunk_rows) | (per > 1 ? kChunkMulti : 0);
      be->h_chunks[v * per + cidx] = cd;
    }
  const int32_t total = per * n_virtual;
  CK(cudaMemcpyAsync(be->chunks, be->h_chunks, sizeof(ChunkDesc) * total, cudaMemcpyHostToDevice, s));
  be->h_status->aux1 = total;   // pinned word as the source of the count
  CK(cudaMemcpyAsync(be->n_chunks, &be->h_status->aux1, 4, cudaMemcpyHostToDevice, s));
  run_ffn(be, L, nmax, 0, false);   // worker-level replies must not depend on what else was grouped
  run_ffn(be, L, nmax, 1, false);   // worker-level replies must not depend on what else was grouped
  CombineParams cp;
  cp.obuf = be->obuf; cp.inv = be->inv; cp.weights = be->weights; cp.y = be->y_dev;
  cp.T = n; cp.k = 0; cp.H = c.hidden; cp.n_shared = n_virtual; cp.Tk = 0; cp.bf16_products = 0;
  cp.shared = nullptr;
  be->launches += launch_combine(cp, s);
  CK(cudaMemcpyAsync(r.y, be->y_dev, (size_t)n * H * 2, cudaMemcpyDefault, s));
  int rc = check_status(be);
  if (rc != EK_OK) return rc;
  CK(cudaGetLastError());
  return EK_OK;
}

// Requests of one layer, each on one expert slot: rows packed back to back, one grouped launch.
int serve_group(ek_backend* be, int layer, std::vector<std::pair<ExpertReq*, int>>& group) {
  const ek_config_t& c = be->cfg;
  Layer& L = be->layers[layer];
  const size_t H = c.hidden;
  cudaStream_t s = be->stream;
  int n_max = 0;
  for (auto& g : group) n_max = std::max(n_max, g.first->n);
  const int nmax = n_max <= 32 ? 32 : n_max <= 64 ? 64 : 128;
  const int chunk_rows = be->ffn_impl == 1 ? 16 : nmax;
  int row = 0, n_chunks = 0;
  for (auto& g : group) {
    ExpertReq& r = *g.first;
    const int per = (r.n + chunk_rows - 1) / chunk_rows;
    CK(cudaMemcpyAsync(be->xp + (size_t)row * H, r.x, (size_t)r.n * H * 2, cudaMemcpyDefault, s));
    for (int cidx = 0; cidx < per; ++cidx) {
      ChunkDesc cd;
      cd.slot = g.second;
      cd.in_row = row + cidx * chunk_rows;
      cd.out_row = row + cidx * chunk_rows;
      cd.n_rows = std::min(chunk_rows, r.n - cidx * chunk_rows) | (per > 1 ? kChunkMulti : 0);
      be->h_chunks[n_chunks++] = cd;
    }
    r.row0 = row;
    row += r.n;
  }
  if (f16_rows(be)) be->launches += launch_rows_to_f16(be->xp, row, c.hidden, s);
  CK(cudaMemcpyAsync(be->chunks, be->h_chunks, sizeof(ChunkDesc) * n_chunks, cudaMemcpyHostToDevice, s));
  be->h_status->aux1 = n_chunks;
  CK(cudaMemcpyAsync(be->n_chunks, &be->h_status->aux1, 4, cudaMemcpyHostToDevice, s));
  run_ffn(be, L, nmax, 0, false);   // worker-level replies must not depend on what else was grouped
  run_ffn(be, L, nmax, 1, false);   // worker-level replies must not depend on what else was grouped
  for (auto& g : group) {
    ExpertReq& r = *g.first;
    CK(cudaMemcpyAsync(r.y, be->obuf + (size_t)r.row0 * H, (size_t)r.n * H * 2, cudaMemcpyDefault, s));
  }
  int rc = check_status(be);
  if (rc != EK_OK) return rc;
  CK(cudaGetLastError());
  return EK_OK;
}

// Serves every queued request; called with the forward lock held.
void serve_pending(ek_backend* be) {
  // When calls have been arriving together, give the callers that were just released a moment to
  // queue their next request: a pass over nine experts costs what a pass over one does.  The window
  // closes when the queue has stopped growing for three polls, at the latest after 20 us; a lone
  // caller (previous pass served one request) never waits.
  if (be->last_batch > 1) {
    const auto t0 = std::chrono::steady_clock::now();
    size_t prev = 0;
    int stable = 0;
    while (std::chrono::steady_clock::now() - t0 < std::chrono::microseconds(20)) {
      size_t cur;
      {
        std::lock_guard<std::mutex> pg(be->pend_mu);
        cur = be->pending.size();
      }
      stable = cur == prev ? stable + 1 : 0;
      prev = cur;
      if (stable >= 3) break;
      const auto p0 = std::chrono::steady_clock::now();
      while (std::chrono::steady_clock::now() - p0 < std::chrono::microseconds(1)) {}
    }
  }
  std::vector<ExpertReq*> batch;
  {
    std::lock_guard<std::mutex> pg(be->pend_mu);
    batch.swap(be->pending);
  }
  if (batch.empty()) return;
  be->last_batch = (int)batch.size();
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  const ek_config_t& c = be->cfg;
  // group by layer, in arrival order; a group is cut when the workspace or the chunk list is full
  std::map<int, std::vector<std::pair<ExpertReq*, int>>> by_layer;
  for (ExpertReq* r : batch) {
    auto it = be->experts.find(r->id);
    if (it == be->experts.end()) {
      r->rc = fail(be, EK_EXPERT_NOT_FOUND, "%s", r->id);
      r->done.store(true, std::memory_order_release);
      continue;
    }
    std::string model; int layer, expert; bool shared;
    parse_id(r->id, model, layer, expert, shared);
    if (shared && c.n_shared_experts > 1) {
      r->rc = serve_shared(be, *r, it->second);
      r->done.store(true, std::memory_order_release);
      continue;
    }
    if (r->n > be->rows_cap - 128) {
      r->rc = fail(be, EK_INVALID_INPUT, "batch of %d rows exceeds the workspace", r->n);
      r->done.store(true, std::memory_order_release);
      continue;
    }
    by_layer[it->second.layer].push_back({r, it->second.slot});
  }
  for (auto& kv : by_layer) {
    auto& all = kv.second;
    size_t i = 0;
    while (i < all.size()) {
      std::vector<std::pair<ExpertReq*, int>> group;
      int rows = 0, chunks = 0;
      while (i < all.size()) {
        const int n = all[i].first->n;
        const int ch = (n + 15) / 16;   // upper bound on its chunks
        if (!group.empty() && (rows + n > be->rows_cap - 128 || chunks + ch > std::min(be->h_chunks_cap, be->max_chunks))) break;
        group.push_back(all[i]);
        rows += n;
        chunks += ch;
        ++i;
      }
      const int rc = serve_group(be, kv.first, group);
      for (auto& g2 : group) {
        g2.first->rc = rc;
        g2.first->done.store(true, std::memory_order_release);
      }
    }
  }
  be->batched_calls += (int64_t)batch.size();
  be->batched_launches += 1;
}

}  // namespace

int32_t ek_expert_forward(ek_backend_t* be, const char* id, const void* x, int32_t n, void* y) {
  if (!be || !id || !x || !y) return EK_INVALID_INPUT;
  if (n < 1) return fail(be, EK_INVALID_INPUT, "empty batch");   // core.rs:55 asserts non-empty
  ExpertReq r;
  r.id = id; r.x = x; r.n = n; r.y = y;
  {
    std::lock_guard<std::mutex> pg(be->pend_mu);
    be->pending.push_back(&r);
  }
  // Whoever finds the forward lock free serves the queue; the others sleep until their request is
  // marked done (or, after a pass that missed them, until they can serve the queue themselves).
  while (!r.done.load(std::memory_order_acquire)) {
    if (be->fwd_mu.try_lock()) {
      if (!r.done.load(std::memory_order_acquire)) {
        cudaSetDevice(be->cfg.device);
        serve_pending(be);
      }
      be->fwd_mu.unlock();
      { std::lock_guard<std::mutex> pg(be->pend_mu); }
      be->pend_cv.notify_all();
    } else {
      std::unique_lock<std::mutex> lk(be->pend_mu);
      be->pend_cv.wait_for(lk, std::chrono::microseconds(100),
                           [&] { return r.done.load(std::memory_order_acquire); });
    }
  }
  return r.rc;
}

static int stage_in(ek_backend* be, const void* x, size_t bytes, const __nv_bfloat16** dev) {
  if (is_device_ptr(x)) {
    *dev = reinterpret_cast<const __nv_bfloat16*>(x);
    return EK_OK;
  }
  // pageable host memory -> pinned staging -> device, all inside the call; memory the caller
  // already pinned is copied from directly
  const void* src = x;
  if (!is_pinned_host(x)) {
    memcpy(be->h_x, x, bytes);
    src = be->h_x;
  }
  CK(cudaMemcpyAsync(be->x_dev, src, bytes, cudaMemcpyHostToDevice, be->stream));
  *dev = be->x_dev;
  return EK_OK;
}

int32_t ek_moe_forward_fused(ek_backend_t* be, int32_t layer, const void* x, int32_t T, void* y,
                             const ek_route_debug_t* dbg) {
  if (!be || !x || !y) return EK_INVALID_INPUT;
  if (T < 1 || T > be->cfg.max_tokens) return fail(be, EK_INVALID_INPUT, "T=%d outside [1,%d]", T, be->cfg.max_tokens);
  cudaSetDevice(be->cfg.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  auto li = be->layers.find(layer);
  if (li == be->layers.end() || !li->second.router_w)
    return fail(be, EK_NOT_FOUND, "layer %d has no router weight registered", layer);
  const ek_config_t& c = be->cfg;
  const size_t bytes = (size_t)T * c.hidden * 2;
  const __nv_bfloat16* xd;
  int rc = stage_in(be, x, bytes, &xd);
  if (rc != EK_OK) return rc;
  const bool y_dev = is_device_ptr(y);
  __nv_bfloat16* yd = y_dev ? reinterpret_cast<__nv_bfloat16*>(y) : be->y_dev;
  rc = run_layer(be, li->second, xd, T, c.top_k, nullptr, yd, nullptr);
  if (rc != EK_OK) return rc;
  cudaStream_t s = be->stream;
  const bool y_pinned = !y_dev && is_pinned_host(y);
  if (!y_dev) CK(cudaMemcpyAsync(y_pinned ? y : be->h_y, be->y_dev, bytes, cudaMemcpyDeviceToHost, s));
  if (dbg) {
    const size_t E = c.n_experts, K = c.top_k;
    if (dbg->logits) CK(cudaMemcpyAsync(dbg->logits, be->logits, T * E * 4, cudaMemcpyDefault, s));
    if (dbg->ids) CK(cudaMemcpyAsync(dbg->ids, be->ids, T * K * 4, cudaMemcpyDefault, s));
    if (dbg->weights) CK(cudaMemcpyAsync(dbg->weights, be->weights, T * K * 4, cudaMemcpyDefault, s));
    if (dbg->counts) CK(cudaMemcpyAsync(dbg->counts, be->counts, E * 4, cudaMemcpyDefault, s));
    if (dbg->offsets) CK(cudaMemcpyAsync(dbg->offsets, be->offsets, (E + 1) * 4, cudaMemcpyDefault, s));
    if (dbg->perm) CK(cudaMemcpyAsync(dbg->perm, be->perm, T * K * 4, cudaMemcpyDefault, s));
  }
  rc = check_status(be);
  if (rc != EK_OK) return rc;
  if (!y_dev && !y_pinned) memcpy(y, be->h_y, bytes);
  return finish_timing(be);
}

int32_t ek_moe_forward_fused_async(ek_backend_t* be, int32_t layer, const void* x, int32_t T, void* y) {
  if (!be || !x || !y) return EK_INVALID_INPUT;
  if (T < 1 || T > be->cfg.max_tokens) return fail(be, EK_INVALID_INPUT, "T=%d outside [1,%d]", T, be->cfg.max_tokens);
  cudaSetDevice(be->cfg.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  auto li = be->layers.find(layer);
  if (li == be->layers.end() || !li->second.router_w)
    return fail(be, EK_NOT_FOUND, "layer %d has no router weight registered", layer);
  return run_layer(be, li->second, reinterpret_cast<const __nv_bfloat16*>(x), T, be->cfg.top_k, nullptr,
                   reinterpret_cast<__nv_bfloat16*>(y), nullptr);
}

int32_t ek_sync(ek_backend_t* be) {
  if (!be) return EK_INVALID_INPUT;
  cudaSetDevice(be->cfg.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  int rc = check_status(be);
  if (rc != EK_OK) return rc;
  return finish_timing(be);
}

int32_t ek_set_stream(ek_backend_t* be, void* stream) {
  if (!be) return EK_INVALID_INPUT;
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  cudaStreamSynchronize(be->stream);
  // (void*)-1 selects the backend's own stream again; NULL is CUDA's default stream
  be->stream = stream == reinterpret_cast<void*>(-1) ? be->own_stream : reinterpret_cast<cudaStream_t>(stream);
  return EK_OK;
}

int32_t ek_moe_forward(ek_backend_t* be, int32_t layer, const void* x, int32_t T, const int32_t* ids, int32_t k,
                       void* out) {
  if (!be || !x || !ids || !out) return EK_INVALID_INPUT;
  const ek_config_t& c = be->cfg;
  if (T < 1 || T > c.max_tokens) return fail(be, EK_INVALID_INPUT, "T=%d outside [1,%d]", T, c.max_tokens);
  if (k < 1 || k > c.top_k) return fail(be, EK_INVALID_INPUT, "k=%d outside [1,%d]", k, c.top_k);
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  auto li = be->layers.find(layer);
  if (li == be->layers.end()) return fail(be, EK_EXPERT_NOT_FOUND, "layer %d holds no experts", layer);
  const size_t bytes = (size_t)T * c.hidden * 2, obytes = bytes * k;
  const __nv_bfloat16* xd;
  int rc = stage_in(be, x, bytes, &xd);
  if (rc != EK_OK) return rc;
  cudaStream_t s = be->stream;
  CK(cudaMemcpyAsync(be->ids, ids, (size_t)T * k * 4, cudaMemcpyDefault, s));
  const bool out_dev = is_device_ptr(out);
  __nv_bfloat16* od = reinterpret_cast<__nv_bfloat16*>(out);
  if (!out_dev) {
    if (be->tk_cap < obytes) {
      cudaStreamSynchronize(s);
      rc = grow(be, (void**)&be->tk_dev, &be->tk_cap, obytes);
      if (rc != EK_OK) return rc;
    }
    if (be->h_tk_cap < obytes) {
      if (be->h_tk) cudaFreeHost(be->h_tk);
      be->h_tk = nullptr; be->h_tk_cap = 0;
      CK(cudaMallocHost(&be->h_tk, obytes));
      be->h_tk_cap = obytes;
    }
    od = be->tk_dev;
  }
  rc = run_layer(be, li->second, xd, T, k, be->ids, nullptr, od);
  if (rc != EK_OK) return rc;
  if (!out_dev) CK(cudaMemcpyAsync(be->h_tk, od, obytes, cudaMemcpyDeviceToHost, s));
  rc = check_status(be);
  if (rc != EK_OK) return rc;
  if (!out_dev) memcpy(out, be->h_tk, obytes);
  return finish_timing(be);
}

int32_t ek_route_from_logits(ek_backend_t* be, const float* logits, int32_t T, const float* bias, int32_t* ids,
                             float* weights, int32_t* counts, int32_t* offsets, int32_t* perm) {
  if (!be || !logits) return EK_INVALID_INPUT;
  const ek_config_t& c = be->cfg;
  if (T < 1 || T > c.max_tokens) return fail(be, EK_INVALID_INPUT, "T=%d outside [1,%d]", T, c.max_tokens);
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  cudaStream_t s = be->stream;
  const size_t E = c.n_experts, K = c.top_k;
  CK(cudaMemcpyAsync(be->logits, logits, T * E * 4, cudaMemcpyDefault, s));
  float* bias_dev = nullptr;
  if (bias) {
    bias_dev = be->bias_scratch;
    CK(cudaMemcpyAsync(bias_dev, bias, E * 4, cudaMemcpyDefault, s));
  }
  RouteParams rp;
  rp.x = nullptr; rp.wg = nullptr; rp.wg_f32 = 0; rp.bias = bias_dev;
  rp.logits = be->logits; rp.ids = be->ids; rp.weights = be->weights; rp.counts = be->counts;
  rp.T = T; rp.H = c.hidden; rp.E = c.n_experts; rp.k = c.top_k;
  rp.scoring = c.scoring; rp.n_group = c.n_group; rp.topk_group = c.topk_group;
  rp.norm = c.norm_topk_prob; rp.scaling = c.routed_scaling; rp.bf16_weights = c.bf16_combine;
  rp.partial = nullptr; rp.n_partials = 0;
  be->launches += launch_route_select(rp, s);
  PermuteParams pp;
  pp.ids = be->ids; pp.counts = be->counts; pp.offsets = be->offsets; pp.perm = be->perm; pp.inv = be->inv;
  pp.T = T; pp.k = c.top_k; pp.E = c.n_experts; pp.e_lo = 0; pp.e_hi = c.n_experts;
  be->launches += launch_permute(pp, s);
  if (ids) CK(cudaMemcpyAsync(ids, be->ids, T * K * 4, cudaMemcpyDefault, s));
  if (weights) CK(cudaMemcpyAsync(weights, be->weights, T * K * 4, cudaMemcpyDefault, s));
  if (counts) CK(cudaMemcpyAsync(counts, be->counts, E * 4, cudaMemcpyDefault, s));
  if (offsets) CK(cudaMemcpyAsync(offsets, be->offsets, (E + 1) * 4, cudaMemcpyDefault, s));
  if (perm) CK(cudaMemcpyAsync(perm, be->perm, T * K * 4, cudaMemcpyDefault, s));
  CK(cudaStreamSynchronize(s));
  CK(cudaGetLastError());
  return EK_OK;
}

int32_t ek_combine(ek_backend_t* be, const void* out, const float* weights, int32_t T, int32_t k,
                   const void* shared, void* y) {
  if (!be || !out || !weights || !y) return EK_INVALID_INPUT;
  const ek_config_t& c = be->cfg;
  if (T < 1 || T > c.max_tokens || k < 1 || k > c.top_k) return fail(be, EK_INVALID_INPUT, "T or k out of range");
  // `out` and `shared` are staged back to back in the output workspace, which holds rows_cap rows
  if ((int64_t)T * k + (shared ? T : 0) > be->rows_cap)
    return fail(be, EK_INVALID_INPUT, "T*k%s = %lld rows exceed the workspace of %d rows: raise max_tokens",
                shared ? " + T" : "", (long long)T * k + (shared ? T : 0), be->rows_cap);
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  cudaStream_t s = be->stream;
  const size_t H = c.hidden;
  // rows [0,T*k) of the output buffer in (token,slot) order, shared rows behind them
  CK(cudaMemcpyAsync(be->obuf, out, (size_t)T * k * H * 2, cudaMemcpyDefault, s));
  if (shared) CK(cudaMemcpyAsync(be->obuf + (size_t)T * k * H, shared, (size_t)T * H * 2, cudaMemcpyDefault, s));
  CK(cudaMemcpyAsync(be->weights, weights, (size_t)T * k * 4, cudaMemcpyDefault, s));
  std::vector<int32_t> ident((size_t)T * k);
  for (size_t i = 0; i < ident.size(); ++i) ident[i] = (int32_t)i;
  CK(cudaMemcpyAsync(be->inv, ident.data(), ident.size() * 4, cudaMemcpyHostToDevice, s));
  CK(cudaStreamSynchronize(s));
  CombineParams cp;
  cp.obuf = be->obuf; cp.inv = be->inv; cp.weights = be->weights; cp.y = be->y_dev;
  cp.T = T; cp.k = k; cp.H = c.hidden; cp.n_shared = shared ? 1 : 0; cp.Tk = T * k;
  cp.bf16_products = c.bf16_combine;
  cp.shared = nullptr;
  be->launches += launch_combine(cp, s);
  CK(cudaMemcpyAsync(y, be->y_dev, (size_t)T * H * 2, cudaMemcpyDefault, s));
  CK(cudaStreamSynchronize(s));
  CK(cudaGetLastError());
  return EK_OK;
}

int32_t ek_w8a16_activate(ek_backend_t* be, const void* w, int32_t w_dtype, const float* scale, int32_t rows,
                          int32_t cols, void* out) {
  if (!be || !w || !scale || !out) return EK_INVALID_INPUT;
  if (w_dtype != EK_F8_E4M3 && w_dtype != EK_I8) return fail(be, EK_INVALID_INPUT, "payload must be F8_E4M3 or I8");
  // the reference reshapes into whole 128x128 blocks (expert_torch.rs:28-46)
  if (rows < 128 || cols < 128 || rows % 128 || cols % 128)
    return fail(be, EK_INVALID_INPUT, "rows and cols must be multiples of 128");
  cudaSetDevice(be->cfg.device);
  std::lock_guard<std::mutex> lg(be->load_mu);
  cudaStream_t s = be->load_stream;
  const size_t n = (size_t)rows * cols, sn = (size_t)(rows / 128) * (cols / 128) * 4;
  int rc = grow(be, &be->stage[0], &be->stage_cap[0], n);
  if (rc != EK_OK) return rc;
  rc = grow(be, (void**)&be->stage_scale[0], &be->stage_scale_cap[0], sn);
  if (rc != EK_OK) return rc;
  rc = grow(be, &be->stage_cvt, &be->stage_cvt_cap, n * 2);
  if (rc != EK_OK) return rc;
  CK(cudaMemcpyAsync(be->stage[0], w, n, cudaMemcpyDefault, s));
  CK(cudaMemcpyAsync(be->stage_scale[0], scale, sn, cudaMemcpyDefault, s));
  be->launches += launch_dequant(be->stage[0], w_dtype, be->stage_scale[0], rows, cols,
                                 reinterpret_cast<__nv_bfloat16*>(be->stage_cvt), s);
  CK(cudaMemcpyAsync(out, be->stage_cvt, n * 2, cudaMemcpyDefault, s));
  CK(cudaStreamSynchronize(s));
  CK(cudaGetLastError());
  return EK_OK;
}

int32_t ek_worker_forward_wire(ek_backend_t* be, const char* expert_id, const void* req, size_t req_len, void* resp,
                               size_t resp_cap, size_t* resp_len) {
  if (!be || !expert_id || !req || !resp_len) return EK_INVALID_INPUT;
  std::vector<ekst::Entry> ent;
  std::string err;
  if (!ekst::parse_blob(req, req_len, ent, err)) return fail(be, EK_SAFETENSOR, "%s", err.c_str());
  const ekst::Entry* data = nullptr;
  for (auto& e : ent)
    if (e.name == "data") data = &e;
  if (!data) return fail(be, EK_SAFETENSOR, "tensor name not found: data");   // EKError::SafeTensorNotFound
  if (data->dtype != "BF16") return fail(be, EK_INVALID_INPUT, "request tensor must be BF16, got %s", data->dtype.c_str());
  if (data->shape.size() != 2) return fail(be, EK_INVALID_INPUT, "request tensor must be 2-D");   // ffn/mod.rs:45
  if (data->shape[1] != be->cfg.hidden) return fail(be, EK_INVALID_INPUT, "request hidden size %lld != %d", (long long)data->shape[1], be->cfg.hidden);
  const int64_t n = data->shape[0];
  if (n < 1 || n > be->cfg.max_tokens) return fail(be, EK_INVALID_INPUT, "request rows %lld outside [1,%d]", (long long)n, be->cfg.max_tokens);
  const std::string hdr = ekst::single_header(n, be->cfg.hidden);
  const size_t payload = (size_t)n * be->cfg.hidden * 2;
  const size_t need = 8 + hdr.size() + payload;
  *resp_len = need;
  if (!resp || resp_cap < need) return fail(be, EK_INVALID_INPUT, "response buffer too small: need %zu bytes", need);
  uint8_t* o = reinterpret_cast<uint8_t*>(resp);
  const uint64_t hl = hdr.size();
  memcpy(o, &hl, 8);
  memcpy(o + 8, hdr.data(), hdr.size());
  // the payload may be unaligned inside the blob; cudaMemcpy from pageable memory does not care
  return ek_expert_forward(be, expert_id, data->data, (int32_t)n, o + 8 + hdr.size());
}


// ---- expert-parallel stages ------------------------------------------------------------------------
// The reference shards experts over worker processes and moves rows by gRPC
// (ek-computation/src/controller/executor.rs:141-226).  Here experts are sharded contiguously over
// the GPUs of one box (expert e lives on rank e / (E / ep_size)); the caller moves rows between
// ranks (all-to-all over NVLink) between these three stages, which all run on the backend stream.

int32_t ek_ep_route(ek_backend_t* be, int32_t layer, const void* x_dev, int32_t T, void* send_rows_dev,
                    int32_t* counts_dev) {
  if (!be || !x_dev || !send_rows_dev || !counts_dev) return EK_INVALID_INPUT;
  if (T < 1 || T > be->cfg.max_tokens) return fail(be, EK_INVALID_INPUT, "T=%d outside [1,%d]", T, be->cfg.max_tokens);
  cudaSetDevice(be->cfg.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  auto li = be->layers.find(layer);
  if (li == be->layers.end() || !li->second.router_w)
    return fail(be, EK_NOT_FOUND, "layer %d has no router weight registered", layer);
  Layer& L = li->second;
  const ek_config_t& c = be->cfg;
  cudaStream_t s = be->stream;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(x_dev);
  RouteParams rp;
  rp.x = x; rp.wg = L.router_w; rp.wg_f32 = L.router_f32; rp.bias = L.router_bias;
  rp.logits = be->logits; rp.ids = be->ids; rp.weights = be->weights; rp.counts = be->counts;
  rp.T = T; rp.H = c.hidden; rp.E = c.n_experts; rp.k = c.top_k;
  rp.scoring = c.scoring; rp.n_group = c.n_group; rp.topk_group = c.topk_group;
  rp.norm = c.norm_topk_prob; rp.scaling = c.routed_scaling; rp.bf16_weights = c.bf16_combine;
  rp.partial = nullptr; rp.n_partials = 0;
  bool tc_done = false;
  if (L.router_tc) {
    RouterTcParams tp;
    if (encode_2d(be, &tp.x_map, x, (uint64_t)c.hidden, (uint64_t)T, 128)) {
      tp.w_map = L.router_map; tp.partial = be->partial; tp.status = be->status;
      tp.T = T; tp.H = c.hidden; tp.E = c.n_experts; tp.n_atoms = (c.hidden + 63) / 64;
      router_tc_plan(T, c.hidden, be->n_sm, &tp.n_splits, &tp.atoms_per_split);
      tp.tmem_cols = 32;
      while (tp.tmem_cols < c.n_experts) tp.tmem_cols *= 2;
      be->launches += launch_router_tc(tp, s);
      rp.partial = be->partial; rp.n_partials = tp.n_splits;
      tc_done = true;
    }
  }
  if (!tc_done) be->launches += launch_router_logits(rp, s);
  be->launches += launch_route_select(rp, s);
  // bucket over ALL experts: rows sorted by global expert id are already grouped by owner rank
  PermuteParams pp;
  pp.ids = be->ids; pp.counts = be->counts; pp.offsets = be->offsets; pp.perm = be->perm; pp.inv = be->inv;
  pp.T = T; pp.k = c.top_k; pp.E = c.n_experts; pp.e_lo = 0; pp.e_hi = c.n_experts;
  be->launches += launch_permute(pp, s);
  be->launches += launch_gather(x, be->perm, be->offsets + c.n_experts, reinterpret_cast<__nv_bfloat16*>(send_rows_dev),
                                T, c.top_k, c.hidden, 0, 0, false, s);
  CK(cudaMemcpyAsync(counts_dev, be->counts, sizeof(int32_t) * c.n_experts, cudaMemcpyDeviceToDevice, s));
  CK(cudaMemcpyAsync(L.last_counts, be->counts, sizeof(int32_t) * c.n_experts, cudaMemcpyDeviceToDevice, s));
  L.have_counts = true;
  CK(cudaGetLastError());
  return EK_OK;
}

int32_t ek_ep_ffn(ek_backend_t* be, int32_t layer, const void* rows_dev, const int32_t* counts_src_host,
                  const void* x_dev, int32_t T, void* out_rows_dev) {
  if (!be || !counts_src_host) return EK_INVALID_INPUT;
  cudaSetDevice(be->cfg.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  auto li = be->layers.find(layer);
  if (li == be->layers.end()) return fail(be, EK_EXPERT_NOT_FOUND, "layer %d holds no experts", layer);
  Layer& L = li->second;
  const ek_config_t& c = be->cfg;
  const int R = c.ep_size, EL = be->n_local, S = c.n_shared_experts;
  if (S > 0 && (!x_dev || T < 1 || T > c.max_tokens)) return fail(be, EK_INVALID_INPUT, "shared expert needs the local tokens");
  // the pinned staging areas are reused per call: wait until the previous call's uploads were consumed
  if (be->ep_uploaded) CK(cudaEventSynchronize(be->ep_upload_done));
  // rows per local expert and where each (source, expert) segment goes in expert order
  std::vector<int> per_expert(EL, 0);
  int64_t n_rows = 0;
  for (int sidx = 0; sidx < R; ++sidx)
    for (int e = 0; e < EL; ++e) {
      const int v = counts_src_host[sidx * EL + e];
      if (v < 0) return fail(be, EK_INVALID_INPUT, "negative row count");
      per_expert[e] += v;
      n_rows += v;
    }
  const int Tsh = S > 0 ? T : 0;
  if (n_rows + (int64_t)S * Tsh > be->rows_cap - 128)
    return fail(be, EK_INVALID_INPUT, "%lld rows arrived, workspace holds %d: raise max_tokens", (long long)n_rows, be->rows_cap);
  if (n_rows > 0 && (!rows_dev || !out_rows_dev)) return EK_INVALID_INPUT;
  std::vector<int> expert_off(EL + 1, 0);
  for (int e = 0; e < EL; ++e) expert_off[e + 1] = expert_off[e] + per_expert[e];
  std::vector<int> fill(EL, 0);
  int n_segs = 0, arrival = 0, max_seg = 0;
  for (int sidx = 0; sidx < R; ++sidx)
    for (int e = 0; e < EL; ++e) {
      const int v = counts_src_host[sidx * EL + e];
      if (v == 0) continue;
      if (!L.host_registered[e]) return fail(be, EK_EXPERT_NOT_FOUND, "expert %d received rows but is not registered", be->e_lo + e);
      RowSegment sg;
      sg.src = arrival; sg.dst = expert_off[e] + fill[e]; sg.n = v; sg.pad = 0;
      be->h_segs[n_segs++] = sg;
      arrival += v;
      fill[e] += v;
      max_seg = std::max(max_seg, v);
    }
  const int rows_total = (int)n_rows;
  const int nmax = pick_nmax(rows_total, EL);
  const int chunk_rows = be->ffn_impl == 1 ? 16 : nmax;
  int n_chunks = 0;
  auto push = [&](int slot, int in_row, int out_row, int n) -> bool {
    for (int c0 = 0; c0 < n; c0 += chunk_rows) {
      if (n_chunks >= be->h_chunks_cap || n_chunks >= be->max_chunks) return false;
      ChunkDesc cd;
      cd.slot = slot; cd.in_row = in_row + c0; cd.out_row = out_row + c0;
      cd.n_rows = std::min(chunk_rows, n - c0) | (n > chunk_rows ? kChunkMulti : 0);
      be->h_chunks[n_chunks++] = cd;
    }
    return true;
  };
  for (int e = 0; e < EL; ++e)
    if (per_expert[e] > 0 && !push(e, expert_off[e], expert_off[e], per_expert[e]))
      return fail(be, EK_INVALID_INPUT, "too many chunks for the workspace");
  for (int j = 0; j < S; ++j) {
    if (!L.host_registered[EL + j]) return fail(be, EK_EXPERT_NOT_FOUND, "shared expert %d of the layer is not registered", j);
    if (!push(EL + j, rows_total, rows_total + j * Tsh, Tsh)) return fail(be, EK_INVALID_INPUT, "too many chunks for the workspace");
  }
  cudaStream_t s = be->stream;
  RowSegment* h_rev = be->h_segs + be->segs_cap;
  RowSegment* d_rev = be->segs + be->segs_cap;
  if (n_segs > 0) {
    for (int i = 0; i < n_segs; ++i) {
      h_rev[i] = be->h_segs[i];
      std::swap(h_rev[i].src, h_rev[i].dst);   // back to arrival order
    }
    CK(cudaMemcpyAsync(be->segs, be->h_segs, sizeof(RowSegment) * n_segs, cudaMemcpyHostToDevice, s));
    CK(cudaMemcpyAsync(d_rev, h_rev, sizeof(RowSegment) * n_segs, cudaMemcpyHostToDevice, s));
    be->launches += launch_segment_copy(reinterpret_cast<const __nv_bfloat16*>(rows_dev), be->xp, be->segs, n_segs,
                                        max_seg, c.hidden, s);
  }
  if (S > 0)
    CK(cudaMemcpyAsync(be->xp + (size_t)rows_total * c.hidden, x_dev, (size_t)T * c.hidden * 2, cudaMemcpyDeviceToDevice, s));
  if (f16_rows(be)) be->launches += launch_rows_to_f16(be->xp, (int64_t)rows_total + (S > 0 ? T : 0), c.hidden, s);
  CK(cudaMemcpyAsync(be->chunks, be->h_chunks, sizeof(ChunkDesc) * n_chunks, cudaMemcpyHostToDevice, s));
  be->h_ep_count[0] = n_chunks;
  CK(cudaMemcpyAsync(be->n_chunks, &be->h_ep_count[0], 4, cudaMemcpyHostToDevice, s));
  CK(cudaEventRecord(be->ep_upload_done, s));
  be->ep_uploaded = true;
  be->ep_rows = rows_total;
  be->ep_T = Tsh;
  mark(be, 0); mark(be, 1); mark(be, 2);
  if (n_chunks > 0) run_ffn(be, L, nmax, 0);
  mark(be, 3);
  if (n_chunks > 0) run_ffn(be, L, nmax, 1);
  mark(be, 4);
  if (n_segs > 0)
    be->launches += launch_segment_copy(be->obuf, reinterpret_cast<__nv_bfloat16*>(out_rows_dev), d_rev, n_segs,
                                        max_seg, c.hidden, s);
  mark(be, 5);
  CK(cudaGetLastError());
  return EK_OK;
}

int32_t ek_ep_combine(ek_backend_t* be, int32_t layer, const void* returned_rows_dev, int32_t T, void* y_dev) {
  if (!be || !returned_rows_dev || !y_dev) return EK_INVALID_INPUT;
  if (T < 1 || T > be->cfg.max_tokens) return fail(be, EK_INVALID_INPUT, "T=%d outside [1,%d]", T, be->cfg.max_tokens);
  cudaSetDevice(be->cfg.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  const ek_config_t& c = be->cfg;
  if (c.n_shared_experts > 0 && be->ep_T != T) return fail(be, EK_INVALID_INPUT, "ek_ep_ffn must run on the same tokens first");
  CombineParams cp;
  cp.obuf = reinterpret_cast<const __nv_bfloat16*>(returned_rows_dev);
  cp.inv = be->inv; cp.weights = be->weights; cp.y = reinterpret_cast<__nv_bfloat16*>(y_dev);
  cp.T = T; cp.k = c.top_k; cp.H = c.hidden; cp.n_shared = c.n_shared_experts; cp.Tk = T * c.top_k;
  cp.bf16_products = c.bf16_combine;
  cp.shared = be->obuf + (size_t)be->ep_rows * c.hidden;   // shared expert rows of the last ek_ep_ffn
  be->launches += launch_combine(cp, be->stream);
  CK(cudaGetLastError());
  return EK_OK;
}

// Expert parallelism without data-dependent exchange sizes (decode-sized batches): every rank
// holds all T_all tokens (all-gathered by the caller), routes them, runs ITS experts on the rows
// routed to them and leaves fp32 partial sums for all tokens; the caller sums the partials across
// ranks (reduce-scatter) and calls ek_ep_finish on its own token slice.
int32_t ek_ep_partial(ek_backend_t* be, int32_t layer, const void* x_all_dev, int32_t T_all, int32_t t0,
                      int32_t T_local, float* partial_dev) {
  if (!be || !x_all_dev || !partial_dev) return EK_INVALID_INPUT;
  const ek_config_t& c = be->cfg;
  if (T_all < 1 || T_all > c.max_tokens) return fail(be, EK_INVALID_INPUT, "T_all=%d outside [1,%d]", T_all, c.max_tokens);
  if (t0 < 0 || T_local < 0 || t0 + T_local > T_all) return fail(be, EK_INVALID_INPUT, "token slice outside the batch");
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  auto li = be->layers.find(layer);
  if (li == be->layers.end() || !li->second.router_w)
    return fail(be, EK_NOT_FOUND, "layer %d has no router weight registered", layer);
  LayerOpts opt;
  opt.sh_t0 = t0;
  opt.sh_T = T_local;
  opt.partial = partial_dev;
  be->ep_rows = T_all * c.top_k;   // shared rows start behind the routed rows
  be->ep_T = T_local;
  return run_layer(be, li->second, reinterpret_cast<const __nv_bfloat16*>(x_all_dev), T_all, c.top_k, nullptr,
                   nullptr, nullptr, opt);
}

int32_t ek_ep_finish(ek_backend_t* be, int32_t layer, const float* reduced_dev, int32_t T_local, void* y_dev) {
  (void)layer;
  if (!be || !reduced_dev || !y_dev) return EK_INVALID_INPUT;
  const ek_config_t& c = be->cfg;
  if (T_local < 1 || T_local > c.max_tokens) return fail(be, EK_INVALID_INPUT, "T_local out of range");
  if (c.n_shared_experts > 0 && be->ep_T != T_local) return fail(be, EK_INVALID_INPUT, "ek_ep_partial must run on the same slice first");
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  be->launches += launch_combine_finish(reduced_dev, be->obuf + (size_t)be->ep_rows * c.hidden, c.n_shared_experts,
                                        T_local, c.hidden, reinterpret_cast<__nv_bfloat16*>(y_dev), be->stream);
  CK(cudaGetLastError());
  return EK_OK;
}

// ---- expert parallel over peer memory ------------------------------------------------------------
namespace {
int check_peer_step(ek_backend* be, int T) {
  const ek_config_t& c = be->cfg;
  PeerTable& pt = be->peers;
  if (!pt.own[0]) return fail(be, EK_INVALID_INPUT, "ek_ep_peer_alloc has not been called");
  for (int r = 0; r < c.ep_size; ++r)
    if (!pt.xall[r]) return fail(be, EK_INVALID_INPUT, "rank %d's buffers have not been opened", r);
  if (T < 1 || T > pt.T_cap) return fail(be, EK_INVALID_INPUT, "T=%d outside [1,%d] (the size given to ek_ep_peer_alloc)", T, pt.T_cap);
  return EK_OK;
}
void free_peers(ek_backend* be) {
  PeerTable& pt = be->peers;
  for (int r = 0; r < EK_EP_MAX_RANKS; ++r) {
    if (pt.opened[r]) {
      cudaIpcCloseMemHandle(pt.xall[r]);
      cudaIpcCloseMemHandle(pt.partial[r]);
      cudaIpcCloseMemHandle(pt.flags[r]);
    }
    pt.opened[r] = false;
    pt.xall[r] = pt.partial[r] = pt.flags[r] = nullptr;
  }
}
}  // namespace

int32_t ek_ep_peer_alloc(ek_backend_t* be, int32_t tokens_per_rank, uint8_t* handles) {
  if (!be || !handles) return EK_INVALID_INPUT;
  const ek_config_t& c = be->cfg;
  static_assert(sizeof(cudaIpcMemHandle_t) == EK_IPC_HANDLE_BYTES, "IPC handle size");
  if (c.ep_size > EK_EP_MAX_RANKS) return fail(be, EK_UNSUPPORTED, "at most %d ranks", EK_EP_MAX_RANKS);
  if (tokens_per_rank < 1 || (int64_t)tokens_per_rank * c.ep_size > c.max_tokens)
    return fail(be, EK_INVALID_INPUT, "%d tokens per rank x %d ranks exceed max_tokens %d", tokens_per_rank, c.ep_size, c.max_tokens);
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  PeerTable& pt = be->peers;
  if (pt.own[0]) return fail(be, EK_INVALID_INPUT, "peer buffers exist already: destroy the backend to resize them");
  const size_t Ta = (size_t)tokens_per_rank * c.ep_size;
  const size_t bytes[3] = {2 * Ta * c.hidden * 2, 2 * Ta * c.hidden * 4, 2 * EK_EP_MAX_RANKS * 4};
  for (int i = 0; i < 3; ++i) {
    CK(cudaMalloc(&pt.own[i], bytes[i]));
    CK(cudaMemset(pt.own[i], 0, bytes[i]));
    cudaIpcMemHandle_t h;
    CK(cudaIpcGetMemHandle(&h, pt.own[i]));
    memcpy(handles + (size_t)i * EK_IPC_HANDLE_BYTES, &h, sizeof h);
  }
  CK(cudaDeviceSynchronize());
  pt.T_cap = tokens_per_rank;
  pt.xall[c.ep_rank] = pt.own[0];
  pt.partial[c.ep_rank] = pt.own[1];
  pt.flags[c.ep_rank] = pt.own[2];
  return EK_OK;
}

int32_t ek_ep_peer_open(ek_backend_t* be, int32_t rank, const uint8_t* handles) {
  if (!be || !handles) return EK_INVALID_INPUT;
  const ek_config_t& c = be->cfg;
  if (rank < 0 || rank >= c.ep_size || rank >= EK_EP_MAX_RANKS) return fail(be, EK_INVALID_INPUT, "rank %d outside the group", rank);
  if (rank == c.ep_rank) return EK_OK;   // the own buffers need no mapping
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  PeerTable& pt = be->peers;
  if (pt.opened[rank]) return fail(be, EK_INVALID_INPUT, "rank %d's buffers are open already", rank);
  void* ptrs[3] = {nullptr, nullptr, nullptr};
  for (int i = 0; i < 3; ++i) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)i * EK_IPC_HANDLE_BYTES, sizeof h);
    // opened with THIS device current: the runtime enables peer access to the owner's device
    const cudaError_t e = cudaIpcOpenMemHandle(&ptrs[i], h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      for (int j = 0; j < i; ++j) cudaIpcCloseMemHandle(ptrs[j]);
      return fail(be, EK_CUDA, "cudaIpcOpenMemHandle for rank %d: %s", rank, cudaGetErrorString(e));
    }
  }
  pt.xall[rank] = ptrs[0];
  pt.partial[rank] = ptrs[1];
  pt.flags[rank] = ptrs[2];
  pt.opened[rank] = true;
  return EK_OK;
}

int32_t ek_ep_peer_close(ek_backend_t* be) {
  if (!be) return EK_INVALID_INPUT;
  cudaSetDevice(be->cfg.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  cudaStreamSynchronize(be->stream);
  free_peers(be);
  return EK_OK;
}

int32_t ek_ep_peer_push(ek_backend_t* be, const void* x_dev, int32_t T, uint32_t step) {
  if (!be || !x_dev) return EK_INVALID_INPUT;
  int rc = check_peer_step(be, T);
  if (rc != EK_OK) return rc;
  const ek_config_t& c = be->cfg;
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  PeerTable& pt = be->peers;
  const int H = c.hidden;
  const size_t Ta = (size_t)T * c.ep_size;
  const size_t off = (size_t)(step & 1u) * Ta * H + (size_t)c.ep_rank * T * H;   // elements into a rank's xall
  be->launches += launch_ep_push(reinterpret_cast<const __nv_bfloat16*>(x_dev), T, H, pt.xall, pt.flags, c.ep_size, c.ep_rank,
                                 step + 1, off, be->ep_counters, be->stream);
  CK(cudaGetLastError());
  return EK_OK;
}

int32_t ek_ep_peer_partial(ek_backend_t* be, int32_t layer, int32_t T, uint32_t step) {
  if (!be) return EK_INVALID_INPUT;
  int rc = check_peer_step(be, T);
  if (rc != EK_OK) return rc;
  const ek_config_t& c = be->cfg;
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  auto li = be->layers.find(layer);
  if (li == be->layers.end() || !li->second.router_w)
    return fail(be, EK_NOT_FOUND, "layer %d has no router weight registered", layer);
  PeerTable& pt = be->peers;
  const int H = c.hidden;
  const size_t Ta = (size_t)T * c.ep_size;
  const size_t par = (size_t)(step & 1u) * Ta * H;
  uint32_t* my_flags = reinterpret_cast<uint32_t*>(pt.flags[c.ep_rank]);
  LayerOpts opt;
  opt.sh_t0 = c.ep_rank * T;
  opt.sh_T = T;
  opt.partial = reinterpret_cast<float*>(pt.partial[c.ep_rank]) + par;
  // the wait for the peers' tokens rides on the first kernel of the pass, the signal that the partial
  // sums are complete on the last one
  opt.wait.flags = my_flags; opt.wait.world = c.ep_size; opt.wait.step_no = step + 1; opt.wait.where = 500;
  PeerSignal sig;
  for (int r = 0; r < EK_EP_MAX_RANKS; ++r) sig.flags.p[r] = r < c.ep_size ? pt.flags[r] : nullptr;
  sig.world = c.ep_size; sig.slot = EK_EP_MAX_RANKS + c.ep_rank; sig.step_no = step + 1;
  sig.ticket = be->front_ticket + 1;
  opt.signal = &sig;
  be->ep_rows = (int)Ta * c.top_k;
  be->ep_T = T;
  rc = run_layer(be, li->second, reinterpret_cast<const __nv_bfloat16*>(pt.xall[c.ep_rank]) + par, (int)Ta, c.top_k, nullptr,
                 nullptr, nullptr, opt);
  if (rc != EK_OK) return rc;
  CK(cudaGetLastError());
  return EK_OK;
}

int32_t ek_ep_peer_finish(ek_backend_t* be, int32_t layer, int32_t T, uint32_t step, void* y_dev) {
  (void)layer;
  if (!be || !y_dev) return EK_INVALID_INPUT;
  int rc = check_peer_step(be, T);
  if (rc != EK_OK) return rc;
  const ek_config_t& c = be->cfg;
  const int H = c.hidden;
  if (c.n_shared_experts > 0 && be->ep_T != T) return fail(be, EK_INVALID_INPUT, "ek_ep_peer_partial must run on the same step first");
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  PeerTable& pt = be->peers;
  const size_t Ta = (size_t)T * c.ep_size;
  const size_t off = (size_t)(step & 1u) * Ta * H + (size_t)c.ep_rank * T * H;   // this rank's token slice in every partial
  const uint32_t* my_flags = reinterpret_cast<const uint32_t*>(pt.flags[c.ep_rank]) + EK_EP_MAX_RANKS;
  be->launches += launch_ep_pull_finish(pt.partial, off, c.ep_size, my_flags, step + 1,
                                        be->obuf + (size_t)be->ep_rows * c.hidden, c.n_shared_experts, T, H,
                                        reinterpret_cast<__nv_bfloat16*>(y_dev), be->status, be->stream);
  CK(cudaGetLastError());
  return EK_OK;
}

int32_t ek_ep_set_owners(ek_backend_t* be, int32_t layer, const int32_t* owners) {
  if (!be) return EK_INVALID_INPUT;
  const ek_config_t& c = be->cfg;
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  auto li = be->layers.find(layer);
  if (li == be->layers.end()) return fail(be, EK_EXPERT_NOT_FOUND, "layer %d holds no experts", layer);
  Layer& L = li->second;
  if (!owners) {
    L.has_owners = false;
    return EK_OK;
  }
  for (int e = 0; e < c.n_experts; ++e) {
    if (owners[e] < 0 || owners[e] >= c.ep_size)
      return fail(be, EK_INVALID_INPUT, "owner %d of expert %d outside [0,%d)", owners[e], e, c.ep_size);
    if (owners[e] == c.ep_rank && (L.host_slot_of[e] < 0 || !L.host_registered[L.host_slot_of[e]]))
      return fail(be, EK_EXPERT_NOT_FOUND, "expert %d is assigned to this rank but not registered here", e);
  }
  CK(cudaMemcpyAsync(L.owners, owners, sizeof(int32_t) * c.n_experts, cudaMemcpyHostToDevice, be->stream));
  CK(cudaStreamSynchronize(be->stream));   // `owners` may be pageable and reused by the caller
  L.has_owners = true;
  return EK_OK;
}

// ---- observability -----------------------------------------------------------------------------

int32_t ek_expert_counts(ek_backend_t* be, int32_t layer, int32_t* counts) {
  if (!be || !counts) return EK_INVALID_INPUT;
  cudaSetDevice(be->cfg.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  std::shared_lock<std::shared_mutex> g(be->reg_mu);
  auto li = be->layers.find(layer);
  if (li == be->layers.end() || !li->second.have_counts) return fail(be, EK_NOT_FOUND, "no forward has run on layer %d", layer);
  CK(cudaMemcpyAsync(counts, li->second.last_counts, sizeof(int32_t) * be->cfg.n_experts, cudaMemcpyDefault, be->stream));
  CK(cudaStreamSynchronize(be->stream));
  return EK_OK;
}

int32_t ek_last_routing(ek_backend_t* be, int32_t T, int32_t* ids, float* weights) {
  if (!be || (!ids && !weights)) return EK_INVALID_INPUT;
  const ek_config_t& c = be->cfg;
  if (T < 1 || T > c.max_tokens) return fail(be, EK_INVALID_INPUT, "T=%d outside [1,%d]", T, c.max_tokens);
  cudaSetDevice(c.device);
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  const size_t n = (size_t)T * c.top_k;
  if (ids) CK(cudaMemcpyAsync(ids, be->ids, n * 4, cudaMemcpyDefault, be->stream));
  if (weights) CK(cudaMemcpyAsync(weights, be->weights, n * 4, cudaMemcpyDefault, be->stream));
  CK(cudaStreamSynchronize(be->stream));
  return EK_OK;
}

int32_t ek_stage_timing_enable(ek_backend_t* be, int32_t on) {
  if (!be) return EK_INVALID_INPUT;
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  be->timing = on != 0;
  be->ev_pass = 0;
  return EK_OK;
}
int32_t ek_stage_times(ek_backend_t* be, float* ms) {
  if (!be || !ms) return EK_INVALID_INPUT;
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  for (int i = 0; i < EK_STAGE_COUNT; ++i) ms[i] = be->stage_ms[i];
  return EK_OK;
}
int64_t ek_kernel_launches(const ek_backend_t* be) { return be ? be->launches.load() : 0; }

int32_t ek_worker_batch_stats(ek_backend_t* be, int64_t* calls, int64_t* batches) {
  if (!be || !calls || !batches) return EK_INVALID_INPUT;
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  *calls = be->batched_calls;
  *batches = be->batched_launches;
  return EK_OK;
}

int32_t ek_set_precise_dequant(ek_backend_t* be, int32_t on) {
  if (!be) return EK_INVALID_INPUT;
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  be->precise = on != 0;
  return EK_OK;
}


int32_t ek_debug_set_ffn_impl(ek_backend_t* be, int32_t impl) {
  if (!be || impl < 0 || impl > 1) return EK_INVALID_INPUT;
  std::lock_guard<std::mutex> fg(be->fwd_mu);
  be->ffn_impl = impl;
  return EK_OK;
}

}  // extern "C"
