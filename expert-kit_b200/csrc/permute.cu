// Bucketing: exclusive scan of the per-expert histogram, stable ranking of the flattened
// [T*k] assignments by expert (ascending token order inside an expert), the inverse map, the
// chunk work list for the grouped GEMMs and the row gather.
//
// Semantics follow NaiveExecutor::break_down_to_egress / assemble_seq_tensors
// (ek-computation/src/controller/executor.rs:283-299,112-133): a stable counting sort.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "ek_internal.h"
#include "bucket.cuh"

namespace ek {

namespace {

// One CTA per expert: offsets[e] = sum of counts of local experts below e, then one ordered
// pass over all assignments, ranking the matches with warp scans.
// With a work list to build (`with_worklist`), the CTA that finishes last does that too: one launch less.
__global__ void __launch_bounds__(256) permute_kernel(const __grid_constant__ PermuteWorklistParams pw) {
  const PermuteParams& p = pw.permute;
  pdl_wait();
  pdl_trigger();
  __shared__ int s_red[8];
  __shared__ int s_base;
  __shared__ int s_last;
  const int e = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // experts this rank serves in this pass: its window, or whatever the owner table says
  auto is_local = [&](int j) { return p.owners ? p.owners[j] == p.rank : (j >= p.e_lo && j < p.e_hi); };
  const bool local = is_local(e);

  // exclusive prefix over the local experts below e
  int part = 0;
  if (p.owners) {
    for (int j = tid; j < e; j += 256) part += is_local(j) ? p.counts[j] : 0;
  } else {
    for (int j = p.e_lo + tid; j < min(e, p.e_hi); j += 256) part += p.counts[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) s_red[warp] = part;
  __syncthreads();
  if (tid == 0) {
    int b = 0;
    for (int w = 0; w < 8; ++w) b += s_red[w];
    s_base = b;
    p.offsets[e] = b;
    if (e == p.E - 1) p.offsets[p.E] = b + (local ? p.counts[e] : 0);
  }
  __syncthreads();
  int running = s_base;
  const int n = p.T * p.k;
  const bool empty = p.counts[e] == 0;

  for (int base = 0; base < (empty ? 0 : n); base += 1024) {
    const int i0 = base + tid * 4;
    int id[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) id[j] = (i0 + j < n) ? p.ids[i0 + j] : -1;
    int c = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) c += (id[j] == e);
    // inclusive warp scan
    int inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int v = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += v;
    }
    __syncthreads();  // protects s_red from the previous round
    if (lane == 31) s_red[warp] = inc;
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      int v = s_red[w];
      if (w < warp) before += v;
      total += v;
    }
    int pos = running + before + inc - c;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (id[j] == e) {
        if (local) {
          p.perm[pos] = i0 + j;
          p.inv[i0 + j] = pos;
          ++pos;
        } else {
          p.inv[i0 + j] = -1;
        }
      }
    }
    running += total;
  }
  if (!pw.with_worklist) return;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned t = atomicAdd(pw.ticket, 1u);
    s_last = t == gridDim.x - 1;
    if (s_last) *pw.ticket = 0;              // launches on one stream do not overlap
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  build_worklist<256>(pw.worklist);
}

// xp[r,:] = x[perm[r] / k, :] for permuted rows, then (optionally) a straight copy of x for
// the shared expert.  16-byte vectors; F16: the rows are written as f16.
template <bool F16>
__global__ void __launch_bounds__(128) gather_kernel(const __nv_bfloat16* __restrict__ x,
                                                     const int32_t* __restrict__ perm,
                                                     const int32_t* __restrict__ n_routed,
                                                     __nv_bfloat16* __restrict__ xp, int32_t T,
                                                     int32_t k, int32_t H, int32_t shared_t0) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int Tk = T * k;
  int src;
  if (r < Tk) {
    if (r >= *n_routed) return;   // rows of non-local experts are not materialised
    src = perm[r] / k;
  } else {
    src = shared_t0 + r - Tk;     // the shared expert's tokens: a slice of x starting at shared_t0
  }
  const uint4* s = reinterpret_cast<const uint4*>(x + (size_t)src * H);
  uint4* d = reinterpret_cast<uint4*>(xp + (size_t)r * H);
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) d[v] = F16 ? bf16x8_to_f16x8(s[v]) : s[v];
}

__global__ void __launch_bounds__(128) rows_to_f16_kernel(__nv_bfloat16* rows, int32_t H) {
  uint4* d = reinterpret_cast<uint4*>(rows + (size_t)blockIdx.x * H);
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) d[v] = bf16x8_to_f16x8(d[v]);
}

}  // namespace

int launch_permute(const PermuteParams& p, cudaStream_t s) {
  PermuteWorklistParams pw;
  pw.permute = p;
  pw.with_worklist = 0;
  if (p.E > 0) launch_pdl(permute_kernel, dim3(p.E), dim3(256), 0, s, pw);
  return 1;
}

int launch_permute_worklist(const PermuteParams& p, const WorklistParams& w, uint32_t* ticket, cudaStream_t s) {
  PermuteWorklistParams pw;
  pw.permute = p;
  pw.worklist = w;
  pw.ticket = ticket;
  pw.with_worklist = 1;
  launch_pdl(permute_kernel, dim3(p.E), dim3(256), 0, s, pw);
  return 1;
}

int launch_gather(const __nv_bfloat16* x, const int32_t* perm, const int32_t* n_routed,
                  __nv_bfloat16* xp, int32_t T, int32_t k, int32_t H, int32_t shared_t0, int32_t shared_T,
                  bool to_f16, cudaStream_t s) {
  const int rows = T * k + shared_T;
  if (rows > 0) {
    if (to_f16) launch_pdl(gather_kernel<true>, dim3(rows), dim3(128), 0, s, x, perm, n_routed, xp, T, k, H, shared_t0);
    else launch_pdl(gather_kernel<false>, dim3(rows), dim3(128), 0, s, x, perm, n_routed, xp, T, k, H, shared_t0);
  }
  return rows > 0 ? 1 : 0;
}

int launch_rows_to_f16(__nv_bfloat16* rows, int64_t n_rows, int32_t H, cudaStream_t s) {
  if (n_rows > 0) rows_to_f16_kernel<<<(unsigned)n_rows, 128, 0, s>>>(rows, H);
  return n_rows > 0 ? 1 : 0;
}

}  // namespace ek

// =============================================================================================
// Bucketing for callers that may not allocate device memory.
//
// Some hosts of this library are not allowed to call cudaMalloc at all: a worker whose device
// memory is carved up front by its own pool and handed out by offset, or a plugin that runs
// inside another runtime's step function where an allocation would synchronise the device or
// break that runtime's memory accounting.  For them the bucketing step is offered in a form
// that owns no handle and allocates nothing: its scratch (the inverse map the ranking kernel
// writes, and the device status word) lives in a file-scope array that every GPU loading this
// library holds until the process exits.
//
// Host code cannot use the array's name as a device address; its address is looked up once per
// device with cudaGetSymbolAddress while that device is current (the first call on a device does
// it).  Every call reads the device status word back and synchronises the stream before it
// returns, so no call may be made on a stream that is being captured.
// All calls share the one array: two calls whose kernels overlap on the same GPU race on it.
// =============================================================================================
namespace {

constexpr int kNoAllocMaxAssignments = EK_NOALLOC_MAX_ASSIGNMENTS;
constexpr int kNoAllocStatusOffset = kNoAllocMaxAssignments * (int)sizeof(int32_t);
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) unsigned char g_bucket_scratch[kNoAllocStatusOffset + 256];

std::mutex g_noalloc_mu;
void* g_noalloc_ptr[kNoAllocMaxDevices] = {};

void noalloc_msg(char* buf, size_t cap, const char* fmt, ...) {
  if (!buf || cap == 0) return;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, cap, fmt, ap);
  va_end(ap);
}

}  // namespace

extern "C" int32_t ek_bucket_noalloc(const int32_t* ids_dev, int32_t T, int32_t k, int32_t n_experts,
                                     int32_t* counts_dev, int32_t* offsets_dev, int32_t* perm_dev,
                                     void* cuda_stream, char* errbuf, size_t errcap) {
  using namespace ek;
  if (!ids_dev || !counts_dev || !offsets_dev || !perm_dev) {
    noalloc_msg(errbuf, errcap, "null pointer argument");
    return EK_INVALID_INPUT;
  }
  if (T < 1 || k < 1 || n_experts < 1 || n_experts > 1024) {
    noalloc_msg(errbuf, errcap, "T, k must be positive and n_experts in [1,1024]");
    return EK_INVALID_INPUT;
  }
  if ((int64_t)T * k > kNoAllocMaxAssignments) {
    noalloc_msg(errbuf, errcap, "T*k = %lld exceeds the built-in scratch of %d assignments",
                (long long)T * k, kNoAllocMaxAssignments);
    return EK_INVALID_INPUT;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) {
    noalloc_msg(errbuf, errcap, "no current CUDA device");
    return EK_CUDA;
  }
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> g(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
      // once per device, with that device current
      cudaError_t e = cudaGetSymbolAddress(&g_noalloc_ptr[dev], g_bucket_scratch);
      if (e != cudaSuccess) {
        g_noalloc_ptr[dev] = nullptr;
        noalloc_msg(errbuf, errcap, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        return EK_CUDA;
      }
    }
    scratch = g_noalloc_ptr[dev];
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
  int32_t* inv = reinterpret_cast<int32_t*>(scratch);
  DevStatus* st = reinterpret_cast<DevStatus*>(reinterpret_cast<unsigned char*>(scratch) + kNoAllocStatusOffset);
  // the array keeps the previous call's contents: the status word must start at zero
  cudaError_t e = cudaMemsetAsync(st, 0, sizeof(DevStatus), s);
  if (e == cudaSuccess) {
    launch_histogram(ids_dev, T * k, n_experts, counts_dev, st, s);   // zeroes counts itself
    PermuteParams pp;
    pp.ids = ids_dev; pp.counts = counts_dev; pp.offsets = offsets_dev; pp.perm = perm_dev; pp.inv = inv;
    pp.T = T; pp.k = k; pp.E = n_experts; pp.e_lo = 0; pp.e_hi = n_experts;
    launch_permute(pp, s);
    e = cudaGetLastError();
  }
  DevStatus host_st = {0, 0, 0, 0};
  if (e == cudaSuccess) e = cudaMemcpyAsync(&host_st, st, sizeof host_st, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    noalloc_msg(errbuf, errcap, "CUDA failure: %s", cudaGetErrorString(e));
    return EK_CUDA;
  }
  if (host_st.code != DEV_OK) {
    noalloc_msg(errbuf, errcap, "assignment %d names expert %d, outside [0,%d)", host_st.aux0, host_st.aux1, n_experts);
    return EK_BOUNDS;
  }
  return EK_OK;
}
