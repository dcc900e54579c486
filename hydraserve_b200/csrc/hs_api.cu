// C ABI of the sampler (include/hs_sampler.h): handle management, launch planning and
// the host-buffer convenience call.  No torch types, no exceptions across the boundary.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/hs_sampler.h"
#include "hs_common.cuh"
#include "hs_state.cuh"
#include "hs_row_kernel.cuh"
#include "hs_row_v3.cuh"
#include "hs_row_topk.cuh"
#include "hs_sharded.cuh"
#include "hs_row_bf16_kernel.cuh"
#include "hs_row_f32_topk.cuh"

namespace {

using hs::u64;

constexpr int kGreedyMaxChunks = 64;
constexpr int kMaxSplit = 4;  // CTAs per row on the candidate path
constexpr int kSideCapMax = 16384;  // side-list entries a CTA can keep in global scratch

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

struct Plan {
  int cluster;
  int slice;
  size_t smem;
  bool global_stage;
};

inline size_t align16(size_t v) { return (v + 15) & ~size_t(15); }

size_t fixed_smem(int cluster) {
  size_t off = align16(sizeof(hs::Exchange));
  off += sizeof(hs::Hist);
  off += (sizeof(u64) + sizeof(uint32_t)) * (hs::kBins / cluster);
  return align16(off);
}

}  // namespace

struct hs_sampler {
  int device = 0;
  int vocab_max = 0, slots_user = 0, slots_total = 0, unique_cap = 0, batch_max = 0;
  int sm_count = 0;
  int smem_optin = 0;
  int force_cluster = 0;
  int force_general = 0;  // route bf16 rows through the general (fp32-stage) kernel too
  int force_split = 0;    // CTAs per candidate row (0 = chosen per call)
  int force_csplit = 0;   // CTAs per counting row (0 = chosen per call)
  int token_draw = 1;     // near-flat counting rows draw by rejection on tokens
  int ctab_tables = 0;    // count tables the hand-over scratch holds
  uint32_t* ctab = nullptr;   // [ctab_tables, kCells]
  int2* crare = nullptr;      // [ctab_tables, kV3RareCap]
  int* crare_n = nullptr;     // [ctab_tables]
  int* count_ticket = nullptr;  // [batch_max]
  int resident_bf16 = 0;  // CTAs of the bf16 kernel that can be resident at once: CTAs per SM x SMs
  int2* side_pair = nullptr;  // [resident_bf16, side_cap] side lists too long for shared memory
  hs::ClassPacked* clist = nullptr;  // [resident_bf16, kCells] class list of the row a CTA works on
  int* scratch_busy = nullptr;  // [resident_bf16] which of those scratch sets are in use
  unsigned long long* split_lists = nullptr;  // [batch_max, kMaxSplit, kSplitCap]
  int* split_n = nullptr;
  int* split_ticket = nullptr;
  int side_cap = 0;
  unsigned long long* phase_clocks = nullptr;  // HS_CREATE_PHASE_CLOCKS: per-row phase timestamps
  hs::Pool pool{};
  u64* greedy_partials = nullptr;
  float* gstage = nullptr;  // global stand-in for the on-chip row copy (very wide rows only)
  size_t gstage_elems = 0;
  // device + pinned staging for the host-buffer call
  void* d_logits = nullptr;
  size_t d_logits_bytes = 0;
  hs_row_params* d_params = nullptr;
  hs_row_out* d_out = nullptr;
  int32_t* d_hist = nullptr;
  size_t d_hist_elems = 0;
  int32_t* d_offsets = nullptr;
  int32_t* d_slots = nullptr;
  hs_row_params* h_params = nullptr;  // pinned
  int32_t* h_small = nullptr;         // pinned: offsets[batch_max+1] then slots[batch_max]
  std::mutex mu;         // the staging buffers of hs_sample_host
  // Every launching call takes launch_mu, and work of one call is ordered after the previous
  // call's on the GPU (an event when the stream changed), because all calls share the
  // sampler's scratch memory and its histograms.
  std::mutex launch_mu;
  cudaEvent_t ev_done = nullptr;
  cudaStream_t last_stream = nullptr;
  bool have_last = false;
  size_t device_bytes = 0;
  unsigned long long launches = 0;
};

namespace {

// The text of the calling thread's last failure (calls may come from several threads).
thread_local char g_last_error[512] = "";

int fail(hs_sampler*, int code, const char* what, cudaError_t e = cudaSuccess) {
  if (e != cudaSuccess)
    std::snprintf(g_last_error, sizeof g_last_error, "%s: %s", what, cudaGetErrorString(e));
  else
    std::snprintf(g_last_error, sizeof g_last_error, "%s", what);
  return code;
}

#define HS_CUDA(h, call)                                              \
  do {                                                                \
    cudaError_t e_ = (call);                                          \
    if (e_ != cudaSuccess) return fail((h), HS_ERR_CUDA, #call, e_);  \
  } while (0)

// Holds the sampler for one call's launches: calls on one sampler are serialised on the host
// (the mutex) and on the GPU (a call on another stream than the previous one first waits for
// that one's work), so they may come from any thread on any stream.
struct Serial {
  hs_sampler* h;
  cudaStream_t stream;
  std::unique_lock<std::mutex> lock;
  cudaError_t status = cudaSuccess;
  Serial(hs_sampler* h_, cudaStream_t s) : h(h_), stream(s), lock(h_->launch_mu) {
    if (h->have_last && h->last_stream != stream) status = cudaStreamWaitEvent(stream, h->ev_done, 0);
  }
  // records the end of this call's work; call once, after the last launch
  cudaError_t done() {
    const cudaError_t e = cudaEventRecord(h->ev_done, stream);
    if (e == cudaSuccess) { h->last_stream = stream; h->have_last = true; }
    return e;
  }
};

template <class T>
bool dmalloc(hs_sampler* h, T** p, size_t bytes) {
  if (cudaMalloc(reinterpret_cast<void**>(p), bytes ? bytes : 1) != cudaSuccess) return false;
  h->device_bytes += bytes;
  return true;
}

bool make_plan(const hs_sampler* h, int vocab, Plan& p) {
  static const int sizes[4] = {1, 2, 4, 8};
  for (int k = 0; k < 4; ++k) {
    const int c = sizes[k];
    if (h->force_cluster && c != h->force_cluster) continue;
    const int slice = ((vocab + c - 1) / c + 7) & ~7;
    const size_t smem = fixed_smem(c) + (size_t)slice * sizeof(float);
    if (smem <= (size_t)h->smem_optin && slice <= hs::kMaxSliceElems) {
      p = Plan{c, slice, smem, false};
      return true;
    }
  }
  const int c = hs::kMaxCluster;
  const int slice = ((vocab + c - 1) / c + 7) & ~7;
  if (slice > hs::kMaxSliceElems) return false;
  p = Plan{c, slice, fixed_smem(c), true};
  return true;
}

int check_common(hs_sampler* h, const void* logits, int dtype, int batch, int vocab) {
  if (!h) return HS_ERR_INVALID;
  if (!logits && batch > 0) return fail(h, HS_ERR_INVALID, "logits is null");
  if (dtype != HS_DTYPE_F32 && dtype != HS_DTYPE_BF16) return fail(h, HS_ERR_INVALID, "unknown dtype");
  if (batch < 0 || vocab < 1) return fail(h, HS_ERR_INVALID, "batch must be >= 0 and vocab >= 1");
  if (vocab > h->vocab_max) return fail(h, HS_ERR_CAPACITY, "vocab exceeds vocab_max given to hs_create");
  if (batch > h->batch_max) return fail(h, HS_ERR_CAPACITY, "batch exceeds batch_max given to hs_create");
  return HS_OK;
}

int launch_rows(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch, int vocab,
                const hs_row_params* params, hs_row_out* out, const float* noise, float* scores_out,
                int32_t* tokens_out, uint32_t flags, cudaStream_t stream) {
  Plan plan;
  hs::RowKernelArgs a{};
  a.logits = logits; a.dtype = dtype; a.row_stride = row_stride; a.vocab = vocab; a.slice = 0;
  a.params = params; a.out = out; a.noise = noise; a.scores_out = scores_out; a.gstage = nullptr;
  a.pool = h->pool; a.flags = flags & HS_SAMPLE_APPEND_TOKEN; a.tokens_out = tokens_out;
  a.token_draw = h->token_draw;
  if (dtype == HS_DTYPE_BF16 && !h->force_general && !(flags & HS_SAMPLE_GENERAL_KERNEL)) {
    // One launch: a CTA per counting row and per part of a candidate row, two resident per
    // SM.  Small batches: several CTAs stream each candidate row so that every SM has work.
    // (as many CTAs per row as fit in one wave, rounded down: a second, partial wave costs more
    // than idle SMs in the first)
    int split = h->force_split ? h->force_split : h->resident_bf16 / batch;
    split = std::max(1, std::min(split, kMaxSplit));
    if (vocab < split * 2 * hs::kSample) split = 1;
    // counting rows: as many CTAs per row as the hand-over scratch allows (the whole batch may
    // be counting rows), so that a small batch still spreads over the SMs
    int csplit = 1;
    if (vocab >= 65536) {
      if ((long long)batch * 4 <= h->ctab_tables) csplit = 4;
      else if ((long long)batch * 2 <= h->ctab_tables) csplit = 2;
    }
    if (h->force_csplit && (long long)batch * h->force_csplit <= h->ctab_tables) csplit = h->force_csplit;
    hs::RowV3Args a3{a, h->clist, h->side_pair, h->side_cap, h->resident_bf16, h->scratch_busy, h->phase_clocks,
                     csplit, h->ctab, h->crare, h->crare_n, h->count_ticket,
                     split, h->split_lists, h->split_n, h->split_ticket, batch};
    const unsigned grid = (unsigned)batch * (unsigned)(csplit + split);
    hs::row_kernel_bf16<<<grid, hs::kThreads, hs::bf16_kernel_smem(), stream>>>(a3);
    HS_CUDA(h, cudaGetLastError());
    h->launches += 1;
    return HS_OK;
  }
  if (!make_plan(h, vocab, plan)) return fail(h, HS_ERR_CAPACITY, "vocabulary too wide for the row kernel");
  // fp32 rows with a small top_k: the candidate kernel, one CTA per row (the other rows' CTAs
  // leave at once); the general kernel below leaves those rows alone
  a.skip_candidate_rows = 0;
  if (dtype == HS_DTYPE_F32 && !h->force_general && !(flags & HS_SAMPLE_GENERAL_KERNEL)) {
    a.skip_candidate_rows = 1;
    hs::F32TopkArgs f{a, h->phase_clocks};
    hs::row_kernel_f32_topk<<<(unsigned)batch, hs::kThreads, hs::layout_cand().total, stream>>>(f);
    HS_CUDA(h, cudaGetLastError());
    h->launches += 1;
  }
  if (plan.global_stage) {
    const size_t need = (size_t)batch * plan.slice * plan.cluster;
    if (need > h->gstage_elems) return fail(h, HS_ERR_CAPACITY, "global stage too small for this batch x vocab");
  }
  a.slice = plan.slice;
  a.gstage = plan.global_stage ? h->gstage : nullptr;

  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)plan.cluster, (unsigned)batch, 1);
  cfg.blockDim = dim3(hs::kThreads, 1, 1);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)plan.cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  HS_CUDA(h, cudaLaunchKernelEx(&cfg, hs::row_kernel, a));
  h->launches += 1;
  return HS_OK;
}

int launch_greedy(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch, int vocab,
                  int32_t* tokens_out, cudaStream_t stream) {
  int chunks = (2 * h->sm_count + batch - 1) / batch;
  chunks = std::max(1, std::min(chunks, kGreedyMaxChunks));
  int chunk = ((vocab + chunks - 1) / chunks + 7) & ~7;
  chunks = (vocab + chunk - 1) / chunk;
  hs::greedy_partial_kernel<<<dim3((unsigned)chunks, (unsigned)batch), hs::kGreedyThreads, 0, stream>>>(
      logits, dtype, row_stride, vocab, chunk, h->greedy_partials);
  HS_CUDA(h, cudaGetLastError());
  hs::greedy_final_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(h->greedy_partials, chunks, batch, tokens_out);
  HS_CUDA(h, cudaGetLastError());
  h->launches += 2;
  return HS_OK;
}

int launch_append(hs_sampler* h, const int32_t* tokens, const int32_t* offsets, const int32_t* slots,
                  int n_slots, int vocab, int max_tokens, cudaStream_t stream) {
  if (n_slots == 0 || max_tokens <= 0) return HS_OK;
  const int threads = 256;
  int bx = std::max(1, std::min((max_tokens + threads - 1) / threads, 64));
  dim3 grid((unsigned)bx, (unsigned)n_slots);
  hs::slots_register_kernel<<<grid, threads, 0, stream>>>(h->pool, tokens, offsets, slots, n_slots, vocab);
  HS_CUDA(h, cudaGetLastError());
  hs::slots_count_kernel<<<grid, threads, 0, stream>>>(h->pool, tokens, offsets, slots, n_slots, vocab);
  HS_CUDA(h, cudaGetLastError());
  hs::slots_classify_kernel<<<grid, threads, 0, stream>>>(h->pool, tokens, offsets, slots, n_slots, vocab);
  HS_CUDA(h, cudaGetLastError());
  h->launches += 3;
  return HS_OK;
}

void release(hs_sampler* h) {
  cudaFree(h->pool.pairs); cudaFree(h->pool.cls); cudaFree(h->pool.heavy); cudaFree(h->pool.n_heavy); cudaFree(h->pool.n); cudaFree(h->pool.pos);
  cudaFree(h->side_pair); cudaFree(h->clist); cudaFree(h->scratch_busy);
  cudaFree(h->ctab); cudaFree(h->crare); cudaFree(h->crare_n); cudaFree(h->count_ticket);
  cudaFree(h->split_lists); cudaFree(h->split_n); cudaFree(h->split_ticket);
  if (h->ev_done) cudaEventDestroy(h->ev_done);
  cudaFree(h->phase_clocks);
  cudaFree(h->pool.error); cudaFree(h->greedy_partials); cudaFree(h->gstage); cudaFree(h->d_logits);
  cudaFree(h->d_params); cudaFree(h->d_out); cudaFree(h->d_hist); cudaFree(h->d_offsets); cudaFree(h->d_slots);
  if (h->h_params) cudaFreeHost(h->h_params);
  if (h->h_small) cudaFreeHost(h->h_small);
}

}  // namespace

// ---- hs_greedy_noalloc: arg max per row with its scratch in a fixed device array --------
namespace {

constexpr int kNoAllocMaxBatch = HS_NOALLOC_MAX_BATCH;
constexpr int kNoAllocChunks = 16;
constexpr int kNoAllocMaxDevices = 64;

// One partial result per (row, chunk).  Every GPU that loads this library holds these
// 128 KB until the process exits.  In host code this name is only a handle for
// cudaGetSymbolAddress; kernels get the device address obtained from it.
static __device__ __align__(256) unsigned long long g_noalloc_partials[kNoAllocMaxBatch * kNoAllocChunks];

struct NoAllocDevice {
  u64* partials = nullptr;  // device address of g_noalloc_partials on that GPU
  bool ready = false;
};
NoAllocDevice g_noalloc_devices[kNoAllocMaxDevices];
std::mutex g_noalloc_mu;
thread_local char g_noalloc_error[256] = "";

int noalloc_fail(int code, const char* what, cudaError_t e = cudaSuccess) {
  if (e != cudaSuccess)
    std::snprintf(g_noalloc_error, sizeof g_noalloc_error, "%s: %s", what, cudaGetErrorString(e));
  else
    std::snprintf(g_noalloc_error, sizeof g_noalloc_error, "%s", what);
  return code;
}

}  // namespace

extern "C" {

const char* hs_greedy_noalloc_error(void) { return g_noalloc_error; }

int hs_greedy_noalloc(const void* logits, int dtype, int64_t row_stride, int batch, int vocab,
                      int32_t* tokens_out, void* stream_) {
  g_noalloc_error[0] = 0;
  if (dtype != HS_DTYPE_F32 && dtype != HS_DTYPE_BF16) return noalloc_fail(HS_ERR_INVALID, "unknown dtype");
  if (batch < 0 || vocab < 1) return noalloc_fail(HS_ERR_INVALID, "batch must be >= 0 and vocab >= 1");
  if (batch > kNoAllocMaxBatch) {
    std::snprintf(g_noalloc_error, sizeof g_noalloc_error,
                  "batch %d exceeds HS_NOALLOC_MAX_BATCH (%d): split the call", batch, kNoAllocMaxBatch);
    return HS_ERR_CAPACITY;
  }
  if (batch == 0) return HS_OK;
  if (!logits || !tokens_out) return noalloc_fail(HS_ERR_INVALID, "logits / tokens_out is null");
  if (row_stride < vocab) return noalloc_fail(HS_ERR_INVALID, "row_stride smaller than vocab");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return noalloc_fail(HS_ERR_CUDA, "cudaGetDevice", e);
  if (dev < 0 || dev >= kNoAllocMaxDevices) return noalloc_fail(HS_ERR_CAPACITY, "device index beyond 63");
  u64* partials = nullptr;
  {
    // Set-up, once per device, with that device current: resolve the array's device address.
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    NoAllocDevice& d = g_noalloc_devices[dev];
    if (!d.ready) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_partials);
      if (e != cudaSuccess) return noalloc_fail(HS_ERR_CUDA, "cudaGetSymbolAddress(g_noalloc_partials)", e);
      d.partials = static_cast<u64*>(p);
      d.ready = true;
    }
    partials = d.partials;
  }
  cudaStream_t stream = (cudaStream_t)stream_;
  int chunks = kNoAllocChunks;
  int chunk = ((vocab + chunks - 1) / chunks + 7) & ~7;
  chunks = (vocab + chunk - 1) / chunk;
  // Every (row, chunk) slot that the final kernel reads is written by the partial kernel of
  // the same call, so nothing left over from an earlier call needs clearing.
  hs::greedy_partial_kernel<<<dim3((unsigned)chunks, (unsigned)batch), hs::kGreedyThreads, 0, stream>>>(
      logits, dtype, row_stride, vocab, chunk, partials);
  e = cudaGetLastError();
  if (e != cudaSuccess) return noalloc_fail(HS_ERR_CUDA, "greedy_partial_kernel launch", e);
  hs::greedy_final_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(partials, chunks, batch, tokens_out);
  e = cudaGetLastError();
  if (e != cudaSuccess) return noalloc_fail(HS_ERR_CUDA, "greedy_final_kernel launch", e);
  return HS_OK;
}

int hs_abi_version(void) { return 1; }

const char* hs_status_string(int status) {
  switch (status) {
    case HS_OK: return "ok";
    case HS_ERR_INVALID: return "invalid argument";
    case HS_ERR_CAPACITY: return "capacity exceeded";
    case HS_ERR_CUDA: return "CUDA error";
    case HS_ERR_UNSUPPORTED: return "unsupported";
    default: return "unknown status";
  }
}

const char* hs_last_error(hs_sampler* h) { return h ? g_last_error : "null sampler"; }

int hs_create(int device, int vocab_max, int slots_max, int unique_cap, int batch_max, hs_sampler** out) {
  return hs_create_ex(device, vocab_max, slots_max, unique_cap, batch_max, 0u, out);
}

int hs_create_ex(int device, int vocab_max, int slots_max, int hist_cap, int batch_max, uint32_t flags,
                 hs_sampler** out) {
  if (!out) return HS_ERR_INVALID;
  *out = nullptr;
  if (vocab_max < 1 || slots_max < 0 || batch_max < 1 || hist_cap < 0) return HS_ERR_INVALID;
  if (batch_max > 65535) return HS_ERR_CAPACITY;
  hs_sampler* h = new (std::nothrow) hs_sampler();
  if (!h) return HS_ERR_INVALID;
  DeviceGuard guard(device);
  if (!guard.ok) { delete h; return HS_ERR_CUDA; }
  h->device = device;
  h->vocab_max = vocab_max;
  h->slots_user = slots_max;
  h->slots_total = slots_max + batch_max;  // the tail serves per-call (stateless) histories
  h->unique_cap = hist_cap == 0 ? vocab_max : std::min(hist_cap, vocab_max);
  h->batch_max = batch_max;
  h->force_general = (flags & HS_CREATE_FORCE_GENERAL) ? 1 : 0;
  {
    const int v = (int)((flags >> 8) & 0xfu);
    if (v == 1 || v == 2 || v == 4 || v == 8) h->force_cluster = v;
  }
  auto bail = [&](int code) { release(h); delete h; return code; };
  if (cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return bail(HS_ERR_CUDA);
  if (cudaDeviceGetAttribute(&h->smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) return bail(HS_ERR_CUDA);
  if (cudaFuncSetAttribute(hs::row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, h->smem_optin) != cudaSuccess) return bail(HS_ERR_CUDA);
  if (cudaFuncSetAttribute(hs::row_kernel_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hs::bf16_kernel_smem()) != cudaSuccess) return bail(HS_ERR_CUDA);
  if (cudaFuncSetAttribute(hs::row_kernel_f32_topk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hs::layout_cand().total) != cudaSuccess) return bail(HS_ERR_CUDA);
  if (cudaFuncSetAttribute(hs::shard_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hs::layout_cand().total) != cudaSuccess) return bail(HS_ERR_CUDA);
  if (cudaFuncSetAttribute(hs::shard_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hs::layout_cand().total) != cudaSuccess) return bail(HS_ERR_CUDA);
  {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, hs::row_kernel_bf16, hs::kThreads,
                                                      hs::bf16_kernel_smem()) != cudaSuccess || per_sm < 1)
      return bail(HS_ERR_CUDA);
    h->resident_bf16 = per_sm * h->sm_count;
  }

  const size_t st = (size_t)h->slots_total;
  h->pool.slots_total = h->slots_total;
  h->pool.unique_cap = h->unique_cap;
  h->pool.pos_stride = vocab_max;
  h->pool.cls_stride = (vocab_max + 15) / 16 + 4;  // words; padded so 128-bit reads of the tail stay inside
  bool ok = true;
  ok = ok && dmalloc(h, &h->pool.pairs, st * h->unique_cap * sizeof(int2));
  ok = ok && dmalloc(h, &h->pool.n, st * sizeof(int32_t));
  ok = ok && dmalloc(h, &h->pool.n_heavy, st * sizeof(int32_t));
  ok = ok && dmalloc(h, &h->pool.heavy, st * h->unique_cap * sizeof(int32_t));
  ok = ok && dmalloc(h, &h->pool.cls, st * (size_t)h->pool.cls_stride * sizeof(uint32_t));
  ok = ok && dmalloc(h, &h->pool.pos, st * (size_t)vocab_max * sizeof(int32_t));
  ok = ok && dmalloc(h, &h->pool.error, sizeof(int32_t));
  ok = ok && dmalloc(h, &h->greedy_partials, (size_t)batch_max * kGreedyMaxChunks * sizeof(u64));
  ok = ok && dmalloc(h, &h->d_params, (size_t)batch_max * sizeof(hs_row_params));
  ok = ok && dmalloc(h, &h->d_out, (size_t)batch_max * sizeof(hs_row_out));
  ok = ok && dmalloc(h, &h->d_offsets, ((size_t)batch_max + 1) * sizeof(int32_t));
  ok = ok && dmalloc(h, &h->d_slots, (size_t)batch_max * sizeof(int32_t));
  // scratch of the bf16 kernel, per resident CTA (not per row of the batch)
  h->side_cap = std::min((vocab_max + 7) & ~7, kSideCapMax);
  ok = ok && dmalloc(h, &h->side_pair, (size_t)h->resident_bf16 * h->side_cap * sizeof(int2));
  ok = ok && dmalloc(h, &h->clist, (size_t)h->resident_bf16 * hs::kCells * sizeof(hs::ClassPacked));
  ok = ok && dmalloc(h, &h->scratch_busy, (size_t)h->resident_bf16 * sizeof(int));
  // hand-over scratch of counting rows split over several CTAs: two tables per resident CTA
  h->ctab_tables = 2 * h->resident_bf16;
  ok = ok && dmalloc(h, &h->ctab, (size_t)h->ctab_tables * hs::kCells * sizeof(uint32_t));
  ok = ok && dmalloc(h, &h->crare, (size_t)h->ctab_tables * hs::kV3RareCap * sizeof(int2));
  ok = ok && dmalloc(h, &h->crare_n, (size_t)h->ctab_tables * sizeof(int));
  ok = ok && dmalloc(h, &h->count_ticket, (size_t)batch_max * sizeof(int));
  ok = ok && cudaEventCreateWithFlags(&h->ev_done, cudaEventDisableTiming) == cudaSuccess;
  ok = ok && dmalloc(h, &h->split_lists, (size_t)batch_max * kMaxSplit * hs::kSplitCap * sizeof(unsigned long long));
  ok = ok && dmalloc(h, &h->split_n, (size_t)batch_max * kMaxSplit * sizeof(int));
  ok = ok && dmalloc(h, &h->split_ticket, (size_t)batch_max * sizeof(int));
  ok = ok && cudaMallocHost(&h->h_params, (size_t)batch_max * sizeof(hs_row_params)) == cudaSuccess;
  ok = ok && cudaMallocHost(&h->h_small, (2 * (size_t)batch_max + 1) * sizeof(int32_t)) == cudaSuccess;
  if (flags & HS_CREATE_PHASE_CLOCKS) {
    const size_t bytes = (size_t)batch_max * hs::kV3PhaseSlots * sizeof(unsigned long long);
    ok = ok && dmalloc(h, &h->phase_clocks, bytes);
    ok = ok && cudaMemset(h->phase_clocks, 0, bytes) == cudaSuccess;
  }
  if (!ok) return bail(HS_ERR_CUDA);
  ok = ok && cudaMemset(h->split_ticket, 0, (size_t)batch_max * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMemset(h->scratch_busy, 0, (size_t)h->resident_bf16 * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMemset(h->count_ticket, 0, (size_t)batch_max * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMemset(h->pool.n, 0, st * sizeof(int32_t)) == cudaSuccess;
  ok = ok && cudaMemset(h->pool.n_heavy, 0, st * sizeof(int32_t)) == cudaSuccess;
  ok = ok && cudaMemset(h->pool.cls, 0, st * (size_t)h->pool.cls_stride * sizeof(uint32_t)) == cudaSuccess;
  ok = ok && cudaMemset(h->pool.pos, 0, st * (size_t)vocab_max * sizeof(int32_t)) == cudaSuccess;
  ok = ok && cudaMemset(h->pool.error, 0, sizeof(int32_t)) == cudaSuccess;
  if (!ok) return bail(HS_ERR_CUDA);
  Plan plan;
  if (!make_plan(h, vocab_max, plan)) return bail(HS_ERR_CAPACITY);
  if (plan.global_stage) {
    h->gstage_elems = (size_t)batch_max * plan.slice * plan.cluster;
    if (!dmalloc(h, &h->gstage, h->gstage_elems * sizeof(float))) return bail(HS_ERR_CUDA);
  }
  if (cudaDeviceSynchronize() != cudaSuccess) return bail(HS_ERR_CUDA);
  *out = h;
  return HS_OK;
}

int hs_destroy(hs_sampler* h) {
  if (!h) return HS_ERR_INVALID;
  {
    DeviceGuard guard(h->device);
    cudaDeviceSynchronize();
    release(h);
  }
  delete h;
  return HS_OK;
}

int hs_slots_reset(hs_sampler* h, const int32_t* slots, int n_slots, void* stream) {
  if (!h || n_slots < 0 || (!slots && n_slots)) return HS_ERR_INVALID;
  if (n_slots == 0) return HS_OK;
  DeviceGuard guard(h->device);
  Serial serial(h, (cudaStream_t)stream);
  HS_CUDA(h, serial.status);
  hs::slots_reset_kernel<<<n_slots, 256, 0, (cudaStream_t)stream>>>(h->pool, slots, n_slots);
  HS_CUDA(h, cudaGetLastError());
  h->launches += 1;
  HS_CUDA(h, serial.done());
  return HS_OK;
}

int hs_slots_append(hs_sampler* h, const int32_t* tokens, const int32_t* offsets, const int32_t* slots,
                    int n_slots, int vocab, int max_tokens_per_slot, void* stream) {
  if (!h || n_slots < 0 || (n_slots && (!offsets || !slots))) return HS_ERR_INVALID;
  if (vocab < 1 || vocab > h->vocab_max) return fail(h, HS_ERR_CAPACITY, "vocab exceeds vocab_max");
  if (n_slots > 65535) return fail(h, HS_ERR_CAPACITY, "too many slots in one call");
  DeviceGuard guard(h->device);
  Serial serial(h, (cudaStream_t)stream);
  HS_CUDA(h, serial.status);
  const int rc = launch_append(h, tokens, offsets, slots, n_slots, vocab, max_tokens_per_slot, (cudaStream_t)stream);
  if (rc != HS_OK) return rc;
  HS_CUDA(h, serial.done());
  return HS_OK;
}

int hs_slot_unique_count(hs_sampler* h, int slot, void* stream, int* out) {
  if (!h || !out || slot < 0 || slot >= h->slots_total) return HS_ERR_INVALID;
  DeviceGuard guard(h->device);
  Serial serial(h, (cudaStream_t)stream);
  HS_CUDA(h, serial.status);
  int32_t v = 0;
  HS_CUDA(h, cudaMemcpyAsync(&v, h->pool.n + slot, sizeof v, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  HS_CUDA(h, cudaStreamSynchronize((cudaStream_t)stream));
  *out = v;
  return HS_OK;
}

int hs_sample(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch, int vocab,
              const hs_row_params* params, hs_row_out* out, const float* noise, float* scores_out,
              uint32_t flags, void* stream) {
  return hs_sample_ex(h, logits, dtype, row_stride, batch, vocab, params, out, noise, scores_out, nullptr,
                      flags, stream);
}

int hs_sample_ex(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch, int vocab,
                 const hs_row_params* params, hs_row_out* out, const float* noise, float* scores_out,
                 int32_t* tokens_out, uint32_t flags, void* stream) {
  int rc = check_common(h, logits, dtype, batch, vocab);
  if (rc != HS_OK) return rc;
  if (batch == 0) return HS_OK;
  if (!params || !out) return fail(h, HS_ERR_INVALID, "params / out is null");
  if (row_stride < vocab) return fail(h, HS_ERR_INVALID, "row_stride smaller than vocab");
  DeviceGuard guard(h->device);
  Serial serial(h, (cudaStream_t)stream);
  HS_CUDA(h, serial.status);
  rc = launch_rows(h, logits, dtype, row_stride, batch, vocab, params, out, noise, scores_out, tokens_out,
                   flags, (cudaStream_t)stream);
  if (rc != HS_OK) return rc;
  HS_CUDA(h, serial.done());
  return HS_OK;
}

int hs_greedy(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch, int vocab,
              int32_t* tokens_out, void* stream) {
  int rc = check_common(h, logits, dtype, batch, vocab);
  if (rc != HS_OK) return rc;
  if (batch == 0) return HS_OK;
  if (!tokens_out) return fail(h, HS_ERR_INVALID, "tokens_out is null");
  if (row_stride < vocab) return fail(h, HS_ERR_INVALID, "row_stride smaller than vocab");
  DeviceGuard guard(h->device);
  Serial serial(h, (cudaStream_t)stream);
  HS_CUDA(h, serial.status);
  rc = launch_greedy(h, logits, dtype, row_stride, batch, vocab, tokens_out, (cudaStream_t)stream);
  if (rc != HS_OK) return rc;
  HS_CUDA(h, serial.done());
  return HS_OK;
}

int hs_sample_host(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch, int vocab,
                   hs_row_params* params, hs_row_out* out, const int32_t* hist_tokens,
                   const int32_t* hist_offsets, uint32_t flags, void* stream_) {
  int rc = check_common(h, logits, dtype, batch, vocab);
  if (rc != HS_OK) return rc;
  if (batch == 0) return HS_OK;
  if (!params || !out) return fail(h, HS_ERR_INVALID, "params / out is null");
  if (row_stride < vocab) return fail(h, HS_ERR_INVALID, "row_stride smaller than vocab");
  cudaStream_t stream = (cudaStream_t)stream_;
  std::lock_guard<std::mutex> lock(h->mu);  // one user of the staging buffers at a time
  DeviceGuard guard(h->device);
  Serial serial(h, stream);
  HS_CUDA(h, serial.status);

  const size_t esz = dtype == HS_DTYPE_BF16 ? 2 : 4;
  const size_t need = (size_t)batch * vocab * esz;
  if (need > h->d_logits_bytes) {
    HS_CUDA(h, cudaStreamSynchronize(stream));
    cudaFree(h->d_logits);
    h->d_logits = nullptr;
    h->d_logits_bytes = 0;
    HS_CUDA(h, cudaMalloc(&h->d_logits, need));
    h->d_logits_bytes = need;
  }
  HS_CUDA(h, cudaMemcpy2DAsync(h->d_logits, (size_t)vocab * esz, logits, (size_t)row_stride * esz,
                               (size_t)vocab * esz, (size_t)batch, cudaMemcpyHostToDevice, stream));

  // Rows marked slot == -2 are penalised with the history passed in this call: it is
  // counted into a per-row scratch slot on the device (the reference's stateless form).
  int32_t* h_offsets = h->h_small;
  int32_t* h_slots = h->h_small + (h->batch_max + 1);
  int n_temp = 0;
  int max_len = 0;
  long long total = 0;
  for (int r = 0; r < batch; ++r) {
    h->h_params[r] = params[r];
    if (params[r].slot == -2) {
      if (!hist_tokens || !hist_offsets) return fail(h, HS_ERR_INVALID, "slot -2 needs hist_tokens / hist_offsets");
      const int len = hist_offsets[r + 1] - hist_offsets[r];
      if (len < 0) return fail(h, HS_ERR_INVALID, "hist_offsets must not decrease");
      h_slots[n_temp] = h->slots_user + r;
      h->h_params[r].slot = h->slots_user + r;
      ++n_temp;
      max_len = std::max(max_len, len);
      total += len;
    } else if (params[r].slot >= h->slots_user || params[r].slot < -2) {
      return fail(h, HS_ERR_INVALID, "params.slot out of range");
    }
  }
  if (n_temp) {
    if ((size_t)total > h->d_hist_elems) {
      HS_CUDA(h, cudaStreamSynchronize(stream));
      cudaFree(h->d_hist);
      h->d_hist = nullptr;
      h->d_hist_elems = 0;
      HS_CUDA(h, cudaMalloc(&h->d_hist, (size_t)total * sizeof(int32_t)));
      h->d_hist_elems = (size_t)total;
    }
    // The append kernels index offsets by position in `slots`, so the participants'
    // tokens are packed back to back.
    long long cursor = 0;
    std::vector<int32_t> packed;
    packed.reserve((size_t)total);
    int idx = 0;
    for (int r = 0; r < batch; ++r) {
      if (params[r].slot != -2) continue;
      h_offsets[idx++] = (int32_t)cursor;
      const int b = hist_offsets[r], e = hist_offsets[r + 1];
      packed.insert(packed.end(), hist_tokens + b, hist_tokens + e);
      cursor += e - b;
    }
    h_offsets[idx] = (int32_t)cursor;
    if (cursor) HS_CUDA(h, cudaMemcpyAsync(h->d_hist, packed.data(), (size_t)cursor * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
    HS_CUDA(h, cudaMemcpyAsync(h->d_offsets, h_offsets, ((size_t)n_temp + 1) * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
    HS_CUDA(h, cudaMemcpyAsync(h->d_slots, h_slots, (size_t)n_temp * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
    if (cursor) HS_CUDA(h, cudaStreamSynchronize(stream));  // `packed` is pageable and about to go away
    hs::slots_reset_kernel<<<n_temp, 256, 0, stream>>>(h->pool, h->d_slots, n_temp);
    HS_CUDA(h, cudaGetLastError());
    h->launches += 1;
    rc = launch_append(h, h->d_hist, h->d_offsets, h->d_slots, n_temp, vocab, max_len, stream);
    if (rc != HS_OK) return rc;
  }
  HS_CUDA(h, cudaMemcpyAsync(h->d_params, h->h_params, (size_t)batch * sizeof(hs_row_params), cudaMemcpyHostToDevice, stream));
  rc = launch_rows(h, h->d_logits, dtype, vocab, batch, vocab, h->d_params, h->d_out, nullptr, nullptr, nullptr, flags, stream);
  if (rc != HS_OK) return rc;
  HS_CUDA(h, cudaMemcpyAsync(out, h->d_out, (size_t)batch * sizeof(hs_row_out), cudaMemcpyDeviceToHost, stream));
  HS_CUDA(h, serial.done());
  HS_CUDA(h, cudaStreamSynchronize(stream));
  return HS_OK;
}

int hs_sharded_partial(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch,
                       int vocab_local, int vocab_offset, const hs_row_params* params,
                       hs_shard_rec* recs_out, void* stream) {
  int rc = check_common(h, logits, dtype, batch, vocab_local);
  if (rc != HS_OK) return rc;
  if (dtype != HS_DTYPE_BF16) return fail(h, HS_ERR_UNSUPPORTED, "sharded sampling takes bf16 slices");
  if (batch == 0) return HS_OK;
  if (!params || !recs_out) return fail(h, HS_ERR_INVALID, "params / recs_out is null");
  if (row_stride < vocab_local || vocab_offset < 0) return fail(h, HS_ERR_INVALID, "bad row_stride / vocab_offset");
  DeviceGuard guard(h->device);
  hs::ShardArgs a{};
  a.base.logits = logits; a.base.dtype = dtype; a.base.row_stride = row_stride; a.base.vocab = vocab_local;
  a.base.params = params; a.base.pool = h->pool;
  a.vocab_offset = vocab_offset;
  a.recs = recs_out;
  Serial serial(h, (cudaStream_t)stream);
  HS_CUDA(h, serial.status);
  hs::shard_partial_kernel<<<(unsigned)batch, hs::kThreads, hs::layout_cand().total, (cudaStream_t)stream>>>(a);
  HS_CUDA(h, cudaGetLastError());
  h->launches += 1;
  HS_CUDA(h, serial.done());
  return HS_OK;
}

int hs_sharded_merge(hs_sampler* h, const hs_shard_rec* recs, int ranks, int batch, int vocab_total,
                     const hs_row_params* params, hs_row_out* out, const float* noise, float* full_lse,
                     void* stream) {
  if (!h) return HS_ERR_INVALID;
  if (batch < 0 || ranks < 1 || ranks > 64 || vocab_total < 1) return fail(h, HS_ERR_INVALID, "bad ranks / batch / vocab_total");
  if (ranks * HS_SHARD_CAND > hs::kCandCap) return fail(h, HS_ERR_CAPACITY, "too many ranks for one merge");
  if (batch == 0) return HS_OK;
  if (!recs || !params || !out) return fail(h, HS_ERR_INVALID, "recs / params / out is null");
  DeviceGuard guard(h->device);
  hs::MergeArgs a{recs, ranks, batch, vocab_total, params, out, noise, full_lse};
  Serial serial(h, (cudaStream_t)stream);
  HS_CUDA(h, serial.status);
  hs::shard_merge_kernel<<<(unsigned)batch, hs::kThreads, hs::layout_cand().total, (cudaStream_t)stream>>>(a);
  HS_CUDA(h, cudaGetLastError());
  h->launches += 1;
  HS_CUDA(h, serial.done());
  return HS_OK;
}

int hs_debug_phase_clocks(hs_sampler* h, int batch, unsigned long long* out_host) {
  if (!h || !out_host || batch < 0 || batch > h->batch_max) return HS_ERR_INVALID;
  if (!h->phase_clocks) return fail(h, HS_ERR_UNSUPPORTED, "create the sampler with HS_CREATE_PHASE_CLOCKS");
  DeviceGuard guard(h->device);
  HS_CUDA(h, cudaMemcpy(out_host, h->phase_clocks, (size_t)batch * hs::kV3PhaseSlots * sizeof(unsigned long long),
                        cudaMemcpyDeviceToHost));
  return HS_OK;
}

int hs_debug_set(hs_sampler* h, int what, int value) {
  if (!h) return HS_ERR_INVALID;
  std::lock_guard<std::mutex> lock(h->launch_mu);
  if (what == 0) {
    if (value != 0 && value != 1 && value != 2 && value != 4) return fail(h, HS_ERR_INVALID, "split must be 0, 1, 2 or 4");
    h->force_split = value;
    return HS_OK;
  }
  if (what == 1) {
    if (value != 0 && value != 1 && value != 2 && value != 4) return fail(h, HS_ERR_INVALID, "counting split must be 0, 1, 2 or 4");
    h->force_csplit = value;
    return HS_OK;
  }
  if (what == 3) {
    h->token_draw = value ? 1 : 0;
    return HS_OK;
  }
  return fail(h, HS_ERR_INVALID, "unknown setting");
}

int hs_query(hs_sampler* h, int what, int vocab, int dtype) {
  if (!h) return HS_ERR_INVALID;
  Plan plan;
  const bool v3 = dtype == HS_DTYPE_BF16 && !h->force_general;
  switch (what) {
    case 0: return v3 ? 1 : (make_plan(h, vocab, plan) ? plan.cluster : HS_ERR_CAPACITY);
    case 1: return v3 ? 0 : (make_plan(h, vocab, plan) ? (plan.global_stage ? 0 : 1) : HS_ERR_CAPACITY);
    case 4: return v3 ? 1 : 0;
    case 2: return h->sm_count;
    case 3: return (int)(h->launches & 0x7fffffffull);
    case 5: return (int)std::min<size_t>(h->device_bytes >> 10, 0x7fffffffu);
    case 6: {
      const size_t per_slot = (size_t)h->unique_cap * (sizeof(int2) + sizeof(int32_t)) +
                              (size_t)h->pool.cls_stride * sizeof(uint32_t) + (size_t)h->vocab_max * sizeof(int32_t) +
                              2 * sizeof(int32_t);
      return (int)std::min<size_t>(per_slot, 0x7fffffffu);
    }
    case 7: return h->resident_bf16;
    case 8: {
      // the flag the append kernels raise when a histogram is asked to hold more distinct ids
      // than hist_cap (those ids were not counted); waits for the device
      DeviceGuard guard(h->device);
      int32_t raised = 0;
      HS_CUDA(h, cudaDeviceSynchronize());
      HS_CUDA(h, cudaMemcpy(&raised, h->pool.error, sizeof raised, cudaMemcpyDeviceToHost));
      return raised ? 1 : 0;
    }
    default: return HS_ERR_INVALID;
  }
}

}  // extern "C"
