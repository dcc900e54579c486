// The fused per-row sampling kernel (general path).
//
// One thread-block cluster owns one logits row.  The row is read from HBM once with
// 128-bit loads, widened to fp32 and kept on chip, a slice per CTA, for the rest of the
// kernel (a global scratch slice stands in when the row is too wide for the cluster's
// shared memory).  Everything after the load works on that resident copy:
//
//   penalties    scatter from the row's sparse (token id, count) list into the slices
//                (distributed shared memory), three separately rounded fp32 steps
//   temperature  true fp32 division, written back; row max / argmax in the same pass
//   top-k        radix descent over order-preserving keys by COUNT (ties at the k-th kept)
//   min-p        threshold test in probability space, relative to the top-k soft-max
//   top-p        radix descent by probability MASS (bucketed prefix sums), ties at the cut
//                resolved towards the lowest token ids
//   draw         Philox4x32-10 inverse CDF over exact integer masses, or the supplied
//                Exp(1) variates (arg max of p / q)
//   logprobs     log soft-max over the kept set, top-N by another count descent
//
// Probability mass is an integer multiple of 2^-40 (hs::mass_of), so every sum is exact
// and independent of accumulation order: the same row always yields the same cut.
#pragma once

#include "hs_common.cuh"
#include "hs_select.cuh"
#include "hs_state.cuh"
#include "../../include/hs_sampler.h"

namespace hs {

struct RowKernelArgs {
  const void* logits;
  int dtype;
  long long row_stride;
  int vocab;
  int slice;            // elements per CTA slice (multiple of 8)
  const hs_row_params* params;
  hs_row_out* out;
  const float* noise;   // [batch, vocab] or null
  float* scores_out;    // [batch, vocab] or null
  float* gstage;        // [batch, slice * cluster] global stage, or null = shared memory
  Pool pool;            // token-count histograms
  uint32_t flags;
  int32_t* tokens_out;  // [batch] or null: the sampled ids once more, as the next step's input ids
  int skip_candidate_rows;  // the general kernel leaves rows with 0 < top_k <= 256 to the fp32 candidate kernel
  int token_draw;       // bf16 counting rows draw near-flat rows by rejection on tokens (tuning / test switch)
};

struct RowCtx : ClusterCtx {
  int row;
  int vocab;
  int slice;
  int base;      // global index of the first element of this CTA's slice
  int n_local;   // elements in this CTA's slice
  int seg;       // elements per warp in the id-ordered walks (multiple of 32)
  float* stage;  // this CTA's slice
  float* smem_stage;
  float* gstage_row;

  __device__ __forceinline__ float* slice_of(unsigned r) {
    if (gstage_row) return gstage_row + (size_t)r * slice;
    return nranks > 1 ? cluster.map_shared_rank(smem_stage, r) : smem_stage;
  }
};

// Every element of the resident fp32 row, for descend_core.
template <bool WITH_MASS>
struct StageFill {
  const float* stage;
  int n_local;
  float m;
  template <class Add>
  __device__ __forceinline__ void operator()(int level, int shift, int bits, uint32_t prefix,
                                             uint32_t lo_key, const Add& add) const {
    const uint32_t mask = (1u << bits) - 1u;
    for (int i0 = threadIdx.x & ~31; i0 < n_local; i0 += kThreads) {
      const int i = i0 + (threadIdx.x & 31);
      bool valid = i < n_local;
      float s = 0.f;
      uint32_t k = 0;
      if (valid) {
        s = stage[i];
        k = key_of(s);
        valid = k >= lo_key && (level == 0 || (k >> (shift + bits)) == prefix);
      }
      add(valid, (k >> shift) & mask, 1u, (WITH_MASS && valid) ? mass_of(s, m) : 0ull);
    }
  }
};

template <bool BY_MASS, bool WITH_MASS>
__device__ Selection descend(RowCtx& c, uint32_t lo_key, u64 target_cnt, float top_p, float m) {
  StageFill<WITH_MASS> fill{c.stage, c.n_local, m};
  return descend_core<BY_MASS, WITH_MASS>(c, fill, lo_key, target_cnt, top_p);
}

// Count and mass of all elements with key >= lo_key, cluster wide.
__device__ void totals_above(RowCtx& c, uint32_t lo_key, float m, bool with_mass, u64& cnt, u64& mass) {
  u64 a = 0, b = 0;
  for (int i = threadIdx.x; i < c.n_local; i += kThreads) {
    const float s = c.stage[i];
    if (key_of(s) >= lo_key) {
      ++a;
      if (with_mass) b += mass_of(s, m);
    }
  }
  block_sum2(*c.x, a, b);
  u64 vals[2] = {a, b};
  u64 all[kMaxCluster][2];
  cluster_allgather<2>(c.cluster, *c.x, vals, all);
  cnt = mass = 0;
  for (unsigned r = 0; r < c.nranks; ++r) { cnt += all[r][0]; mass += all[r][1]; }
}

constexpr int kCandidateTopKMax = 256;  // largest top_k the candidate paths serve

struct KeptSet {
  uint32_t cut_key;  // kept: key > cut_key, or key == cut_key and global id <= tie_limit
  int tie_limit;
  __device__ __forceinline__ bool has(uint32_t k, int gid) const {
    return k > cut_key || (k == cut_key && gid <= tie_limit);
  }
};

// Global id of the t-th (1-based) element, in ascending id order, whose key equals `key`.
__device__ int find_tth_equal(RowCtx& c, uint32_t key, u64 t) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w0 = warp * c.seg;
  const int w1 = min(w0 + c.seg, c.n_local);
  u64 mine = 0;
  for (int i = w0 + lane; i < w1; i += 32) mine += key_of(c.stage[i]) == key;
  const u64 wtot = warp_sum_u64(mine);
  u64 pre, pre_unused, tot, tot_unused;
  block_warp_prefix2(*c.x, wtot, 0, pre, pre_unused, tot, tot_unused);
  u64 vals[1] = {tot};
  u64 all[kMaxCluster][1];
  cluster_allgather<1>(c.cluster, *c.x, vals, all);
  u64 cta_pre = 0;
  for (unsigned r = 0; r < c.rank; ++r) cta_pre += all[r][0];
  if (threadIdx.x == 0) c.x->bcast[6] = 0;
  __syncthreads();
  const u64 before = cta_pre + pre;
  if (before < t && t <= before + wtot) {  // this warp holds the t-th
    u64 running = before;
    for (int i0 = w0; i0 < w1; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < w1 && key_of(c.stage[i]) == key;
      const uint32_t ballot = __ballot_sync(0xffffffffu, hit);
      const u64 n = __popc(ballot);
      if (running + n >= t) {
        const int nth = (int)(t - running);  // 1-based among set bits
        const int pos = __fns(ballot, 0, nth);
        if (lane == 0) c.x->bcast[6] = (u64)(c.base + i0 + pos) + 1;
        break;
      }
      running += n;
    }
  }
  __syncthreads();
  u64 v2[1] = {c.x->bcast[6]};
  cluster_allgather<1>(c.cluster, *c.x, v2, all);
  int result = 0x7fffffff;
  for (unsigned r = 0; r < c.nranks; ++r)
    if (all[r][0]) result = (int)(all[r][0] - 1);
  return result;
}

// Inverse CDF over the kept set in ascending id order: the first kept element at which
// the running integer mass exceeds `target` (0 <= target < total kept mass).
__device__ int draw_inverse_cdf(RowCtx& c, const KeptSet& kept, float m, u64 target) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w0 = warp * c.seg;
  const int w1 = min(w0 + c.seg, c.n_local);
  u64 mine = 0;
  for (int i = w0 + lane; i < w1; i += 32) {
    const float s = c.stage[i];
    if (kept.has(key_of(s), c.base + i)) mine += mass_of(s, m);
  }
  const u64 wtot = warp_sum_u64(mine);
  u64 pre, pre_unused, tot, tot_unused;
  block_warp_prefix2(*c.x, wtot, 0, pre, pre_unused, tot, tot_unused);
  u64 vals[1] = {tot};
  u64 all[kMaxCluster][1];
  cluster_allgather<1>(c.cluster, *c.x, vals, all);
  u64 cta_pre = 0;
  for (unsigned r = 0; r < c.rank; ++r) cta_pre += all[r][0];
  if (threadIdx.x == 0) c.x->bcast[6] = 0;
  __syncthreads();
  const u64 before = cta_pre + pre;
  if (before <= target && target < before + wtot) {
    u64 running = before;
    for (int i0 = w0; i0 < w1; i0 += 32) {
      const int i = i0 + lane;
      u64 q = 0;
      if (i < w1) {
        const float s = c.stage[i];
        if (kept.has(key_of(s), c.base + i)) q = mass_of(s, m);
      }
      const u64 incl = warp_scan_u64(q);
      const uint32_t ballot = __ballot_sync(0xffffffffu, running + incl > target);
      if (ballot) {
        const int pos = __ffs(ballot) - 1;
        if (lane == 0) c.x->bcast[6] = (u64)(c.base + i0 + pos) + 1;
        break;
      }
      running += shfl_u64(incl, 31);
    }
  }
  __syncthreads();
  u64 v2[1] = {c.x->bcast[6]};
  cluster_allgather<1>(c.cluster, *c.x, v2, all);
  int result = -1;
  for (unsigned r = 0; r < c.nranks; ++r)
    if (all[r][0]) result = (int)(all[r][0] - 1);
  return result;
}

// arg max over the kept set of fl(fl(e / z) / noise), lowest id on ties: what
// torch.multinomial(p, 1) computes on CPU from its Exp(1) variates.
__device__ int draw_with_noise(RowCtx& c, const KeptSet& kept, float m, float zf,
                               const float* noise_row) {
  u64 best = 0;
  for (int i = threadIdx.x; i < c.n_local; i += kThreads) {
    const float s = c.stage[i];
    const int gid = c.base + i;
    if (!kept.has(key_of(s), gid)) continue;
    const float p = __fdiv_rn(expf(s - m), zf);
    const float ratio = __fdiv_rn(p, noise_row[gid]);
    const u64 packed = ((u64)__float_as_uint(ratio) << 32) | (uint32_t)(~(uint32_t)gid);
    best = packed > best ? packed : best;
  }
  best = block_max_u64(*c.x, best);
  u64 vals[1] = {best};
  u64 all[kMaxCluster][1];
  cluster_allgather<1>(c.cluster, *c.x, vals, all);
  for (unsigned r = 0; r < c.nranks; ++r) best = all[r][0] > best ? all[r][0] : best;
  return (int)(~(uint32_t)(best & 0xffffffffu));
}

// Writes the n_want highest kept scores (ties: lowest ids) as log-probabilities, sorted by
// (value descending, id ascending), into out->top_ids / out->top_logprobs.
__device__ void write_top_logprobs(RowCtx& c, const KeptSet& kept, uint32_t key_n, u64 above_n,
                                   int n_want, float m, float log_z, hs_row_out* out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w0 = warp * c.seg;
  const int w1 = min(w0 + c.seg, c.n_local);
  const u64 need_ties = (u64)n_want - above_n;
  u64 gt = 0, eq = 0;
  for (int i = w0 + lane; i < w1; i += 32) {
    const uint32_t k = key_of(c.stage[i]);
    gt += k > key_n;
    eq += (k == key_n) && kept.has(k, c.base + i);
  }
  const u64 wgt = warp_sum_u64(gt), weq = warp_sum_u64(eq);
  u64 pgt, peq, tgt, teq;
  block_warp_prefix2(*c.x, wgt, weq, pgt, peq, tgt, teq);
  u64 vals[2] = {tgt, teq};
  u64 all[kMaxCluster][2];
  cluster_allgather<2>(c.cluster, *c.x, vals, all);
  u64 run_gt = pgt, run_eq = peq;
  for (unsigned r = 0; r < c.rank; ++r) { run_gt += all[r][0]; run_eq += all[r][1]; }
  for (int i0 = w0; i0 < w1; i0 += 32) {
    const int i = i0 + lane;
    bool is_gt = false, is_eq = false;
    float s = 0.f;
    if (i < w1) {
      s = c.stage[i];
      const uint32_t k = key_of(s);
      is_gt = k > key_n;
      is_eq = (k == key_n) && kept.has(k, c.base + i);
    }
    const uint32_t bg = __ballot_sync(0xffffffffu, is_gt);
    const uint32_t be = __ballot_sync(0xffffffffu, is_eq);
    const uint32_t lt = (1u << lane) - 1u;
    int slot = -1;
    if (is_gt) slot = (int)(run_gt + __popc(bg & lt));
    if (is_eq) {
      const u64 r = run_eq + __popc(be & lt);
      if (r < need_ties) slot = (int)(above_n + r);
    }
    if (slot >= 0 && slot < HS_MAX_LOGPROBS) {
      out->top_ids[slot] = c.base + i;
      out->top_logprobs[slot] = (s - m) - log_z;
    }
    run_gt += __popc(bg);
    run_eq += __popc(be);
  }
  __threadfence();
  c.sync_all();
  if (c.rank == 0 && warp == 0) {  // n_want <= 20 entries: rank sort inside one warp
    int id = 0x7fffffff;
    float v = 0.f;
    if (lane < n_want) {
      id = *((volatile int32_t*)&out->top_ids[lane]);
      v = *((volatile float*)&out->top_logprobs[lane]);
    }
    const uint32_t kv = key_of(v);
    int pos = 0;
    for (int j = 0; j < n_want; ++j) {
      const uint32_t kj = __shfl_sync(0xffffffffu, kv, j);
      const int idj = __shfl_sync(0xffffffffu, id, j);
      if (kj > kv || (kj == kv && idj < id)) ++pos;
    }
    __syncwarp();
    if (lane < n_want) {
      out->top_ids[pos] = id;
      out->top_logprobs[pos] = v;
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1) row_kernel(const RowKernelArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  if (a.skip_candidate_rows) {
    // fp32 rows with a small top_k are sampled by the candidate kernel launched next to this
    // one (every CTA of the row's cluster sees the same parameters and leaves together)
    const hs_row_params& p = a.params[blockIdx.y];
    if (p.temperature != 0.0f && p.top_k > 0 && p.top_k <= kCandidateTopKMax && p.top_k < a.vocab) return;
  }
  RowCtx c{{cg::this_cluster()}};
  c.rank = c.cluster.block_rank();
  c.nranks = c.cluster.num_blocks();
  c.row = blockIdx.y;
  c.vocab = a.vocab;
  c.slice = a.slice;
  c.base = (int)c.rank * a.slice;
  c.n_local = max(0, min(a.slice, a.vocab - c.base));
  c.seg = ((c.n_local + kThreads - 1) / kThreads) * 32;

  size_t off = 0;
  c.x = reinterpret_cast<Exchange*>(smem_raw + off);
  off += (sizeof(Exchange) + 15) & ~size_t(15);
  c.hist = reinterpret_cast<Hist*>(smem_raw + off);
  off += sizeof(Hist);
  const int per = kBins / (int)c.nranks;
  c.red_mass = reinterpret_cast<u64*>(smem_raw + off);
  off += sizeof(u64) * per;
  c.red_cnt = reinterpret_cast<uint32_t*>(smem_raw + off);
  off += sizeof(uint32_t) * per;
  off = (off + 15) & ~size_t(15);
  c.smem_stage = reinterpret_cast<float*>(smem_raw + off);
  c.gstage_row = a.gstage ? a.gstage + (size_t)c.row * ((size_t)a.slice * c.nranks) : nullptr;
  c.stage = c.gstage_row ? c.gstage_row + c.base : c.smem_stage;
  if (threadIdx.x == 0) c.x->ring_phase = 0;

  const int tid = threadIdx.x;
  const hs_row_params P = a.params[c.row];
  hs_row_out* out = a.out + c.row;
  const bool greedy = P.temperature == 0.0f;

  // ---- A. the one read of the row from HBM -----------------------------------------
  {
    const long long gofs = (long long)c.row * a.row_stride + c.base;
    if (a.dtype == HS_DTYPE_BF16) {
      const unsigned short* src = reinterpret_cast<const unsigned short*>(a.logits) + gofs;
      const bool vec = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
      const int nvec = vec ? c.n_local / 8 : 0;
      const uint4* src4 = reinterpret_cast<const uint4*>(src);
      for (int i = tid; i < nvec; i += kThreads) {
        const uint4 w = __ldcs(src4 + i);
        float4 lo, hi;
        lo.x = canonical(__uint_as_float(w.x << 16)); lo.y = canonical(__uint_as_float(w.x & 0xffff0000u));
        lo.z = canonical(__uint_as_float(w.y << 16)); lo.w = canonical(__uint_as_float(w.y & 0xffff0000u));
        hi.x = canonical(__uint_as_float(w.z << 16)); hi.y = canonical(__uint_as_float(w.z & 0xffff0000u));
        hi.z = canonical(__uint_as_float(w.w << 16)); hi.w = canonical(__uint_as_float(w.w & 0xffff0000u));
        float4* dst = reinterpret_cast<float4*>(c.stage + 8 * i);
        dst[0] = lo;
        dst[1] = hi;
      }
      for (int i = nvec * 8 + tid; i < c.n_local; i += kThreads)
        c.stage[i] = canonical(__uint_as_float((uint32_t)src[i] << 16));
    } else {
      const float* src = reinterpret_cast<const float*>(a.logits) + gofs;
      const bool vec = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
      const int nvec = vec ? c.n_local / 4 : 0;
      const float4* src4 = reinterpret_cast<const float4*>(src);
      for (int i = tid; i < nvec; i += kThreads) {
        float4 w = __ldcs(src4 + i);
        w.x = canonical(w.x); w.y = canonical(w.y); w.z = canonical(w.z); w.w = canonical(w.w);
        reinterpret_cast<float4*>(c.stage)[i] = w;
      }
      for (int i = nvec * 4 + tid; i < c.n_local; i += kThreads) c.stage[i] = canonical(src[i]);
    }
  }
  c.sync_all();

  // ---- B. penalties from the row's resident (id, count) list -------------------------
  const bool slot_ok = P.slot >= 0 && P.slot < a.pool.slots_total;
  const bool penalised = slot_ok && (P.repetition_penalty != 1.0f || P.presence_penalty != 0.0f ||
                                     P.frequency_penalty != 0.0f);
  if (penalised) {
    const int n_unique = min(a.pool.n[P.slot], a.pool.unique_cap);
    const int2* pairs = a.pool.pairs + (size_t)P.slot * a.pool.unique_cap;
    for (int j = (int)c.rank * kThreads + tid; j < n_unique; j += (int)c.nranks * kThreads) {
      const int2 e = pairs[j];
      const int id = e.x;
      if (id < 0 || id >= a.vocab) continue;
      const unsigned r = (unsigned)(id / a.slice);
      float* p = c.slice_of(r) + (id - (int)r * a.slice);
      float v = *p;
      v = v < 0.0f ? __fmul_rn(v, P.repetition_penalty) : __fdiv_rn(v, P.repetition_penalty);
      v = __fsub_rn(v, P.presence_penalty);
      v = __fsub_rn(v, __fmul_rn(P.frequency_penalty, (float)e.y));
      *p = canonical(v);
    }
    if (c.gstage_row) __threadfence();
    c.sync_all();
  }

  // ---- C. temperature, row max, arg max ----------------------------------------------
  u64 best = 0;
  for (int i = tid; i < c.n_local; i += kThreads) {
    float v = c.stage[i];
    if (!greedy) {
      v = canonical(__fdiv_rn(v, P.temperature));
      c.stage[i] = v;
    }
    const u64 packed = ((u64)key_of(v) << 32) | (uint32_t)(~(uint32_t)(c.base + i));
    best = packed > best ? packed : best;
  }
  best = block_max_u64(*c.x, best);
  {
    u64 vals[1] = {best};
    u64 all[kMaxCluster][1];
    cluster_allgather<1>(c.cluster, *c.x, vals, all);
    for (unsigned r = 0; r < c.nranks; ++r) best = all[r][0] > best ? all[r][0] : best;
  }
  const uint32_t max_key = (uint32_t)(best >> 32);
  const int argmax_id = (int)(~(uint32_t)(best & 0xffffffffu));
  const float m = score_of(max_key);

  KeptSet kept{0u, 0x7fffffff};
  int token = argmax_id;
  int status = P.slot >= a.pool.slots_total ? 64 : 0;  // a slot this sampler does not have: no penalties
  u64 n_topk = (u64)a.vocab, n_minp = (u64)a.vocab, n_kept = (u64)a.vocab;
  u64 q_kept = 0;
  bool have_totals = false;
  long long cut_ties = -1;

  if (!greedy) {
    u64 cnt = 0, mass = 0;
    if (P.top_k > 0 && P.top_k < a.vocab) {
      Selection sk = descend<false, true>(c, 0u, (u64)P.top_k, 1.0f, m);
      if (!sk.ok) status |= 1;
      kept.cut_key = sk.key;
      cnt = sk.above_cnt + sk.bin_cnt;
      mass = sk.above_mass + sk.bin_mass;
      have_totals = sk.ok;
      n_topk = cnt;
    }
    if (P.min_p > 0.0f) {
      if (!have_totals) totals_above(c, kept.cut_key, m, true, cnt, mass);
      const float z1 = mass_to_float(mass);
      const float thr = __fmul_rn(__fdiv_rn(1.0f, z1), P.min_p);
      uint32_t lowest = 0xffffffffu;
      for (int i = tid; i < c.n_local; i += kThreads) {
        const float s = c.stage[i];
        const uint32_t k = key_of(s);
        if (k >= kept.cut_key && !(__fdiv_rn(expf(s - m), z1) < thr)) lowest = min(lowest, k);
      }
      lowest = ~block_max_u32(*c.x, ~lowest);
      u64 vals[1] = {(u64)lowest};
      u64 all[kMaxCluster][1];
      cluster_allgather<1>(c.cluster, *c.x, vals, all);
      for (unsigned r = 0; r < c.nranks; ++r) lowest = min(lowest, (uint32_t)all[r][0]);
      if (lowest != 0xffffffffu && lowest > kept.cut_key) {
        kept.cut_key = lowest;
        have_totals = false;
      }
    }
    if (P.top_p < 1.0f) {
      Selection sp = descend<true, true>(c, kept.cut_key, 0, P.top_p, m);
      n_minp = sp.total_cnt;
      if (sp.ok && sp.bin_cnt > 0) {
        const u64 qv = sp.bin_mass / sp.bin_cnt;  // all elements of the bin share one score
        u64 t = sp.bin_cnt;
        if (qv > 0) {
          const u64 want = sp.target - sp.above_mass;
          t = (want + qv - 1) / qv;
          if (t < 1) t = 1;
          if (t > sp.bin_cnt) t = sp.bin_cnt;
        }
        kept.cut_key = sp.key;
        cnt = sp.above_cnt + t;
        mass = sp.above_mass + t * qv;
        cut_ties = (long long)t;
        have_totals = true;
        if (t < sp.bin_cnt) kept.tie_limit = find_tth_equal(c, sp.key, t);
      } else {
        status |= 1;
        cnt = sp.total_cnt;
        mass = sp.total_mass;
        have_totals = true;
      }
    } else {
      if (!have_totals) totals_above(c, kept.cut_key, m, true, cnt, mass);
      have_totals = true;
      n_minp = cnt;
    }
    n_kept = cnt;
    q_kept = mass;

    // ---- draw ------------------------------------------------------------------------
    if (q_kept == 0) {
      token = argmax_id;
      status |= 1;
    } else if (a.noise) {
      token = draw_with_noise(c, kept, m, mass_to_float(q_kept), a.noise + (size_t)c.row * a.vocab);
    } else {
      const Philox4 r = philox4x32_10(0u, 0u, 0u, 0u, (uint32_t)P.seed, (uint32_t)(P.seed >> 32));
      const u64 r64 = ((u64)r.v[0] << 32) | r.v[1];
      const u64 target = __umul64hi(r64, q_kept);
      token = draw_inverse_cdf(c, kept, m, target);
      if (token < 0) { token = argmax_id; status |= 1; }
    }
  } else if (P.n_logprobs >= 0) {
    u64 cnt;
    totals_above(c, 0u, m, true, cnt, q_kept);
  }

  // ---- D. log-probabilities ----------------------------------------------------------
  float log_z = 0.f;
  if (P.n_logprobs >= 0) {
    log_z = (float)(log((double)q_kept) - (double)kMassShift * 0.6931471805599453);
    const unsigned owner = (unsigned)(token / a.slice);
    if (c.rank == owner && tid == 0) {
      const float s = c.stage[token - (int)owner * a.slice];
      out->logprob = (s - m) - log_z;
    }
    int n_want = min(P.n_logprobs, a.vocab);
    if ((u64)n_want > n_kept) n_want = (int)n_kept;
    if (n_want > 0) {
      Selection sn = descend<false, false>(c, kept.cut_key, (u64)n_want, 1.0f, m);
      if (sn.ok) {
        write_top_logprobs(c, kept, sn.key, sn.above_cnt, n_want, m, log_z, out);
      } else {
        n_want = 0;
        status |= 1;
      }
    }
    if (c.rank == 0 && tid == 0) out->n_top = n_want;
  } else if (c.rank == 0 && tid == 0) {
    out->n_top = 0;
    out->logprob = 0.f;
  }

  // ---- E. optional dump of the final scores (parity tests) ----------------------------
  if (a.scores_out) {
    float* dst = a.scores_out + (size_t)c.row * a.vocab + c.base;
    for (int i = tid; i < c.n_local; i += kThreads) {
      const float s = c.stage[i];
      dst[i] = (greedy || kept.has(key_of(s), c.base + i)) ? s : __int_as_float(0xff800000);
    }
  }

  if (c.rank == 0 && tid == 0) {
    out->token = token;
    out->status = status;
    out->n_kept = (int32_t)n_kept;
    out->n_after_topk = (int32_t)n_topk;
    out->n_after_minp = (int32_t)n_minp;
    out->n_after_topp = (int32_t)n_kept;
    out->cut_bits = __float_as_uint(score_of(kept.cut_key));
    out->n_cut_ties = (int32_t)cut_ties;
    out->row_max = m;
    out->log_z = log_z;
    if (a.tokens_out) a.tokens_out[c.row] = token;
    if ((a.flags & HS_SAMPLE_APPEND_TOKEN) && slot_ok && token >= 0 && token < a.vocab) {
      if (!slot_append_one(a.pool, P.slot, token)) out->status = status | 2;
    }
  }
  // No CTA may leave while a peer can still read its shared memory.
  c.sync_all();
}

}  // namespace hs
