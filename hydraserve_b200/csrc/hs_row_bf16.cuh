// The fused per-row sampling kernel for bf16 logits (the serving default).
//
// A bf16 row has at most 65,536 distinct values, and only the tokens of the request's
// history get a different (fp32) score from their penalties.  The kernel therefore splits
// the row into two populations:
//
//   N  the tokens without a penalty.  They are described exactly by COUNTS per distinct
//      bf16 value: 8,192 bins cover every value with 2^-16 <= |x| < 2^16, one value per bin.
//      Their probability mass is count * mass(value): no exp per token, no mass histogram.
//   S  the side list: penalised tokens (fp32 scores), plus the few unpenalised tokens whose
//      value lies outside the bin window (zeros, denormals, infinities).  Individual
//      (id, score) pairs in a global scratch list.
//
// The row is read from HBM once with 128-bit loads; in the same pass its raw bf16 bits go
// to shared memory (a slice per CTA of the thread-block cluster) and its values are counted
// into the CTA's bins with shared-memory atomics.  The penalty pass then walks the row's
// resident (token id, count) list: it fetches each raw value from the owning CTA's slice
// through distributed shared memory, takes it out of the bins, marks the slot in the slice,
// and stores the penalised score in S.  After the per-CTA bins are summed across the
// cluster every CTA holds the row's full value histogram.
//
// Selection (top-k by count, min-p by threshold, top-p by probability mass, top-N for the
// log-probabilities) is a radix descent over 32-bit order-preserving keys of the scores:
// S elements are histogrammed individually, N bins are injected as (count, count * mass).
// As soon as the bucket that holds the answer has at most kListCap members they are
// gathered into one small list, sorted, and the exact key is read off a prefix sum.
// Probability mass is an integer multiple of 2^-40, so all sums are exact and
// order-independent.  The resident slice is only revisited to turn "the j-th token with
// value v" into a token id (draw, tie-breaks towards the lowest id, top-N ids).
#pragma once

#include "hs_common.cuh"
#include "hs_select.cuh"
#include "hs_row_kernel.cuh"
#include "../../include/hs_sampler.h"

namespace hs {

constexpr int kValueBins = 8192;            // 2 signs x 32 binades x 128 mantissas
constexpr uint32_t kWinBase = 111u << 7;    // smallest binned magnitude: 2^-16
constexpr uint32_t kSentinel = 0xFFFFu;     // marks a slice slot whose token moved to S
constexpr int kListCap = 256;               // members resolved by sorting instead of another radix level
constexpr int kPhaseSlots = 12;
constexpr int kRareCap = 256;               // out-of-window tokens remembered per CTA before a sweep

struct ListEntry {
  uint32_t key;  // 32-bit key of the score
  int32_t id;    // token id of an S element, -1 for a value bin
  uint32_t cnt;  // tokens this entry stands for
  uint32_t raw;  // bf16 bits of a value bin
  u64 q;         // mass of one token
};

struct Row16Args {
  RowKernelArgs base;
  int2* s_pair;    // [batch, s_cap] side list: (token id or -1, fp32 bits of the score)
  int s_cap;
  unsigned long long* phase_clocks;  // [batch, kPhaseSlots] SM clock at phase boundaries, or null
};

// Shared-memory layout of one CTA (offsets in bytes); the slice of raw bf16 bits follows.
struct Layout16 {
  size_t x, bins, hist, red_mass, red_cnt, bins_red, glist, list, rare, small, stage;
};
__host__ __device__ inline Layout16 layout16(int nranks) {
  Layout16 l{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = (off + bytes + 15) & ~size_t(15);
    return at;
  };
  l.x = take(sizeof(Exchange));
  l.bins = take(sizeof(uint32_t) * kValueBins);
  l.hist = take(sizeof(Hist));
  l.red_mass = take(sizeof(u64) * (kBins / nranks));
  l.red_cnt = take(sizeof(uint32_t) * (kBins / nranks));
  l.bins_red = take(sizeof(uint32_t) * (kValueBins / nranks));
  l.glist = take(sizeof(ListEntry) * 2 * kListCap);
  l.list = take(sizeof(ListEntry) * kListCap);
  l.rare = take(sizeof(int) * kRareCap);
  l.small = take(sizeof(int) * 8);
  l.stage = off;
  return l;
}

__device__ __forceinline__ int bin_of_raw(uint32_t raw) {
  const uint32_t idx = (raw & 0x7fffu) - kWinBase;
  if (idx >= 4096u) return -1;
  return (raw & 0x8000u) ? 4095 - (int)idx : 4096 + (int)idx;
}
__device__ __forceinline__ uint32_t raw_of_bin(int b) {
  return b >= 4096 ? (uint32_t)(b - 4096) + kWinBase : 0x8000u | ((uint32_t)(4095 - b) + kWinBase);
}

struct Ctx16 : ClusterCtx {
  int row, vocab, slice, base, n_local, seg;
  uint16_t* stage;      // this CTA's slice of raw bf16 bits
  uint32_t* bins;       // kValueBins counts: local, then the whole row's
  uint32_t* bins_red;   // kValueBins / nranks, reduce-scatter buffer
  ListEntry* glist;     // [2][kListCap] gather buffers (appends go to the leader's)
  int* glist_n;         // [3] append counters (the leader's), rotated so clearing never races a reader
  int gather_seq;
  ListEntry* list;      // [kListCap] this CTA's sorted copy
  int* s_extra;         // leader: number of out-of-window tokens appended to S
  int2* s_pair;
  int n_s;
  int s_cap;
  float T;
  bool greedy;
  float m;

  __device__ __forceinline__ float score_of_value(float v) const {
    return greedy ? canonical(v) : canonical(__fdiv_rn(v, T));
  }
  __device__ __forceinline__ float score_of_raw(uint32_t raw) const {
    return score_of_value(__uint_as_float(raw << 16));
  }
  __device__ __forceinline__ uint16_t* slice_of(unsigned r) {
    return nranks > 1 ? cluster.map_shared_rank(stage, r) : stage;
  }
};

// Calls f(id, score) for this CTA's share of the side list.  The list lives in global
// memory (L2); eight entries per thread are fetched before any is processed, so a pass
// costs about one L2 round trip per eight entries instead of one per entry.
template <class F>
__device__ __forceinline__ void for_each_side(const Ctx16& c, F&& f) {
  const int stride = (int)c.nranks * kThreads;
  for (int j0 = (int)c.rank * kThreads + threadIdx.x; j0 < c.n_s; j0 += 8 * stride) {
    int2 e[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j = j0 + u * stride;
      e[u] = j < c.n_s ? c.s_pair[j] : make_int2(-1, 0);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (e[u].x >= 0) f(e[u].x, __int_as_float(e[u].y));
  }
}

// The kept set: key > cut_key, or key == cut_key and token id <= tie_limit.
// (KeptSet is declared in hs_row_kernel.cuh.)

// ---- fills for descend_core ----------------------------------------------------------
// All elements of the row: S individually, N as bins (this CTA injects its share of bins).
template <bool WITH_MASS>
struct UnionFill {
  Ctx16* c;
  template <class Add>
  __device__ __forceinline__ void operator()(int level, int shift, int bits, uint32_t prefix,
                                             uint32_t lo_key, const Add& add) const {
    const uint32_t mask = (1u << bits) - 1u;
    const int lane = threadIdx.x & 31;
    for_each_side(*c, [&](int, float s) {
      const uint32_t k = key_of(s);
      const bool valid = k >= lo_key && (level == 0 || (k >> (shift + bits)) == prefix);
      add(valid, (k >> shift) & mask, 1u, (WITH_MASS && valid) ? mass_of(s, c->m) : 0ull);
    });
    const int per = kValueBins / (int)c->nranks;
    const int b_end = ((int)c->rank + 1) * per;
    for (int b0 = (int)c->rank * per + (threadIdx.x & ~31); b0 < b_end; b0 += kThreads) {
      const int b = b0 + lane;
      uint32_t cnt = b < b_end ? c->bins[b] : 0u;
      float s = 0.f;
      uint32_t k = 0;
      if (cnt) {
        s = c->score_of_raw(raw_of_bin(b));
        k = key_of(s);
        if (!(k >= lo_key && (level == 0 || (k >> (shift + bits)) == prefix))) cnt = 0;
      }
      add(cnt != 0, (k >> shift) & mask, cnt, (WITH_MASS && cnt) ? (u64)cnt * mass_of(s, c->m) : 0ull);
    }
  }
};

// Tokens whose score key equals `key`, keyed by ~id (so a descending walk is ascending id).
struct TieFill {
  Ctx16* c;
  uint32_t key;
  int raw;  // bf16 bits of the value bin with that key, or -1
  template <class Add>
  __device__ __forceinline__ void operator()(int level, int shift, int bits, uint32_t prefix,
                                             uint32_t, const Add& add) const {
    const uint32_t mask = (1u << bits) - 1u;
    const int lane = threadIdx.x & 31;
    for_each_side(*c, [&](int id, float s) {
      const uint32_t k = ~(uint32_t)id;
      const bool valid = key_of(s) == key && (level == 0 || (k >> (shift + bits)) == prefix);
      add(valid, (k >> shift) & mask, 1u, 0ull);
    });
    if (raw >= 0) {
      for (int i0 = threadIdx.x & ~31; i0 < c->n_local; i0 += kThreads) {
        const int i = i0 + lane;
        bool valid = i < c->n_local && c->stage[i] == (uint16_t)raw;
        const uint32_t k = ~(uint32_t)(c->base + i);
        valid = valid && (level == 0 || (k >> (shift + bits)) == prefix);
        add(valid, (k >> shift) & mask, 1u, 0ull);
      }
    }
  }
};

// Kept S elements keyed by ~id, with their mass (the S part of the inverse-CDF draw).
struct SideDrawFill {
  Ctx16* c;
  KeptSet kept;
  template <class Add>
  __device__ __forceinline__ void operator()(int level, int shift, int bits, uint32_t prefix,
                                             uint32_t, const Add& add) const {
    const uint32_t mask = (1u << bits) - 1u;
    for_each_side(*c, [&](int id, float s) {
      const uint32_t k = ~(uint32_t)id;
      const bool valid = kept.has(key_of(s), id) && (level == 0 || (k >> (shift + bits)) == prefix);
      add(valid, (k >> shift) & mask, 1u, valid ? mass_of(s, c->m) : 0ull);
    });
  }
};

// ---- gathering a few entries from the whole cluster into the leader CTA ------------------
// Gather g appends to the leader's buffer g % 2 through counter g % 3 and, before its
// barrier, clears counter (g + 1) % 3, whose last readers finished two barriers ago.
struct GatherSlot {
  ListEntry* dst;    // leader's buffer
  int* dst_n;        // leader's counter
  ListEntry* local;  // this CTA's buffer of the same index
  int clear;         // counter to clear for the next gather
};
__device__ __forceinline__ GatherSlot begin_gather(Ctx16& c) {
  const int g = c.gather_seq++;
  GatherSlot s;
  ListEntry* lead = c.nranks > 1 ? c.cluster.map_shared_rank(c.glist, 0) : c.glist;
  int* lead_n = c.nranks > 1 ? c.cluster.map_shared_rank(c.glist_n, 0) : c.glist_n;
  s.dst = lead + (g & 1) * kListCap;
  s.dst_n = lead_n + g % 3;
  s.local = c.glist + (g & 1) * kListCap;
  s.clear = (g + 1) % 3;
  return s;
}
__device__ __forceinline__ void end_gather(Ctx16& c, const GatherSlot& s) {
  if (c.rank == 0 && threadIdx.x == 0) c.glist_n[s.clear] = 0;
  c.sync_all();
}

// ---- small-list resolution -----------------------------------------------------------
// Gathers into every CTA's `list` the members (S elements, N bins) with key >= lo_key whose
// top `levels` radix digits equal `prefix` (levels = 0: no prefix test), sorted by
// (key descending, bins before elements, id ascending).  Returns the member count; the
// caller guarantees it does not exceed kListCap.  One cluster barrier.
__device__ int gather_members(Ctx16& c, uint32_t lo_key, int levels, uint32_t prefix, bool with_mass) {
  const int tid = threadIdx.x;
  const GatherSlot g = begin_gather(c);
  ListEntry* dst = g.dst;
  int* dst_n = g.dst_n;
  const int drop = levels == 0 ? 32 : (levels == 1 ? 21 : (levels == 2 ? 10 : 0));
  auto matches = [&](uint32_t k) {
    if (k < lo_key) return false;
    return levels == 0 || (levels == 3 ? k == prefix : (k >> drop) == prefix);
  };
  for_each_side(c, [&](int id, float s) {
    const uint32_t k = key_of(s);
    if (!matches(k)) return;
    const int slot = atomicAdd(dst_n, 1);
    if (slot < kListCap) dst[slot] = ListEntry{k, id, 1u, 0u, with_mass ? mass_of(s, c.m) : 0ull};
  });
  const int per = kValueBins / (int)c.nranks;
  for (int b = (int)c.rank * per + tid; b < ((int)c.rank + 1) * per; b += kThreads) {
    const uint32_t cnt = c.bins[b];
    if (!cnt) continue;
    const uint32_t raw = raw_of_bin(b);
    const float s = c.score_of_raw(raw);
    const uint32_t k = key_of(s);
    if (!matches(k)) continue;
    const int slot = atomicAdd(dst_n, 1);
    if (slot < kListCap) dst[slot] = ListEntry{k, -1, cnt, raw, with_mass ? mass_of(s, c.m) : 0ull};
  }
  end_gather(c, g);
  const int n = min(*dst_n, kListCap);
  // bring the entries here, then rank sort: position = number of entries that precede
  if (c.rank != 0 && tid < n) g.local[tid] = dst[tid];
  __syncthreads();
  ListEntry mine;
  int pos = 0;
  if (tid < n) {
    mine = g.local[tid];
    for (int j = 0; j < n; ++j) {
      const uint32_t kj = g.local[j].key;
      const int idj = g.local[j].id;
      pos += (kj > mine.key || (kj == mine.key && idj < mine.id)) ? 1 : 0;
    }
    c.list[pos] = mine;
  }
  __syncthreads();
  return n;
}

// Inclusive prefix sums of (count, count * q) over the first n entries of the sorted list;
// thread i < n gets those of entry i.  Also returns the totals.
__device__ __forceinline__ void list_scan(Ctx16& c, int n, u64& incl_cnt, u64& incl_mass, u64& tot_cnt,
                                          u64& tot_mass) {
  const int tid = threadIdx.x;
  u64 a = 0, b = 0;
  if (tid < n) { a = c.list[tid].cnt; b = (u64)c.list[tid].cnt * c.list[tid].q; }
  const u64 ia = warp_scan_u64(a), ib = warp_scan_u64(b);
  u64 pa, pb;
  block_warp_prefix2(*c.x, shfl_u64(ia, 31), shfl_u64(ib, 31), pa, pb, tot_cnt, tot_mass);
  incl_cnt = pa + ia;
  incl_mass = pb + ib;
}

// Completes a descent that stopped early: gathers the members of the selected bucket and
// finds the exact key where the running count / mass reaches the target.
template <bool BY_MASS>
__device__ Selection resolve(Ctx16& c, Selection sel, uint32_t lo_key) {
  if (!sel.ok || sel.levels == 3) return sel;
  const int n = gather_members(c, lo_key, sel.levels, sel.prefix, true);
  u64 ic, im, tc, tm;
  list_scan(c, n, ic, im, tc, tm);
  const int tid = threadIdx.x;
  const u64 want = sel.target - (BY_MASS ? sel.above_mass : sel.above_cnt);
  if (tid == 0) c.x->bcast[7] = 0;
  __syncthreads();
  if (tid < n) {
    const u64 mine_c = c.list[tid].cnt, mine_m = mine_c * c.list[tid].q;
    const u64 incl = BY_MASS ? im : ic;
    const u64 excl = incl - (BY_MASS ? mine_m : mine_c);
    if (excl < want && want <= incl) { c.x->bcast[0] = c.list[tid].key; c.x->bcast[7] = 1; }
  }
  __syncthreads();
  if (c.x->bcast[7] == 0) {
    sel.ok = false;
    __syncthreads();
    return sel;
  }
  const uint32_t key = (uint32_t)c.x->bcast[0];
  u64 ac = 0, am = 0, bc = 0, bm = 0;
  if (tid < n) {
    const u64 mc = c.list[tid].cnt, mm = mc * c.list[tid].q;
    if (c.list[tid].key > key) { ac = mc; am = mm; }
    if (c.list[tid].key == key) { bc = mc; bm = mm; }
  }
  block_sum2(*c.x, ac, am);
  block_sum2(*c.x, bc, bm);
  sel.key = key;
  sel.prefix = key;
  sel.levels = 3;
  sel.above_cnt += ac;
  sel.above_mass += am;
  sel.bin_cnt = bc;
  sel.bin_mass = bm;
  __syncthreads();
  return sel;
}

template <bool BY_MASS, bool WITH_MASS>
__device__ Selection select_union(Ctx16& c, uint32_t lo_key, u64 target, float top_p) {
  UnionFill<WITH_MASS> fill{&c};
  Selection sel = descend_core<BY_MASS, WITH_MASS>(c, fill, lo_key, target, top_p, (u64)kListCap);
  return resolve<BY_MASS>(c, sel, lo_key);
}

// ---- replicated work on the value bins (every CTA holds the whole row's bins) ----------
// Highest non-empty bin, or -1.
__device__ int highest_bin(Ctx16& c) {
  int best = -1;
  for (int b = threadIdx.x; b < kValueBins; b += kThreads)
    if (c.bins[b]) best = b;  // ascending b per thread: the last hit is the highest
  return (int)block_max_u32(*c.x, (uint32_t)(best + 1)) - 1;
}
// The bin whose score key equals `key`, or -1.
__device__ int bin_with_key(Ctx16& c, uint32_t key) {
  int found = -1;
  for (int b = threadIdx.x; b < kValueBins; b += kThreads)
    if (c.bins[b] && key_of(c.score_of_raw(raw_of_bin(b))) == key) found = b;
  return (int)block_max_u32(*c.x, (uint32_t)(found + 1)) - 1;
}
// Lowest bin index whose score key is >= key (kValueBins when there is none).  Keys grow
// with the bin index, so tokens in lower bins can never reach `key`.
__device__ int lowest_bin_at_or_above(Ctx16& c, uint32_t key) {
  int best = kValueBins;
  for (int b = threadIdx.x; b < kValueBins; b += kThreads)
    if (key_of(c.score_of_raw(raw_of_bin(b))) >= key) best = min(best, b);
  return kValueBins - (int)block_max_u32(*c.x, (uint32_t)(kValueBins - best));
}
// Count and mass of the N tokens with score key >= lo_key (strict = false) or > lo_key.
__device__ void bins_totals(Ctx16& c, uint32_t lo_key, bool strict, bool with_mass, u64& cnt, u64& mass) {
  u64 a = 0, b = 0;
  for (int i = threadIdx.x; i < kValueBins; i += kThreads) {
    const uint32_t n = c.bins[i];
    if (!n) continue;
    const float s = c.score_of_raw(raw_of_bin(i));
    const uint32_t k = key_of(s);
    if (strict ? k > lo_key : k >= lo_key) {
      a += n;
      if (with_mass) b += (u64)n * mass_of(s, c.m);
    }
  }
  block_sum2(*c.x, a, b);
  cnt = a;
  mass = b;
}
// Count and mass of the S elements with key >= lo_key, cluster wide.  One cluster barrier.
__device__ void side_totals(Ctx16& c, uint32_t lo_key, bool with_mass, u64& cnt, u64& mass) {
  u64 a = 0, b = 0;
  for_each_side(c, [&](int, float s) {
    if (key_of(s) >= lo_key) {
      ++a;
      if (with_mass) b += mass_of(s, c.m);
    }
  });
  block_sum2(*c.x, a, b);
  const u64 vals[2] = {a, b};
  const uint32_t ph = cluster_publish<2>(c.cluster, *c.x, vals);
  cnt = ring_reduce<RingOp::Sum>(c.cluster, *c.x, ph, 0);
  mass = ring_reduce<RingOp::Sum>(c.cluster, *c.x, ph, 1);
}

// ---- id look-ups in the resident slices ------------------------------------------------
// Number of tokens with raw value `raw` and id <= id_limit, cluster wide.  One barrier.
__device__ u64 count_raw_upto(Ctx16& c, uint32_t raw, int id_limit) {
  u64 a = 0, b = 0;
  for (int i = threadIdx.x; i < c.n_local; i += kThreads)
    a += (c.stage[i] == (uint16_t)raw && c.base + i <= id_limit) ? 1 : 0;
  block_sum2(*c.x, a, b);
  const u64 vals[1] = {a};
  const uint32_t ph = cluster_publish<1>(c.cluster, *c.x, vals);
  return ring_reduce<RingOp::Sum>(c.cluster, *c.x, ph, 0);
}
// Token id of the n-th (1-based, ascending id) token whose raw value is `raw`; every CTA
// gets the answer (0x7fffffff when there is none).  Two cluster barriers.
__device__ int find_nth_raw(Ctx16& c, uint32_t raw, u64 n) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w0 = warp * c.seg;
  const int w1 = min(w0 + c.seg, c.n_local);
  const uint16_t want = (uint16_t)raw;
  u64 mine = 0;
  for (int i = w0 + lane; i < w1; i += 32) mine += c.stage[i] == want;
  const u64 wtot = warp_sum_u64(mine);
  u64 pre, pre_unused, tot, tot_unused;
  block_warp_prefix2(*c.x, wtot, 0, pre, pre_unused, tot, tot_unused);
  const u64 vals[1] = {tot};
  const uint32_t ph = cluster_publish<1>(c.cluster, *c.x, vals);
  const u64 cta_pre = ring_prefix(c.cluster, *c.x, ph, 0, c.rank);
  if (threadIdx.x == 0) c.x->bcast[6] = 0;
  __syncthreads();
  const u64 before = cta_pre + pre;
  if (before < n && n <= before + wtot) {
    u64 running = before;
    for (int i0 = w0; i0 < w1; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < w1 && c.stage[i] == want;
      const uint32_t ballot = __ballot_sync(0xffffffffu, hit);
      const u64 cnt = __popc(ballot);
      if (running + cnt >= n) {
        const int pos = __fns(ballot, 0, (int)(n - running));
        if (lane == 0) c.x->bcast[6] = (u64)(c.base + i0 + pos) + 1;
        break;
      }
      running += cnt;
    }
  }
  __syncthreads();
  const u64 v2[1] = {c.x->bcast[6]};
  const uint32_t ph2 = cluster_publish<1>(c.cluster, *c.x, v2);
  const u64 found = ring_reduce<RingOp::Max>(c.cluster, *c.x, ph2, 0);
  return found ? (int)(found - 1) : 0x7fffffff;
}
// Largest id among the `t` lowest-id tokens (N and S together) whose score key is `key`.
__device__ int tie_id_limit(Ctx16& c, uint32_t key, u64 t) {
  const int b = bin_with_key(c, key);
  TieFill fill{&c, key, b >= 0 ? (int)raw_of_bin(b) : -1};
  // ids are below 2^21: the top radix digit of ~id is all ones, start at the second level
  Selection sel = descend_core<false, false>(c, fill, 0u, t, 1.0f, 0, 1, 0x7FFu);
  return sel.ok ? (int)(~sel.key) : 0x7fffffff;
}

__global__ void __launch_bounds__(kThreads, 1) row_kernel_bf16(const Row16Args args) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const RowKernelArgs& a = args.base;
  Ctx16 c{{cg::this_cluster()}};
  c.rank = c.cluster.block_rank();
  c.nranks = c.cluster.num_blocks();
  c.row = blockIdx.y;
  c.vocab = a.vocab;
  c.slice = a.slice;
  c.base = (int)c.rank * a.slice;
  c.n_local = max(0, min(a.slice, a.vocab - c.base));
  c.seg = ((c.n_local + kThreads - 1) / kThreads) * 32;
  c.gather_seq = 0;

  const int per_bins = kValueBins / (int)c.nranks;
  const Layout16 lay = layout16((int)c.nranks);
  c.x = reinterpret_cast<Exchange*>(smem_raw + lay.x);
  c.bins = reinterpret_cast<uint32_t*>(smem_raw + lay.bins);
  c.hist = reinterpret_cast<Hist*>(smem_raw + lay.hist);
  c.red_mass = reinterpret_cast<u64*>(smem_raw + lay.red_mass);
  c.red_cnt = reinterpret_cast<uint32_t*>(smem_raw + lay.red_cnt);
  c.bins_red = reinterpret_cast<uint32_t*>(smem_raw + lay.bins_red);
  c.glist = reinterpret_cast<ListEntry*>(smem_raw + lay.glist);
  c.list = reinterpret_cast<ListEntry*>(smem_raw + lay.list);
  int* rare_id = reinterpret_cast<int*>(smem_raw + lay.rare);
  int* small = reinterpret_cast<int*>(smem_raw + lay.small);
  c.glist_n = small;        // [0..2]
  c.s_extra = small + 3;
  int* rare_n = small + 4;
  c.stage = reinterpret_cast<uint16_t*>(smem_raw + lay.stage);

  const int tid = threadIdx.x;
  const hs_row_params P = a.params[c.row];
  hs_row_out* out = a.out + c.row;
  c.greedy = P.temperature == 0.0f;
  c.T = P.temperature;
  c.m = 0.f;
  c.s_pair = args.s_pair + (size_t)c.row * args.s_cap;
  c.s_cap = args.s_cap;
  c.n_s = 0;

  unsigned long long* clocks = args.phase_clocks ? args.phase_clocks + (size_t)c.row * kPhaseSlots : nullptr;
  auto mark = [&](int slot) {
    if (clocks && c.rank == 0 && tid == 0) clocks[slot] = clock64();
  };
  mark(0);
  for (int b = tid; b < kValueBins; b += kThreads) c.bins[b] = 0;
  if (tid < 8) small[tid] = 0;
  if (tid == 0) c.x->ring_phase = 0;
  __syncthreads();

  // ---- A. the one read of the row from HBM: raw bits to the slice, values to the bins --
  {
    const unsigned short* src = reinterpret_cast<const unsigned short*>(a.logits) +
                                ((long long)c.row * a.row_stride + c.base);
    auto count_one = [&](uint32_t raw, int local) {
      const int b = bin_of_raw(raw);
      if (b >= 0) {
        atomicAdd(&c.bins[b], 1u);
      } else {
        const int slot = atomicAdd(rare_n, 1);
        if (slot < kRareCap) rare_id[slot] = local;
      }
    };
    const bool vec = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    const int nvec = vec ? c.n_local / 8 : 0;
    const uint4* src4 = reinterpret_cast<const uint4*>(src);
    uint4* dst4 = reinterpret_cast<uint4*>(c.stage);
    constexpr int kInFlight = 8;  // 128-bit loads issued per thread before any is consumed
    for (int i0 = tid; i0 < nvec; i0 += kInFlight * kThreads) {
      uint4 w[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int i = i0 + u * kThreads;
        if (i < nvec) w[u] = __ldcs(src4 + i);
      }
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int i = i0 + u * kThreads;
        if (i >= nvec) break;
        dst4[i] = w[u];
        const uint32_t words[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          count_one(words[k] & 0xffffu, 8 * i + 2 * k);
          count_one(words[k] >> 16, 8 * i + 2 * k + 1);
        }
      }
    }
    for (int i = nvec * 8 + tid; i < c.n_local; i += kThreads) {
      const uint32_t raw = src[i];
      c.stage[i] = (uint16_t)raw;
      count_one(raw, i);
    }
  }
  __syncthreads();  // so far every CTA has only touched its own slice and bins
  mark(1);

  // ---- B. penalties: move the history's tokens from the bins to the side list ----------
  // Every CTA walks the whole (id, count) list and handles the ids that live in its own
  // slice: the raw value comes from local shared memory, the list position is the S slot.
  const bool penalised = P.slot >= 0 && (P.repetition_penalty != 1.0f || P.presence_penalty != 0.0f ||
                                          P.frequency_penalty != 0.0f);
  int status = 0;
  int n_listed = 0;
  u64 side_best = 0;  // (key << 32 | ~id) of the best S element this thread has seen
  if (penalised) {
    n_listed = min(min(a.pool.n[P.slot], a.pool.unique_cap), args.s_cap);
    const int2* pairs = a.pool.pairs + (size_t)P.slot * a.pool.unique_cap;  // (token id, count)
    for (int j0 = tid; j0 < n_listed; j0 += 8 * kThreads) {
      int2 e[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int j = j0 + u * kThreads;
        e[u] = j < n_listed ? pairs[j] : make_int2(0x7fffffff, 0);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int j = j0 + u * kThreads;
        const int id = e[u].x;
        const int local = id - c.base;
        if ((unsigned)local >= (unsigned)c.n_local) {
          // not in this CTA's slice; rank 0 voids entries that are not tokens of this row
          if (c.rank == 0 && j < n_listed && (id < 0 || id >= a.vocab)) c.s_pair[j] = make_int2(-1, 0);
          continue;
        }
        const uint32_t raw = c.stage[local];
        c.stage[local] = (uint16_t)kSentinel;
        const int b = bin_of_raw(raw);
        if (b >= 0) atomicSub(&c.bins[b], 1u);
        float v = canonical(__uint_as_float(raw << 16));
        v = v < 0.0f ? __fmul_rn(v, P.repetition_penalty) : __fdiv_rn(v, P.repetition_penalty);
        v = __fsub_rn(v, P.presence_penalty);
        v = __fsub_rn(v, __fmul_rn(P.frequency_penalty, (float)e[u].y));
        const float s = c.score_of_value(v);
        c.s_pair[j] = make_int2(id, __float_as_int(s));
        const u64 packed = ((u64)key_of(s) << 32) | (uint32_t)(~(uint32_t)id);
        side_best = packed > side_best ? packed : side_best;
      }
    }
    __syncthreads();
  }
  // Unpenalised tokens outside the bin window join the side list with their own score.
  // First count this CTA's survivors (a penalised token is already in S), then, once the
  // counts of the lower-ranked CTAs are known, append them behind the listed entries.
  const int n_rare = *rare_n;
  const bool sweep = n_rare > kRareCap;
  auto is_rare = [&](int local) {
    const uint32_t raw = c.stage[local];
    return raw != kSentinel && bin_of_raw(raw) < 0;
  };
  {
    int mine = 0;
    auto look = [&](int local) {
      if (!is_rare(local)) return;
      ++mine;
      const float s = c.score_of_value(canonical(__uint_as_float((uint32_t)c.stage[local] << 16)));
      const u64 packed = ((u64)key_of(s) << 32) | (uint32_t)(~(uint32_t)(c.base + local));
      side_best = packed > side_best ? packed : side_best;
    };
    if (sweep) { for (int i = tid; i < c.n_local; i += kThreads) look(i); }
    else { for (int t = tid; t < n_rare; t += kThreads) look(rare_id[t]); }
    if (mine) atomicAdd(c.s_extra, mine);
  }
  side_best = block_max_u64(*c.x, side_best);
  mark(2);

  // ---- C. sum the per-CTA bins across the cluster; row maximum --------------------------
  uint32_t phase;
  {
    __syncthreads();
    const u64 vals[2] = {side_best, (u64)*c.s_extra};
    phase = cluster_publish<2>(c.cluster, *c.x, vals);  // first cluster-wide barrier
  }
  side_best = ring_reduce<RingOp::Max>(c.cluster, *c.x, phase, 0);
  {
    const int extra_total = (int)ring_reduce<RingOp::Sum>(c.cluster, *c.x, phase, 1);
    const int extra_before = (int)ring_prefix(c.cluster, *c.x, phase, 1, c.rank);
    c.n_s = n_listed + extra_total;
    if (c.n_s > args.s_cap) { c.n_s = args.s_cap; status |= 4; }
    if (*c.s_extra > 0) {  // CTA-uniform
      __syncthreads();
      if (tid == 0) *c.s_extra = 0;  // reused as the local append cursor
      __syncthreads();
      auto move_out = [&](int local) {
        if (!is_rare(local)) return;
        const int slot = n_listed + extra_before + atomicAdd(c.s_extra, 1);
        const uint32_t raw = c.stage[local];
        c.stage[local] = (uint16_t)kSentinel;
        if (slot >= args.s_cap) return;
        c.s_pair[slot] = make_int2(c.base + local,
                                   __float_as_int(c.score_of_value(canonical(__uint_as_float(raw << 16)))));
      };
      if (sweep) { for (int i = tid; i < c.n_local; i += kThreads) move_out(i); }
      else { for (int t = tid; t < n_rare; t += kThreads) move_out(rare_id[t]); }
    }
  }
  __threadfence();  // the side list is read by every CTA of the cluster after the next barrier
  if (c.nranks > 1) {
    for (int b = tid; b < per_bins; b += kThreads) {
      const int gb = (int)c.rank * per_bins + b;
      uint32_t sum = 0;
#pragma unroll
      for (unsigned r = 0; r < (unsigned)kMaxCluster; ++r) {
        if (r >= c.nranks) break;
        sum += c.cluster.map_shared_rank(c.bins, r)[gb];
      }
      c.bins_red[b] = sum;
    }
    c.sync_all();
    for (int gb = tid; gb < kValueBins; gb += kThreads) {
      const unsigned r = (unsigned)(gb / per_bins);
      c.bins[gb] = c.cluster.map_shared_rank(c.bins_red, r)[gb - (int)r * per_bins];
    }
    __syncthreads();
  } else {
    __syncthreads();
  }
  const int top_bin = highest_bin(c);
  const uint32_t side_key = (uint32_t)(side_best >> 32);
  const int side_arg = (int)(~(uint32_t)(side_best & 0xffffffffu));
  const uint32_t bins_key = top_bin >= 0 ? key_of(c.score_of_raw(raw_of_bin(top_bin))) : 0u;
  const bool any_side = side_best != 0;
  const uint32_t max_key = (top_bin >= 0 && (!any_side || bins_key >= side_key)) ? bins_key : side_key;
  c.m = score_of(max_key);
  const float m = c.m;

  mark(3);
  KeptSet kept{0u, 0x7fffffff};
  int token = -1;
  u64 n_topk = (u64)a.vocab, n_minp = (u64)a.vocab, n_kept = (u64)a.vocab;
  u64 q_kept = 0;
  bool have_totals = false;
  long long cut_ties = -1;

  if (c.greedy) {
    // arg max with the lowest id on ties, over both populations
    int id_bins = 0x7fffffff;
    if (top_bin >= 0 && bins_key >= side_key) id_bins = find_nth_raw(c, raw_of_bin(top_bin), 1);
    if (!any_side || (top_bin >= 0 && bins_key > side_key)) token = id_bins;
    else if (top_bin < 0 || side_key > bins_key) token = side_arg;
    else token = min(id_bins, side_arg);
    if (P.n_logprobs >= 0) {
      u64 cn, cs, ms;
      bins_totals(c, 0u, false, true, cn, q_kept);
      side_totals(c, 0u, true, cs, ms);
      q_kept += ms;
    }
  } else {
    u64 cnt = 0, mass = 0;
    auto refresh_totals = [&]() {
      u64 cn, mn, cs, ms;
      bins_totals(c, kept.cut_key, false, true, cn, mn);
      side_totals(c, kept.cut_key, true, cs, ms);
      cnt = cn + cs;
      mass = mn + ms;
      have_totals = true;
    };
    if (P.top_k > 0 && P.top_k < a.vocab) {
      Selection sk = select_union<false, true>(c, 0u, (u64)P.top_k, 1.0f);
      if (!sk.ok) status |= 1;
      kept.cut_key = sk.key;
      cnt = sk.above_cnt + sk.bin_cnt;
      mass = sk.above_mass + sk.bin_mass;
      have_totals = sk.ok;
      n_topk = cnt;
    }
    mark(4);
    if (P.min_p > 0.0f) {
      if (!have_totals) refresh_totals();
      const float z1 = mass_to_float(mass);
      const float thr = __fmul_rn(__fdiv_rn(1.0f, z1), P.min_p);
      uint32_t lowest = 0xffffffffu;
      auto consider = [&](float s) {
        const uint32_t k = key_of(s);
        if (k >= kept.cut_key && !(__fdiv_rn(expf(s - m), z1) < thr)) lowest = min(lowest, k);
      };
      for (int b = tid; b < kValueBins; b += kThreads)
        if (c.bins[b]) consider(c.score_of_raw(raw_of_bin(b)));
      for_each_side(c, [&](int, float s) { consider(s); });
      lowest = ~block_max_u32(*c.x, ~lowest);
      {
        const u64 vals[1] = {(u64)lowest};
        const uint32_t ph = cluster_publish<1>(c.cluster, *c.x, vals);
        lowest = (uint32_t)ring_reduce<RingOp::Min>(c.cluster, *c.x, ph, 0);
      }
      if (lowest != 0xffffffffu && lowest > kept.cut_key) {
        kept.cut_key = lowest;
        have_totals = false;
      }
    }
    mark(5);
    if (P.top_p < 1.0f) {
      Selection sp = select_union<true, true>(c, kept.cut_key, 0, P.top_p);
      n_minp = sp.total_cnt;
      if (sp.ok && sp.bin_cnt > 0) {
        const u64 qv = sp.bin_mass / sp.bin_cnt;  // every token at the cut key has the same mass
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
        mark(6);
        if (t < sp.bin_cnt) kept.tie_limit = tie_id_limit(c, sp.key, t);
      } else {
        status |= 1;
        cnt = sp.total_cnt;
        mass = sp.total_mass;
        have_totals = true;
      }
    } else {
      if (!have_totals) refresh_totals();
      n_minp = cnt;
    }
    n_kept = cnt;
    q_kept = mass;
    mark(7);

    // ---- draw --------------------------------------------------------------------------
    if (q_kept == 0) {
      status |= 1;
      token = any_side ? side_arg : 0;
    } else if (a.noise) {
      const float zf = mass_to_float(q_kept);
      const float* noise_row = a.noise + (size_t)c.row * a.vocab;
      u64 best = 0;
      auto race = [&](float s, int gid) {
        if (!kept.has(key_of(s), gid)) return;
        const float p = __fdiv_rn(expf(s - m), zf);
        const float ratio = __fdiv_rn(p, noise_row[gid]);
        const u64 packed = ((u64)__float_as_uint(ratio) << 32) | (uint32_t)(~(uint32_t)gid);
        best = packed > best ? packed : best;
      };
      for (int i = tid; i < c.n_local; i += kThreads) {
        const uint32_t raw = c.stage[i];
        if (raw != kSentinel) race(c.score_of_raw(raw), c.base + i);
      }
      for_each_side(c, [&](int id, float s) { race(s, id); });
      best = block_max_u64(*c.x, best);
      {
        const u64 vals[1] = {best};
        const uint32_t ph = cluster_publish<1>(c.cluster, *c.x, vals);
        best = ring_reduce<RingOp::Max>(c.cluster, *c.x, ph, 0);
      }
      token = (int)(~(uint32_t)(best & 0xffffffffu));
    } else {
      // Inverse CDF over exact integer masses: first the kept N tokens ordered by
      // (value descending, id ascending), then the kept S tokens by ascending id.
      const Philox4 r = philox4x32_10(0u, 0u, 0u, 0u, (uint32_t)P.seed, (uint32_t)(P.seed >> 32));
      const u64 r64 = ((u64)r.v[0] << 32) | r.v[1];
      const u64 target = __umul64hi(r64, q_kept);
      // kept N mass: bins above the cut, plus the kept part of the bin at the cut
      const int cut_bin = bin_with_key(c, kept.cut_key);
      u64 cut_bin_kept = 0;
      if (cut_bin >= 0) {
        cut_bin_kept = c.bins[cut_bin];
        if (kept.tie_limit != 0x7fffffff) cut_bin_kept = count_raw_upto(c, raw_of_bin(cut_bin), kept.tie_limit);
      }
      // each thread owns kPerBins consecutive bins, walking down from the top
      constexpr int kPerBins = kValueBins / kThreads;
      const int b_hi = kValueBins - 1 - kPerBins * tid;
      auto kept_in_bin = [&](int b, u64& q) -> u64 {
        u64 n = c.bins[b];
        q = 0;
        if (!n) return 0;
        const float s = c.score_of_raw(raw_of_bin(b));
        const uint32_t k = key_of(s);
        if (k < kept.cut_key) return 0;
        if (k == kept.cut_key) n = cut_bin_kept;
        if (n) q = mass_of(s, m);
        return n;
      };
      u64 chunk = 0;
#pragma unroll 1
      for (int u = 0; u < kPerBins; ++u) {
        u64 q;
        const u64 n = kept_in_bin(b_hi - u, q);
        chunk += n * q;
      }
      const u64 incl = warp_scan_u64(chunk);
      u64 pre, pre_unused, q_bins, tot_unused;
      block_warp_prefix2(*c.x, shfl_u64(incl, 31), 0, pre, pre_unused, q_bins, tot_unused);
      if (target < q_bins) {
        if (tid == 0) c.x->bcast[5] = 0;
        __syncthreads();
        u64 run = pre + incl - chunk;
        if (run <= target && target < run + chunk) {
#pragma unroll 1
          for (int u = 0; u < kPerBins; ++u) {
            u64 q;
            const u64 n = kept_in_bin(b_hi - u, q);
            const u64 w = n * q;
            if (w && target < run + w) {
              c.x->bcast[4] = (target - run) / q + 1;
              c.x->bcast[5] = (u64)raw_of_bin(b_hi - u) + 1;
              break;
            }
            run += w;
          }
        }
        __syncthreads();
        if (c.x->bcast[5] != 0) {
          token = find_nth_raw(c, (uint32_t)(c.x->bcast[5] - 1), c.x->bcast[4]);
        }
        if (token < 0 || token == 0x7fffffff) { token = any_side ? side_arg : 0; status |= 1; }
      } else {
        SideDrawFill fill{&c, kept};
        Selection sd = descend_core<true, true>(c, fill, 0u, target - q_bins + 1, -1.0f, 0, 1, 0x7FFu);
        if (sd.ok) token = (int)(~sd.key);
        else { token = any_side ? side_arg : 0; status |= 1; }
      }
    }
  }

  mark(8);
  // ---- D. log-probabilities -------------------------------------------------------------
  float log_z = 0.f;
  if (P.n_logprobs >= 0) {
    log_z = (float)(log((double)q_kept) - (double)kMassShift * 0.6931471805599453);
    if (token >= 0 && token < a.vocab) {
      const unsigned owner = (unsigned)(token / a.slice);
      bool in_side = true;
      if (c.rank == owner) {
        const uint32_t raw = c.stage[token - (int)owner * a.slice];
        if (raw != kSentinel) {
          in_side = false;
          if (tid == 0) out->logprob = (c.score_of_raw(raw) - m) - log_z;
        }
      }
      // a side token is found by whichever thread scans it; harmless if the owner already wrote
      for_each_side(c, [&](int id, float s) {
        if (id == token && in_side) out->logprob = (s - m) - log_z;
      });
    }
    int n_want = min(P.n_logprobs, a.vocab);
    if ((u64)n_want > n_kept) n_want = (int)n_kept;
    if (n_want > 0) {
      Selection sn = select_union<false, false>(c, kept.cut_key, (u64)n_want, 1.0f);
      if (sn.ok) {
        const u64 need = (u64)n_want - sn.above_cnt;
        u64 ties = sn.bin_cnt;
        if (sn.key == kept.cut_key && cut_ties >= 0) ties = (u64)cut_ties;
        int limit = sn.key == kept.cut_key ? kept.tie_limit : 0x7fffffff;
        if (need < ties) limit = tie_id_limit(c, sn.key, need);
        // collect exactly n_want tokens: score above the N-th key, or at it with a low enough id
        const GatherSlot g = begin_gather(c);
        ListEntry* dst = g.dst;
        int* dst_n = g.dst_n;
        auto take = [&](float s, int gid) {
          const uint32_t k = key_of(s);
          if (k > sn.key || (k == sn.key && gid <= limit)) {
            const int slot = atomicAdd(dst_n, 1);
            if (slot < kListCap) dst[slot] = ListEntry{k, gid, 1u, 0u, 0ull};
          }
        };
        // in the slice only values whose bin reaches the N-th key can qualify
        const int b_min = lowest_bin_at_or_above(c, sn.key);
        for (int i = tid; i < c.n_local; i += kThreads) {
          const uint32_t raw = c.stage[i];
          if (bin_of_raw(raw) < b_min) continue;  // also skips moved-out slots (bin -1)
          take(c.score_of_raw(raw), c.base + i);
        }
        for_each_side(c, [&](int id, float s) { take(s, id); });
        end_gather(c, g);
        if (c.rank == 0 && tid < 32) {
          const int n = min(*dst_n, HS_MAX_LOGPROBS);
          uint32_t kv = 0;
          int id = 0x7fffffff;
          if (tid < n) { kv = dst[tid].key; id = dst[tid].id; }
          int pos = 0;
          for (int j = 0; j < n; ++j) {
            const uint32_t kj = __shfl_sync(0xffffffffu, kv, j);
            const int idj = __shfl_sync(0xffffffffu, id, j);
            if (kj > kv || (kj == kv && idj < id)) ++pos;
          }
          if (tid < n) {
            out->top_ids[pos] = id;
            out->top_logprobs[pos] = (score_of(kv) - m) - log_z;
          }
          if (tid == 0 && n != n_want) status |= 8;
        }
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

  mark(9);
  // ---- E. optional dump of the final scores (parity tests) -------------------------------
  if (a.scores_out) {
    float* dst = a.scores_out + (size_t)c.row * a.vocab;
    const float ninf = __int_as_float(0xff800000);
    for (int i = tid; i < c.n_local; i += kThreads) {
      const uint32_t raw = c.stage[i];
      if (raw == kSentinel) continue;
      const float s = c.score_of_raw(raw);
      dst[c.base + i] = (c.greedy || kept.has(key_of(s), c.base + i)) ? s : ninf;
    }
    for_each_side(c, [&](int id, float s) {
      dst[id] = (c.greedy || kept.has(key_of(s), id)) ? s : ninf;
    });
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
    if ((a.flags & HS_SAMPLE_APPEND_TOKEN) && P.slot >= 0 && token >= 0 && token < a.vocab) {
      if (!slot_append_one(a.pool, P.slot, token)) out->status = status | 2;
    }
  }
  // No CTA may leave while a peer can still read its shared memory.
  c.sync_all();
  mark(10);
}

}  // namespace hs
