// Radix selection over a thread-block cluster: per-level histograms of count and exact
// probability mass in shared memory, merged across the cluster through distributed shared
// memory, and a descending scan that finds the bucket where a running count or mass
// reaches its target.  The elements are supplied by a `Fill` functor, so the same core
// serves a row resident as fp32, a sparse side list plus per-value counts, or ids.
#pragma once

#include "hs_common.cuh"

namespace hs {

struct Hist {
  uint32_t cnt[kBins];  // after the merge: full_cnt
  uint32_t l0[kBins];   // after the merge: full_mass (u64) spans l0 and l1
  uint32_t l1[kBins];
  uint32_t l2[kBins];
};

struct Selection {
  uint32_t key;               // selected key; when `levels` < 3 only its top bits (prefix) are known
  uint32_t prefix;            // resolved high bits, right aligned
  int levels;                 // radix levels resolved: 3 = the full 32-bit key
  u64 above_cnt, above_mass;  // over elements with key above the selected key / bucket
  u64 bin_cnt, bin_mass;      // over elements inside the selected key / bucket
  u64 total_cnt, total_mass;  // over all elements with key >= lo
  u64 target;                 // the count / mass that was searched for
  bool ok;
};

struct ClusterCtx {
  cg::cluster_group cluster;
  unsigned rank, nranks;
  Hist* hist;
  uint32_t* red_cnt;
  u64* red_mass;
  Exchange* x;
  __device__ __forceinline__ void sync_all() {
    if (nranks > 1) cluster.sync(); else __syncthreads();
  }
};

__device__ __forceinline__ int level_shift(int level) { return level == 0 ? 21 : (level == 1 ? 10 : 0); }
__device__ __forceinline__ int level_bits(int level) { return level < 2 ? 11 : 10; }

// Adds a contribution (count, mass) to a bucket of the CTA-local level histogram.  Plain
// shared-memory atomics: the hardware combines lanes that hit the same address (measured
// ~29 atomics/clk/SM for one address, ~7 for random addresses, which are bank-conflict
// bound), so no software pre-aggregation is done.
template <bool WITH_MASS>
struct HistAdder {
  Hist* h;
  __device__ __forceinline__ void operator()(bool valid, uint32_t bin, uint32_t count, u64 mass) const {
    if (!valid) return;
    atomicAdd(&h->cnt[bin], count);
    if (WITH_MASS) {
      const uint32_t a0 = (uint32_t)mass & kLimbMask;
      const uint32_t a1 = (uint32_t)(mass >> kLimbBits) & kLimbMask;
      const uint32_t a2 = (uint32_t)(mass >> (2 * kLimbBits));
      if (a0) atomicAdd(&h->l0[bin], a0);
      if (a1) atomicAdd(&h->l1[bin], a1);
      if (a2) atomicAdd(&h->l2[bin], a2);
    }
  }
};

// Smallest integer mass A with float(A / total) > top_p, i.e. the cumulative mass at which
// the reference's `cumulative > top_p` first becomes true (sampling.py:136).
__device__ __forceinline__ u64 top_p_target(u64 total, float top_p) {
  const double tot = (double)total;
  const float up = __uint_as_float(__float_as_uint(top_p) + 1u);
  const double mid = 0.5 * ((double)top_p + (double)up);
  double guess = floor(mid * tot) - 2.0;
  u64 a = guess < 1.0 ? 1ull : (u64)guess;
  for (int i = 0; i < 8; ++i) {
    if ((float)((double)a / tot) > top_p) break;
    ++a;
  }
  if (a > total) a = total;
  if (a < 1) a = 1;
  return a;
}

// The same value, worked out by the 32 lanes of one warp together (all must call): lane l tries
// the l-th candidate above the first guess and the lowest that passes wins, so the slow
// double-precision divisions run side by side instead of one after the other.
__device__ __forceinline__ u64 top_p_target_warp(u64 total, float top_p) {
  const double tot = (double)total;
  const float up = __uint_as_float(__float_as_uint(top_p) + 1u);
  const double mid = 0.5 * ((double)top_p + (double)up);
  const double guess = floor(mid * tot) - 2.0;
  const u64 a0 = guess < 1.0 ? 1ull : (u64)guess;
  const u64 mine = a0 + (threadIdx.x & 31);
  const bool pass = (threadIdx.x & 31) >= 8 || (float)((double)mine / tot) > top_p;  // (the scalar version stops after 8 steps too)
  const uint32_t votes = __ballot_sync(0xffffffffu, pass);
  u64 a = a0 + (u64)(__ffs(votes) - 1);
  if (a > total) a = total;
  if (a < 1) a = 1;
  return a;
}

// Walks keys downwards from the top until the running count (BY_MASS = false) or mass
// (BY_MASS = true) reaches the target.  fill(level, shift, bits, prefix, lo_key, add)
// must call add(valid, bucket, count, mass), with all lanes of each warp together, where
// valid marks an element with key >= lo_key whose bits above `shift + bits` equal `prefix`
// (level 0: all), and bucket = (key >> shift) & mask.
// Stops early, with sel.levels < 3, once the selected bucket holds at most stop_pop
// elements (stop_pop = 0: always resolve all 32 bits).
template <bool BY_MASS, bool WITH_MASS, class Fill>
__device__ Selection descend_core(ClusterCtx& c, Fill& fill, uint32_t lo_key, u64 target_cnt,
                                  float top_p, u64 stop_pop = 0, int first_level = 0,
                                  uint32_t prefix0 = 0) {
  static_assert(WITH_MASS || !BY_MASS, "a mass descent needs masses");
  Hist& h = *c.hist;
  u64* full_mass = reinterpret_cast<u64*>(h.l0);
  uint32_t* full_cnt = h.cnt;
  Selection sel;
  sel.above_cnt = sel.above_mass = 0;
  sel.total_cnt = sel.total_mass = 0;
  sel.bin_cnt = sel.bin_mass = 0;
  sel.target = target_cnt;
  sel.ok = true;
  sel.levels = first_level;
  uint32_t prefix = prefix0;
  const int per = kBins / (int)c.nranks;
  const int tid = threadIdx.x;
  const HistAdder<WITH_MASS> add{&h};

  for (int level = first_level; level < 3; ++level) {
    const int shift = level_shift(level);
    const int bits = level_bits(level);
    for (int b = tid; b < kBins; b += kThreads) {
      h.cnt[b] = 0;
      if (WITH_MASS) { h.l0[b] = 0; h.l1[b] = 0; h.l2[b] = 0; }
    }
    __syncthreads();
    fill(level, shift, bits, prefix, lo_key, add);
    c.sync_all();
    // reduce-scatter: this CTA sums buckets [rank*per, (rank+1)*per) over the cluster
    for (int b = tid; b < per; b += kThreads) {
      const int gb = (int)c.rank * per + b;
      uint32_t cn = 0;
      u64 ms = 0;
#pragma unroll
      for (unsigned r = 0; r < (unsigned)kMaxCluster; ++r) {
        if (r >= c.nranks) break;
        const Hist* rh = c.nranks > 1 ? c.cluster.map_shared_rank(c.hist, r) : c.hist;
        cn += rh->cnt[gb];
        if (WITH_MASS)
          ms += (u64)rh->l0[gb] + ((u64)rh->l1[gb] << kLimbBits) + ((u64)rh->l2[gb] << (2 * kLimbBits));
      }
      c.red_cnt[b] = cn;
      c.red_mass[b] = ms;
    }
    c.sync_all();
    // all-gather the merged buckets into this CTA (over the now unused local arrays)
    for (int gb = tid; gb < kBins; gb += kThreads) {
      const unsigned r = (unsigned)(gb / per);
      const int b = gb - (int)r * per;
      const uint32_t* rc = c.nranks > 1 ? c.cluster.map_shared_rank(c.red_cnt, r) : c.red_cnt;
      const u64* rm = c.nranks > 1 ? c.cluster.map_shared_rank(c.red_mass, r) : c.red_mass;
      full_cnt[gb] = rc[b];
      full_mass[gb] = WITH_MASS ? rm[b] : 0ull;
    }
    if (tid == 0) c.x->bcast[7] = 0;
    __syncthreads();
    // scan buckets from the top: thread t owns kPer consecutive buckets ending at `hi`
    constexpr int kPer = kBins / kThreads;
    const int hi = kBins - 1 - kPer * tid;
    u64 c_sum = 0, m_sum = 0;
#pragma unroll
    for (int u = 0; u < kPer; ++u) { c_sum += full_cnt[hi - u]; m_sum += full_mass[hi - u]; }
    u64 ia = warp_scan_u64(c_sum);
    u64 ib = warp_scan_u64(m_sum);
    u64 pa, pb, ta, tb;
    block_warp_prefix2(*c.x, shfl_u64(ia, 31), shfl_u64(ib, 31), pa, pb, ta, tb);
    u64 ex_cnt = pa + ia - c_sum;   // exclusive prefix over buckets above `hi`
    u64 ex_mass = pb + ib - m_sum;
    if (level == first_level) {
      sel.total_cnt = ta;
      sel.total_mass = tb;
      if (BY_MASS && top_p >= 0.0f) sel.target = top_p_target(tb, top_p);  // top_p < 0: explicit mass target
    }
    const u64 want = sel.target - (BY_MASS ? sel.above_mass : sel.above_cnt);
    {
      const u64 ex = BY_MASS ? ex_mass : ex_cnt;
      const u64 mine = BY_MASS ? m_sum : c_sum;
      if (ex < want && want <= ex + mine) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
          const u64 bc = full_cnt[hi - u], bm = full_mass[hi - u];
          const u64 e = BY_MASS ? ex_mass : ex_cnt;
          if (want <= e + (BY_MASS ? bm : bc)) {
            c.x->bcast[0] = (u64)(hi - u);
            c.x->bcast[1] = ex_cnt;
            c.x->bcast[2] = ex_mass;
            c.x->bcast[3] = bc;
            c.x->bcast[4] = bm;
            c.x->bcast[7] = 1;
            break;
          }
          ex_cnt += bc;
          ex_mass += bm;
        }
      }
    }
    __syncthreads();
    if (c.x->bcast[7] == 0) {  // nothing reaches the target (non-finite input)
      sel.ok = false;
      sel.key = lo_key;
      sel.prefix = prefix;
      sel.bin_cnt = sel.bin_mass = 0;
      __syncthreads();
      return sel;
    }
    const uint32_t bin = (uint32_t)c.x->bcast[0];
    sel.above_cnt += c.x->bcast[1];
    sel.above_mass += c.x->bcast[2];
    sel.bin_cnt = c.x->bcast[3];
    sel.bin_mass = c.x->bcast[4];
    prefix = (prefix << bits) | bin;
    sel.levels = level + 1;
    __syncthreads();  // bcast and the aliased arrays are reused by the next level
    if (stop_pop && level < 2 && sel.bin_cnt <= stop_pop) break;
  }
  sel.prefix = prefix;
  sel.key = sel.levels == 3 ? prefix : (prefix << (sel.levels == 1 ? 21 : 10));
  return sel;
}

}  // namespace hs
