// The fused per-row sampling kernel for bf16 logits (the serving default): one CTA per row.
//
// Everything the sampler needs to know about a bf16 row fits in COUNTS.  A token's final
// score is a function of its raw bf16 value and of how often the request's history holds
// it, so tokens fall into classes (count class c in {0, 1, 2}, value bin b), and all tokens
// of a class share one score and one probability mass.  The kernel streams the row from
// HBM once, 128 bits at a time, together with the request's dense 2-bit count classes
// (V/4 bytes), and counts tokens per class with shared-memory atomics: three tables of
// 6,144 one-value bins (2^-14 <= |x| < 2^10).  The few tokens that do not fit a class --
// history count >= 3 (listed per request), or a value outside the bin window -- become
// individual (id, score) entries of a small side list.
//
// Selection (top-k by count, min-p by threshold, top-p by probability mass, top-N for the
// log-probabilities) is a radix descent over 32-bit order-preserving keys of the class
// scores: each non-empty class contributes (count, count * mass) to a bucket, the buckets
// are scanned from the top, and once the deciding bucket holds few members they are
// gathered, sorted and resolved exactly.  Probability mass is an integer multiple of 2^-40,
// so all sums are exact and order-independent.
//
// Token ids are only needed at the very end ("a uniformly chosen member of this class",
// "the lowest ids of this tie group").  A class of more than kV3ListCap tokens is sampled by
// rejection: Philox-drawn positions are probed until one belongs to the class (exactly
// uniform over its members); a lone CTA issues scattered reads slowly, so a smaller class,
// or one the probes keep missing, is found by scanning the row once more for its bit
// pattern.  Lowest-id tie-breaks walk the row hierarchically.
//
// A row's CTA keeps the count table, a short side list and (once the table has served, in its
// place) the selection histograms in shared memory, about 88 KB, so that two CTAs share an
// SM and one row's barrier-bound selection phases overlap another row's counting.  The list
// of the row's non-empty classes (16 bytes each) lives in per-CTA global scratch and is
// streamed from L2.  What is left of L1 is small, so the streaming loads go past it.
#pragma once

#include "hs_common.cuh"
#include "hs_select.cuh"
#include "hs_state.cuh"
#include "hs_row_kernel.cuh"
#include "../../include/hs_sampler.h"

namespace hs {

constexpr int kV3Half = 3072;                 // 24 binades x 128 mantissas
constexpr int kV3Bins = 2 * kV3Half;          // per count class
constexpr int kCells = 3 * kV3Bins;           // count classes 0, 1, 2
constexpr uint32_t kV3Base = 113u << 7;       // smallest binned magnitude: 2^-14
constexpr int kV3ListCap = 256;               // members resolved by sorting
constexpr int kV3RejectMin = 128;             // classes of up to this many tokens are found by scanning the row, larger ones by rejection
constexpr int kV3ScanCap = 1024;              // ids one class scan can hold (in the gather and list buffers)
#ifndef HS_RARE_CAP
#define HS_RARE_CAP 512
#endif
#ifndef HS_SIDE_SHARED
#define HS_SIDE_SHARED 1024
#endif
constexpr int kV3RareCap = HS_RARE_CAP;               // out-of-window tokens remembered before a sweep
constexpr int kV3SideShared = HS_SIDE_SHARED;           // side-list entries kept in shared memory (else global scratch)
constexpr int kV3PhaseSlots = 64;
#ifndef HS_DEFER_CAP
#define HS_DEFER_CAP 2048
#endif
constexpr int kV3DeferCap = HS_DEFER_CAP;             // chunks the counting loop sets aside for the token-by-token pass
constexpr int kSplitCap = 4096;               // candidate entries one CTA of a split row can hand over

struct V3Entry {
  uint32_t key;  // 32-bit key of the score
  int32_t id;    // token id of a side element, -1 for a class
  uint32_t cnt;  // tokens this entry stands for
  uint32_t cell; // class index (count class * kV3Bins + bin) of a class entry
  u64 q;         // mass of one token
};

struct LocalHist {
  uint32_t ent[kBins];  // entries (classes + side elements) per bucket
  uint32_t cnt[kBins];
  uint32_t l0[kBins], l1[kBins], l2[kBins];  // mass in 14-bit limbs: 32-bit shared atomics only
  __device__ __forceinline__ u64 mass(int b) const {
    return (u64)l0[b] + ((u64)l1[b] << kLimbBits) + ((u64)l2[b] << (2 * kLimbBits));
  }
};

// A non-empty class with its score key and mass, computed once per row.  Stored in 16 bytes
// in the CTA's global scratch and handed to the visitors of for_each_class unpacked.
struct __align__(16) ClassPacked {
  uint32_t key;  // 32-bit key of the class score
  uint32_t cnt;  // tokens in the class
  u64 qc;        // bits 0..47: mass of one token (<= 2^40); bits 48..63: count class * kV3Bins + bin
};
struct ClassEntry {
  uint32_t key, cnt, cell;
  u64 q;  // mass of one token
  u64 w;  // cnt * q
};
__device__ __forceinline__ ClassEntry unpack_class(const uint4& v) {
  ClassEntry e;
  e.key = v.x;
  e.cnt = v.y;
  e.cell = v.w >> 16;
  e.q = ((u64)(v.w & 0xffffu) << 32) | v.z;
  e.w = (u64)e.cnt * e.q;
  return e;
}
__device__ __forceinline__ uint4 pack_class(uint32_t key, uint32_t cnt, uint32_t cell, u64 q) {
  return make_uint4(key, cnt, (uint32_t)q, (uint32_t)(q >> 32) | (cell << 16));
}

struct RowV3Args {
  RowKernelArgs base;
  ClassPacked* clist;  // [n_scratch, kCells] scratch: the class list of the row a CTA is working on
  int2* s_pair;   // [n_scratch, s_cap] side lists too long for shared memory: (token id or -1, fp32 bits of the score)
  int s_cap;
  int n_scratch;       // scratch sets: as many as CTAs of the kernel can be resident at once
  int* scratch_busy;   // [n_scratch] 1 while a CTA holds the set
  unsigned long long* phase_clocks;  // [batch, kV3PhaseSlots] or null
  int csplit;                        // CTAs per row on the counting path (1, 2 or 4)
  uint32_t* ctab;                    // [batch, csplit, kCells] count tables handed over by the parts of a row
  int2* crare;                       // [batch, csplit, kV3RareCap] their rare lists
  int* crare_n;                      // [batch, csplit]
  int* count_ticket;                 // [batch] arrival counter (returns to 0)
  int split;                         // CTAs per row on the candidate path
  unsigned long long* split_lists;   // [batch, split, kSplitCap] candidate lists of the row's CTAs
  int* split_n;                      // [batch, split] their lengths
  int* split_ticket;                 // [batch] arrival counter (returns to 0)
  int batch;                         // rows in the launch
};

// Shared memory of a counting row.  The selection histograms and the two member buffers are
// only needed after the count table has been turned into the class list, and take its place.
struct LayoutV3 {
  size_t x, tab, hist, gbuf, list, side, rare, defer, small, total;
};
__host__ __device__ inline LayoutV3 layout_v3() {
  LayoutV3 l{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = (off + bytes + 15) & ~size_t(15);
    return at;
  };
  l.x = take(sizeof(Exchange));
  l.tab = take(sizeof(uint32_t) * kCells);
  {
    size_t in_tab = l.tab;
    auto sub = [&](size_t bytes) {
      const size_t at = in_tab;
      in_tab = (in_tab + bytes + 15) & ~size_t(15);
      return at;
    };
    l.hist = sub(sizeof(LocalHist));
    l.gbuf = sub(sizeof(V3Entry) * kV3ListCap);
    l.list = sub(sizeof(V3Entry) * kV3ListCap);
  }
  l.side = take(sizeof(int2) * kV3SideShared);
  l.rare = take(sizeof(int2) * kV3RareCap);
  l.defer = take(sizeof(int) * kV3DeferCap);
  l.small = take(sizeof(int) * 32);
  l.total = off;
  return l;
}
static_assert(sizeof(LocalHist) + 2 * sizeof(V3Entry) * kV3ListCap + 32 <= sizeof(uint32_t) * kCells,
              "the selection buffers fit in the count table's place");

__device__ __forceinline__ int v3_bin_of_raw(uint32_t raw) {
  const uint32_t idx = (raw & 0x7fffu) - kV3Base;
  if (idx >= (uint32_t)kV3Half) return -1;
  return (raw & 0x8000u) ? kV3Half - 1 - (int)idx : kV3Half + (int)idx;
}
__device__ __forceinline__ uint32_t v3_raw_of_bin(int b) {
  return b >= kV3Half ? (uint32_t)(b - kV3Half) + kV3Base
                      : 0x8000u | ((uint32_t)(kV3Half - 1 - b) + kV3Base);
}

struct Ctx3 {
  Exchange* x;
  uint32_t* tab;     // [kCells] tokens per class
  LocalHist* hist;
  V3Entry* gbuf;     // gather buffer
  V3Entry* list;     // sorted members
  int* gbuf_n;
  int* step_n = nullptr;  // two counters the early-exit scan alternates between
  int row, vocab;
  unsigned long long* dbg = nullptr;
  int lo, hi;                    // token range this CTA streams in the candidate path (lo a multiple of 8)
  const unsigned short* logits;  // this row
  const uint32_t* cls;           // this row's 2-bit classes, or null (no penalties)
  bool vec;                      // row start is 16-byte aligned
  Pool pool;
  int slot;
  int2* s_pair;
  int n_s, s_cap;
  ClassPacked* cl;   // this row's non-empty classes (global scratch of this CTA)
  // entry i of the row's class list
  __device__ __forceinline__ ClassEntry class_at(int i) const {
    return unpack_class(__ldcg(reinterpret_cast<const uint4*>(cl) + i));
  }
  int n_cl;
  float T, rp, pp, fp;
  bool greedy;
  float m;
  // Linear bucketing of the first level of a mass descent (see descend_local): bucket =
  // (score - lin_lo) * lin_scale, which grows with the key like the key's own top bits do,
  // but spreads a row whose scores lie close together over all buckets.
  bool lin = false;
  float lin_lo = 0.f, lin_scale = 0.f;
  __device__ __forceinline__ uint32_t lin_bucket(uint32_t key) const {
    const float t = (hs::score_of(key) - lin_lo) * lin_scale;
    return (uint32_t)min(max(__float2int_rz(t), 0), kBins - 1);
  }

  __device__ __forceinline__ float score_of_value(float v) const {
    return greedy ? canonical(v) : canonical(__fdiv_rn(v, T));
  }
  // score of a token with raw value bits `raw` that the history holds `count` times
  __device__ __forceinline__ float score_of(uint32_t raw, int count) const {
    float v = canonical(__uint_as_float(raw << 16));
    if (count > 0) {
      v = v < 0.0f ? __fmul_rn(v, rp) : __fdiv_rn(v, rp);
      v = __fsub_rn(v, pp);
      v = __fsub_rn(v, __fmul_rn(fp, (float)count));
    }
    return score_of_value(v);
  }
  __device__ __forceinline__ float cell_score(int cell) const {
    const int c = cell / kV3Bins;
    return score_of(v3_raw_of_bin(cell - c * kV3Bins), c);
  }
  __device__ __forceinline__ int class_of(int id) const {
    return cls ? (int)((cls[id >> 4] >> ((id & 15) * 2)) & 3u) : 0;
  }
  // exact history count of a token of class 3
  __device__ __forceinline__ int heavy_count(int id) const {
    const int q = (pool.pos + (size_t)slot * pool.pos_stride)[id];
    return q > 0 ? (pool.pairs + (size_t)slot * pool.unique_cap)[q - 1].y : 0;
  }
  // score of the token at position id, whatever population it belongs to
  __device__ __forceinline__ float element_score(int id, uint32_t raw, int c) const {
    return score_of(raw, c == 3 ? heavy_count(id) : c);
  }
};

template <class F>
__device__ __forceinline__ void for_each_side3(const Ctx3& c, F&& f) {
  for (int j0 = threadIdx.x; j0 < c.n_s; j0 += 4 * kThreads) {
    int2 e[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * kThreads;
      e[u] = j < c.n_s ? c.s_pair[j] : make_int2(-1, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (e[u].x >= 0) f(e[u].x, __int_as_float(e[u].y));
  }
}
// Calls f(entry) for the row's non-empty classes, thread t taking entries t, t + kThreads, ...
// (four 16-byte loads in flight per thread; the list sits in L2).
template <class F>
__device__ __forceinline__ void for_each_class(const Ctx3& c, F&& f) {
  const uint4* src = reinterpret_cast<const uint4*>(c.cl);
  for (int i0 = threadIdx.x; i0 < c.n_cl; i0 += 4 * kThreads) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * kThreads;
      if (i < c.n_cl) v[u] = __ldcg(src + i);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * kThreads;
      if (i >= c.n_cl) break;
      f(unpack_class(v[u]));
    }
  }
}

// ---- radix descent inside one CTA ----------------------------------------------------
struct LocalAdder {
  LocalHist* h;
  __device__ __forceinline__ void operator()(bool valid, uint32_t bin, uint32_t count, u64 mass) const {
    if (!valid) return;
    atomicAdd(&h->ent[bin], 1u);
    atomicAdd(&h->cnt[bin], count);
    const uint32_t a0 = (uint32_t)mass & kLimbMask;
    const uint32_t a1 = (uint32_t)(mass >> kLimbBits) & kLimbMask;
    const uint32_t a2 = (uint32_t)(mass >> (2 * kLimbBits));
    if (a0) atomicAdd(&h->l0[bin], a0);
    if (a1) atomicAdd(&h->l1[bin], a1);
    if (a2) atomicAdd(&h->l2[bin], a2);
  }
};

template <bool BY_MASS, class Fill>
__device__ Selection descend_local(Ctx3& c, Fill& fill, uint32_t lo_key, u64 target_cnt, float top_p,
                                   u64 stop_pop = 0, int first_level = 0, uint32_t prefix0 = 0) {
  LocalHist& h = *c.hist;
  Selection sel;
  sel.above_cnt = sel.above_mass = 0;
  sel.total_cnt = sel.total_mass = 0;
  sel.bin_cnt = sel.bin_mass = 0;
  sel.target = target_cnt;
  sel.ok = true;
  sel.levels = first_level;
  uint32_t prefix = prefix0;
  const int tid = threadIdx.x;
  const LocalAdder add{&h};
  for (int level = first_level; level < 3; ++level) {
    const int shift = level_shift(level);
    const int bits = level_bits(level);
    for (int b = tid; b < kBins; b += kThreads) { h.ent[b] = 0; h.cnt[b] = 0; h.l0[b] = 0; h.l1[b] = 0; h.l2[b] = 0; }
    if (tid == 0) c.x->bcast[7] = 0;
    __syncthreads();
    if (c.dbg && tid == 0 && BY_MASS && level == first_level) c.dbg[16] = clock64();
    fill(level, shift, bits, prefix, lo_key, add);
    __syncthreads();
    if (c.dbg && tid == 0 && BY_MASS && level == first_level) c.dbg[17] = clock64();
    constexpr int kPer = kBins / kThreads;
    const int hi = kBins - 1 - kPer * tid;
    u64 c_sum = 0, m_sum = 0;
#pragma unroll
    for (int u = 0; u < kPer; ++u) { c_sum += h.cnt[hi - u]; m_sum += h.mass(hi - u); }
    const u64 ia = warp_scan_u64(c_sum);
    const u64 ib = warp_scan_u64(m_sum);
    if (c.dbg && tid == 0 && BY_MASS && level == first_level) c.dbg[30] = clock64();
    u64 pa, pb, ta, tb;
    block_warp_prefix2(*c.x, shfl_u64(ia, 31), shfl_u64(ib, 31), pa, pb, ta, tb);
    if (c.dbg && tid == 0 && BY_MASS && level == first_level) c.dbg[31] = clock64();
    u64 ex_cnt = pa + ia - c_sum;
    u64 ex_mass = pb + ib - m_sum;
    if (level == first_level) {
      sel.total_cnt = ta;
      sel.total_mass = tb;
      if (BY_MASS && top_p >= 0.0f) {
        // (double precision, slow: the lanes of one warp try neighbouring candidates at once)
        if (tid < 32) {
          const u64 t = top_p_target_warp(tb, top_p);
          if (tid == 0) c.x->bcast[6] = t;
        }
        __syncthreads();
        sel.target = c.x->bcast[6];
      }
    }
    if (c.dbg && tid == 0 && BY_MASS && level == first_level) c.dbg[32] = clock64();
    const u64 want = sel.target - (BY_MASS ? sel.above_mass : sel.above_cnt);
    {
      const u64 ex = BY_MASS ? ex_mass : ex_cnt;
      const u64 mine = BY_MASS ? m_sum : c_sum;
      if (ex < want && want <= ex + mine) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
          const u64 bc = h.cnt[hi - u], bm = h.mass(hi - u);
          const u64 e = BY_MASS ? ex_mass : ex_cnt;
          if (want <= e + (BY_MASS ? bm : bc)) {
            c.x->bcast[0] = (u64)(hi - u);
            c.x->bcast[1] = ex_cnt;
            c.x->bcast[2] = ex_mass;
            c.x->bcast[3] = bc;
            c.x->bcast[4] = bm;
            c.x->bcast[5] = h.ent[hi - u];
            c.x->bcast[7] = 1;
            break;
          }
          ex_cnt += bc;
          ex_mass += bm;
        }
      }
    }
    __syncthreads();
    if (c.x->bcast[7] == 0) {
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
    const u64 entries = c.x->bcast[5];
    prefix = (prefix << bits) | bin;
    sel.levels = level + 1;
    __syncthreads();
    if (c.dbg && tid == 0 && BY_MASS && level == first_level) c.dbg[18] = clock64();
    if (stop_pop && level < 2 && entries <= stop_pop) break;  // few enough members to sort
    if (c.lin && level == 0) {
      // the linear buckets did not separate the row: once more, by the key's own bits
      c.lin = false;
      sel.above_cnt = sel.above_mass = 0;
      prefix = prefix0;
      level = first_level - 1;
    }
  }
  sel.prefix = prefix;
  sel.key = sel.levels == 3 ? prefix : (prefix << (sel.levels == 1 ? 21 : 10));
  return sel;
}

// All tokens of the row: side elements individually, classes as (count, count * mass).
template <bool WITH_MASS>
struct UnionFill3 {
  Ctx3* c;
  template <class Add>
  __device__ __forceinline__ void operator()(int level, int shift, int bits, uint32_t prefix,
                                             uint32_t lo_key, const Add& add) const {
    const uint32_t mask = (1u << bits) - 1u;
    auto ok = [&](uint32_t k) { return k >= lo_key && (level == 0 || (k >> (shift + bits)) == prefix); };
    const bool lin = c->lin && level == 0;
    for_each_side3(*c, [&](int, float s) {
      const uint32_t k = key_of(s);
      const bool valid = ok(k);
      add(valid, lin ? c->lin_bucket(k) : (k >> shift) & mask, 1u, (WITH_MASS && valid) ? mass_of(s, c->m) : 0ull);
    });
    for_each_class(*c, [&](const ClassEntry& e) {
      add(ok(e.key), lin ? c->lin_bucket(e.key) : (e.key >> shift) & mask, e.cnt, WITH_MASS ? e.w : 0ull);
    });
  }
};

// Kept side elements keyed by ~id with their mass: the side part of the draw.
struct SideDrawFill3 {
  Ctx3* c;
  uint32_t cut_key;
  template <class Add>
  __device__ __forceinline__ void operator()(int level, int shift, int bits, uint32_t prefix,
                                             uint32_t, const Add& add) const {
    const uint32_t mask = (1u << bits) - 1u;
    for_each_side3(*c, [&](int id, float s) {
      const uint32_t k = ~(uint32_t)id;
      const bool valid = key_of(s) > cut_key && (level == 0 || (k >> (shift + bits)) == prefix);
      add(valid, (k >> shift) & mask, 1u, valid ? mass_of(s, c->m) : 0ull);
    });
  }
};

// Gathers the members (side elements, classes) with key >= lo_key whose top `levels` radix
// digits equal `prefix` into `list`, sorted by (key descending, classes first, id ascending).
__device__ int gather_members3(Ctx3& c, uint32_t lo_key, int levels, uint32_t prefix) {
  const int tid = threadIdx.x;
  if (tid == 0) *c.gbuf_n = 0;
  __syncthreads();
  const int drop = levels == 1 ? 21 : (levels == 2 ? 10 : 0);
  const bool lin = c.lin && levels == 1;
  auto matches = [&](uint32_t k) {
    if (k < lo_key) return false;
    if (lin) return c.lin_bucket(k) == prefix;
    return levels == 0 || (levels == 3 ? k == prefix : (k >> drop) == prefix);
  };
  for_each_side3(c, [&](int id, float s) {
    const uint32_t k = key_of(s);
    if (!matches(k)) return;
    const int slot = atomicAdd(c.gbuf_n, 1);
    if (slot < kV3ListCap) c.gbuf[slot] = V3Entry{k, id, 1u, 0u, mass_of(s, c.m)};
  });
  for_each_class(c, [&](const ClassEntry& e) {
    if (!matches(e.key)) return;
    const int slot = atomicAdd(c.gbuf_n, 1);
    if (slot < kV3ListCap) c.gbuf[slot] = V3Entry{e.key, -1, e.cnt, e.cell, e.q};
  });
  __syncthreads();
  if (c.dbg && tid == 0) c.dbg[20] = clock64();
  const int n = min(*c.gbuf_n, kV3ListCap);
  if (tid < n) {
    const V3Entry mine = c.gbuf[tid];
    int pos = 0;
    for (int j = 0; j < n; ++j) {
      const uint32_t kj = c.gbuf[j].key;
      const int idj = c.gbuf[j].id;
      // classes (id -1) sort before side elements of the same key; two classes of one key
      // are ordered by their class index
      const bool before = kj > mine.key ||
                          (kj == mine.key && (idj < mine.id || (idj == mine.id && c.gbuf[j].cell < mine.cell)));
      pos += before ? 1 : 0;
    }
    c.list[pos] = mine;
  }
  __syncthreads();
  return n;
}

template <bool BY_MASS>
__device__ Selection resolve3(Ctx3& c, Selection sel, uint32_t lo_key) {
  if (!sel.ok || sel.levels == 3) return sel;
  if (c.dbg && threadIdx.x == 0 && BY_MASS) { c.dbg[19] = clock64(); c.dbg[23] = (unsigned long long)sel.levels; }
  const int n = gather_members3(c, lo_key, sel.levels, sel.prefix);
  const int tid = threadIdx.x;
  if (c.dbg && tid == 0 && BY_MASS) { c.dbg[21] = clock64(); c.dbg[24] = (unsigned long long)n; }
  u64 a = 0, b = 0;
  if (tid < n) { a = c.list[tid].cnt; b = a * c.list[tid].q; }
  const u64 ia = warp_scan_u64(a), ib = warp_scan_u64(b);
  u64 pa, pb, tc, tm;
  block_warp_prefix2(*c.x, shfl_u64(ia, 31), shfl_u64(ib, 31), pa, pb, tc, tm);
  if (c.dbg && tid == 0 && BY_MASS) c.dbg[34] = clock64();
  const u64 want = sel.target - (BY_MASS ? sel.above_mass : sel.above_cnt);
  if (tid == 0) c.x->bcast[7] = 0;
  __syncthreads();
  if (tid < n) {
    const u64 incl = BY_MASS ? pb + ib : pa + ia;
    const u64 excl = incl - (BY_MASS ? b : a);
    if (excl < want && want <= incl) { c.x->bcast[0] = c.list[tid].key; c.x->bcast[7] = 1; }
  }
  __syncthreads();
  if (c.x->bcast[7] == 0) {
    sel.ok = false;
    __syncthreads();
    return sel;
  }
  const uint32_t key = (uint32_t)c.x->bcast[0];
  if (c.dbg && tid == 0 && BY_MASS) c.dbg[35] = clock64();
  // the list is sorted by key: what lies above the key's group and the group itself are read
  // off the running sums at the group's two ends
  if (tid < n && c.list[tid].key == key) {
    if (tid == 0 || c.list[tid - 1].key != key) { c.x->bcast[1] = pa + ia - a; c.x->bcast[2] = pb + ib - b; }
    if (tid == n - 1 || c.list[tid + 1].key != key) { c.x->bcast[3] = pa + ia; c.x->bcast[4] = pb + ib; }
  }
  __syncthreads();
  const u64 ac = c.x->bcast[1], am = c.x->bcast[2];
  const u64 bc = c.x->bcast[3] - ac, bm = c.x->bcast[4] - am;
  sel.key = key;
  sel.prefix = key;
  sel.levels = 3;
  sel.above_cnt += ac;
  sel.above_mass += am;
  sel.bin_cnt = bc;
  sel.bin_mass = bm;
  __syncthreads();
  if (c.dbg && tid == 0 && BY_MASS) c.dbg[36] = clock64();
  return sel;
}

template <bool BY_MASS, bool WITH_MASS>
__device__ Selection select_union3(Ctx3& c, uint32_t lo_key, u64 target, float top_p) {
  UnionFill3<WITH_MASS> fill{&c};
  Selection sel = descend_local<BY_MASS>(c, fill, lo_key, target, top_p, (u64)kV3ListCap);
  return resolve3<BY_MASS>(c, sel, lo_key);
}

// Count and mass of all tokens with key >= lo_key.
__device__ void totals3(Ctx3& c, uint32_t lo_key, u64& cnt, u64& mass) {
  u64 a = 0, b = 0;
  for_each_side3(c, [&](int, float s) {
    if (key_of(s) >= lo_key) { ++a; b += mass_of(s, c.m); }
  });
  for_each_class(c, [&](const ClassEntry& e) {
    if (e.key >= lo_key) { a += e.cnt; b += e.w; }
  });
  block_sum2(*c.x, a, b);
  cnt = a;
  mass = b;
}

// ---- the tie group of a key: the classes (at most one per count class, scores grow with
// the bin) and the side elements whose score key equals it ---------------------------------
struct Group {
  uint32_t key;
  int cell0, cell1, cell2;  // class index per count class, or -1
  __device__ __forceinline__ int cell_of(int cc) const { return cc == 0 ? cell0 : (cc == 1 ? cell1 : cell2); }
};
__device__ Group find_group(Ctx3& c, uint32_t key) {
  if (threadIdx.x < 3) c.x->bcast[threadIdx.x] = 0;
  __syncthreads();
  for_each_class(c, [&](const ClassEntry& e) {
    if (e.key == key) c.x->bcast[e.cell / kV3Bins] = (u64)e.cell + 1;
  });
  __syncthreads();
  Group g;
  g.key = key;
  g.cell0 = (int)c.x->bcast[0] - 1;
  g.cell1 = (int)c.x->bcast[1] - 1;
  g.cell2 = (int)c.x->bcast[2] - 1;
  __syncthreads();
  return g;
}
// Does the token at position id (raw bits, 2-bit class cc) belong to the group?
__device__ __forceinline__ bool in_group(const Ctx3& c, const Group& g, int id, uint32_t raw, int cc) {
  if (cc < 3) {
    const int b = v3_bin_of_raw(raw);
    if (b >= 0) return g.cell_of(cc) == cc * kV3Bins + b;
    return key_of(c.score_of(raw, cc)) == g.key;  // outside the bin window: a side element
  }
  return key_of(c.score_of(raw, c.heavy_count(id))) == g.key;
}

// Loads chunk i (8 tokens) of the row and its classes.
__device__ __forceinline__ void load_chunk(const Ctx3& c, int i, uint32_t (&raw)[8], uint32_t& cls16) {
  const uint4 w = reinterpret_cast<const uint4*>(c.logits)[i];
  raw[0] = w.x & 0xffffu; raw[1] = w.x >> 16; raw[2] = w.y & 0xffffu; raw[3] = w.y >> 16;
  raw[4] = w.z & 0xffffu; raw[5] = w.z >> 16; raw[6] = w.w & 0xffffu; raw[7] = w.w >> 16;
  cls16 = c.cls ? reinterpret_cast<const unsigned short*>(c.cls)[i] : 0u;
}
// Bit k set: token 8*i + k belongs to the group.
__device__ __forceinline__ uint32_t chunk_members(const Ctx3& c, const Group& g, int i, const uint4& w,
                                                  uint32_t cls16) {
  const uint32_t words[4] = {w.x, w.y, w.z, w.w};
  uint32_t memb = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    memb |= (in_group(c, g, 8 * i + 2 * k, words[k] & 0xffffu, (cls16 >> (4 * k)) & 3) ? 1u : 0u) << (2 * k);
    memb |= (in_group(c, g, 8 * i + 2 * k + 1, words[k] >> 16, (cls16 >> (4 * k + 2)) & 3) ? 1u : 0u) << (2 * k + 1);
  }
  return memb;
}
// Members in chunks [b, e) seen by this lane (lanes of a warp interleave), four 128-bit
// loads in flight per lane.
__device__ __forceinline__ u64 count_members(const Ctx3& c, const Group& g, int b, int e) {
  const int lane = threadIdx.x & 31;
  const uint4* src4 = reinterpret_cast<const uint4*>(c.logits);
  const unsigned short* cls16p = reinterpret_cast<const unsigned short*>(c.cls);
  u64 mine = 0;
  for (int i0 = b + lane; i0 < e; i0 += 4 * 32) {
    uint4 w[4];
    uint32_t cl[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + 32 * u;
      if (i < e) { w[u] = src4[i]; cl[u] = cls16p ? cls16p[i] : 0u; }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + 32 * u;
      if (i < e) mine += __popc(chunk_members(c, g, i, w[u], cl[u]));
    }
  }
  return mine;
}

// Token id of the n-th (1-based, ascending id) member of the group (classes and side
// elements whose score key is g.key), or 0x7fffffff.  The row is cut into one segment per
// warp, members are counted, and the segment that holds the n-th is cut again until one
// warp can rank its members with ballots.
__device__ int nth_in_group(Ctx3& c, const Group& g, u64 n) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
  const int n8 = c.vec ? c.vocab / 8 : 0;
  int b = 0, e = n8;
  u64 before = 0;
  bool in_tail = false;
  int result = 0x7fffffff;
  while (true) {
    if (e - b <= 4 * 32) break;
    const int seg = (e - b + kWarps - 1) / kWarps;
    const int mb = min(b + warp * seg, e), me = min(mb + seg, e);
    const u64 wtot = warp_sum_u64(count_members(c, g, mb, me));
    u64 pre, pre_unused, tot, tot_unused;
    block_warp_prefix2(*c.x, wtot, 0, pre, pre_unused, tot, tot_unused);
    if (before + tot < n) { before += tot; in_tail = true; break; }
    if (before + pre < n && n <= before + pre + wtot && lane == 0) {
      c.x->bcast[4] = (u64)mb;
      c.x->bcast[5] = (u64)me;
      c.x->bcast[6] = before + pre;
    }
    __syncthreads();
    b = (int)c.x->bcast[4];
    e = (int)c.x->bcast[5];
    before = c.x->bcast[6];
    __syncthreads();
  }
  if (tid == 0) c.x->bcast[6] = 0;
  __syncthreads();
  if (!in_tail && warp == 0) {
    // at most 128 chunks: rank members with warp scans
    const uint4* src4 = reinterpret_cast<const uint4*>(c.logits);
    const unsigned short* cls16p = reinterpret_cast<const unsigned short*>(c.cls);
    u64 running = before;
    for (int i0 = b; i0 < e && running < n; i0 += 32) {
      const int i = i0 + lane;
      uint32_t memb = 0;
      if (i < e) memb = chunk_members(c, g, i, src4[i], cls16p ? cls16p[i] : 0u);
      const u64 incl = warp_scan_u64((u64)__popc(memb));
      u64 rank = running + incl - __popc(memb);
      for (int k = 0; k < 8; ++k) {
        if (!((memb >> k) & 1u)) continue;
        if (++rank == n) c.x->bcast[6] = (u64)(8 * i + k) + 1;
      }
      running += shfl_u64(incl, 31);
    }
    if (running < n) before = running;  // not reached inside the vector part: look in the tail
    if (lane == 0 && running < n) c.x->bcast[5] = running;
  }
  __syncthreads();
  if (c.x->bcast[6] == 0) {
    // scalar tail of the row (all of it when the row is not 16-byte aligned)
    if (!in_tail) before = c.x->bcast[5];
    if (warp == 0) {
      u64 running = in_tail ? before : c.x->bcast[5];
      for (int id0 = n8 * 8; id0 < c.vocab && running < n; id0 += 32) {
        const int id = id0 + lane;
        const bool mbr = id < c.vocab && in_group(c, g, id, c.logits[id], c.class_of(id));
        const uint32_t ballot = __ballot_sync(0xffffffffu, mbr);
        const u64 rank = running + __popc(ballot & ((1u << lane) - 1u)) + 1;
        if (mbr && rank == n) c.x->bcast[6] = (u64)id + 1;
        running += __popc(ballot);
      }
    }
    __syncthreads();
  }
  const u64 found = c.x->bcast[6];
  __syncthreads();
  if (found) result = (int)(found - 1);
  return result;
}

// Token id of the n-th (1-based, ascending id) of the `members` tokens of ONE class (count
// class and one-value bin `cell`), for classes of at most kV3ScanCap tokens, or -1 when the row
// has no 16-byte aligned view.  The row is walked from the end that is nearer to the n-th
// member, 16,384 tokens per step, and the walk stops soon after the step that reaches it (it
// looks every fourth step): members are spread evenly over the row, so on average a third of
// it is read.  A class is one bf16 bit
// pattern and a normal number (the bin window holds neither zeros nor NaNs), so two tokens are
// compared with it by one native bf16x2 equality per 32-bit word; a hit looks its count class
// up in the 16 class bits that travel with its chunk.  The ids found (in the gather and list
// buffers, which are contiguous) are ranked among themselves.
static_assert(kV3ScanCap * sizeof(int) <= 2 * kV3ListCap * sizeof(V3Entry), "scan ids fit the two buffers");
// (Not inlined, and handed plain values instead of the row's context: inside the kernel's main
// body its eight 128-bit registers in flight were spilled to local memory, which this kernel's
// small L1 turns into round trips to L2 inside the loop.)
struct ScanArgs {
  const unsigned short* logits;
  const uint32_t* cls;
  int vocab;
  int* ids;       // [kV3ScanCap]
  int* slot_n;    // ids used
  int* step_n;    // [2]
  u64* result;    // id + 1 of the answer, or 0
  unsigned long long* dbg;
};
__device__ __noinline__ void scan_small_class(const ScanArgs c, uint32_t raw, int cc, int n, int members) {
  const int tid = threadIdx.x;
  const uint32_t vv = raw | (raw << 16);
  const __nv_bfloat162 vv2 = *reinterpret_cast<const __nv_bfloat162*>(&vv);
  int* ids = c.ids;
  const bool forward = 2 * n <= members + 1;
  const int need = forward ? n : members - n + 1;  // counted from the end the walk starts at
  if (tid == 0) { *c.slot_n = 0; c.step_n[0] = 0; c.step_n[1] = 0; *c.result = 0; }
  __syncthreads();
  if (c.dbg && tid == 0) c.dbg[40] = clock64();
  const int n8 = c.vocab / 8;
  const uint4* src4 = reinterpret_cast<const uint4*>(c.logits);
  const unsigned short* cls16p = reinterpret_cast<const unsigned short*>(c.cls);
  // Members found are counted in two counters that take turns from one look to the next:
  // after a look's barrier every thread reads that turn's counter, which nobody adds to before
  // the barrier after next, so all threads see the same running total and leave together.
  auto note = [&](int id, int parity) {
    const int slot = atomicAdd(c.slot_n, 1);
    if (slot < kV3ScanCap) ids[slot] = id;
    atomicAdd(c.step_n + parity, 1);
  };
  // the few tokens after the last whole chunk: first when walking backwards, last otherwise
  auto tail = [&](int parity) {
    for (int id = n8 * 8 + tid; id < c.vocab; id += kThreads)
      if ((uint32_t)c.logits[id] == raw && (c.cls ? (int)((c.cls[id >> 4] >> ((id & 15) * 2)) & 3u) : 0) == cc) note(id, parity);
  };
  if (!forward) tail(0);
  constexpr int kBatch = 4;
  constexpr int kStep = kBatch * kThreads;  // chunks per step
  constexpr int kCheckShift = 2;            // the walk looks whether it may stop every 2^kCheckShift steps
  const int n_steps = (n8 + kStep - 1) / kStep;
  uint4 w[kBatch], wn[kBatch];
  uint32_t cl[kBatch], cn[kBatch];
  // chunk u of step s for this thread (steps are numbered in walking order)
  auto chunk_of = [&](int s, int u) { return (forward ? s : n_steps - 1 - s) * kStep + u * kThreads + tid; };
  auto fetch = [&](uint4 (&dw)[kBatch], uint32_t (&dc)[kBatch], int s) {
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = chunk_of(s, u);
      const bool in = s < n_steps && i < n8;
      dw[u] = in ? __ldcg(src4 + i) : make_uint4(~vv, ~vv, ~vv, ~vv);
      dc[u] = (in && cls16p) ? (uint32_t)__ldcg(cls16p + i) : 0u;
    }
  };
  fetch(w, cl, 0);
  bool reached = false;
  int total = 0, seen[2] = {0, 0};
  for (int s = 0; s < n_steps; ++s) {
    fetch(wn, cn, s + 1);
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const uint32_t m0 = __heq2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].x), vv2);
      const uint32_t m1 = __heq2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].y), vv2);
      const uint32_t m2 = __heq2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].z), vv2);
      const uint32_t m3 = __heq2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].w), vv2);
      if (m0 | m1 | m2 | m3) {
        const int id = 8 * chunk_of(s, u);
        uint32_t hits = ((m0 & 1u) | ((m0 >> 15) & 2u)) | (((m1 & 1u) | ((m1 >> 15) & 2u)) << 2) |
                        (((m2 & 1u) | ((m2 >> 15) & 2u)) << 4) | (((m3 & 1u) | ((m3 >> 15) & 2u)) << 6);
        while (hits) {
          const int q = __ffs(hits) - 1;
          hits &= hits - 1;
          if ((int)((cl[u] >> (2 * q)) & 3u) == cc) note(id + q, (s >> kCheckShift) & 1);
        }
      }
    }
    // (a look every few steps: a barrier after every step would make each one wait for its
    // slowest load)
    if ((s & ((1 << kCheckShift) - 1)) == (1 << kCheckShift) - 1) {
      const int turn = (s >> kCheckShift) & 1;
      __syncthreads();
      const int now = c.step_n[turn];
      total += now - seen[turn];
      seen[turn] = now;
      if (total >= need) { reached = true; break; }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) { w[u] = wn[u]; cl[u] = cn[u]; }
  }
  if (forward && !reached) tail(0);
  if (c.dbg && tid == 0) c.dbg[43] = clock64();
  __syncthreads();
  if (c.dbg && tid == 0) c.dbg[41] = clock64();
  const int found = min(*c.slot_n, kV3ScanCap);
  // every member on the near side of the last step's far end was noted: the one that `need - 1`
  // others precede (follow, when walking backwards) is the answer
  for (int t = tid; t < found; t += kThreads) {
    const int mine = ids[t];
    int before = 0;
    for (int j = 0; j < found; ++j) before += (forward ? ids[j] < mine : ids[j] > mine) ? 1 : 0;
    if (before + 1 == need) *c.result = (u64)mine + 1;
  }
  __syncthreads();
  if (c.dbg && tid == 0) { c.dbg[42] = clock64(); c.dbg[44] = (unsigned long long)found; }
}
__device__ __forceinline__ int nth_in_small_class(Ctx3& c, int cell, u64 n, u64 members) {
  if (!c.vec || members > (u64)kV3ScanCap || n < 1 || n > members) return -1;
  const int cc = cell / kV3Bins;
  const ScanArgs sa{c.logits, c.cls, c.vocab, reinterpret_cast<int*>(c.gbuf), c.gbuf_n, c.step_n, &c.x->bcast[6], c.dbg};
  scan_small_class(sa, v3_raw_of_bin(cell - cc * kV3Bins), cc, (int)n, (int)members);
  const u64 hit = c.x->bcast[6];
  __syncthreads();
  return hit ? (int)(hit - 1) : 0x7fffffff;
}

// Appends to the gather buffer the ids of all group members with id <= id_limit.
__device__ void emit_group_upto(Ctx3& c, const Group& g, int id_limit) {
  const int n8 = c.vec ? c.vocab / 8 : 0;
  const int last = min(n8, id_limit / 8 + 1);
  const uint4* src4 = reinterpret_cast<const uint4*>(c.logits);
  const unsigned short* cls16p = reinterpret_cast<const unsigned short*>(c.cls);
  auto emit = [&](int id) {
    const int slot = atomicAdd(c.gbuf_n, 1);
    if (slot < kV3ListCap) c.gbuf[slot] = V3Entry{g.key, id, 1u, 0u, 0ull};
  };
  for (int i = threadIdx.x; i < last; i += kThreads) {
    uint32_t memb = chunk_members(c, g, i, src4[i], cls16p ? cls16p[i] : 0u);
    while (memb) {
      const int k = __ffs(memb) - 1;
      memb &= memb - 1;
      if (8 * i + k <= id_limit) emit(8 * i + k);
    }
  }
  for (int id = n8 * 8 + threadIdx.x; id < c.vocab && id <= id_limit; id += kThreads)
    if (in_group(c, g, id, c.logits[id], c.class_of(id))) emit(id);
  __syncthreads();
}

// A uniformly chosen token of ONE class (count class and one-value bin `cell`) by rejection:
// Philox-drawn positions are probed, `trials` (<= kRandomTrials) per thread and round with
// their loads in flight together; trial t = (round * trials + j) * kThreads + thread, and
// the lowest hitting trial wins.  A lone CTA sustains well under one scattered load per
// clock, so a probe reads the value first and the class map only when the value matches.
// Returns -1 if max_rounds pass without a hit.
constexpr int kRandomTrials = 8;
__device__ int random_in_class(Ctx3& c, int cell, int trials, uint64_t seed, int max_rounds) {
  const int tid = threadIdx.x;
  const int cc = cell / kV3Bins;
  const uint32_t value = v3_raw_of_bin(cell - cc * kV3Bins);
  for (int round = 0; round < max_rounds; ++round) {
    int id[kRandomTrials];
    uint32_t raw[kRandomTrials];
#pragma unroll
    for (int j = 0; j < kRandomTrials / 2; ++j) {
      if (2 * j < trials) {
        const Philox4 r = philox4x32_10((uint32_t)round, (uint32_t)tid, 1u + (uint32_t)j, 0u, (uint32_t)seed,
                                        (uint32_t)(seed >> 32));
        id[2 * j] = (int)__umul64hi(((u64)r.v[0] << 32) | r.v[1], (u64)c.vocab);
        id[2 * j + 1] = (int)__umul64hi(((u64)r.v[2] << 32) | r.v[3], (u64)c.vocab);
      }
    }
#pragma unroll
    for (int j = 0; j < kRandomTrials; ++j) raw[j] = j < trials ? (uint32_t)c.logits[id[j]] : ~value;
    uint32_t key = 0;
    int mine = -1;
#pragma unroll
    for (int j = kRandomTrials - 1; j >= 0; --j) {
      if (j < trials && raw[j] == value && c.class_of(id[j]) == cc) {
        key = (uint32_t)((kRandomTrials - j) * kThreads - tid);
        mine = id[j];
      }
    }
    const uint32_t best = block_max_u32(*c.x, key);
    if (best) {
      if (key == best) c.x->bcast[6] = (u64)mine;
      __syncthreads();
      const int token = (int)c.x->bcast[6];
      __syncthreads();
      return token;
    }
  }
  return -1;
}

// A token of the kept set drawn with probability proportional to its mass, by rejection on
// TOKENS: a Philox-drawn position is accepted when a second number, uniform on [0, 2^40), lies
// below the token's integer mass (2^40 stands for the row maximum) and the token is kept.  The
// first accepted trial wins (trial t = (round * kTokenTrials + j) * kThreads + thread), which
// makes the draw exact and reproducible.  The chance per trial is the kept mass over
// vocab * 2^40: high on near-flat rows -- exactly where the draw by classes is slow (many
// small classes, whose members must be looked for) -- and hopeless on peaked ones, so the
// caller asks for it only when a round is almost sure to succeed (with one trial per thread
// on the flattest rows, else two).  A top-p cut that splits a
// tie group keeps the group's `cut_ties` lowest ids: a member of the group that is hit stands
// for the group as a whole and is accepted with probability cut_ties / group_cnt; the caller
// then picks one of the kept members (group_hit).  Returns -1 if max_rounds pass without a hit.
constexpr int kTokenTrials = 2;
__device__ int draw_by_token_rejection(Ctx3& c, const KeptSet& kept, bool tie_split, u64 cut_ties, u64 group_cnt,
                                       uint64_t seed, int max_rounds, int trials, bool& group_hit) {
  const int tid = threadIdx.x;
  group_hit = false;
  for (int round = 0; round < max_rounds; ++round) {
    int id[kTokenTrials];
    u64 u[kTokenTrials];
    uint32_t raw[kTokenTrials];
    int cc[kTokenTrials];
#pragma unroll
    for (int j = 0; j < kTokenTrials; ++j) {
      if (j >= trials) break;
      const Philox4 r = philox4x32_10((uint32_t)round, (uint32_t)tid, (uint32_t)j, 2u, (uint32_t)seed, (uint32_t)(seed >> 32));
      id[j] = (int)__umul64hi(((u64)r.v[0] << 32) | r.v[1], (u64)c.vocab);
      u[j] = ((u64)r.v[2] << 8) | (r.v[3] >> 24);
    }
#pragma unroll
    for (int j = 0; j < kTokenTrials; ++j) {
      if (j >= trials) break;
      raw[j] = (uint32_t)c.logits[id[j]];
      cc[j] = c.class_of(id[j]);
    }
    u64 best = 0;
#pragma unroll
    for (int j = 0; j < kTokenTrials; ++j) {
      if (j >= trials) break;
      const float s = c.element_score(id[j], raw[j], cc[j]);
      const uint32_t k = key_of(s);
      if (k < kept.cut_key || !(u[j] < mass_of(s, c.m))) continue;
      bool group = false;
      if (k == kept.cut_key && tie_split) {
        const Philox4 r = philox4x32_10((uint32_t)round, (uint32_t)tid, (uint32_t)j, 3u, (uint32_t)seed, (uint32_t)(seed >> 32));
        if (!(__umul64hi(((u64)r.v[0] << 32) | r.v[1], group_cnt) < cut_ties)) continue;
        group = true;
      }
      const u64 packed = ((u64)((kTokenTrials - j) * kThreads - tid) << 33) | ((u64)(group ? 1u : 0u) << 32) | (uint32_t)id[j];
      best = packed > best ? packed : best;
    }
    best = block_max_u64(*c.x, best);
    if (best) {
      group_hit = ((best >> 32) & 1ull) != 0;
      return (int)(uint32_t)best;
    }
  }
  return -1;
}

}  // namespace hs
