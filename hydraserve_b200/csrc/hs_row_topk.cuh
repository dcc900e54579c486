// Rows with a small top_k: the candidate path, and the list finisher shared with the
// vocabulary-sharded merge.
//
// With top_k = k, only the k highest scores (and ties at the k-th) can ever be sampled or
// reported, so nothing needs counting: the row is streamed once from HBM and compared, two
// tokens per instruction, against a lower bound of the k-th highest score.  The bound comes
// from the row itself: among the first 16,384 tokens, those the history does not hold are
// ranked by raw value (no scoring needed: their score grows with it), and the k-th highest is
// a valid bound for the whole row; whenever the candidate list grows past 2,048 entries
// the bound is raised to the list's k-th highest score and the list is compacted.  Scores
// grow with the raw value inside a history-count class, so the bound turns into one raw
// threshold per class (binary search over the 65,536 bf16 values); a token whose history
// count is 3 or more is always scored exactly.
//
// What is left, at most a few thousand (score key, token id) pairs in shared memory, is
// sorted by (score descending, id ascending).  In that order every filter of the reference
// is a prefix: top-k with ties, min-p, top-p (a cut inside a tie group keeps the lowest ids),
// the top-N log-probabilities; the draw is an inverse CDF over exact integer masses.
#pragma once

#include <cuda_bf16.h>

#include "hs_common.cuh"
#include "hs_select.cuh"
#include "hs_row_v3.cuh"

#ifndef HS_CAND_BATCH
#define HS_CAND_BATCH 4
#endif

namespace hs {

constexpr int kTopKMax = 256;      // largest top_k served by the candidate path
constexpr int kCandCap = 4096;     // candidate list capacity (shared memory, 8 bytes each)
constexpr int kCandSoft = 2048;    // raise the bound once the list is this long
constexpr int kSortAll = 128;      // a merged list this short is sorted whole instead of cut first
constexpr int kSample = 16384;     // tokens sampled (their raw values only) to get the first bound

// (score key << 32) | ~id : sorting these descending orders by score, then by ascending id
__device__ __forceinline__ u64 cand_pack(uint32_t key, int id) {
  return ((u64)key << 32) | (uint32_t)(~(uint32_t)id);
}
__device__ __forceinline__ uint32_t cand_key(u64 p) { return (uint32_t)(p >> 32); }
__device__ __forceinline__ int cand_id(u64 p) { return (int)(~(uint32_t)(p & 0xffffffffu)); }

// Signed 16-bit image of bf16 bits whose integer order is the float order.
__device__ __forceinline__ int t16_of_raw(uint32_t raw) {
  const uint32_t t = raw ^ ((raw & 0x8000u) ? 0x7fffu : 0u);
  return (int)(short)t;
}
__device__ __forceinline__ uint32_t raw_of_t16(int t) {
  const uint32_t u = (uint32_t)t & 0xffffu;
  return u ^ ((u & 0x8000u) ? 0x7fffu : 0u);
}

struct CandCtx {
  u64* cand;        // [kCandCap]
  int* n;           // entries in the list
  int* lost;        // set when an append did not fit; lost[2] is scratch of the stream's looks at the list
  uint32_t* count;  // [kBins] radix counters
  int* thr;         // [4] per-class signed 16-bit thresholds
  unsigned long long* dbg;  // optional phase clocks of this row (tuning aid), or null
};

// The k-th highest key among the n list entries (n >= k >= 1).  The keys of a candidate list
// lie close together, so the 2,048 counters are laid over [lowest key, highest key] instead of
// over fixed bit fields: one counting pass usually leaves a bucket with a handful of keys,
// which are then ranked among themselves; a fuller bucket is counted again over its own range.
__device__ uint32_t cand_kth_key(Exchange& x, CandCtx& L, int n, int k) {
  const int tid = threadIdx.x;
  constexpr int kResolve = 64;  // in-bucket keys ranked directly
  uint32_t lo_key = 0xffffffffu, hi_key = 0u;
  for (int i = tid; i < n; i += kThreads) {
    const uint32_t key = cand_key(L.cand[i]);
    lo_key = min(lo_key, key);
    hi_key = max(hi_key, key);
  }
  hi_key = block_max_u32(x, hi_key);
  lo_key = ~block_max_u32(x, ~lo_key);
  int want = k;
  for (int pass = 0; pass < 4; ++pass) {
    if (lo_key == hi_key) return lo_key;
    const uint32_t span = hi_key - lo_key;
    const int shift = max(0, 32 - __clz(span) - 11);  // (span >> shift) < 2048
    for (int b = tid; b < kBins; b += kThreads) L.count[b] = 0;
    if (tid == 0) L.thr[3] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += kThreads) {
      const uint32_t key = cand_key(L.cand[i]);
      if (key >= lo_key && key <= hi_key) atomicAdd(&L.count[(key - lo_key) >> shift], 1u);
    }
    __syncthreads();
    constexpr int kPer = kBins / kThreads;
    const int hi = kBins - 1 - kPer * tid;
    u64 sum = 0;
#pragma unroll
    for (int u = 0; u < kPer; ++u) sum += L.count[hi - u];
    const u64 incl = warp_scan_u64(sum);
    u64 pre, pu, tot, tu;
    block_warp_prefix2(x, shfl_u64(incl, 31), 0, pre, pu, tot, tu);
    u64 ex = pre + incl - sum;
    if (ex < (u64)want && (u64)want <= ex + sum) {
#pragma unroll
      for (int u = 0; u < kPer; ++u) {
        const u64 bc = L.count[hi - u];
        if ((u64)want <= ex + bc) {
          x.bcast[0] = (u64)(hi - u);
          x.bcast[1] = ex;
          x.bcast[2] = bc;
          break;
        }
        ex += bc;
      }
    }
    __syncthreads();
    const uint32_t bucket = (uint32_t)x.bcast[0];
    const int in_bucket = (int)x.bcast[2];
    want -= (int)x.bcast[1];
    // the bucket's key range (clamped to the range that was counted)
    const uint32_t b_lo = lo_key + (bucket << shift);
    const uint32_t b_hi = shift == 0 ? b_lo : min(hi_key, b_lo + ((1u << shift) - 1u));
    __syncthreads();
    lo_key = b_lo;
    hi_key = b_hi;
    if (shift == 0) return b_lo;  // a bucket was one key
    if (in_bucket <= kResolve) {
      // rank the bucket's keys among themselves (the counters have served: they hold the keys now)
      for (int i = tid; i < n; i += kThreads) {
        const uint32_t key = cand_key(L.cand[i]);
        if (key >= lo_key && key <= hi_key) L.count[atomicAdd(&L.thr[3], 1)] = key;
      }
      __syncthreads();
      if (tid < in_bucket) {
        const uint32_t mine = L.count[tid];
        int greater = 0, at_least = 0;
        for (int j = 0; j < in_bucket; ++j) {
          const uint32_t other = L.count[j];
          greater += other > mine ? 1 : 0;
          at_least += other >= mine ? 1 : 0;
        }
        if (greater < want && want <= at_least) x.bcast[0] = (u64)mine;  // equal keys write the same value
      }
      __syncthreads();
      const uint32_t key = (uint32_t)x.bcast[0];
      __syncthreads();
      return key;
    }
  }
  // not reached: every pass narrows the range by a factor of 2,048
  return lo_key;
}

// Drops list entries with key < bound (in place).  Returns the new length.
__device__ int cand_compact(CandCtx& L, int n, uint32_t bound) {
  const int tid = threadIdx.x;
  constexpr int kPer = kCandCap / kThreads;
  u64 mine[kPer];
#pragma unroll
  for (int u = 0; u < kPer; ++u) {
    const int i = tid + u * kThreads;
    mine[u] = i < n ? L.cand[i] : 0ull;
  }
  __syncthreads();
  if (tid == 0) *L.n = 0;
  __syncthreads();
#pragma unroll
  for (int u = 0; u < kPer; ++u) {
    const int i = tid + u * kThreads;
    if (i < n && mine[u] != 0ull && cand_key(mine[u]) >= bound) L.cand[atomicAdd(L.n, 1)] = mine[u];
  }
  __syncthreads();
  return *L.n;
}

// Per count class, the lowest raw value (as signed 16-bit image) whose score reaches `bound`
// (32768 if none does).  Scores grow with the value inside a class, so warp cc searches the
// 65,536 values of class cc 32 at a time: four rounds of one evaluation per lane and a ballot.
__device__ void cand_thresholds(const Ctx3& c, CandCtx& L, uint32_t bound) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < 3) {
    const int cc = warp;
    // every t < lo fails, every t >= hi passes (hi = 32768 stands for "none")
    int lo = -32768, hi = 32768;
#pragma unroll 1
    while (lo < hi) {
      const int step = (hi - lo + 31) >> 5;
      const int t = lo + (lane + 1) * step - 1;  // last value of this lane's block
      const bool pass = t >= hi || key_of(c.score_of(raw_of_t16(t), cc)) >= bound;
      const uint32_t votes = __ballot_sync(0xffffffffu, pass);
      if (votes == 0) { lo = hi; break; }
      const int f = __ffs(votes) - 1;  // the answer lies in block f
      hi = min(lo + (f + 1) * step - 1, hi);
      lo = lo + f * step;
    }
    if (lane == 0) {
      // -0.0 scores like +0.0 but sits one step below it in the integer order
      if (lo == 0) lo = -1;
      L.thr[cc] = lo;
    }
  }
  __syncthreads();
}

// Calls hit(id, raw, count class) for every token of the row whose score key can reach the
// bound the thresholds stand for: raw value (as signed 16-bit image) >= thr[class] for the
// classes 0, 1, 2; tokens of class 3 are never reported (they are listed per request).
// One pass, eight tokens per 128-bit load and one native bf16x2 comparison per two tokens
// against the most permissive threshold; a hit looks its class up.  Loads go past L1 (the
// counting kernel, which also uses this, has almost none).
template <class Hit>
__device__ void stream_at_or_above(const Ctx3& c, const int* thr, Hit&& hit) {
  const int tid = threadIdx.x;
  int t_min = thr[0];
  if (c.cls) t_min = min(t_min, min(thr[1], thr[2]));
  // threshold as a bf16 value (NaN = nothing passes, -inf = everything passes)
  uint32_t tb = t_min > 32640 ? 0x7fc0u : raw_of_t16(t_min);
  if (t_min <= -32641) tb = 0xff80u;
  const uint32_t pair = tb * 0x10001u;
  const __nv_bfloat162 thr2 = *reinterpret_cast<const __nv_bfloat162*>(&pair);
  auto look = [&](int id, uint32_t raw) {
    const int cc = c.class_of(id);
    if (cc != 3 && t16_of_raw(raw) >= thr[cc]) hit(id, raw, cc);
  };
  const int n8 = c.vec ? c.vocab / 8 : 0;
  const uint4* src4 = reinterpret_cast<const uint4*>(c.logits);
  constexpr int kInFlight = 8;
  for (int base = 0; base < n8; base += kInFlight * kThreads) {
    uint4 w[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int i = base + tid + u * kThreads;
      if (i < n8) w[u] = __ldcg(src4 + i);
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int i = base + tid + u * kThreads;
      if (i >= n8) break;
      const uint32_t m0 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].x), thr2);
      const uint32_t m1 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].y), thr2);
      const uint32_t m2 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].z), thr2);
      const uint32_t m3 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].w), thr2);
      if (!(m0 | m1 | m2 | m3)) continue;  // the common case
      uint32_t hits = ((m0 & 1u) | ((m0 >> 15) & 2u)) | (((m1 & 1u) | ((m1 >> 15) & 2u)) << 2) |
                      (((m2 & 1u) | ((m2 >> 15) & 2u)) << 4) | (((m3 & 1u) | ((m3 >> 15) & 2u)) << 6);
#pragma unroll 1
      while (hits) {
        const int q = __ffs(hits) - 1;
        hits &= hits - 1;
        const uint32_t word = q < 2 ? w[u].x : (q < 4 ? w[u].y : (q < 6 ? w[u].z : w[u].w));
        look(8 * i + q, (word >> (16 * (q & 1))) & 0xffffu);
      }
    }
  }
  for (int id = n8 * 8 + tid; id < c.vocab; id += kThreads) {
    const uint32_t raw = c.logits[id];
    if (t16_of_raw(raw) >= t_min) look(id, raw);
  }
}

// A lower bound (as signed 16-bit image of a raw value) of the k-th highest raw value among
// the tokens of [begin, end) that the history does not hold, or -32768 when none is found.
// The sampled tokens are cut into groups of eight (one 128-bit load); the k highest group
// maxima are k different tokens, so the k-th highest maximum is such a bound, and with
// k much smaller than the number of groups it is about as tight as the k-th highest token.
// Each thread keeps its (at most four) group maxima in registers; the k-th highest of them
// is found with two count-only radix levels of eight bits.
constexpr int kSampleGroups = 4;  // per thread: kSample = kSampleGroups * 8 * kThreads
static_assert(kSample == kSampleGroups * 8 * kThreads, "one 128-bit load per group");
struct SampleRegs {
  uint4 w[kSampleGroups];
  uint32_t cl[kSampleGroups];
};
// Starts the loads of the sample (nothing waits for them here).
__device__ __forceinline__ void sample_fetch(const Ctx3& c, int begin, int end, SampleRegs& r) {
  const int tid = threadIdx.x;
  const bool vec = c.vec && (begin & 7) == 0;
  const int n8 = vec ? (end - begin) / 8 : 0;  // whole 8-token chunks read as 128-bit words
  const uint4* src4 = reinterpret_cast<const uint4*>(c.logits) + (begin >> 3);
  const unsigned short* cls16p = c.cls ? reinterpret_cast<const unsigned short*>(c.cls) + (begin >> 3) : nullptr;
#pragma unroll
  for (int u = 0; u < kSampleGroups; ++u) {
    const int i = tid + u * kThreads;
    if (i < n8) { r.w[u] = src4[i]; r.cl[u] = cls16p ? cls16p[i] : 0u; }
  }
}
__device__ int sample_kth_t16(const Ctx3& c, CandCtx& L, int begin, int end, int k, const SampleRegs& r) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kGroups = kSampleGroups;
  const bool vec = c.vec && (begin & 7) == 0;
  const int n8 = vec ? (end - begin) / 8 : 0;
  int top[kGroups];  // value + 32768 of the group maximum, 0 = no token
  {
#pragma unroll
    for (int u = 0; u < kGroups; ++u) {
      top[u] = 0;
      if (tid + u * kThreads >= n8) continue;
      const uint32_t words[4] = {r.w[u].x, r.w[u].y, r.w[u].z, r.w[u].w};
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (((r.cl[u] >> (2 * q)) & 3u) == 0)
          top[u] = max(top[u], t16_of_raw((words[q >> 1] >> (16 * (q & 1))) & 0xffffu) + 32768);
    }
  }
  if (!vec) {
    // a part that is not 16-byte aligned: thread-strided groups over the scalar view
    for (int id = begin + tid; id < end; id += kThreads)
      if (c.class_of(id) == 0) top[0] = max(top[0], t16_of_raw(c.logits[id]) + 32768);
  }
  // k-th highest of the positive maxima: bins of L.count, 256 per level
  int prefix = 0, want = k;
  for (int level = 0; level < 2; ++level) {
    if (tid < 256) L.count[tid] = 0;
    __syncthreads();
#pragma unroll
    for (int u = 0; u < kGroups; ++u) {
      if (top[u] <= 0) continue;
      if (level == 0) atomicAdd(&L.count[top[u] >> 8], 1u);
      else if ((top[u] >> 8) == prefix) atomicAdd(&L.count[top[u] & 255], 1u);
    }
    if (tid == 0) L.thr[3] = -1;
    __syncthreads();
    if (warp == 0) {
      // lane l owns bins 255 - 8 l ... 248 - 8 l (descending)
      const int hi = 255 - 8 * lane;
      uint32_t sum = 0;
#pragma unroll
      for (int u = 0; u < 8; ++u) sum += L.count[hi - u];
      uint32_t incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      uint32_t ex = incl - sum;
      if (ex < (uint32_t)want && (uint32_t)want <= incl) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint32_t bc = L.count[hi - u];
          if ((uint32_t)want <= ex + bc) {
            L.thr[3] = hi - u;
            c.x->bcast[1] = ex;
            break;
          }
          ex += bc;
        }
      }
    }
    __syncthreads();
    const int found = L.thr[3];
    const int above = (int)c.x->bcast[1];
    __syncthreads();
    if (found < 0) return -32768;  // fewer than k groups with a token outside the history
    want -= above;
    if (level == 0) prefix = found; else return ((prefix << 8) | found) - 32768;
  }
  return -32768;
}

// Streams the row and leaves in L every token whose score can be among the top k (ties at
// the k-th included).  Returns the list length, or -1 when the list overflowed (the caller
// then uses the counting path).
__device__ int topk_candidates(Ctx3& c, CandCtx& L, int k) {
  const int tid = threadIdx.x;
  if (tid == 0) { *L.n = 0; *L.lost = 0; }
  __syncthreads();
  // A hit is stored unscored, (raw bits, count class, id), by the one lane that found it;
  // scores are computed later for the whole list at once with every lane busy.
  auto push = [&](int id, uint32_t raw, int cc) {
    const int slot = atomicAdd(L.n, 1);
    if (slot < kCandCap) L.cand[slot] = ((u64)raw << 48) | ((u64)cc << 32) | (uint32_t)id;
    else *L.lost = 1;
  };
  auto score_pending = [&](int from, int to) {
    for (int i = from + tid; i < to; i += kThreads) {
      const u64 e = L.cand[i];
      const int id = (int)(uint32_t)e;
      int cc = (int)(e >> 32) & 7;
      bool valid = true;
      if (cc == 4) {  // found by the stream, which does not look at count classes
        cc = c.class_of(id);
        valid = cc != 3;  // tokens held three times or more come from the request's list
      }
      L.cand[i] = valid ? cand_pack(key_of(c.element_score(id, (uint32_t)(e >> 48), cc)), id) : 0ull;
    }
    __syncthreads();
  };
  // 1. Tokens the history holds three times or more are candidates by definition (their score
  // does not follow from a class threshold); they come from the request's list, not the stream.
  // The chain heavy -> pairs -> logits is three dependent reads; it is started for list entry
  // `tid` before the sample is fetched and worked off between the sample's steps, so that
  // the waits overlap.
  const int sample_end = min(c.hi, c.lo + kSample);
  int n_heavy = 0, hv_q = -1;
  if (c.cls) {
    n_heavy = load_now_s32(c.pool.n_heavy + c.slot);
    if (tid < c.pool.unique_cap) hv_q = load_now_s32(c.pool.heavy + (size_t)c.slot * c.pool.unique_cap + tid);
  }
  SampleRegs sample;
  sample_fetch(c, c.lo, sample_end, sample);
  n_heavy = min(n_heavy, c.pool.unique_cap);
  const int2* pairs = c.pool.pairs + (size_t)c.slot * c.pool.unique_cap;
  int2 hv_pair = make_int2(-1, 0);
  if (tid < n_heavy && hv_q >= 0 && hv_q < c.pool.unique_cap) hv_pair = load_now_int2(pairs + hv_q);  // (id, count)
  const bool hv_mine = hv_pair.x >= c.lo && hv_pair.x < c.hi;
  uint32_t hv_raw = 0;
  if (hv_mine) hv_raw = load_now_u16(c.logits + hv_pair.x);
  // the first bound: from the group maxima of the sampled tokens outside the history
  const int t_k = sample_kth_t16(c, L, c.lo, sample_end, k, sample);
  if (c.cls) {
    auto add_scored = [&](int id, uint32_t raw, int count) {  // the exact count is at hand
      const int slot = atomicAdd(L.n, 1);
      if (slot < kCandCap) L.cand[slot] = cand_pack(key_of(c.score_of(raw, count)), id);
      else *L.lost = 1;
    };
    if (hv_mine) add_scored(hv_pair.x, hv_raw, hv_pair.y);
    const int32_t* heavy = c.pool.heavy + (size_t)c.slot * c.pool.unique_cap;
    for (int j = tid + kThreads; j < n_heavy; j += kThreads) {
      const int q = heavy[j];
      if (q < 0 || q >= c.pool.unique_cap) continue;
      const int2 pr = pairs[q];  // (id, count)
      if (pr.x < c.lo || pr.x >= c.hi) continue;
      add_scored(pr.x, c.logits[pr.x], pr.y);
    }
  }
  __syncthreads();
  if (*L.lost) return -1;
  int n = min(*L.n, kCandCap);
  uint32_t bound = t_k > -32768 ? key_of(c.score_of(raw_of_t16(t_k), 0)) : 0u;
  if (L.dbg && tid == 0) L.dbg[3] = clock64();
  cand_thresholds(c, L, bound);
  if (L.dbg && tid == 0) L.dbg[4] = clock64();
  int refreshes = 0;
  // 2. the rest of the row: eight tokens per 128-bit load, one native bf16x2 comparison per
  // two tokens against the most permissive class threshold; the rare hit is looked at closely
  const int first8 = c.lo / 8;  // lo is a multiple of 8
  const int n8 = c.vec ? c.hi / 8 : first8;
  const uint4* src4 = reinterpret_cast<const uint4*>(c.logits);
  constexpr int kBatch = HS_CAND_BATCH;  // two batches of loads: the next is on its way while this one is compared
  int n_scored = n;
  uint4 w[kBatch], wn[kBatch];
  auto fetch = [&](uint4 (&dst)[kBatch], int base) {
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = base + tid + u * kThreads;
      if (i < n8) dst[u] = __ldcs(src4 + i);
    }
  };
  fetch(w, first8);
  int iteration = 0, next_look = 1, last_look = -1, last_seen = n;
  for (int base = first8; base < n8; base += kBatch * kThreads, ++iteration) {
    // threshold as a bf16 value (NaN = nothing passes, -inf = everything passes)
    int t_min = L.thr[0];
    if (c.cls) t_min = min(t_min, min(L.thr[1], L.thr[2]));
    uint32_t tb = t_min > 32640 ? 0x7fc0u : raw_of_t16(t_min);
    if (t_min <= -32641) tb = 0xff80u;
    const uint32_t pair = tb * 0x10001u;
    const __nv_bfloat162 thr2 = *reinterpret_cast<const __nv_bfloat162*>(&pair);
    fetch(wn, base + kBatch * kThreads);
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = base + tid + u * kThreads;
      if (i >= n8) break;
      const uint32_t m0 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].x), thr2);
      const uint32_t m1 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].y), thr2);
      const uint32_t m2 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].z), thr2);
      const uint32_t m3 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[u].w), thr2);
      if (!(m0 | m1 | m2 | m3)) continue;  // the common case
      uint32_t hits = ((m0 & 1u) | ((m0 >> 15) & 2u)) | (((m1 & 1u) | ((m1 >> 15) & 2u)) << 2) |
                      (((m2 & 1u) | ((m2 >> 15) & 2u)) << 4) | (((m3 & 1u) | ((m3 >> 15) & 2u)) << 6);
#pragma unroll 1
      while (hits) {
        const int q = __ffs(hits) - 1;
        hits &= hits - 1;
        const uint32_t word = q < 2 ? w[u].x : (q < 4 ? w[u].y : (q < 6 ? w[u].z : w[u].w));
        const uint32_t raw = (word >> (16 * (q & 1))) & 0xffffu;
        push(8 * i + q, raw, 4);
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) w[u] = wn[u];
    // A look at the list's length now and then (a barrier: every look makes the batch wait for
    // its slowest load): after the second batch, then the sooner the faster the list grows, so
    // that it cannot run from the soft limit past its capacity between two looks.
    if (iteration != next_look) continue;
    if (tid == 0) L.lost[2] = *L.n;  // (a spare slot two behind the flag)
    // raise the bound when the list is getting long (block-uniform decision)
    const bool refresh = __syncthreads_or(*L.n >= kCandSoft);
    {
      const int seen = L.lost[2];  // (what thread 0 saw: the same value for all)
      const int per_batch = max(0, seen - last_seen) / (iteration - last_look);
      last_seen = seen;
      last_look = iteration;
      constexpr int kRoom = (kCandCap - kCandSoft) / 2;  // (half: hits come in bursts)
      next_look = iteration + (per_batch * 8 <= kRoom ? 8 : (per_batch * 4 <= kRoom ? 4 : (per_batch * 2 <= kRoom ? 2 : 1)));
    }
    if (refresh) {
      if (*L.lost) return -1;
      n = min(*L.n, kCandCap);
      score_pending(n_scored, n);
      bound = cand_kth_key(*c.x, L, n, k);
      n = cand_compact(L, n, bound);
      n_scored = n;
      cand_thresholds(c, L, bound);
      ++refreshes;
      last_seen = n;
    }
  }
  __syncthreads();
  if (L.dbg && tid == 0) { L.dbg[5] = clock64(); L.dbg[6] = (unsigned long long)refreshes; L.dbg[7] = (unsigned long long)*L.n; }
  // scalar tail (or the whole remainder of a row that is not 16-byte aligned)
  for (int id = max(n8 * 8, c.lo) + tid; id < c.hi; id += kThreads) {
    const uint32_t raw = c.logits[id];
    const int cc = c.class_of(id);
    if (cc != 3 && t16_of_raw(raw) >= L.thr[cc]) push(id, raw, cc);
  }
  __syncthreads();
  if (*L.lost) return -1;
  n = min(*L.n, kCandCap);
  score_pending(n_scored, n);
  return n;
}

// Sorts the first n list entries descending (bitonic, n padded to a power of two with zeros).
// A compare-exchange step of stride <= 32 stays inside the 64 entries one warp handles, so
// only the wider steps (and the changes between the two kinds) need the block barrier.
__device__ void cand_sort(CandCtx& L, int n) {
  if (n <= 128) {
    // short list: every entry counts the entries above it (entries are distinct: they end
    // in the token id) and moves to that position
    const int i = threadIdx.x;
    const u64 mine = i < n ? L.cand[i] : 0ull;
    int rank = 0;
    if (i < n)
      for (int j = 0; j < n; ++j) rank += L.cand[j] > mine ? 1 : 0;
    __syncthreads();
    if (i < n) L.cand[rank] = mine;
    __syncthreads();
    return;
  }
  int p = 1;
  while (p < n) p <<= 1;
  if (p < 64) p = 64;
  for (int i = n + threadIdx.x; i < p; i += kThreads) L.cand[i] = 0ull;
  __syncthreads();
  for (int size = 2; size <= p; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < p / 2; t += kThreads) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool desc = (lo & size) == 0;
        const u64 a = L.cand[lo], b = L.cand[hi];
        if ((a < b) == desc) { L.cand[lo] = b; L.cand[hi] = a; }
      }
      // the next step: stride / 2, or size (the first stride of the next size)
      const int next = stride > 1 ? (stride >> 1) : size;
      if (stride > 32 || next > 32) __syncthreads(); else __syncwarp();
    }
  }
  __syncthreads();
}

struct FinishOut {
  int token;
  int status;
  u64 n_topk, n_minp, n_kept;
  long long cut_ties;
  uint32_t cut_key;
  float m, log_z;
};

// Everything after top-k on a list sorted by (score descending, id ascending): min-p, top-p,
// draw, log-probabilities.  n = tokens that survived top-k (ties included), n >= 1.
// `mass` is scratch for n 64-bit values.  WARP = true: run by ONE warp (reductions are
// shuffles, no block barrier); false: by the whole CTA.
template <bool WARP>
__device__ FinishOut finish_impl(Exchange& x, const u64* cand, u64* mass, int n, const hs_row_params& P,
                                 const float* noise_row, hs_row_out* out, unsigned long long* dbg) {
  const int tid = WARP ? (int)(threadIdx.x & 31) : (int)threadIdx.x;
  constexpr int kLanes = WARP ? 32 : kThreads;
  auto sync = [&]() { if (WARP) __syncwarp(); else __syncthreads(); };
  auto sum = [&](u64 v) -> u64 {
    if (WARP) return warp_sum_u64(v);
    u64 unused = 0;
    block_sum2(x, v, unused);
    return v;
  };
  FinishOut r;
  r.status = 0;
  r.n_topk = (u64)n;
  const float m = score_of(cand_key(cand[0]));
  r.m = m;
  // masses and their inclusive prefix, each thread owning a contiguous run of entries
  const int per = (n + kLanes - 1) / kLanes;
  const int i0 = min(tid * per, n), i1 = min(i0 + per, n);
  u64 run = 0;
  for (int i = i0; i < i1; ++i) { run += mass_of(score_of(cand_key(cand[i])), m); mass[i] = run; }
  const u64 incl = warp_scan_u64(run);
  u64 my_off, z1;
  if (WARP) {
    my_off = incl - run;
    z1 = shfl_u64(incl, 31);
  } else {
    u64 pre, pu, tu;
    block_warp_prefix2(x, shfl_u64(incl, 31), 0, pre, pu, z1, tu);
    my_off = pre + incl - run;
  }
  for (int i = i0; i < i1; ++i) mass[i] += my_off;  // mass[i] = inclusive cumulative mass
  sync();
  // min-p: the passing tokens are a prefix
  int n1 = n;
  if (P.min_p > 0.0f) {
    const float z1f = mass_to_float(z1);
    const float thr = __fmul_rn(__fdiv_rn(1.0f, z1f), P.min_p);
    u64 pass = 0;
    for (int i = tid; i < n; i += kLanes) {
      const float s = score_of(cand_key(cand[i]));
      pass += !(__fdiv_rn(expf(s - m), z1f) < thr) ? 1 : 0;
    }
    n1 = max(1, (int)sum(pass));
  }
  r.n_minp = (u64)n1;
  if (dbg && tid == 0) dbg[9] = clock64();
  // top-p: shortest prefix whose mass reaches the target
  int n2 = n1;
  r.cut_ties = -1;
  if (P.top_p < 1.0f) {
    const u64 z2 = mass[n1 - 1];
    const u64 target = top_p_target(z2, P.top_p);
    u64 below = 0;
    for (int i = tid; i < n1; i += kLanes) below += mass[i] < target ? 1 : 0;
    n2 = min(n1, (int)sum(below) + 1);
    const uint32_t ck = cand_key(cand[n2 - 1]);
    u64 ties = 0;
    for (int i = tid; i < n2; i += kLanes) ties += cand_key(cand[i]) == ck ? 1 : 0;
    r.cut_ties = (long long)sum(ties);
  }
  r.n_kept = (u64)n2;
  r.cut_key = cand_key(cand[n2 - 1]);
  const u64 z3 = mass[n2 - 1];
  if (dbg && tid == 0) dbg[10] = clock64();
  // draw
  if (noise_row) {
    const float zf = mass_to_float(z3);
    u64 best = 0;
    for (int i = tid; i < n2; i += kLanes) {
      const int id = cand_id(cand[i]);
      const float p = __fdiv_rn(expf(score_of(cand_key(cand[i])) - m), zf);
      const float ratio = __fdiv_rn(p, noise_row[id]);
      const u64 packed = ((u64)__float_as_uint(ratio) << 32) | (uint32_t)(~(uint32_t)id);
      best = packed > best ? packed : best;
    }
    best = WARP ? warp_max_u64(best) : block_max_u64(x, best);
    r.token = (int)(~(uint32_t)(best & 0xffffffffu));
  } else {
    const Philox4 ph = philox4x32_10(0u, 0u, 0u, 0u, (uint32_t)P.seed, (uint32_t)(P.seed >> 32));
    const u64 target = __umul64hi(((u64)ph.v[0] << 32) | ph.v[1], z3);
    u64 le = 0;
    for (int i = tid; i < n2; i += kLanes) le += mass[i] <= target ? 1 : 0;
    r.token = cand_id(cand[min((int)sum(le), n2 - 1)]);
  }
  if (dbg && tid == 0) dbg[11] = clock64();
  // log-probabilities over the kept set
  r.log_z = 0.f;
  if (P.n_logprobs >= 0) {
    r.log_z = (float)(log((double)z3) - (double)kMassShift * 0.6931471805599453);
    const int n_want = min(P.n_logprobs, n2);
    for (int i = tid; i < n2; i += kLanes) {
      const float lp = (score_of(cand_key(cand[i])) - m) - r.log_z;
      if (i < n_want) { out->top_ids[i] = cand_id(cand[i]); out->top_logprobs[i] = lp; }
      if (cand_id(cand[i]) == r.token) out->logprob = lp;
    }
    if (tid == 0) out->n_top = n_want;
  } else if (tid == 0) {
    out->n_top = 0;
    out->logprob = 0.f;
  }
  return r;
}

constexpr int kWarpFinish = 1024;  // lists up to this length are finished by one warp

// The finisher, called by the whole CTA (the list complete and visible to all threads);
// every thread gets the result.
__device__ FinishOut finish_sorted(Exchange& x, const u64* cand, u64* mass, int n, const hs_row_params& P,
                                   const float* noise_row, hs_row_out* out, unsigned long long* dbg = nullptr) {
  if (n > kWarpFinish) return finish_impl<false>(x, cand, mass, n, P, noise_row, out, dbg);
  __shared__ FinishOut shared_result;
  if (threadIdx.x < 32) {
    const FinishOut r = finish_impl<true>(x, cand, mass, n, P, noise_row, out, dbg);
    if (threadIdx.x == 0) shared_result = r;
  }
  __syncthreads();
  const FinishOut r = shared_result;
  __syncthreads();
  return r;
}

__device__ __forceinline__ void write_finish(const FinishOut& r, hs_row_out* out) {
  out->token = r.token;
  out->status = r.status;
  out->n_kept = (int32_t)r.n_kept;
  out->n_after_topk = (int32_t)r.n_topk;
  out->n_after_minp = (int32_t)r.n_minp;
  out->n_after_topp = (int32_t)r.n_kept;
  out->cut_bits = __float_as_uint(score_of(r.cut_key));
  out->n_cut_ties = (int32_t)r.cut_ties;
  out->row_max = r.m;
  out->log_z = r.log_z;
}

}  // namespace hs
