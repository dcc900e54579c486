// The candidate path for fp32 logits: rows with 0 < top_k <= 256 and fp32 logits (the reference's
// HYDRASERVE_FP32_LOGITS mode; its CPU-runnable check) without the general kernel's resident
// row.  One CTA per row.  A lower bound of the row's k-th highest score comes from 512 groups of
// eight neighbouring tokens spread over the row (each thread scores one group and keeps the
// best: 512 different tokens, so the k-th highest of them is a valid bound); the bound becomes,
// per count class, the lowest logit VALUE whose score reaches it (scores grow with the value
// inside a class: a search over the 2^32 ordered float patterns, 32 at a time with ballots); the
// row is streamed once, four values per 128-bit load, against the most permissive of those
// values; the rare hit is listed as it is and the listed hits are scored together whenever the
// list is looked at.  The list is cut back whenever it gets long, and finished exactly like a
// bf16 candidate row's (hs_row_topk.cuh).  Rows this kernel does not serve return at once; a
// list that overflows (more ties than it holds) reports status 4 and the row is sampled again
// by the general kernel.
#pragma once

#include "hs_row_bf16_kernel.cuh"

namespace hs {

static_assert(kTopKMax == kCandidateTopKMax, "both kernels agree on which rows are candidate rows");

// score of a token with logit x that the history holds `count` times
__device__ __forceinline__ float score_of_float(const Ctx3& c, float x, int count) {
  float v = canonical(x);
  if (count > 0) {
    v = v < 0.0f ? __fmul_rn(v, c.rp) : __fdiv_rn(v, c.rp);
    v = __fsub_rn(v, c.pp);
    v = __fsub_rn(v, __fmul_rn(c.fp, (float)count));
  }
  return c.score_of_value(v);
}

// Per count class (thr[0..2]), the lowest logit value whose score key reaches `bound`, NaN when
// none does.  Warp cc searches the ordered patterns from -inf to +inf.
__device__ void f32_thresholds(const Ctx3& c, uint32_t bound, float* thr) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < 3) {
    const int cc = warp;
    const u64 first = (u64)key_of(__int_as_float(0xff800000));       // -inf
    const u64 none = (u64)key_of(__int_as_float(0x7f800000)) + 1ull;  // one past +inf
    // every pattern below lo fails, every pattern from hi on passes (hi = none: nothing does)
    u64 lo = first, hi = none;
#pragma unroll 1
    while (lo < hi) {
      const u64 step = (hi - lo + 31ull) >> 5;
      const u64 t = lo + (u64)(lane + 1) * step - 1ull;  // last pattern of this lane's block
      const bool pass = t >= hi || key_of(score_of_float(c, score_of((uint32_t)t), cc)) >= bound;
      const uint32_t votes = __ballot_sync(0xffffffffu, pass);
      if (votes == 0) { lo = hi; break; }
      const int f = __ffs(votes) - 1;  // the answer lies in block f
      hi = min(lo + (u64)(f + 1) * step - 1ull, hi);
      lo = lo + (u64)f * step;
    }
    if (lane == 0) thr[cc] = lo >= none ? __int_as_float(0x7fc00000) : score_of((uint32_t)lo);
  }
  __syncthreads();
}

struct F32TopkArgs {
  RowKernelArgs base;
  unsigned long long* phase_clocks;
};

__global__ void __launch_bounds__(kThreads, 2) row_kernel_f32_topk(const F32TopkArgs args) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const RowKernelArgs& a = args.base;
  const int row = blockIdx.x;
  const hs_row_params P = a.params[row];
  if (!is_candidate_row(P, a.vocab)) return;  // the general kernel's row
  const LayoutCand lay = layout_cand();
  Ctx3 c;
  c.x = reinterpret_cast<Exchange*>(smem_raw + lay.x);
  int* small = reinterpret_cast<int*>(smem_raw + lay.small);
  CandCtx L{reinterpret_cast<u64*>(smem_raw + lay.cand), small + 4, small + 5,
            reinterpret_cast<uint32_t*>(smem_raw + lay.count), small + 8, nullptr};
  float* thr = reinterpret_cast<float*>(small + 12);  // [3]
  const int tid = threadIdx.x;
  c.row = row;
  c.vocab = a.vocab;
  c.lo = 0;
  c.hi = a.vocab;
  c.greedy = false;
  c.logits = nullptr;
  const float* logits = reinterpret_cast<const float*>(a.logits) + (long long)row * a.row_stride;
  const bool vec = (reinterpret_cast<uintptr_t>(logits) & 15u) == 0;
  hs_row_out* out = a.out + row;
  c.T = P.temperature; c.rp = P.repetition_penalty; c.pp = P.presence_penalty; c.fp = P.frequency_penalty;
  c.pool = a.pool;
  c.slot = P.slot;
  const bool slot_ok = P.slot >= 0 && P.slot < a.pool.slots_total;
  const bool penalised = slot_ok && (c.rp != 1.0f || c.pp != 0.0f || c.fp != 0.0f);
  c.cls = penalised ? a.pool.cls + (size_t)P.slot * a.pool.cls_stride : nullptr;
  c.s_pair = nullptr; c.n_s = 0; c.s_cap = 0; c.cl = nullptr; c.n_cl = 0; c.m = 0.f;
  c.tab = nullptr; c.hist = nullptr; c.gbuf = nullptr; c.list = nullptr; c.gbuf_n = nullptr;
  if (tid < 16) small[tid] = 0;
  __syncthreads();
  const int k = P.top_k;  // (0 < k <= kTopKMax and k < vocab)

  auto push = [&](int id, float x, int count) {
    const int slot = atomicAdd(L.n, 1);
    if (slot < kCandCap) L.cand[slot] = cand_pack(key_of(score_of_float(c, x, count)), id);
    else *L.lost = 1;
  };

  // 1. the first bound: every thread scores eight tokens and lists its best.  The eight are
  // neighbours (two 128-bit loads, one 32-byte sector, one or two words of the class map); the
  // 512 groups are spread evenly over the row and do not overlap, so the 512 listed tokens are
  // different tokens.  (A row without a 16-byte aligned view, or of fewer than about 4,100
  // tokens, goes without a bound: everything is listed.)
  uint32_t bound = 0;
  {
    const int n4_all = vec ? c.vocab / 4 : 0;
    const bool sampled = n4_all >= 2 * kThreads + 2;
    u64 best = 0;
    if (sampled) {
      const int i = (int)(((long long)tid * (n4_all - 2)) / kThreads);  // groups at least two chunks apart
      const float4 a4 = reinterpret_cast<const float4*>(logits)[i], b4 = reinterpret_cast<const float4*>(logits)[i + 1];
      const float xs[8] = {a4.x, a4.y, a4.z, a4.w, b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int id = 4 * i + j;
        const int cc = c.class_of(id);
        if (cc == 3 || xs[j] != xs[j]) continue;  // (listed per request and taken below; NaN)
        const u64 e = cand_pack(key_of(score_of_float(c, xs[j], cc)), id);
        best = e > best ? e : best;
      }
    }
    L.cand[tid] = best;
    __syncthreads();
    if (sampled) bound = cand_kth_key(*c.x, L, kThreads, k);
    __syncthreads();
  }
  // 2. tokens the history holds three times or more: from the request's list, with their count
  if (c.cls) {
    const int n_heavy = min(c.pool.n_heavy[c.slot], c.pool.unique_cap);
    const int32_t* heavy = c.pool.heavy + (size_t)c.slot * c.pool.unique_cap;
    const int2* pairs = c.pool.pairs + (size_t)c.slot * c.pool.unique_cap;
    for (int j = tid; j < n_heavy; j += kThreads) {
      const int q = heavy[j];
      if (q < 0 || q >= c.pool.unique_cap) continue;
      const int2 pr = pairs[q];  // (id, count)
      if (pr.x < 0 || pr.x >= c.vocab) continue;
      const float x = logits[pr.x];
      if (x == x) push(pr.x, x, pr.y);
    }
  }
  __syncthreads();
  // (read by every thread before the barrier in f32_thresholds: after it the stream adds to the list)
  int n_scored = min(*L.n, kCandCap);  // the often-repeated tokens, scored when they were listed
  f32_thresholds(c, bound, thr);

  // 3. the row, once: four values per 128-bit load against the most permissive threshold
  // A hit is listed unscored, (value bits, id), by the lane that found it: looking its count
  // class up there would stall the stream on a scattered load per hit.  The listed hits are
  // scored in bulk, all lanes busy, whenever the list is looked at; a token of a penalised
  // class that does not reach its own threshold drops out then.
  auto look = [&](int id, float x) {
    const int slot = atomicAdd(L.n, 1);
    if (slot < kCandCap) L.cand[slot] = ((u64)__float_as_uint(x) << 32) | (uint32_t)id;
    else *L.lost = 1;
  };
  auto score_pending = [&](int from, int to) {
#pragma unroll 1
    for (int i = from + tid; i < to; i += kThreads) {
      const u64 e = L.cand[i];
      const int id = (int)(uint32_t)e;
      const float x = __uint_as_float((uint32_t)(e >> 32));
      const int cc = c.class_of(id);
      const bool valid = cc != 3 && x >= thr[cc];  // (three times or more: listed above already)
      L.cand[i] = valid ? cand_pack(key_of(score_of_float(c, x, cc)), id) : 0ull;
    }
    __syncthreads();
  };
  const int n4 = vec ? c.vocab / 4 : 0;
  const float4* src4 = reinterpret_cast<const float4*>(logits);
  constexpr int kBatch = 4;
  // One buffer: a chunk's successor is requested as soon as the chunk has been tested, so a
  // request has a whole pass of the loop to arrive, and the registers hold one batch only.
  float4 w[kBatch];
#pragma unroll
  for (int u = 0; u < kBatch; ++u) {
    const int i = tid + u * kThreads;
    if (i < n4) w[u] = __ldcs(src4 + i);
  }
  int iteration = 0, next_look = 1, last_look = -1, last_seen = 0;
  for (int base = 0; base < n4; base += kBatch * kThreads, ++iteration) {
    float t_min = thr[0];
    if (c.cls) t_min = fminf(t_min, fminf(thr[1], thr[2]));  // (a NaN threshold, "none", is ignored by fminf)
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = base + tid + u * kThreads;
      if (i < n4) {
        const float4 v = w[u];
        if (i + kBatch * kThreads < n4) w[u] = __ldcs(src4 + i + kBatch * kThreads);
        if (!(v.x >= t_min || v.y >= t_min || v.z >= t_min || v.w >= t_min)) continue;  // the common case
        if (v.x >= t_min) look(4 * i, v.x);
        if (v.y >= t_min) look(4 * i + 1, v.y);
        if (v.z >= t_min) look(4 * i + 2, v.z);
        if (v.w >= t_min) look(4 * i + 3, v.w);
      }
    }
    // a look at the list's length now and then, the sooner the faster it grows (see the bf16
    // candidate stream)
    if (iteration != next_look) continue;
    if (tid == 0) L.lost[2] = *L.n;
    const bool refresh = __syncthreads_or(*L.n >= kCandSoft);
    {
      const int seen = L.lost[2];
      const int per_batch = max(0, seen - last_seen) / (iteration - last_look);
      last_seen = seen;
      last_look = iteration;
      constexpr int kRoom = (kCandCap - kCandSoft) / 2;
      next_look = iteration + (per_batch * 8 <= kRoom ? 8 : (per_batch * 4 <= kRoom ? 4 : (per_batch * 2 <= kRoom ? 2 : 1)));
    }
    // raise the bound when the list is getting long (block-uniform decision)
    if (refresh) {
      if (*L.lost) break;
      const int n_now = min(*L.n, kCandCap);
      score_pending(n_scored, n_now);
      bound = cand_kth_key(*c.x, L, n_now, k);
      n_scored = last_seen = cand_compact(L, n_now, bound);
      f32_thresholds(c, bound, thr);
    }
  }
  __syncthreads();
  {
    float t_min = thr[0];
    if (c.cls) t_min = fminf(t_min, fminf(thr[1], thr[2]));
    for (int id = n4 * 4 + tid; id < c.vocab; id += kThreads) {
      const float x = logits[id];
      if (x >= t_min) look(id, x);
    }
  }
  __syncthreads();
  if (!*L.lost) score_pending(n_scored, min(*L.n, kCandCap));
  int n = *L.lost ? -1 : min(*L.n, kCandCap);
  if (n < 0) {
    // more ties than the list holds: the general kernel samples this row
    if (tid == 0) { out->token = 0; out->status = 4; out->n_top = 0; out->n_kept = 0; out->logprob = 0.f; }
    return;
  }
  {
    // (without a cut the pass still drops the entries the scoring voided)
    const uint32_t cut = n > k && n > kSortAll ? cand_kth_key(*c.x, L, n, k) : 0u;
    n = cand_compact(L, n, cut);
  }
  cand_sort(L, n);
  if (n > k) {
    // a list that was sorted whole: top-k keeps the first k entries and the ties of the k-th
    const uint32_t cut = cand_key(L.cand[k - 1]);
    u64 keep = 0, unused = 0;
    for (int i = tid; i < n; i += kThreads) keep += cand_key(L.cand[i]) >= cut ? 1 : 0;
    block_sum2(*c.x, keep, unused);
    n = (int)keep;
  }
  const float* noise_row = a.noise ? a.noise + (size_t)row * a.vocab : nullptr;
  FinishOut r = finish_sorted(*c.x, L.cand, reinterpret_cast<u64*>(smem_raw + lay.mass), n, P, noise_row, out, nullptr);
  if (P.slot >= a.pool.slots_total) r.status |= 64;  // a slot this sampler does not have: no penalties
  if (a.scores_out) {
    float* dst = a.scores_out + (size_t)row * a.vocab;
    for (int id = tid; id < c.vocab; id += kThreads) dst[id] = __int_as_float(0xff800000);
    __syncthreads();
    for (int i = tid; i < (int)r.n_kept; i += kThreads) dst[cand_id(L.cand[i])] = score_of(cand_key(L.cand[i]));
  }
  if (tid == 0) {
    write_finish(r, out);
    if (a.tokens_out) a.tokens_out[row] = r.token;
    if ((a.flags & HS_SAMPLE_APPEND_TOKEN) && slot_ok && r.token >= 0 && r.token < a.vocab) {
      if (!slot_append_one(a.pool, P.slot, r.token)) out->status = r.status | 2;
    }
  }
}

}  // namespace hs
