// Vocabulary-sharded sampling: every GPU holds a contiguous slice of the vocabulary (the
// output of a tensor-parallel LM head).  Each rank reduces its slice of a row to a small
// record -- the top-k candidates (ties at the k-th included), the slice's maximum score and
// its soft-max denominator -- the records are exchanged (NCCL all-gather, about half a
// kilobyte per row per rank), and every rank finishes the row from the union of the
// candidates.  Exact because top_k bounds the candidate set: a token outside its own
// slice's top k cannot be inside the row's.
#pragma once

#include "hs_row_v3.cuh"
#include "hs_row_topk.cuh"

namespace hs {

struct ShardArgs {
  RowKernelArgs base;   // logits = this rank's slice, vocab = slice width, params of all rows
  int vocab_offset;     // global id of the slice's first token
  hs_shard_rec* recs;   // [batch]
};

// smem: Exchange | cand[kCandCap] | mass[kCandCap] | count[kBins] | small[16]
struct LayoutCand {
  size_t x, cand, mass, count, small, total;
};
__host__ __device__ inline LayoutCand layout_cand() {
  LayoutCand l{};
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t at = off; off = (off + bytes + 15) & ~size_t(15); return at; };
  l.x = take(sizeof(Exchange));
  l.cand = take(sizeof(u64) * kCandCap);
  l.mass = take(sizeof(u64) * kCandCap);
  l.count = take(sizeof(uint32_t) * kBins);
  l.small = take(sizeof(int) * 16);
  l.total = off;
  return l;
}

__global__ void __launch_bounds__(kThreads, 2) shard_partial_kernel(const ShardArgs args) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const RowKernelArgs& a = args.base;
  const LayoutCand lay = layout_cand();
  Ctx3 c;
  c.x = reinterpret_cast<Exchange*>(smem_raw + lay.x);
  int* small = reinterpret_cast<int*>(smem_raw + lay.small);
  CandCtx L{reinterpret_cast<u64*>(smem_raw + lay.cand), small + 4, small + 5,
            reinterpret_cast<uint32_t*>(smem_raw + lay.count), small + 8, nullptr};
  const int tid = threadIdx.x;
  c.row = blockIdx.x;
  c.vocab = a.vocab;
  c.lo = 0;
  c.hi = a.vocab;
  c.logits = reinterpret_cast<const unsigned short*>(a.logits) + (long long)c.row * a.row_stride;
  c.vec = (reinterpret_cast<uintptr_t>(c.logits) & 15u) == 0;
  const hs_row_params P = a.params[c.row];
  c.greedy = P.temperature == 0.0f;
  c.T = P.temperature; c.rp = P.repetition_penalty; c.pp = P.presence_penalty; c.fp = P.frequency_penalty;
  c.pool = a.pool;
  c.slot = P.slot;
  const bool slot_ok = P.slot >= 0 && P.slot < a.pool.slots_total;
  const bool penalised = slot_ok && (c.rp != 1.0f || c.pp != 0.0f || c.fp != 0.0f);
  c.cls = penalised ? a.pool.cls + (size_t)P.slot * a.pool.cls_stride : nullptr;
  c.s_pair = nullptr; c.n_s = 0; c.s_cap = 0; c.cl = nullptr; c.n_cl = 0; c.m = 0.f;
  c.tab = nullptr; c.hist = nullptr; c.gbuf = nullptr; c.list = nullptr; c.gbuf_n = nullptr;
  hs_shard_rec* rec = args.recs + c.row;
  if (tid < 16) small[tid] = 0;
  __syncthreads();
  const int k = min(max(P.top_k, 1), c.vocab);
  int n = topk_candidates(c, L, k);
  int status = P.slot >= a.pool.slots_total ? 64 : 0;  // a slot this sampler does not have: no penalties
  // list overflow: what is in the list is partly unscored, so the record carries no candidates
  // and the merge reports the row as failed
  if (n < 0) { status |= 16; n = 0; }
  if (n > k) {
    const uint32_t cut = cand_kth_key(*c.x, L, n, k);
    n = cand_compact(L, n, cut);
  } else if (n > 0) {
    n = cand_compact(L, n, 0u);  // drops entries the scoring pass voided
  }
  cand_sort(L, n);
  if (n > HS_SHARD_CAND) { status |= 32; n = HS_SHARD_CAND; }  // more ties than the record holds
  __syncthreads();
  const float m = n > 0 ? score_of(cand_key(L.cand[0])) : 0.f;
  // The record's candidates leave shared memory now: the list's place is needed below.
  for (int i = tid; i < HS_SHARD_CAND; i += kThreads) {
    rec->ids[i] = i < n ? cand_id(L.cand[i]) + args.vocab_offset : -1;
    rec->scores[i] = i < n ? score_of(cand_key(L.cand[i])) : 0.f;
  }
  __syncthreads();
  // Soft-max denominator of the whole slice, relative to the slice maximum (exact integer
  // mass).  A token's mass follows from its value and count class, so the slice (streamed a
  // moment ago, it sits in L2) is COUNTED per class into three tables of one-value bins, in the
  // candidate list's place, and every non-empty class contributes count x mass: one exponential
  // per class instead of one per token.  Tokens held three times or more, and values outside
  // the bin window, are rare and add their mass directly.
  u64 z = 0, unused = 0;
  {
    uint32_t* tab = reinterpret_cast<uint32_t*>(smem_raw + lay.cand);
    static_assert(sizeof(uint32_t) * kCells <= sizeof(u64) * kCandCap * 2 + sizeof(uint32_t) * kBins,
                  "the count tables fit in the place of the candidate list, its masses and the counters");
    for (int i = tid; i < kCells; i += kThreads) tab[i] = 0;
    __syncthreads();
    const int n8 = c.vec ? c.vocab / 8 : 0;
    const uint4* src4 = reinterpret_cast<const uint4*>(c.logits);
    const unsigned short* cls16p = reinterpret_cast<const unsigned short*>(c.cls);
    const uint32_t tab_at = (uint32_t)__cvta_generic_to_shared(tab);
    auto take = [&](int id, uint32_t raw, int cc) {
      const int b = cc == 3 ? -1 : v3_bin_of_raw(raw);
      if (b >= 0) asm volatile("red.shared.add.u32 [%0], 1;" ::"r"(tab_at + 4u * (uint32_t)(cc * kV3Bins + b)) : "memory");
      else z += mass_of(c.element_score(id, raw, cc), m);
    };
    for (int i = tid; i < n8; i += kThreads) {
      const uint4 w = __ldcg(src4 + i);
      const uint32_t cl = cls16p ? (uint32_t)cls16p[i] : 0u;
      const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int q = 0; q < 8; ++q)
        take(8 * i + q, (words[q >> 1] >> (16 * (q & 1))) & 0xffffu, (int)((cl >> (2 * q)) & 3u));
    }
    for (int id = n8 * 8 + tid; id < c.vocab; id += kThreads) take(id, c.logits[id], c.class_of(id));
    __syncthreads();
    for (int cell = tid; cell < kCells; cell += kThreads) {
      const uint32_t count = tab[cell];
      if (count) z += (u64)count * mass_of(c.cell_score(cell), m);
    }
  }
  block_sum2(*c.x, z, unused);
  if (tid == 0) {
    rec->row_max = m;
    rec->pad = 0.f;
    rec->z_mass = z;
    rec->n = n;
    rec->status = status;
  }
}

struct MergeArgs {
  const hs_shard_rec* recs;  // [ranks][batch]
  int ranks, batch, vocab_total;
  const hs_row_params* params;
  hs_row_out* out;
  const float* noise;        // [batch, vocab_total] or null
  float* full_lse;           // [batch] log-sum-exp over the whole vocabulary, or null
};

__global__ void __launch_bounds__(kThreads, 2) shard_merge_kernel(const MergeArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const LayoutCand lay = layout_cand();
  Exchange* x = reinterpret_cast<Exchange*>(smem_raw + lay.x);
  int* small = reinterpret_cast<int*>(smem_raw + lay.small);
  CandCtx L{reinterpret_cast<u64*>(smem_raw + lay.cand), small + 4, small + 5,
            reinterpret_cast<uint32_t*>(smem_raw + lay.count), small + 8, nullptr};
  u64* mass = reinterpret_cast<u64*>(smem_raw + lay.mass);
  const int tid = threadIdx.x, row = blockIdx.x;
  const hs_row_params P = a.params[row];
  hs_row_out* out = a.out + row;
  if (tid < 16) small[tid] = 0;
  __syncthreads();
  int status = 0;
  // union of the ranks' candidates
  for (int i = tid; i < a.ranks * HS_SHARD_CAND; i += kThreads) {
    const hs_shard_rec* rec = a.recs + (size_t)(i / HS_SHARD_CAND) * a.batch + row;
    const int j = i % HS_SHARD_CAND;
    if (j < rec->n && rec->ids[j] >= 0) {
      const int slot = atomicAdd(L.n, 1);
      if (slot < kCandCap) L.cand[slot] = cand_pack(key_of(rec->scores[j]), rec->ids[j]);
    }
    if (j == 0 && rec->status) atomicOr(small + 6, rec->status);
  }
  __syncthreads();
  int n = min(*L.n, kCandCap);
  status = small[6];
  if (n == 0) {
    if (tid == 0) { out->token = 0; out->status = status | 1; out->n_top = 0; out->n_kept = 0; }
    return;
  }
  const int k = P.top_k > 0 ? P.top_k : n;
  if (n > k) {
    const uint32_t cut = cand_kth_key(*x, L, n, k);
    n = cand_compact(L, n, cut);
  }
  cand_sort(L, n);
  const float* noise_row = a.noise ? a.noise + (size_t)row * a.vocab_total : nullptr;
  FinishOut r = finish_sorted(*x, L.cand, mass, n, P, noise_row, out);
  r.status |= status;
  if (tid == 0) {
    write_finish(r, out);
    if (a.full_lse) {
      // log sum exp over the whole vocabulary from the slices' (max, denominator) pairs
      double acc = 0.0;
      for (int rk = 0; rk < a.ranks; ++rk) {
        const hs_shard_rec* rec = a.recs + (size_t)rk * a.batch + row;
        if (rec->n > 0) acc += (double)rec->z_mass * 9.094947017729282e-13 * exp((double)rec->row_max - (double)r.m);
      }
      a.full_lse[row] = (float)((double)r.m + log(acc));
    }
  }
}

}  // namespace hs
