// The bf16 row kernel: one launch per step, one CTA per work item, two CTAs resident per SM.
// An item is a row for the counting path (hs_row_v3.cuh; also the plain arg-max rows of a
// mixed batch) or one part of a row for the candidate path (small top_k, hs_row_topk.cuh);
// the hardware hands the items out in grid order as SMs free up, the long ones first.  No CTA
// waits for another: the last part of a candidate row to arrive finishes that row, and a row
// whose candidate list overflowed is counted by the CTA that found out.
#pragma once
#include <type_traits>

#include "hs_row_v3.cuh"
#include "hs_row_topk.cuh"
#include "hs_sharded.cuh"

namespace hs {

// One chunk of eight tokens the counting loop could not take in its branch-free form (a
// value outside the bin window, a token of count class 3): token by token, out of line so
// that the unrolled loop stays small.
__device__ __noinline__ void count_chunk_slow(uint32_t* tab, int* rare_n, int2* rare, uint4 w, uint32_t cl, int i) {
  const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll 1
  for (int k = 0; k < 8; ++k) {
    const uint32_t raw = (words[k >> 1] >> (16 * (k & 1))) & 0xffffu;
    const int cc = (int)((cl >> (2 * k)) & 3u);
    if (cc == 3) continue;  // listed per request; scored individually with its exact count
    const int b = v3_bin_of_raw(raw);
    if (b >= 0) {
      atomicAdd(&tab[cc * kV3Bins + b], 1u);
    } else {
      const int slot = atomicAdd(rare_n, 1);
      if (slot < kV3RareCap) rare[slot] = make_int2(8 * i + k, (int)(raw | ((uint32_t)cc << 16)));
    }
  }
}

// The counting path for one row (also: plain arg max of a row in a mixed batch).  part < 0:
// this CTA counts the whole row.  part >= 0: the row's tokens are counted by args.csplit CTAs,
// each a contiguous range; every part leaves its count table and rare list in global scratch,
// and the part that arrives last (a ticket) adds the others' to its own and goes on alone.
__device__ __forceinline__ void count_row(const RowV3Args& args, unsigned char* smem_raw, int row_index, int part) {
  const RowKernelArgs& a = args.base;
  const LayoutV3 lay = layout_v3();
  Ctx3 c;
  c.x = reinterpret_cast<Exchange*>(smem_raw + lay.x);
  c.tab = reinterpret_cast<uint32_t*>(smem_raw + lay.tab);
  c.hist = reinterpret_cast<LocalHist*>(smem_raw + lay.hist);   // in the count table's place, once it has served
  c.gbuf = reinterpret_cast<V3Entry*>(smem_raw + lay.gbuf);
  c.list = reinterpret_cast<V3Entry*>(smem_raw + lay.list);
  int2* side_shared = reinterpret_cast<int2*>(smem_raw + lay.side);
  int2* rare = reinterpret_cast<int2*>(smem_raw + lay.rare);  // (id, raw bits | count class << 16)
  int* small = reinterpret_cast<int*>(smem_raw + lay.small);
  c.gbuf_n = small;
  c.step_n = small + 24;
  int* rare_n = small + 1;
  int* side_n = small + 2;
  int* defer_n = small + 27;
  int* defer = reinterpret_cast<int*>(smem_raw + lay.defer);
  const int tid = threadIdx.x;
  c.row = row_index;
  c.vocab = a.vocab;
  c.logits = reinterpret_cast<const unsigned short*>(a.logits) + (long long)c.row * a.row_stride;
  c.vec = (reinterpret_cast<uintptr_t>(c.logits) & 15u) == 0;
  const hs_row_params P = a.params[c.row];
  hs_row_out* out = a.out + c.row;
  c.greedy = P.temperature == 0.0f;
  c.T = P.temperature;
  c.rp = P.repetition_penalty;
  c.pp = P.presence_penalty;
  c.fp = P.frequency_penalty;
  c.pool = a.pool;
  c.slot = P.slot;
  const bool slot_ok = P.slot >= 0 && P.slot < a.pool.slots_total;
  const bool penalised = slot_ok && (P.repetition_penalty != 1.0f || P.presence_penalty != 0.0f ||
                                     P.frequency_penalty != 0.0f);
  c.cls = penalised ? a.pool.cls + (size_t)P.slot * a.pool.cls_stride : nullptr;
  c.s_pair = nullptr;
  c.s_cap = 0;
  c.n_s = 0;
  c.cl = nullptr;
  c.n_cl = 0;
  c.m = 0.f;
  unsigned long long* clocks = args.phase_clocks ? args.phase_clocks + (size_t)c.row * kV3PhaseSlots : nullptr;
  c.dbg = clocks;
  auto mark = [&](int slot) {
    if (clocks && tid == 0) clocks[slot] = clock64();
  };
  mark(0);
  int status = P.slot >= a.pool.slots_total ? 64 : 0;  // a slot this sampler does not have: no penalties

  // ---- plain greedy rows of a mixed batch: arg max only -----------------------------------
  if (c.greedy && !penalised && P.n_logprobs < 0) {
    if (part > 0) return;  // (one CTA walks the whole row)
    u64 best = 0;
    auto consider = [&](uint32_t raw, int id) {
      const u64 packed = ((u64)key_of(canonical(__uint_as_float(raw << 16))) << 32) | (uint32_t)(~(uint32_t)id);
      best = packed > best ? packed : best;
    };
    const int n8 = c.vec ? c.vocab / 8 : 0;
    for (int i = tid; i < n8; i += kThreads) {
      uint32_t raw[8], cls16;
      load_chunk(c, i, raw, cls16);
#pragma unroll
      for (int k = 0; k < 8; ++k) consider(raw[k], 8 * i + k);
    }
    for (int id = n8 * 8 + tid; id < c.vocab; id += kThreads) consider(c.logits[id], id);
    best = block_max_u64(*c.x, best);
    if (a.scores_out) {
      float* dst = a.scores_out + (size_t)c.row * a.vocab;
      for (int id = tid; id < c.vocab; id += kThreads) dst[id] = canonical(__uint_as_float((uint32_t)c.logits[id] << 16));
    }
    if (tid == 0) {
      out->token = (int)(~(uint32_t)(best & 0xffffffffu));
      if (a.tokens_out) a.tokens_out[c.row] = out->token;
      out->logprob = 0.f; out->n_top = 0; out->status = status;
      out->n_kept = a.vocab; out->n_after_topk = a.vocab; out->n_after_minp = a.vocab; out->n_after_topp = a.vocab;
      out->cut_bits = 0xff800000u; out->n_cut_ties = -1;
      out->row_max = score_of((uint32_t)(best >> 32)); out->log_z = 0.f;
    }
    return;
  }

  // The side list needs (id, count, value) of the tokens held three times or more: three
  // dependent reads.  Thread t starts the chain for list entry t here and takes one step of
  // it at each stop below, so that it has run its course by the time the row is counted.
  int n_heavy = 0, hv_q = -1;
  int2 hv_pair = make_int2(-1, 0);
  uint32_t hv_raw = 0;
  if (penalised) {
    n_heavy = a.pool.n_heavy[P.slot];
    if (tid < a.pool.unique_cap) hv_q = load_now_s32(a.pool.heavy + (size_t)P.slot * a.pool.unique_cap + tid);
  }
  // this CTA's range of 8-token chunks [chunk_lo, chunk_hi); the last part also takes the
  // tokens after the last whole chunk
  const int n8_row = c.vec ? c.vocab / 8 : 0;
  const int parts = part < 0 ? 1 : args.csplit;
  const int my_part = part < 0 ? 0 : part;
  const int per_part = (n8_row + parts - 1) / parts;
  const int chunk_lo = min(my_part * per_part, n8_row), chunk_hi = min(chunk_lo + per_part, n8_row);
  const bool last_part = my_part == parts - 1;
  // small[16..18] / [19..21]: highest (+ 1) / lowest non-empty cell per count class; [22]: lowest side key
  if (tid < 32) small[tid] = (tid >= 19 && tid <= 22) ? -1 : 0;
  if (tid == 0) c.x->bcast[5] = 0;  // highest side element, (key, ~id)
  __syncthreads();
  for (int i = tid; i < kCells; i += kThreads) c.tab[i] = 0;
  __syncthreads();
  // (more often-repeated tokens than the side list holds: the general kernel's row)
  if (n_heavy > min(a.pool.unique_cap, args.s_cap)) status |= 4;
  n_heavy = min(n_heavy, min(a.pool.unique_cap, args.s_cap));
  if (tid < n_heavy && hv_q >= 0 && hv_q < a.pool.unique_cap)
    hv_pair = load_now_int2(a.pool.pairs + (size_t)P.slot * a.pool.unique_cap + hv_q);  // (id, count)

  // ---- A. the one read of the row from HBM: count tokens per (count class, value) --------
  {
    auto count_one = [&](uint32_t raw, int cc, int id) {
      if (cc == 3) return;  // listed per request; handled below with its exact count
      const int b = v3_bin_of_raw(raw);
      if (b >= 0) {
        atomicAdd(&c.tab[cc * kV3Bins + b], 1u);
      } else {
        const int slot = atomicAdd(rare_n, 1);
        if (slot < kV3RareCap) rare[slot] = make_int2(id, (int)(raw | ((uint32_t)cc << 16)));
      }
    };
    const uint4* src4 = reinterpret_cast<const uint4*>(c.logits);
    const unsigned short* cls16p = reinterpret_cast<const unsigned short*>(c.cls);
    // Eight tokens at a time without a branch per token.  Per 32-bit word (two tokens):
    // |x| + (0x8000 - base) sets bit 15 of a half iff |x| >= base and leaves |x| - base in its
    // low bits; |x| + (0x8000 - top) sets it iff |x| >= top; a byte permute with sign
    // replication turns the two sign bits into two 16-bit masks, and one LOP3 leaves, per half,
    // the bin relative to the middle of a class table as a signed 16-bit number (idx for
    // x >= 0, -1 - idx for x < 0).  Per token: sign-extending extraction (one permute), class
    // offset and table address (two multiply-adds on the FMA pipe), the reduction.  A chunk
    // with a value outside the window or a token of count class 3 (rare) takes the per-token
    // path.  Written as PTX where one instruction is meant.
    constexpr uint32_t kLoAdd = (0x8000u - kV3Base) * 0x00010001u;
    constexpr uint32_t kHiAdd = (0x8000u - (kV3Base + (uint32_t)kV3Half)) * 0x00010001u;
    constexpr uint32_t kClassBytes = (uint32_t)(kV3Bins * 4);
    const uint32_t tab_mid = (uint32_t)__cvta_generic_to_shared(c.tab + kV3Half);
    auto take_chunk = [&](const uint4& w4, uint32_t cl4, int i) {
      const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
      uint32_t rel2[4];
      uint32_t wnd = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint32_t mag, mask;
        asm("and.b32 %0, %1, 0x7fff7fff;" : "=r"(mag) : "r"(words[k]));
        const uint32_t lo = mag + kLoAdd, ht = mag + kHiAdd;
        asm("lop3.b32 %0, %1, %2, %3, 0xef;" : "=r"(wnd) : "r"(lo), "r"(ht), "r"(wnd));     // wnd | ~lo | ht
        asm("prmt.b32 %0, %1, 0, 0xBB99;" : "=r"(mask) : "r"(words[k]));                     // 0xffff per negative half
        asm("lop3.b32 %0, %1, 0x7fff7fff, %2, 0x6a;" : "=r"(rel2[k]) : "r"(lo), "r"(mask));  // (lo & 0x7fff7fff) ^ mask
      }
      // bits 15 / 31 of wnd: a value outside the window; bit 2J of cl & (cl >> 1): token J is of class 3
      if (((wnd & 0x80008000u) | (cl4 & (cl4 >> 1) & 0x5555u)) == 0) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int kShift = 2 * (2 * k + h);
            uint32_t r;
            if (h == 0) asm("prmt.b32 %0, %1, 0, 0x9910;" : "=r"(r) : "r"(rel2[k]));  // low half, sign extended
            else asm("prmt.b32 %0, %1, 0, 0xBB32;" : "=r"(r) : "r"(rel2[k]));          // high half, sign extended
            uint32_t base;
            if (kShift < 14) base = (cl4 & (3u << kShift)) * (kClassBytes >> kShift) + tab_mid;
            else base = (cl4 >> 14) * kClassBytes + tab_mid;
            const uint32_t addr = r * 4u + base;
            asm volatile("red.shared.add.u32 [%0], 1;" ::"r"(addr) : "memory");
          }
        }
      } else {
        // set aside: a call here would save and restore the loop's registers through local
        // memory (round trips to L2 with this kernel's small L1), a few thousand cycles a time
        const int slot = atomicAdd(defer_n, 1);
        if (slot < kV3DeferCap) defer[slot] = i;
      }
    };
    // Two batches of loads: the next one is on its way while this one is counted.  The main
    // loop runs without bounds checks; what is left over is taken chunk by chunk.
    constexpr int kInFlight = 2;  // 128-bit loads per thread and batch
    constexpr int kStride = kInFlight * kThreads;
    const int n_full = (chunk_hi - chunk_lo) / kStride;
    int i0 = chunk_lo + tid;
    if (hv_pair.x >= 0 && hv_pair.x < c.vocab) hv_raw = load_now_u16(c.logits + hv_pair.x);
    if (n_full > 0) {
      uint4 w[kInFlight], wn[kInFlight];
      uint32_t cl[kInFlight], cn[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        w[u] = __ldcg(src4 + i0 + u * kThreads);  // past L1: almost all of it is shared memory here
        cl[u] = cls16p ? (uint32_t)__ldcg(cls16p + i0 + u * kThreads) : 0u;
        wn[u] = w[u];
        cn[u] = cl[u];
      }
      for (int it = 0; it < n_full; ++it) {
        if (it + 1 < n_full) {
#pragma unroll
          for (int u = 0; u < kInFlight; ++u) {
            wn[u] = __ldcg(src4 + i0 + kStride + u * kThreads);
            cn[u] = cls16p ? (uint32_t)__ldcg(cls16p + i0 + kStride + u * kThreads) : 0u;
          }
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) take_chunk(w[u], cl[u], i0 + u * kThreads);
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) { w[u] = wn[u]; cl[u] = cn[u]; }
        i0 += kStride;
      }
    }
    for (int i = i0; i < chunk_hi; i += kThreads) take_chunk(__ldcg(src4 + i), cls16p ? (uint32_t)__ldcg(cls16p + i) : 0u, i);
    // the chunks that were set aside, token by token, one thread per chunk
    __syncthreads();
    {
      const int n_defer = *defer_n;
      if (n_defer <= kV3DeferCap) {
        for (int j = tid; j < n_defer; j += kThreads) {
          const int i = defer[j];
          count_chunk_slow(c.tab, rare_n, rare, __ldcg(src4 + i), cls16p ? (uint32_t)__ldcg(cls16p + i) : 0u, i);
        }
      } else {
        // more than the list holds (a row full of values outside the bin window): every chunk of
        // the range is looked at again and those the loop did not take are counted now
        for (int i = chunk_lo + tid; i < chunk_hi; i += kThreads) {
          const uint4 w4 = __ldcg(src4 + i);
          const uint32_t cl4 = cls16p ? (uint32_t)__ldcg(cls16p + i) : 0u;
          const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
          bool slow = (cl4 & (cl4 >> 1) & 0x5555u) != 0u;
#pragma unroll
          for (int q = 0; q < 8; ++q) slow = slow || v3_bin_of_raw((words[q >> 1] >> (16 * (q & 1))) & 0xffffu) < 0;
          if (slow) count_chunk_slow(c.tab, rare_n, rare, w4, cl4, i);
        }
      }
    }
    if (last_part)
      for (int id = n8_row * 8 + tid; id < c.vocab; id += kThreads) count_one(c.logits[id], c.class_of(id), id);
  }
  __syncthreads();
  if (parts > 1) {
    // Hand this part's counts over: table and rare list to global scratch, then a ticket.  The
    // part that draws the last ticket adds the other parts' to its own and goes on; the
    // others are done.  Nobody waits for anybody.
    const size_t mine = (size_t)c.row * parts + my_part;
    uint32_t* gtab = args.ctab + mine * kCells;
    for (int i = tid; i < kCells / 4; i += kThreads)
      reinterpret_cast<uint4*>(gtab)[i] = reinterpret_cast<const uint4*>(c.tab)[i];
    const int nr = *rare_n;
    for (int t = tid; t < min(nr, kV3RareCap); t += kThreads) args.crare[mine * kV3RareCap + t] = rare[t];
    if (tid == 0) args.crare_n[mine] = nr;
    __threadfence();
    __syncthreads();
    if (tid == 0) small[14] = atomicAdd(&args.count_ticket[c.row], 1);
    __syncthreads();
    if (small[14] != parts - 1) return;
    __threadfence();
    if (tid == 0) args.count_ticket[c.row] = 0;
    for (int g = 0; g < parts; ++g) {
      if (g == my_part) continue;
      const size_t theirs = (size_t)c.row * parts + g;
      const uint4* src = reinterpret_cast<const uint4*>(args.ctab + theirs * kCells);
      for (int i = tid; i < kCells / 4; i += kThreads) {
        const uint4 v = __ldcg(src + i);
        uint4 t = reinterpret_cast<uint4*>(c.tab)[i];
        t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        reinterpret_cast<uint4*>(c.tab)[i] = t;
      }
      // their rare list goes behind this CTA's (a total beyond the capacity is swept up below)
      const int ng = ((volatile int*)args.crare_n)[theirs];
      __syncthreads();
      const int have = *rare_n;
      __syncthreads();
      if (have <= kV3RareCap && ng <= kV3RareCap) {
        for (int t = tid; t < ng; t += kThreads)
          if (have + t < kV3RareCap) rare[have + t] = __ldcg(args.crare + theirs * kV3RareCap + t);
      }
      if (tid == 0) *rare_n = have + ng;
      __syncthreads();
    }
  }
  mark(1);
  // Global scratch (class list, long side lists) is held per RESIDENT CTA: a CTA claims one of
  // the n_scratch sets (as many as CTAs can be resident, so one is always free), starting its
  // search at the pair of its SM, and gives it back at the end.
  if (tid == 0) {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    int got = -1;
    for (int k = 0; k < 2 * args.n_scratch && got < 0; ++k) {
      const int at = (int)((2u * smid + (unsigned)k) % (unsigned)args.n_scratch);
      if (atomicCAS(&args.scratch_busy[at], 0, 1) == 0) got = at;
    }
    small[15] = got;
  }
  __syncthreads();
  const int scratch = small[15];
  if (scratch < 0) {  // cannot happen while n_scratch covers the resident CTAs; fail the row, do not wait
    if (tid == 0) { out->token = 0; out->status = 128; out->n_top = 0; out->n_kept = 0; }
    return;
  }
  auto release_scratch = [&]() {
    __syncthreads();
    if (tid == 0) { __threadfence(); atomicExch(&args.scratch_busy[scratch], 0); }
  };
  c.s_pair = args.s_pair + (size_t)scratch * args.s_cap;
  c.s_cap = args.s_cap;
  c.cl = args.clist + (size_t)scratch * kCells;


  // ---- B. the side list: tokens with history count >= 3, and values outside the bin window
  // It is walked by every selection, so it lives in shared memory when it fits.
  u64 side_best = 0;
  uint32_t side_worst = 0xffffffffu;  // this thread's lowest side key
  const int n_rare = *rare_n;
  if (n_rare <= kV3RareCap && n_heavy + kV3RareCap <= kV3SideShared) {
    c.s_pair = side_shared;
    c.s_cap = kV3SideShared;
  }
  {
    auto put = [&](int slot, int id, float s) {
      if (slot >= c.s_cap) return;  // (reported below, from the counts, by every thread alike)
      c.s_pair[slot] = make_int2(id, __float_as_int(s));
      const u64 packed = ((u64)key_of(s) << 32) | (uint32_t)(~(uint32_t)id);
      side_best = packed > side_best ? packed : side_best;
      side_worst = min(side_worst, key_of(s));
    };
    if (penalised) {
      if (tid < n_heavy) {  // the entry whose reads were started early
        if (hv_pair.x < 0 || hv_pair.x >= c.vocab) c.s_pair[tid] = make_int2(-1, 0);
        else put(tid, hv_pair.x, c.score_of(hv_raw, hv_pair.y));
      }
      const int32_t* heavy = a.pool.heavy + (size_t)P.slot * a.pool.unique_cap;
      const int2* pairs = a.pool.pairs + (size_t)P.slot * a.pool.unique_cap;
      for (int j = tid + kThreads; j < n_heavy; j += kThreads) {
        const int q = heavy[j];
        const int2 pr = q >= 0 && q < a.pool.unique_cap ? pairs[q] : make_int2(-1, 0);  // (id, count)
        if (pr.x < 0 || pr.x >= c.vocab) { c.s_pair[j] = make_int2(-1, 0); continue; }
        put(j, pr.x, c.score_of(c.logits[pr.x], pr.y));
      }
    }
    if (clocks && tid == 0) clocks[10] = clock64();
    if (n_rare <= kV3RareCap) {
      for (int t = tid; t < n_rare; t += kThreads) {
        const int2 e = rare[t];
        put(n_heavy + t, e.x, c.score_of((uint32_t)e.y & 0xffffu, (e.y >> 16) & 3));
      }
      if (n_heavy + n_rare > c.s_cap) status |= 4;
      c.n_s = min(n_heavy + n_rare, c.s_cap);
    } else {
      // too many to remember: sweep the row again for out-of-window values
      for (int id = tid; id < c.vocab; id += kThreads) {
        const uint32_t raw = c.logits[id];
        const int cc = c.class_of(id);
        if (cc == 3 || v3_bin_of_raw(raw) >= 0) continue;
        put(n_heavy + atomicAdd(side_n, 1), id, c.score_of(raw, cc));
      }
      __syncthreads();
      // more than the list holds: the row is reported for the general kernel (the record is
      // written by thread 0, so the decision has to be every thread's, not the one whose token
      // found no room)
      if (n_heavy + *side_n > c.s_cap) status |= 4;
      c.n_s = min(n_heavy + *side_n, c.s_cap);
    }
  }
  if (clocks && tid == 0) clocks[11] = clock64();
  // ---- C. row maximum and minimum --------------------------------------------------------------
  // Scores grow with the bin inside a count class, so the highest and lowest non-empty bin of
  // each class decide (with the side list).  One pass over the table; warps combine with
  // REDUX and meet in shared memory, one barrier (which also publishes the side list).
  {
    uint32_t top[3] = {0u, 0u, 0u}, bot[3] = {0xffffffffu, 0xffffffffu, 0xffffffffu};
    constexpr int kPerClass = kV3Bins / kThreads;  // a thread's cells tid + u * kThreads: count class u / kPerClass
    static_assert(kV3Bins % kThreads == 0, "a thread's u-th cell has the same count class for all threads");
#pragma unroll
    for (int k = 0; k < 3; ++k) {
#pragma unroll 4
      for (int u = 0; u < kPerClass; ++u) {
        const uint32_t cell = (uint32_t)(tid + (k * kPerClass + u) * kThreads);
        if (c.tab[cell]) { top[k] = cell + 1u; bot[k] = min(bot[k], cell); }
      }
    }
    const int lane = tid & 31;
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      const uint32_t t = __reduce_max_sync(0xffffffffu, top[k]);
      const uint32_t l = __reduce_min_sync(0xffffffffu, bot[k]);
      if (lane == 0) {
        if (t) atomicMax(reinterpret_cast<unsigned*>(small) + 16 + k, t);
        if (l != 0xffffffffu) atomicMin(reinterpret_cast<unsigned*>(small) + 19 + k, l);
      }
    }
    const u64 sb = warp_max_u64(side_best);
    const uint32_t sl = __reduce_min_sync(0xffffffffu, side_worst);
    if (lane == 0) {
      if (sb) atomicMax(&c.x->bcast[5], sb);
      if (sl != 0xffffffffu) atomicMin(reinterpret_cast<unsigned*>(small) + 22, sl);
    }
  }
  __syncthreads();
  side_best = c.x->bcast[5];
  mark(2);
  uint32_t cells_key = 0, min_key = reinterpret_cast<unsigned*>(small)[22], cells_min_key = 0xffffffffu;
  {
    // six scores (highest and lowest non-empty cell of three count classes): lanes 0..5 of every
    // warp work one out each and the warp combines them
    const int lane = tid & 31;
    const bool top = lane < 3;
    const uint32_t mark_at = reinterpret_cast<unsigned*>(small)[(top ? 16 : 19) + lane % 3];
    const bool valid = lane < 6 && (top ? mark_at != 0u : mark_at != 0xffffffffu);
    uint32_t key = 0;
    if (valid) key = key_of(c.cell_score(top ? (int)mark_at - 1 : (int)mark_at));
    cells_key = __reduce_max_sync(0xffffffffu, valid && top ? key : 0u);
    cells_min_key = __reduce_min_sync(0xffffffffu, valid && !top ? key : 0xffffffffu);
  }
  min_key = min(min_key, cells_min_key);
  if (clocks && tid == 0) clocks[25] = clock64();
  const uint32_t side_key = (uint32_t)(side_best >> 32);
  const int side_arg = (int)(~(uint32_t)(side_best & 0xffffffffu));
  const bool any_side = side_best != 0;
  const uint32_t max_key = max(cells_key, side_key);
  c.m = score_of(max_key);
  const float m = c.m;

  KeptSet kept{0u, 0x7fffffff};
  int token = -1;
  u64 n_topk = (u64)a.vocab, n_minp = (u64)a.vocab, n_kept = (u64)a.vocab;
  u64 q_kept = 0;
  bool have_totals = false;
  long long cut_ties = -1;
  u64 cut_group_cnt = 0;   // members at the cut key (kept or not)
  bool tie_split = false;
  Group cut_group{0u, -1, -1, -1};
  bool have_cut_group = false;
  auto need_cut_group = [&]() {
    if (!have_cut_group) { cut_group = find_group(c, kept.cut_key); have_cut_group = true; }
  };
  auto need_tie_limit = [&]() {
    if (tie_split && kept.tie_limit == 0x7fffffff) {
      need_cut_group();
      kept.tie_limit = nth_in_group(c, cut_group, (u64)cut_ties);
    }
  };
  // per-class raw thresholds of a score bound (see cand_thresholds), for the walks that only
  // need the few tokens at or above a key
  CandCtx bound_ctx{nullptr, nullptr, nullptr, nullptr, small + 8, nullptr};
  int* low_id = small + 3;
  // what the draw found: a member of one class (cell, its size, the n-th by ascending id)
  int draw_cell = -1;
  u64 draw_members = 0, draw_nth = 0;
  bool token_known = false;

  {
  // ---- the row's non-empty classes, each with its key and mass computed once ---------------
  // Thread t owns classes t, t + kThreads, ... (the populated value range spreads evenly over
  // the threads) and writes its entries back to back; the order is fixed by the counts alone.
  {
    constexpr int kPerCells = kCells / kThreads;
    int mine = 0;
#pragma unroll 4
    for (int u = 0; u < kPerCells; ++u) mine += c.tab[tid + u * kThreads] != 0;
    const u64 incl = warp_scan_u64((u64)mine);
    u64 pre, pre_unused, tot, tot_unused;
    block_warp_prefix2(*c.x, shfl_u64(incl, 31), 0, pre, pre_unused, tot, tot_unused);
    int at = (int)(pre + incl) - mine;
    if (clocks && tid == 0) clocks[26] = clock64();
    for (int u = 0; u < kPerCells; ++u) {
      const int cell = tid + u * kThreads;
      const uint32_t n = c.tab[cell];
      if (!n) continue;
      const float s = c.cell_score(cell);
      const u64 q = mass_of(s, m);
      reinterpret_cast<uint4*>(c.cl)[at] = pack_class(key_of(s), n, (uint32_t)cell, q);
      ++at;
    }
    c.n_cl = (int)tot;
    __syncthreads();
  }
  mark(3);  // (the count table has served: the selection histograms take its place)

  if (c.greedy) {
    // arg max with penalties: the lowest id among the tokens whose score key is the maximum
    if (tid == 0) *low_id = side_key == max_key ? side_arg : 0x7fffffff;
    cand_thresholds(c, bound_ctx, max_key);  // (ends with a barrier)
    stream_at_or_above(c, bound_ctx.thr, [&](int id, uint32_t raw, int cc) {
      if (v3_bin_of_raw(raw) >= 0 && key_of(c.score_of(raw, cc)) == max_key) atomicMin(low_id, id);
    });
    __syncthreads();
    token = *low_id;
    __syncthreads();
    if (token == 0x7fffffff) { token = any_side ? side_arg : 0; status |= 1; }
    if (P.n_logprobs >= 0) {
      u64 cn;
      totals3(c, 0u, cn, q_kept);
    }
  } else {
    u64 cnt = 0, mass = 0;
    if (P.top_k > 0 && P.top_k < a.vocab) {
      Selection sk = select_union3<false, true>(c, 0u, (u64)P.top_k, 1.0f);
      if (!sk.ok) status |= 1;
      kept.cut_key = sk.key;
      cnt = sk.above_cnt + sk.bin_cnt;
      mass = sk.above_mass + sk.bin_mass;
      have_totals = sk.ok;
      n_topk = cnt;
      cut_group_cnt = sk.bin_cnt;
    }
    mark(4);
    if (P.min_p > 0.0f) {
      if (!have_totals) { totals3(c, kept.cut_key, cnt, mass); have_totals = true; }
      const float z1 = mass_to_float(mass);
      const float thr = __fmul_rn(__fdiv_rn(1.0f, z1), P.min_p);
      uint32_t lowest = 0xffffffffu;
      auto consider = [&](float s) {
        const uint32_t k = key_of(s);
        if (k >= kept.cut_key && !(__fdiv_rn(expf(s - m), z1) < thr)) lowest = min(lowest, k);
      };
      for_each_class(c, [&](const ClassEntry& e) { consider(score_of(e.key)); });
      for_each_side3(c, [&](int, float s) { consider(s); });
      lowest = ~block_max_u32(*c.x, ~lowest);
      if (lowest != 0xffffffffu && lowest > kept.cut_key) {
        kept.cut_key = lowest;
        have_totals = false;
      }
    }
    mark(5);
    if (P.top_p < 1.0f) {
      {
        // first level over the scores' own range (from the lowest class that can be kept to the
        // row maximum) instead of the key's top bits: one level separates a near-flat row
        const float lo = score_of(max(kept.cut_key, cells_min_key == 0xffffffffu ? min_key : cells_min_key));
        const float range = m - lo;
        c.lin = range > 0.f && range < 3.0e38f;
        c.lin_lo = lo;
        c.lin_scale = c.lin ? __fdiv_rn(2047.5f, range) : 0.f;
      }
      Selection sp = select_union3<true, true>(c, kept.cut_key, 0, P.top_p);
      c.lin = false;
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
        cut_group_cnt = sp.bin_cnt;
        tie_split = t < sp.bin_cnt;
        have_totals = true;
      } else {
        status |= 1;
        cnt = sp.total_cnt;
        mass = sp.total_mass;
        have_totals = true;
      }
    } else {
      if (!have_totals) { totals3(c, kept.cut_key, cnt, mass); have_totals = true; }
      n_minp = cnt;
    }
    n_kept = cnt;
    q_kept = mass;
    mark(6);

  }
  }

  // ---- draw ------------------------------------------------------------------------------
  if (!c.greedy) {
    if (q_kept == 0) {
      status |= 1;
      token = any_side ? side_arg : 0;
    } else if (a.noise) {
      // reference draws: arg max of fl(fl(e / z) / noise) over the kept set, lowest id on ties
      need_tie_limit();
      const float zf = mass_to_float(q_kept);
      const float* noise_row = a.noise + (size_t)c.row * a.vocab;
      u64 best = 0;
      for (int id = tid; id < c.vocab; id += kThreads) {
        const float s = c.element_score(id, c.logits[id], c.class_of(id));
        if (!kept.has(key_of(s), id)) continue;
        const float p = __fdiv_rn(expf(s - m), zf);
        const float ratio = __fdiv_rn(p, noise_row[id]);
        const u64 packed = ((u64)__float_as_uint(ratio) << 32) | (uint32_t)(~(uint32_t)id);
        best = packed > best ? packed : best;
      }
      best = block_max_u64(*c.x, best);
      token = (int)(~(uint32_t)(best & 0xffffffffu));
    } else {
      // Near-flat rows: rejection on tokens, when one round is all but sure to accept.
      bool by_tokens = false;
      if (a.token_draw && mass_to_float(q_kept) * (float)(kTokenTrials * kThreads) >= 4.0f * (float)c.vocab) {
        bool group_hit;
        // (a sixteenth of the trials accepted on average: one per thread is plenty)
        const int trials = mass_to_float(q_kept) * 16.0f >= (float)c.vocab ? 1 : kTokenTrials;
        const int t = draw_by_token_rejection(c, kept, tie_split, cut_ties > 0 ? (u64)cut_ties : 0ull, cut_group_cnt, P.seed, 4,
                                              trials, group_hit);
        if (t >= 0) {
          token = t;
          if (group_hit) {
            // one of the kept members of the group the cut splits: its lowest ids
            need_cut_group();
            const Philox4 r = philox4x32_10(0u, 0u, 0u, 4u, (uint32_t)P.seed, (uint32_t)(P.seed >> 32));
            const u64 nth = 1 + __umul64hi(((u64)r.v[0] << 32) | r.v[1], (u64)cut_ties);
            token = nth_in_group(c, cut_group, nth);
            if (token == 0x7fffffff) { token = any_side ? side_arg : 0; status |= 1; }
          }
          token_known = true;
          by_tokens = true;
        }
      }
      if (!by_tokens) {
        // Inverse CDF over exact integer masses in the order: classes above the cut (by class
        // index), the tie group at the cut (its lowest ids), side elements above the cut (by id).
        const Philox4 r = philox4x32_10(0u, 0u, 0u, 0u, (uint32_t)P.seed, (uint32_t)(P.seed >> 32));
        const u64 r64 = ((u64)r.v[0] << 32) | r.v[1];
        const u64 target = __umul64hi(r64, q_kept);
        // classes above the cut in the order (thread, step): thread t owns entries t, t + kThreads, ...
        u64 chunk = 0;
        for_each_class(c, [&](const ClassEntry& e) { if (e.key > kept.cut_key) chunk += e.w; });
        const u64 incl = warp_scan_u64(chunk);
        u64 pre, pre_unused, q_cells, tot_unused;
        block_warp_prefix2(*c.x, shfl_u64(incl, 31), 0, pre, pre_unused, q_cells, tot_unused);
        mark(12);
        // the group at the cut key: cut_ties members when top-p split it, else all of them
        u64 group_kept = cut_ties >= 0 ? (u64)cut_ties : 0;
        u64 q_cut = 0;
        if (cut_ties < 0) {
          // cut by top-k / min-p / nothing: everything at the cut key is kept; count it
          u64 gc = 0, gm = 0;
          for_each_class(c, [&](const ClassEntry& e) { if (e.key == kept.cut_key) gc += e.cnt; });
          for_each_side3(c, [&](int, float s) { if (key_of(s) == kept.cut_key) gc += 1; });
          block_sum2(*c.x, gc, gm);
          group_kept = gc;
        }
        q_cut = mass_of(score_of(kept.cut_key), m);
        const u64 q_group = group_kept * q_cut;
        mark(13);
        if (target < q_cells) {
          if (tid == 0) c.x->bcast[5] = 0;
          __syncthreads();
          u64 run = pre + incl - chunk;
          if (run <= target && target < run + chunk) {
            bool done = false;
            for (int i = tid; i < c.n_cl && !done; i += kThreads) {
              const ClassEntry e = c.class_at(i);
              if (e.key <= kept.cut_key) continue;
              if (e.w && target < run + e.w) {
                c.x->bcast[3] = e.cnt;
                c.x->bcast[4] = (target - run) / e.q + 1;
                c.x->bcast[5] = (u64)e.cell + 1;
                done = true;
              }
              run += e.w;
            }
          }
          __syncthreads();
          draw_cell = (int)c.x->bcast[5] - 1;
          draw_members = c.x->bcast[3];
          draw_nth = c.x->bcast[4];
          __syncthreads();
          if (draw_cell < 0) { token = any_side ? side_arg : 0; status |= 1; token_known = true; }
        } else if (target < q_cells + q_group) {
          need_cut_group();
          const u64 nth = q_cut ? (target - q_cells) / q_cut + 1 : 1;
          token = nth_in_group(c, cut_group, nth);  // the kept members are the lowest ids
          if (token == 0x7fffffff) { token = any_side ? side_arg : 0; status |= 1; }
          token_known = true;
        } else {
          SideDrawFill3 fill{&c, kept.cut_key};
          Selection sd = descend_local<true>(c, fill, 0u, target - q_cells - q_group + 1, -1.0f, 0, 1, 0x7FFu);
          if (sd.ok) token = (int)(~sd.key);
          else { token = any_side ? side_arg : 0; status |= 1; }
          token_known = true;
        }
      }
      mark(14);
      if (!token_known) {
        // a uniformly chosen member of ONE class (not of other classes that share its key):
        // large classes by rejection (about vocab / members scattered probes, which a lone CTA
        // issues slowly), classes of up to kV3RejectMin tokens by one scan of the row
        const int cell = draw_cell;
        const u64 members = draw_members, nth = draw_nth;
        if (clocks && tid == 0) clocks[15] = members;
        if (cell >= 0) {
          Group g{key_of(c.cell_score(cell)), -1, -1, -1};
          if (cell < kV3Bins) g.cell0 = cell; else if (cell < 2 * kV3Bins) g.cell1 = cell; else g.cell2 = cell;
          if (members > (u64)kV3RejectMin) {
            const u64 per_round = ((u64)c.vocab + members - 1) / members;  // probes for ~63 % success
            const int trials = (int)min((u64)kRandomTrials, max(1ull, (per_round + kThreads - 1) / kThreads));
            // a class the scan can hold gets a few rounds, then the scan; a larger one many
            token = random_in_class(c, cell, trials, P.seed, members <= (u64)kV3ScanCap ? 4 : 32);
            if (token < 0 && members <= (u64)kV3ScanCap) token = nth_in_small_class(c, cell, nth, members);
          } else {
            token = nth_in_small_class(c, cell, nth, members);
          }
          if (token < 0) {
            Group only = g;
            only.key = 0xffffffffu;  // no out-of-class member can match
            token = nth_in_group(c, only, nth);
          }
        }
        if (token < 0 || token == 0x7fffffff) { token = any_side ? side_arg : 0; status |= 1; }
      }
    }
  }
  mark(7);

  // ---- D. log-probabilities -------------------------------------------------------------
  float log_z = 0.f;
  if (P.n_logprobs >= 0) {
    if (tid == 0) c.x->bcast[6] = (u64)__float_as_uint((float)(log((double)q_kept) - (double)kMassShift * 0.6931471805599453));
    __syncthreads();
    log_z = __uint_as_float((uint32_t)c.x->bcast[6]);
    __syncthreads();
    if (tid == 0 && token >= 0 && token < a.vocab)
      out->logprob = (c.element_score(token, c.logits[token], c.class_of(token)) - m) - log_z;
    int n_want = min(P.n_logprobs, a.vocab);
    if ((u64)n_want > n_kept) n_want = (int)n_kept;
    if (n_want > 0) {
      Selection sn = select_union3<false, false>(c, kept.cut_key, (u64)n_want, 1.0f);
      if (sn.ok) {
        const int need = n_want - (int)sn.above_cnt;  // lowest ids of the group at the N-th key
        // The tokens above the N-th key (fewer than N) and the group at it: side elements come
        // from the side list, the rest from one walk of the row against per-class raw
        // thresholds.  The group's ids go to a list of their own (the member list's memory);
        // a group too large for it is walked the slow way.
        int* tie_ids = reinterpret_cast<int*>(c.list);
        constexpr int kTieCap = (int)(kV3ListCap * sizeof(V3Entry) / sizeof(int));
        int* tie_n = small + 3;
        if (tid == 0) { *c.gbuf_n = 0; *tie_n = 0; }
        __syncthreads();
        auto take = [&](uint32_t k, int id) {
          if (k > sn.key) {
            const int slot = atomicAdd(c.gbuf_n, 1);
            if (slot < kV3ListCap) c.gbuf[slot] = V3Entry{k, id, 1u, 0u, 0ull};
          } else if (k == sn.key && need > 0) {
            const int slot = atomicAdd(tie_n, 1);
            if (slot < kTieCap) tie_ids[slot] = id;
          }
        };
        for_each_side3(c, [&](int id, float s) { take(key_of(s), id); });
        cand_thresholds(c, bound_ctx, sn.key);  // (ends with a barrier)
        stream_at_or_above(c, bound_ctx.thr, [&](int id, uint32_t raw, int cc) {
          if (v3_bin_of_raw(raw) < 0) return;  // outside the bin window: a side element, taken above
          take(key_of(c.score_of(raw, cc)), id);
        });
        __syncthreads();
        if (need > 0) {
          const int n_tie = *tie_n;
          if (n_tie <= kTieCap) {
            // the `need` lowest ids of the group: each id counts the ids below it
            for (int t = tid; t < n_tie; t += kThreads) {
              const int mine = tie_ids[t];
              int below = 0;
              for (int j = 0; j < n_tie; ++j) below += tie_ids[j] < mine ? 1 : 0;
              if (below < need) {
                const int slot = atomicAdd(c.gbuf_n, 1);
                if (slot < kV3ListCap) c.gbuf[slot] = V3Entry{sn.key, mine, 1u, 0u, 0ull};
              }
            }
          } else {
            const Group g = sn.key == kept.cut_key && have_cut_group ? cut_group : find_group(c, sn.key);
            const int last_id = nth_in_group(c, g, (u64)need);
            emit_group_upto(c, g, last_id == 0x7fffffff ? -1 : last_id);
          }
        }
        __syncthreads();
        if (tid < 32) {
          const int n = min(*c.gbuf_n, HS_MAX_LOGPROBS);
          uint32_t kv = 0;
          int id = 0x7fffffff;
          if (tid < n) { kv = c.gbuf[tid].key; id = c.gbuf[tid].id; }
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
    if (tid == 0) out->n_top = n_want;
  } else if (tid == 0) {
    out->n_top = 0;
    out->logprob = 0.f;
  }
  mark(8);

  // ---- E. optional dump of the final scores (parity tests) -------------------------------
  if (a.scores_out) {
    need_tie_limit();
    float* dst = a.scores_out + (size_t)c.row * a.vocab;
    const float ninf = __int_as_float(0xff800000);
    for (int id = tid; id < c.vocab; id += kThreads) {
      const float s = c.element_score(id, c.logits[id], c.class_of(id));
      dst[id] = (c.greedy || kept.has(key_of(s), id)) ? s : ninf;
    }
  }

  if (tid == 0) {
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
  (void)cut_group_cnt;
  release_scratch();
  mark(9);
}


// Rows with 0 < top_k <= kTopKMax take the candidate path.
__device__ __forceinline__ bool is_candidate_row(const hs_row_params& P, int vocab) {
  return P.temperature != 0.0f && P.top_k > 0 && P.top_k <= kTopKMax && P.top_k < vocab;
}

// One part of a candidate row (a contiguous range of its tokens).  The CTA that brings in the
// row's last part finishes the row.  Returns true when the row's candidate list overflowed
// and the caller (the finishing CTA) has to count the row after all.
__device__ __forceinline__ bool cand_part(const RowV3Args& args, unsigned char* smem_raw, int row_index, int part) {
  const RowKernelArgs& a = args.base;
  const LayoutCand lay = layout_cand();
  Ctx3 c;
  c.x = reinterpret_cast<Exchange*>(smem_raw + lay.x);
  int* small = reinterpret_cast<int*>(smem_raw + lay.small);
  CandCtx L{reinterpret_cast<u64*>(smem_raw + lay.cand), small + 4, small + 5,
            reinterpret_cast<uint32_t*>(smem_raw + lay.count), small + 8, nullptr};
  const int tid = threadIdx.x;
  c.row = row_index;
  c.vocab = a.vocab;
  const hs_row_params P = a.params[c.row];
  c.greedy = false;
  // the row is streamed by args.split CTAs, each taking a contiguous range of tokens
  const int split = args.split;
  const int width = (((a.vocab + split - 1) / split) + 7) & ~7;
  c.lo = min(part * width, a.vocab);
  c.hi = min(c.lo + width, a.vocab);
  c.logits = reinterpret_cast<const unsigned short*>(a.logits) + (long long)c.row * a.row_stride;
  c.vec = (reinterpret_cast<uintptr_t>(c.logits) & 15u) == 0;
  hs_row_out* out = a.out + c.row;
  c.T = P.temperature; c.rp = P.repetition_penalty; c.pp = P.presence_penalty; c.fp = P.frequency_penalty;
  c.pool = a.pool;
  c.slot = P.slot;
  const bool slot_ok = P.slot >= 0 && P.slot < a.pool.slots_total;
  const bool penalised = slot_ok && (c.rp != 1.0f || c.pp != 0.0f || c.fp != 0.0f);
  c.cls = penalised ? a.pool.cls + (size_t)P.slot * a.pool.cls_stride : nullptr;
  c.s_pair = nullptr; c.n_s = 0; c.s_cap = 0; c.cl = nullptr; c.n_cl = 0; c.m = 0.f;
  c.tab = nullptr; c.hist = nullptr; c.gbuf = nullptr; c.list = nullptr; c.gbuf_n = nullptr;
  unsigned long long* clocks = args.phase_clocks ? args.phase_clocks + (size_t)c.row * kV3PhaseSlots : nullptr;
  auto mark = [&](int slot) {
    if (clocks && tid == 0) clocks[slot] = clock64();
  };
  mark(0);
  L.dbg = clocks;
  if (tid < 16) small[tid] = 0;
  __syncthreads();
  int n = c.hi > c.lo ? topk_candidates(c, L, min(P.top_k, c.hi - c.lo)) : 0;
  mark(1);
  // a lone CTA cuts its list at the k-th highest score now; a part of a split row hands its
  // candidates over as they are unless they would crowd the merged list
  if (n > P.top_k && (split == 1 || n > kCandCap / split)) {
    const uint32_t cut = cand_kth_key(*c.x, L, n, P.top_k);
    n = cand_compact(L, n, cut);
  } else if (n > 0) {
    n = cand_compact(L, n, 0u);  // drops entries the scoring pass voided
  }
  if (split > 1) {
    // hand this CTA's candidates over; the CTA that arrives last finishes the row
    static_assert(kSplitCap >= kCandCap, "a part's whole list fits in its hand-over block");
    u64* mine = args.split_lists + ((size_t)c.row * split + part) * kSplitCap;
    for (int i = tid; i < n; i += kThreads) mine[i] = L.cand[i];
    if (tid == 0) args.split_n[c.row * split + part] = n;  // -1: this part overflowed
    __threadfence();
    __syncthreads();
    if (tid == 0) small[6] = atomicAdd(&args.split_ticket[c.row], 1);
    __syncthreads();
    if (small[6] != split - 1) return false;
    mark(12);
    __threadfence();
    if (tid == 0) args.split_ticket[c.row] = 0;
    // all parts' lengths first, then all copies at once (one wait instead of one per part)
    if (tid < split) small[12 + tid] = ((volatile int*)args.split_n)[c.row * split + tid];  // -1: that part overflowed
    __syncthreads();
    {
      int at = 0;
      bool overflow = false;
      for (int g = 0; g < split; ++g) {
        const int ng = small[12 + g];
        if (ng < 0) { overflow = true; continue; }
        const u64* theirs = args.split_lists + ((size_t)c.row * split + g) * kSplitCap;
        for (int i = tid; i < ng; i += kThreads)
          if (at + i < kCandCap) L.cand[at + i] = ((volatile const u64*)theirs)[i];
        at += ng;
      }
      n = (overflow || at > kCandCap) ? -1 : at;
    }
    __syncthreads();
    mark(13);
    if (n > kSortAll) {
      const uint32_t cut = cand_kth_key(*c.x, L, n, P.top_k);
      n = cand_compact(L, n, cut);
    }
  }
  if (n < 0) return true;  // more ties than a candidate list holds: the row is counted instead
  mark(14);
  cand_sort(L, n);
  mark(15);
  if (n > P.top_k) {
    // a list that was sorted whole: top-k keeps the first k entries and the ties of the k-th
    const uint32_t cut = cand_key(L.cand[P.top_k - 1]);
    u64 keep = 0, unused = 0;
    for (int i = tid; i < n; i += kThreads) keep += cand_key(L.cand[i]) >= cut ? 1 : 0;
    block_sum2(*c.x, keep, unused);
    n = (int)keep;
  }
  mark(2);
  const float* noise_row = a.noise ? a.noise + (size_t)c.row * a.vocab : nullptr;
  FinishOut r = finish_sorted(*c.x, L.cand, reinterpret_cast<u64*>(smem_raw + lay.mass), n, P, noise_row, out, clocks);
  if (P.slot >= a.pool.slots_total) r.status |= 64;  // a slot this sampler does not have: no penalties
  if (a.scores_out) {
    float* dst = a.scores_out + (size_t)c.row * a.vocab;
    for (int id = tid; id < c.vocab; id += kThreads) dst[id] = __int_as_float(0xff800000);
    __syncthreads();
    for (int i = tid; i < (int)r.n_kept; i += kThreads) dst[cand_id(L.cand[i])] = score_of(cand_key(L.cand[i]));
  }
  if (tid == 0) {
    write_finish(r, out);
    if (a.tokens_out) a.tokens_out[c.row] = r.token;
    if ((a.flags & HS_SAMPLE_APPEND_TOKEN) && slot_ok && r.token >= 0 && r.token < a.vocab) {
      if (!slot_append_one(a.pool, P.slot, r.token)) out->status = r.status | 2;
    }
  }
  mark(8);
  return false;
}

// Shared memory of the persistent kernel: the larger of the two paths' layouts.
__host__ __device__ inline size_t bf16_kernel_smem() {
  const size_t a = layout_v3().total, b = layout_cand().total;
  return a > b ? a : b;
}

// One CTA per work item, two CTAs resident per SM; the hardware hands out the items in grid
// order, long ones first: batch * csplit items = part p of row r on the counting path (a CTA
// whose row is not a counting row leaves at once), then batch * split items = part p of row r
// on the candidate path (likewise).  No CTA waits for another.
__global__ void __launch_bounds__(kThreads, 2) row_kernel_bf16(const RowV3Args args) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int item = blockIdx.x;
  const int n_count = args.batch * args.csplit;
  bool count = item < n_count;
  // counting items are laid out part-major, so that the parts of one row start on different SMs
  int row = count ? item % args.batch : (item - n_count) / args.split;
  int part = count ? item / args.batch : (item - n_count) % args.split;
  if (is_candidate_row(args.base.params[row], args.base.vocab) == count) return;  // the other path's row
  // (tuning aid: when each item started and ended, in ns of the global timer, slots 48.. of its row)
  unsigned long long* when = nullptr;
  if (args.phase_clocks && threadIdx.x == 0) {
    when = args.phase_clocks + (size_t)row * kV3PhaseSlots + (count ? 48 : 56) + 2 * part;
    when[0] = global_timer_ns();
  }
  if (!count) {
    if (!cand_part(args, smem_raw, row, part)) {
      if (when) when[1] = global_timer_ns();
      return;
    }
    __syncthreads();
    part = -1;  // more ties than a candidate list holds: this CTA counts the whole row
  } else if (args.csplit == 1) {
    part = -1;
  }
  count_row(args, smem_raw, row, part);
  if (when) when[1] = global_timer_ns();
}

}  // namespace hs
