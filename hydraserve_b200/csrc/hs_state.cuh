// Device-resident token-count histograms (one per request slot) and the plain-greedy
// arg-max kernels.
//
// A slot is the device form of the `counts` dict the reference rebuilds per row per step
// (sampling.py:106-110).  It holds
//   pairs[]   the distinct token ids seen so far with their counts, (id, count), 8 bytes each
//   pos[]     dense index: pos[token] = 1 + position in pairs (0 = unseen); touched only
//             when tokens are appended
//   cls[]     dense 2-bit class per token, min(count, 3), sixteen tokens per 32-bit word: what
//             the bf16 sampling kernel streams next to the logits (V/4 bytes per row)
//   heavy[]   positions in pairs of the ids whose count reached 3: the only tokens whose
//             exact count the bf16 kernels need (one look-up gives id and count)
#pragma once

#include "hs_common.cuh"
#include "../../include/hs_sampler.h"

namespace hs {

struct Pool {
  int2* pairs;     // [slots_total, unique_cap] (token id, count)
  int32_t* n;      // [slots_total]
  int32_t* pos;    // [slots_total, pos_stride]
  uint32_t* cls;   // [slots_total, cls_stride] 2-bit classes
  int32_t* heavy;  // [slots_total, unique_cap] positions in pairs
  int32_t* n_heavy;  // [slots_total]
  int32_t* error;  // [1] sticky: 1 = a slot overflowed unique_cap
  int slots_total;
  int unique_cap;
  long long pos_stride;
  long long cls_stride;  // words per slot
};

// Sets the 2-bit class of `token` to min(count, 3); returns the previous class.
__device__ __forceinline__ uint32_t set_class(uint32_t* cls, int token, int count) {
  const uint32_t want = (uint32_t)min(count, 3);
  uint32_t* word = cls + (token >> 4);
  const int shift = (token & 15) * 2;
  uint32_t old = *word;
  while (true) {
    const uint32_t cur = (old >> shift) & 3u;
    if (cur >= want) return cur;  // classes only grow between resets
    const uint32_t next = (old & ~(3u << shift)) | (want << shift);
    const uint32_t seen = atomicCAS(word, old, next);
    if (seen == old) return cur;
    old = seen;
  }
}

// Empties each listed slot by walking its id list (no dense clear).
__global__ void slots_reset_kernel(Pool p, const int32_t* slots, int n_slots) {
  const int s = blockIdx.x < n_slots ? slots[blockIdx.x] : -1;
  if (s < 0 || s >= p.slots_total) return;
  const int n = min(p.n[s], p.unique_cap);
  const int2* pairs = p.pairs + (size_t)s * p.unique_cap;
  int32_t* pos = p.pos + (size_t)s * p.pos_stride;
  uint32_t* cls = p.cls + (size_t)s * p.cls_stride;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const int id = pairs[j].x;
    if (id >= 0 && id < p.pos_stride) {
      pos[id] = 0;
      cls[id >> 4] = 0;  // every non-zero field of the word belongs to a listed id
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) { p.n[s] = 0; p.n_heavy[s] = 0; }
}

// Pass 1 of an append: give every token id not yet in the slot a list position.
__global__ void slots_register_kernel(Pool p, const int32_t* tokens, const int32_t* offsets,
                                      const int32_t* slots, int n_slots, int vocab) {
  const int row = blockIdx.y;
  const int s = row < n_slots ? slots[row] : -1;
  if (s < 0 || s >= p.slots_total) return;
  const int t0 = offsets[row], t1 = offsets[row + 1];
  int2* pairs = p.pairs + (size_t)s * p.unique_cap;
  int32_t* pos = p.pos + (size_t)s * p.pos_stride;
  for (int j = t0 + blockIdx.x * blockDim.x + threadIdx.x; j < t1; j += gridDim.x * blockDim.x) {
    const int t = tokens[j];
    if (t < 0 || t >= vocab || t >= p.pos_stride) continue;  // ignored, as in the reference
    if (atomicCAS(&pos[t], 0, -1) == 0) {
      const int idx = atomicAdd(&p.n[s], 1);
      if (idx < p.unique_cap) {
        pairs[idx] = make_int2(t, 0);
        pos[t] = idx + 1;
      } else {
        atomicSub(&p.n[s], 1);
        pos[t] = 0;
        *p.error = 1;
      }
    }
  }
}

// Pass 2 of an append: count.
__global__ void slots_count_kernel(Pool p, const int32_t* tokens, const int32_t* offsets,
                                   const int32_t* slots, int n_slots, int vocab) {
  const int row = blockIdx.y;
  const int s = row < n_slots ? slots[row] : -1;
  if (s < 0 || s >= p.slots_total) return;
  const int t0 = offsets[row], t1 = offsets[row + 1];
  int2* pairs = p.pairs + (size_t)s * p.unique_cap;
  const int32_t* pos = p.pos + (size_t)s * p.pos_stride;
  for (int j = t0 + blockIdx.x * blockDim.x + threadIdx.x; j < t1; j += gridDim.x * blockDim.x) {
    const int t = tokens[j];
    if (t < 0 || t >= vocab || t >= p.pos_stride) continue;
    const int q = pos[t];
    if (q > 0) atomicAdd(&pairs[q - 1].y, 1);
  }
}

// Pass 3 of an append: with the counts final, refresh the 2-bit classes and list the ids
// whose count reached 3 (the thread that moves a class to 3 does the listing).
__global__ void slots_classify_kernel(Pool p, const int32_t* tokens, const int32_t* offsets,
                                      const int32_t* slots, int n_slots, int vocab) {
  const int row = blockIdx.y;
  const int s = row < n_slots ? slots[row] : -1;
  if (s < 0 || s >= p.slots_total) return;
  const int t0 = offsets[row], t1 = offsets[row + 1];
  const int2* pairs = p.pairs + (size_t)s * p.unique_cap;
  const int32_t* pos = p.pos + (size_t)s * p.pos_stride;
  uint32_t* cls = p.cls + (size_t)s * p.cls_stride;
  int32_t* heavy = p.heavy + (size_t)s * p.unique_cap;
  for (int j = t0 + blockIdx.x * blockDim.x + threadIdx.x; j < t1; j += gridDim.x * blockDim.x) {
    const int t = tokens[j];
    if (t < 0 || t >= vocab || t >= p.pos_stride) continue;
    const int q = pos[t];
    if (q <= 0) continue;
    const int count = pairs[q - 1].y;
    const uint32_t before = set_class(cls, t, count);
    if (count >= 3 && before < 3u) {
      const int idx = atomicAdd(&p.n_heavy[s], 1);
      if (idx < p.unique_cap) heavy[idx] = q - 1;
    }
  }
}

// One token appended by a single thread (the sampling kernel's epilogue).
__device__ __forceinline__ bool slot_append_one(const Pool& p, int s, int token) {
  int2* pairs = p.pairs + (size_t)s * p.unique_cap;
  int32_t* pos = p.pos + (size_t)s * p.pos_stride;
  uint32_t* cls = p.cls + (size_t)s * p.cls_stride;
  int count;
  const int q = pos[token];
  if (q > 0) {
    count = (pairs[q - 1].y += 1);
  } else {
    const int n = p.n[s];
    if (n >= p.unique_cap) return false;
    pairs[n] = make_int2(token, 1);
    pos[token] = n + 1;
    p.n[s] = n + 1;
    count = 1;
  }
  if (count <= 3) {
    uint32_t* word = cls + (token >> 4);
    const int shift = (token & 15) * 2;
    *word = (*word & ~(3u << shift)) | ((uint32_t)count << shift);
    if (count == 3) {
      const int h = p.n_heavy[s];
      if (h < p.unique_cap) { (p.heavy + (size_t)s * p.unique_cap)[h] = pos[token] - 1; p.n_heavy[s] = h + 1; }
    }
  }
  return true;
}

// ---- plain greedy: arg max per row, lowest id on ties (reference sampling.py:69-73) ---
constexpr int kGreedyThreads = 512;

// Each CTA scans one chunk of one row and leaves (key << 32 | ~id) of its best element.
__global__ void __launch_bounds__(kGreedyThreads) greedy_partial_kernel(
    const void* logits, int dtype, long long row_stride, int vocab, int chunk, u64* partials) {
  __shared__ u64 warp_best[kGreedyThreads / 32];
  const int row = blockIdx.y;
  const int begin = blockIdx.x * chunk;
  const int n = max(0, min(chunk, vocab - begin));
  const int tid = threadIdx.x;
  u64 best = 0;
  auto consider = [&](float f, int gid) {
    const u64 packed = ((u64)key_of(canonical(f)) << 32) | (uint32_t)(~(uint32_t)gid);
    best = packed > best ? packed : best;
  };
  const long long gofs = (long long)row * row_stride + begin;
  if (dtype == HS_DTYPE_BF16) {
    const unsigned short* src = reinterpret_cast<const unsigned short*>(logits) + gofs;
    const bool vec = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    const int nvec = vec ? n / 8 : 0;
    const uint4* src4 = reinterpret_cast<const uint4*>(src);
    for (int i = tid; i < nvec; i += kGreedyThreads) {
      const uint4 w = __ldcs(src4 + i);
      const int g = begin + 8 * i;
      consider(__uint_as_float(w.x << 16), g + 0); consider(__uint_as_float(w.x & 0xffff0000u), g + 1);
      consider(__uint_as_float(w.y << 16), g + 2); consider(__uint_as_float(w.y & 0xffff0000u), g + 3);
      consider(__uint_as_float(w.z << 16), g + 4); consider(__uint_as_float(w.z & 0xffff0000u), g + 5);
      consider(__uint_as_float(w.w << 16), g + 6); consider(__uint_as_float(w.w & 0xffff0000u), g + 7);
    }
    for (int i = nvec * 8 + tid; i < n; i += kGreedyThreads)
      consider(__uint_as_float((uint32_t)src[i] << 16), begin + i);
  } else {
    const float* src = reinterpret_cast<const float*>(logits) + gofs;
    const bool vec = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    const int nvec = vec ? n / 4 : 0;
    const float4* src4 = reinterpret_cast<const float4*>(src);
    for (int i = tid; i < nvec; i += kGreedyThreads) {
      const float4 w = __ldcs(src4 + i);
      const int g = begin + 4 * i;
      consider(w.x, g); consider(w.y, g + 1); consider(w.z, g + 2); consider(w.w, g + 3);
    }
    for (int i = nvec * 4 + tid; i < n; i += kGreedyThreads) consider(src[i], begin + i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const u64 t = __shfl_xor_sync(0xffffffffu, best, o);
    best = t > best ? t : best;
  }
  if ((tid & 31) == 0) warp_best[tid >> 5] = best;
  __syncthreads();
  if (tid < 32) {
    best = tid < kGreedyThreads / 32 ? warp_best[tid] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const u64 t = __shfl_xor_sync(0xffffffffu, best, o);
      best = t > best ? t : best;
    }
    if (tid == 0) partials[(size_t)row * gridDim.x + blockIdx.x] = best;
  }
}

__global__ void greedy_final_kernel(const u64* partials, int chunks, int batch, int32_t* tokens_out) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= batch) return;
  u64 best = 0;
  for (int g = 0; g < chunks; ++g) {
    const u64 t = partials[(size_t)row * chunks + g];
    best = t > best ? t : best;
  }
  tokens_out[row] = (int32_t)(~(uint32_t)(best & 0xffffffffu));
}

}  // namespace hs
