// Device-side building blocks of the sampler: order-preserving keys, fixed-point
// probability mass, Philox4x32-10, and block / cluster wide reductions and scans.
#pragma once

#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cg = cooperative_groups;

namespace hs {

constexpr int kThreads = 512;           // threads per CTA of the row kernels (128 registers each: no spills)
constexpr int kWarps = kThreads / 32;
constexpr int kMaxCluster = 8;          // portable cluster limit
constexpr int kBinBits = 11;            // radix digit of the first two select levels
constexpr int kBins = 1 << kBinBits;    // 2048
constexpr int kMassShift = 40;          // probability mass is an integer multiple of 2^-40
constexpr int kLimbBits = 14;           // mass limbs accumulated with 32-bit shared atomics
constexpr uint32_t kLimbMask = (1u << kLimbBits) - 1;
constexpr int kMaxSliceElems = 262143;  // keeps every 14-bit limb sum below 2^32

typedef unsigned long long u64;

// ---- order-preserving key of an fp32 score: a > b  <=>  key(a) > key(b) -------------
__device__ __forceinline__ uint32_t key_of(float f) {
  uint32_t u = __float_as_uint(f);
  return u ^ (uint32_t)(((int32_t)u >> 31) | 0x80000000);
}
__device__ __forceinline__ float score_of(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k ^ 0x80000000u) : ~k;
  return __uint_as_float(u);
}
// -0.0 and +0.0 compare equal in the reference; give them one key.
__device__ __forceinline__ float canonical(float f) {
  return (__float_as_uint(f) == 0x80000000u) ? 0.0f : f;
}

// Hint: bring `bytes` (a multiple of 16) starting at the 16-byte aligned global address p
// into L2.  No completion to wait for, nothing is written.
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Loads the compiler must issue where they are written (it may otherwise sink a load to its
// first use, which defeats starting a chain of dependent reads early).
__device__ __forceinline__ int load_now_s32(const int* p) {
  int v;
  asm volatile("ld.global.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ int2 load_now_int2(const int2* p) {
  int2 v;
  asm volatile("ld.global.v2.s32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t load_now_u16(const unsigned short* p) {
  unsigned short v;
  asm volatile("ld.global.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- probability mass as an exact integer -------------------------------------------
// e = exp(s - m) in (0, 1]; mass = round(e * 2^40).  Sums of masses are exact and do not
// depend on the order of accumulation, which makes every cut reproducible.
__device__ __forceinline__ u64 mass_of(float s, float m) {
  float e = expf(s - m);
  return __float2ull_rn(e * 1099511627776.0f);
}
__device__ __forceinline__ float mass_to_float(u64 q) {
  return __ull2float_rn(q) * 9.094947017729282e-13f;  // 2^-40
}

// ---- Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as
// 1, 2, 3", SC'11), the counter-based generator behind the seeded draw -----------------
struct Philox4 {
  uint32_t v[4];
};
__device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                 uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  Philox4 r;
  r.v[0] = c0; r.v[1] = c1; r.v[2] = c2; r.v[3] = c3;
  return r;
}

// ---- warp / block primitives ---------------------------------------------------------
__device__ __forceinline__ u64 shfl_xor_u64(u64 v, int lane_mask) {
  const uint32_t lo = __shfl_xor_sync(0xffffffffu, (uint32_t)v, lane_mask);
  const uint32_t hi = __shfl_xor_sync(0xffffffffu, (uint32_t)(v >> 32), lane_mask);
  return ((u64)hi << 32) | lo;
}
__device__ __forceinline__ u64 shfl_u64(u64 v, int src) {
  return __shfl_sync(0xffffffffu, v, src);
}
// Sum over the warp of values below 2^62: three 22-bit limbs, one REDUX each (a chain of
// five dependent 64-bit shuffle steps costs several times as much).
__device__ __forceinline__ u64 warp_sum_u64(u64 v) {
  const uint32_t l0 = __reduce_add_sync(0xffffffffu, (uint32_t)v & 0x3fffffu);
  const uint32_t l1 = __reduce_add_sync(0xffffffffu, (uint32_t)(v >> 22) & 0x3fffffu);
  const uint32_t l2 = __reduce_add_sync(0xffffffffu, (uint32_t)(v >> 44));
  return (u64)l0 + ((u64)l1 << 22) + ((u64)l2 << 44);
}
// Maximum over the warp: the high words first, then the low words of the lanes that hold it.
__device__ __forceinline__ u64 warp_max_u64(u64 v) {
  const uint32_t hi = (uint32_t)(v >> 32);
  const uint32_t top = __reduce_max_sync(0xffffffffu, hi);
  const uint32_t lo = __reduce_max_sync(0xffffffffu, hi == top ? (uint32_t)v : 0u);
  return ((u64)top << 32) | lo;
}
__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) {
  return __reduce_max_sync(0xffffffffu, v);
}
__device__ __forceinline__ uint32_t warp_min_u32(uint32_t v) {
  return __reduce_min_sync(0xffffffffu, v);
}
// Inclusive scan over the lanes of a warp.
__device__ __forceinline__ u64 warp_scan_u64(u64 v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    u64 t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

// Scratch every CTA owns for the collective helpers below.
struct Exchange {
  u64 warp_a[kWarps];
  u64 warp_b[kWarps];
  u64 ring[2][4];      // values this CTA publishes to its cluster, double buffered
  u64 bcast[8];        // results broadcast within the CTA
  uint32_t ring_phase;
};

// Sum of (a, b) over the CTA; every thread gets the totals.  Two barriers.
__device__ __forceinline__ void block_sum2(Exchange& x, u64& a, u64& b) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = warp_sum_u64(a);
  b = warp_sum_u64(b);
  __syncthreads();  // protects warp_a / warp_b against the previous reader
  if (lane == 0) { x.warp_a[warp] = a; x.warp_b[warp] = b; }
  __syncthreads();
  u64 ta = lane < kWarps ? x.warp_a[lane] : 0ull, tb = lane < kWarps ? x.warp_b[lane] : 0ull;
  a = warp_sum_u64(ta);
  b = warp_sum_u64(tb);
}
__device__ __forceinline__ uint32_t block_max_u32(Exchange& x, uint32_t v) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max_u32(v);
  __syncthreads();
  if (lane == 0) x.warp_a[warp] = v;
  __syncthreads();
  return warp_max_u32(lane < kWarps ? (uint32_t)x.warp_a[lane] : 0u);
}
__device__ __forceinline__ u64 block_max_u64(Exchange& x, u64 v) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max_u64(v);
  __syncthreads();
  if (lane == 0) x.warp_a[warp] = v;
  __syncthreads();
  return warp_max_u64(lane < kWarps ? x.warp_a[lane] : 0ull);
}
// Exclusive prefix of (a, b) over the warps of the CTA, given per-warp totals held by
// every lane of each warp; also returns the CTA totals.  Two barriers.
__device__ __forceinline__ void block_warp_prefix2(Exchange& x, u64 wa, u64 wb, u64& pre_a,
                                                   u64& pre_b, u64& tot_a, u64& tot_b) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { x.warp_a[warp] = wa; x.warp_b[warp] = wb; }
  __syncthreads();
  u64 ia = warp_scan_u64(lane < kWarps ? x.warp_a[lane] : 0ull);
  u64 ib = warp_scan_u64(lane < kWarps ? x.warp_b[lane] : 0ull);
  tot_a = shfl_u64(ia, 31);
  tot_b = shfl_u64(ib, 31);
  u64 ea = shfl_u64(ia, warp) - x.warp_a[warp];
  u64 eb = shfl_u64(ib, warp) - x.warp_b[warp];
  pre_a = ea;
  pre_b = eb;
}

// ---- cluster primitives --------------------------------------------------------------
// Every CTA of the cluster publishes up to four 64-bit values; all CTAs read all of
// them.  ring_publish, then any cluster-wide barrier, then ring_read.  The buffer is
// double buffered, so no barrier is needed after the read.  `vals` must be CTA-uniform.
template <int N>
__device__ __forceinline__ uint32_t ring_publish(Exchange& x, const u64 (&vals)[N]) {
  static_assert(N <= 4, "ring holds four values");
  __syncthreads();
  const uint32_t phase = x.ring_phase & 1u;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) x.ring[phase][i] = vals[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) x.ring_phase = phase ^ 1u;
  return phase;
}
template <int N>
__device__ __forceinline__ void ring_read(cg::cluster_group& cluster, Exchange& x, uint32_t phase,
                                          u64 (&out)[kMaxCluster][N]) {
  const unsigned nranks = cluster.num_blocks();
  for (unsigned r = 0; r < nranks; ++r) {
    const Exchange* remote = nranks > 1 ? cluster.map_shared_rank(&x, r) : &x;
#pragma unroll
    for (int i = 0; i < N; ++i) out[r][i] = remote->ring[phase][i];
  }
}
// Reductions over the published values of all CTAs, read straight from the ring.
enum class RingOp { Sum, Max, Min };
template <RingOp OP>
__device__ __forceinline__ u64 ring_reduce(cg::cluster_group& cluster, Exchange& x, uint32_t phase, int i) {
  const unsigned nranks = cluster.num_blocks();
  u64 acc = OP == RingOp::Min ? ~0ull : 0ull;
#pragma unroll
  for (unsigned r = 0; r < (unsigned)kMaxCluster; ++r) {
    if (r >= nranks) break;
    const Exchange* remote = nranks > 1 ? cluster.map_shared_rank(&x, r) : &x;
    const u64 v = remote->ring[phase][i];
    if (OP == RingOp::Sum) acc += v;
    else if (OP == RingOp::Max) acc = v > acc ? v : acc;
    else acc = v < acc ? v : acc;
  }
  return acc;
}
// Sum over the CTAs of rank < my_rank (exclusive prefix in rank order).
__device__ __forceinline__ u64 ring_prefix(cg::cluster_group& cluster, Exchange& x, uint32_t phase, int i,
                                           unsigned my_rank) {
  const unsigned nranks = cluster.num_blocks();
  u64 acc = 0;
#pragma unroll
  for (unsigned r = 0; r < (unsigned)kMaxCluster; ++r) {
    if (r >= my_rank || r >= nranks) break;
    const Exchange* remote = nranks > 1 ? cluster.map_shared_rank(&x, r) : &x;
    acc += remote->ring[phase][i];
  }
  return acc;
}
// publish + one cluster barrier; returns the ring phase to reduce from.
template <int N>
__device__ __forceinline__ uint32_t cluster_publish(cg::cluster_group& cluster, Exchange& x,
                                                    const u64 (&vals)[N]) {
  const uint32_t phase = ring_publish<N>(x, vals);
  if (cluster.num_blocks() > 1) cluster.sync();
  return phase;
}

// publish + barrier + read in one call.  out[rank][i].
template <int N>
__device__ __forceinline__ void cluster_allgather(cg::cluster_group& cluster, Exchange& x,
                                                  const u64 (&vals)[N], u64 (&out)[kMaxCluster][N]) {
  const uint32_t phase = ring_publish<N>(x, vals);
  if (cluster.num_blocks() > 1) cluster.sync();
  ring_read<N>(cluster, x, phase, out);
}

}  // namespace hs
