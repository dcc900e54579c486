/*
 * hs_sampler.h -- C ABI of the B200 (sm_100a) per-step token sampler.
 *
 * The reference (HydraServe) has no FFI: its boundary for this path is the Python
 * module hydraserve/engine/sampling.py.  Each entry point below names the piece of that
 * module it stands in for.  Plain C types only; every function returns an hs_status
 * (0 = ok, negative = error) and never throws or aborts.  Unless a parameter says
 * "host", pointers are DEVICE pointers valid on the sampler's device, and work is
 * enqueued on the given CUDA stream (a cudaStream_t passed as void*) without
 * synchronising it.
 *
 * Threads and streams.  Every function may be called from any thread, on any stream: the
 * reference's callers are the serving loop, each worker's command loop and, concurrently,
 * the threads that replay a first token on a side stream (hydraserve/engine/pd_service.py:
 * 916-967, pd_worker.py:305-308, 475-480).  Calls on ONE sampler do not run concurrently:
 * they take a lock for the time of their launches, and a call enqueued on another stream
 * than the previous call first waits (on the GPU, through an event) for that call's work,
 * because all calls share the sampler's scratch memory and histograms.  Two samplers never
 * wait for each other.  hs_last_error returns the calling thread's last message.
 */
#ifndef HS_SAMPLER_H
#define HS_SAMPLER_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HS_MAX_LOGPROBS 20 /* reference sampling.py:38 */

typedef enum {
  HS_OK = 0,
  HS_ERR_INVALID = -1,   /* bad argument (null pointer, negative size, unknown dtype) */
  HS_ERR_CAPACITY = -2,  /* vocabulary, batch, slot or history beyond what hs_create sized */
  HS_ERR_CUDA = -3,      /* a CUDA runtime call failed; see hs_last_error */
  HS_ERR_UNSUPPORTED = -4
} hs_status;

typedef enum { HS_DTYPE_F32 = 0, HS_DTYPE_BF16 = 1 } hs_dtype;

/* Bits of hs_row_params.flags. */
#define HS_ROW_PLAIN_GREEDY 1u /* temperature 0, no penalties, no logprobs: argmax only */

/* Bits of the `flags` argument of hs_sample / hs_sample_ex. */
#define HS_SAMPLE_APPEND_TOKEN 1u   /* after sampling, count the sampled token in the row's slot */
#define HS_SAMPLE_GENERAL_KERNEL 2u /* bf16 rows too take the general kernel (rows reported with status bit 4) */

/* Bits of the `flags` argument of hs_create_ex (tests and tuning; a serving process passes 0). */
#define HS_CREATE_FORCE_GENERAL 1u /* every row, bf16 included, takes the general (fp32-resident) kernel */
#define HS_CREATE_PHASE_CLOCKS 2u  /* the bf16 kernel records phase time stamps, see hs_debug_phase_clocks */
#define HS_CREATE_CLUSTER(n) (((uint32_t)(n) & 0xfu) << 8) /* general kernel: n = 1, 2, 4 or 8 CTAs per row */

/* One row's sampling parameters: the numeric fields of SamplingParams
 * (reference sampling.py:8-19) in the fp32 precision the reference computes in. */
typedef struct hs_row_params {
  float temperature;        /* 0 = greedy (sampling.py:122) */
  float top_p;              /* (0,1]; 1 = off */
  float min_p;              /* [0,1]; 0 = off */
  float repetition_penalty; /* 1 = off */
  float presence_penalty;   /* 0 = off */
  float frequency_penalty;  /* 0 = off */
  int32_t top_k;            /* 0 = off */
  int32_t n_logprobs;       /* -1 = none, else 0..20 (sampling.py:152-155) */
  uint64_t seed;            /* (seed + (step+1)*0x1E3779B97F4A7C15) mod 2^63 (sampling.py:148) */
  uint32_t flags;           /* HS_ROW_* */
  int32_t slot;             /* token-count histogram to penalise with, or -1 for none.  A row with a
                               slot and a row without one may be served by different code paths, and
                               the path decides which token a seeded draw lands on (the distribution
                               is the same): present a request the same way every time it is sampled
                               with the same inputs, e.g. -1 while its history is still empty */
} hs_row_params;

/* One row's result: the fields of TokenSample (reference sampling.py:47-51) plus what the
 * parity tests need to compare candidate sets. */
typedef struct hs_row_out {
  int32_t token;         /* sampled / argmax token id */
  float logprob;         /* log-probability of `token` (valid when n_logprobs >= 0) */
  int32_t n_top;         /* number of valid entries in top_ids / top_logprobs */
  int32_t status;        /* 0 ok.  bit 0 (1): selection fell back (non-finite input); 2: the sampled token
                            could not be counted (histogram full); 4: more individually scored tokens than
                            the bf16 kernel keeps (values outside 2^-14 <= |x| < 2^10, history counts >= 3):
                            sample the row again with HS_SAMPLE_GENERAL_KERNEL; 8: fewer top log-probabilities
                            found than expected; 16 / 32: a vocabulary shard's record was cut short;
                            64: params.slot is not a slot of this sampler (the row got no penalties);
                            128: the row found no free scratch block (more CTAs resident than the
                            sampler was sized for: an internal error, the row is not sampled) */
  int32_t n_kept;        /* size of the final candidate set */
  int32_t n_after_topk;  /* candidates left by top-k (ties at the k-th value kept) */
  int32_t n_after_minp;  /* ... and by min-p */
  int32_t n_after_topp;  /* ... and by top-p (== n_kept) */
  uint32_t cut_bits;     /* fp32 bits of the lowest kept score */
  int32_t n_cut_ties;    /* how many tokens scoring exactly the cut are kept (lowest ids) */
  float row_max;         /* largest score after penalties and temperature */
  float log_z;           /* log of the soft-max denominator over the kept set, relative to row_max */
  int32_t top_ids[HS_MAX_LOGPROBS];
  float top_logprobs[HS_MAX_LOGPROBS];
} hs_row_out;

typedef struct hs_sampler hs_sampler;

/* Create a sampler on `device`.  vocab_max: largest vocabulary any call will pass.
 * slots_max: number of resident token-count histograms (one per request in flight); the
 *   sampler adds batch_max more, [slots_max, slots_max + batch_max), for histories that live
 *   for one call only.
 * hist_cap: most distinct token ids one histogram can hold (<= vocab_max; 0 = vocab_max); a
 *   request's history cannot hold more distinct ids than its context length.  Device memory
 *   per slot: 12 * hist_cap + 4.25 * vocab_max bytes (hs_query what = 6).
 * batch_max: most rows per call.  Allocates all device memory the sampler will ever use
 *   (hs_query what = 5).  The environment is not consulted. */
int hs_create(int device, int vocab_max, int slots_max, int hist_cap, int batch_max,
              hs_sampler** out);
int hs_create_ex(int device, int vocab_max, int slots_max, int hist_cap, int batch_max,
                 uint32_t flags /* HS_CREATE_* */, hs_sampler** out);
int hs_destroy(hs_sampler* h);

/* Token-count histograms: the device-resident form of the `counts` dict the reference
 * rebuilds per row per step (sampling.py:106-110).
 * hs_slots_reset empties the listed slots.  hs_slots_append counts tokens
 * tokens[offsets[i] .. offsets[i+1]) into slot slots[i]; ids outside [0, vocab) are
 * ignored as in the reference (sampling.py:108).  slots must not repeat within a call. */
int hs_slots_reset(hs_sampler* h, const int32_t* slots, int n_slots, void* stream);
int hs_slots_append(hs_sampler* h, const int32_t* tokens, const int32_t* offsets,
                    const int32_t* slots, int n_slots, int vocab, int max_tokens_per_slot,
                    void* stream);
/* Host-side count of distinct ids in a slot (synchronises the stream); for tests. */
int hs_slot_unique_count(hs_sampler* h, int slot, void* stream, int* out);

/* sample_logits (reference sampling.py:54-83) for rows of one batch.
 * logits: [batch, vocab] of `dtype`, row r starting at logits + r*row_stride elements.
 * noise: NULL, or [batch, vocab] fp32 Exp(1) variates; when given, the draw is
 *   argmax(p / noise) as torch.multinomial does on CPU (sampling.py:150) instead of the
 *   Philox stream.  For parity tests.
 * scores_out: NULL, or [batch, vocab] fp32 that receives the reference's final `scores`
 *   (penalised, temperature-scaled, -inf where filtered).  For parity tests. */
int hs_sample(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch,
              int vocab, const hs_row_params* params, hs_row_out* out, const float* noise,
              float* scores_out, uint32_t flags, void* stream);
/* hs_sample that also leaves the sampled ids in tokens_out[batch] (device, int32; NULL = as
 * hs_sample): the next decode step's input ids.  The reference copies them in from the host
 * every step (hydraserve/model/runtime.py:682); with this buffer and HS_SAMPLE_APPEND_TOKEN a
 * decode loop can run step after step on one stream without reading anything back, and fetch
 * the records of several steps later (or never). */
int hs_sample_ex(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch,
                 int vocab, const hs_row_params* params, hs_row_out* out, const float* noise,
                 float* scores_out, int32_t* tokens_out, uint32_t flags, void* stream);

/* The all-rows-plain-greedy fast path (reference sampling.py:69-73): argmax per row,
 * lowest id on ties, int32 token ids to tokens_out[batch]. */
int hs_greedy(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch,
              int vocab, int32_t* tokens_out, void* stream);

/* No counterpart in the reference.  hs_greedy for callers that must not allocate device
 * memory: a serving worker that has handed all of the GPU's memory to its framework's
 * caching allocator (a raw cudaMalloc can fail there), or a step on the latency-critical
 * decode path, where the device-wide synchronisation that cudaMalloc and cudaFree imply is
 * not acceptable.  It needs no hs_sampler: it runs on the CURRENT device, calls no
 * cudaMalloc / cudaFree / allocating library routine, and keeps its per-row partial results
 * in a fixed 128 KB device array inside the library (each GPU that loads the library holds
 * that array until the process exits).  Limits and rules:
 *   - batch <= HS_NOALLOC_MAX_BATCH; a larger batch is refused with HS_ERR_CAPACITY and a
 *     message from hs_greedy_noalloc_error() (split the call);
 *   - the first call on each device resolves the array's address (once per device, under a
 *     lock); make that first call before any stream capture;
 *   - all calls on one GPU share the array: two calls whose kernels can overlap on the GPU
 *     (different streams, no ordering) race.  Calls on one stream are fine.  Nothing needs to
 *     start at zero: every slot a call reads is written by that same call.
 * Results are identical to hs_greedy (lowest id on ties). */
#define HS_NOALLOC_MAX_BATCH 1024
int hs_greedy_noalloc(const void* logits, int dtype, int64_t row_stride, int batch, int vocab,
                      int32_t* tokens_out, void* stream);
/* Message for the calling thread's last failed hs_greedy_noalloc ("" after a success). */
const char* hs_greedy_noalloc_error(void);

/* Same as hs_sample but every pointer is a HOST pointer; copies in and out on `stream`
 * through pinned staging buffers owned by the sampler and synchronises before returning.
 * hist_tokens/hist_offsets: flat per-row histories (offsets has batch+1 entries), or NULL;
 * rows whose params.slot is -2 are penalised with their history from these arrays
 * (rebuilt on the device for this call, the reference's stateless behaviour). */
int hs_sample_host(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch,
                   int vocab, hs_row_params* params, hs_row_out* out,
                   const int32_t* hist_tokens, const int32_t* hist_offsets, uint32_t flags,
                   void* stream);

/* Vocabulary-sharded sampling (no counterpart in the reference, which has no tensor-parallel
 * LM head; the result equals sample_logits on the concatenated row, sampling.py:54-163).
 * Each rank reduces its contiguous slice of every row to an hs_shard_rec with
 * hs_sharded_partial; the records of all ranks are exchanged by the caller (an all-gather,
 * e.g. NCCL over NVLink) into recs[ranks][batch]; hs_sharded_merge finishes the rows from the
 * union of the candidates.  Needs 0 < top_k <= HS_SHARD_CAND - 8 on every row; token ids in
 * the records and results are global (slice-local id + vocab_offset).  Histories, when
 * penalties are on, are slots of THIS rank's sampler filled with slice-local ids. */
#define HS_SHARD_CAND 64
typedef struct hs_shard_rec {
  float row_max;       /* highest score of the slice (after penalties and temperature) */
  float pad;
  uint64_t z_mass;     /* sum over the slice of round(exp(score - row_max) * 2^40) */
  int32_t n;           /* candidates that follow: the slice's top_k, ties at the k-th included */
  int32_t status;      /* 0 ok; 16: candidate list overflowed; 32: more ties than the record holds */
  int32_t ids[HS_SHARD_CAND];    /* global token ids, descending score then ascending id */
  float scores[HS_SHARD_CAND];
} hs_shard_rec;
int hs_sharded_partial(hs_sampler* h, const void* logits, int dtype, int64_t row_stride, int batch,
                       int vocab_local, int vocab_offset, const hs_row_params* params,
                       hs_shard_rec* recs_out, void* stream);
/* noise: NULL or [batch, vocab_total] Exp(1) variates (parity tests).  full_lse: NULL or
 * [batch] floats receiving log-sum-exp of the scores over the whole vocabulary. */
int hs_sharded_merge(hs_sampler* h, const hs_shard_rec* recs, int ranks, int batch, int vocab_total,
                     const hs_row_params* params, hs_row_out* out, const float* noise,
                     float* full_lse, void* stream);

/* Introspection. */
const char* hs_last_error(hs_sampler* h);
const char* hs_status_string(int status);
int hs_abi_version(void);
/* what: 0 = CTAs per row (cluster size) hs_sample would use for (vocab, dtype),
 *       1 = 1 if the general kernel would hold that row in shared memory, 0 if in global scratch
 *           (the bf16 kernels do not hold the row at all),
 *       2 = number of SMs, 3 = kernels launched by this sampler so far (low 31 bits),
 *       4 = 1 if (vocab, dtype) takes the bf16 kernel (candidate / counting paths), 0 if the general one,
 *       5 = device memory held by the sampler, in KiB, 6 = device bytes per histogram slot,
 *       7 = CTAs of the bf16 kernel that can be resident at once (CTAs per SM x SMs),
 *       8 = 1 if hs_slots_append was ever given more distinct ids for one histogram than hist_cap
 *           (the ids beyond it were not counted and get no penalty; the flag stays up), else 0;
 *           waits for the device.  A caller that sizes hist_cap by its context length, as the
 *           Python host does, never sees it; hs_sample's own one-token append reports status 2
 *           for the row instead. */
int hs_query(hs_sampler* h, int what, int vocab, int dtype);
/* Tuning aid: a sampler created with HS_CREATE_PHASE_CLOCKS records, per row of the last launch,
 * 64 counters: the SM clock at the phases of the row's CTA (slots 0..47), and when each of the
 * row's work items started and ended, in ns of the global timer (slots 48..55: up to four
 * counting parts, 56..63: up to four candidate parts).  Copies batch x 64 counters to out_host (synchronises the device). */
int hs_debug_phase_clocks(hs_sampler* h, int batch, unsigned long long* out_host);
/* Tests and tuning.  what = 0: CTAs per candidate row, what = 1: CTAs per counting row; value 1, 2
 * or 4 (0 = chosen per call).  what = 3: near-flat counting rows draw by rejection on tokens
 * (1, the default) or always class by class (0). */
int hs_debug_set(hs_sampler* h, int what, int value);

#ifdef __cplusplus
}
#endif
#endif /* HS_SAMPLER_H */
