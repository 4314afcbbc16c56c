/* colinfer_b200.h -- C ABI of the B200 (sm_100a) logits -> token path.
 *
 * Every entry point takes plain device pointers and sizes, launches on the CUDA stream it is given (a cudaStream_t
 * passed as void*), performs no host synchronisation and no allocation (except where stated), and returns a
 * cudaError_t value as int (0 = success; cudaErrorInvalidValue = 1 for a bad shape, as the reference's launch_*
 * functions do, csrc/sampling.cu:79, 112).  Inputs are borrowed, outputs are caller-allocated.  No entry point ever
 * traps or asserts on the device: anomalies are reported through the optional per-row status words.
 *
 * "Reference" citations name files of the colinfer tree (engine/..., csrc/...).
 */
#ifndef COLINFER_B200_H
#define COLINFER_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Per-slot sampling parameters: the device buffers of the reference's SamplerParams (engine/runtime/sampler.py:23-31),
 * each [B], plus this project's optional penalty fields (NULL = neutral). */
typedef struct colinfer_sampler_params {
    const float*   temperature;        /* [B]  <= 0 selects the argmax of the slot's rows */
    const int32_t* top_k;              /* [B]  <= 0 or >= V disables top-k */
    const float*   top_p;              /* [B]  >= 1 disables top-p */
    const float*   log_min_p;          /* [B]  -inf disables min-p */
    const int64_t* seed;               /* [B]  may be NULL when explicit uniforms are passed */
    const float*   repetition_penalty; /* [B] or NULL (= 1) */
    const float*   presence_penalty;   /* [B] or NULL (= 0) */
    const float*   frequency_penalty;  /* [B] or NULL (= 0) */
    const int32_t* history;            /* [B, hist_stride] token ids of each slot, or NULL */
    const int32_t* hist_len;           /* [B] valid ids per slot, or NULL (= hist_stride) */
    int32_t        hist_stride;
} colinfer_sampler_params;

/* Per-row description of the processed distribution, written by colinfer_sample when `stats` is not NULL.
 * The kept set of the row is { t : logit'(t) >= lcut } (logit' = after penalties and mask) and
 * P(t) = exp(logit'(t) / tc - lmax / tc) / (mass_q * 2^-30) on that set.
 * Masses are integers in units of 2^-30 of the largest token's, so that every sum is exact and a row's result does not
 * depend on the batch or the grid.  A token more than about 21.5 temperatures below the row's maximum has mass 0: it is
 * never drawn, processed_probs gives it 0, and the rejection verify treats it as a token the target excludes.  Against an
 * fp32 softmax this moves at most V * 2^-31 of the probability (7e-5 at 151,936 tokens). */
typedef struct colinfer_row_stats {
    float    lmax;      /* largest logit' of the row */
    float    lcut;      /* smallest kept logit' value (a threshold; -inf keeps all) */
    float    tc;        /* max(temperature, 1e-6) */
    int32_t  status;    /* COLINFER_ROW_* bits */
    int64_t  argmax;    /* lowest index of the largest logit' */
    uint64_t mass_q;    /* kept mass in units of 2^-30 */
} colinfer_row_stats;

enum {
    COLINFER_ROW_DEGENERATE = 1,  /* no finite maximum (every token masked, or an infinite logit): argmax emitted */
    COLINFER_ROW_TIMEOUT    = 2,  /* a bounded on-chip wait gave up; the row's outputs are undefined */
    COLINFER_ROW_HIST_SLOW  = 4,  /* more distinct history ids than the fast table holds: same result, slower */
    COLINFER_ROW_SELECT_SLOW = 8  /* a candidate list overflowed or the estimated band missed the pivot: the exact radix
                                     select ran instead; same result, slower */
};

enum { COLINFER_F32 = 0, COLINFER_BF16 = 1 };

/* Flags of colinfer_sample (per call: the library keeps no settings between calls). */
enum {
    COLINFER_FORCE_DISTRIBUTION = 1, /* build the distribution even for temperature <= 0 (processed_probs does) */
    /* which kernel runs (tests and benchmarks; results are the same): default automatic -- few rows take the
       cluster-resident kernel, one 8-CTA cluster per row, more rows the streaming kernel */
    COLINFER_KERNEL_STREAM   = 0x100, /* the streaming kernel */
    COLINFER_KERNEL_CLUSTER1 = 0x200, /* the cluster-resident kernel with clusters of 1, */
    COLINFER_KERNEL_CLUSTER2 = 0x300, /* 2, */
    COLINFER_KERNEL_CLUSTER4 = 0x400, /* 4, */
    COLINFER_KERNEL_CLUSTER8 = 0x500, /* 8 CTAs */
    COLINFER_TEST_DROP_COPY = 0x2000, /* test flag (cluster-resident kernel): the bulk copies of a row are never issued, so its
                                         bounded waits run out: rows report COLINFER_ROW_TIMEOUT and the kernel returns */
    COLINFER_TEST_MISS_BAND = 0x4000 /* test flag: misplace the estimated top-p band so that the exact retry paths run;
                                        results are unchanged, rows report COLINFER_ROW_SELECT_SLOW */
};

/* Replaces ops().philox_uniform (csrc/sampling.cu:25-35, csrc/bindings.cpp:538-544):
 * out[b, i] = U(0, 1] of Philox4x32-10 keyed by mix(seed[b]) at counter offset[b] + i.  out is [B, n] fp32. */
int colinfer_philox_uniform(const int64_t* seed, const int64_t* offset, float* out, int B, int n, void* stream);

/* Replaces apply_mask (engine/runtime/sampler.py:50-56): out = logits with every token whose bit (t % 32 of int32 word
 * t / 32) is clear set to -inf.  logits, out: [rows, V] fp32 (out may alias logits); mask: [rows, W] int32, W >= ceil(V/32). */
int colinfer_apply_mask(const float* logits, const int32_t* mask, float* out, int64_t rows, int V, int W, void* stream);

/* Replaces draw / sample (engine/spec/accept.py:43-52, engine/runtime/sampler.py:59-62) fused with apply_mask and the
 * penalties: one pass over HBM per row.
 *   logits  [B, R, V] fp32 or bf16 (dtype), contiguous
 *   mask    [B, mask_rows, W] int32 or NULL; row r of slot b uses mask[b, r]
 *   pos     [B] int32 or int64 (pos_is_i64) device positions: row r draws the uniform at counter pos[b] + r
 *   u       [B, R] explicit uniforms in (0, 1], or NULL to use Philox(seed, pos)
 *   out_ids [B, R] int64 (may be NULL when only stats are wanted; then u, pos and seed may be NULL too)
 *   stats   [B, R] or NULL;  status [B, R] int32 or NULL */
int colinfer_sample(const void* logits, int dtype, const int32_t* mask, int mask_rows, int W,
                    const colinfer_sampler_params* params, const void* pos, int pos_is_i64, const float* u,
                    int64_t* out_ids, colinfer_row_stats* stats, int32_t* status,
                    int B, int R, int V, int flags, void* stream);

/* Replaces processed_probs (engine/spec/accept.py:23-33).  logits [R, V] fp32; temperature, top_k, top_p, log_min_p:
 * 1-element device arrays; out [R, V] fp32 renormalised probabilities; scratch: R colinfer_row_stats (device). */
int colinfer_processed_probs(const float* logits, const float* temperature, const int32_t* top_k, const float* top_p,
                             const float* log_min_p, float* out, colinfer_row_stats* scratch, int R, int V, void* stream);

/* colinfer_processed_probs for callers that have no scratch to give (no counterpart in the reference; added for hosts
 * that bind this ABI without an allocator of their own -- e.g. one that replays the call from a captured CUDA graph or
 * runs under a fixed memory budget, where cudaMalloc is illegal or forbidden).  The per-row statistics live in a
 * fixed 128 KB array inside the library's device image, held by every GPU that loads the library until the process
 * exits.  Same arguments and results as colinfer_processed_probs, minus `scratch`.
 *   - R may not exceed colinfer_noalloc_max_rows() (4096): larger R returns cudaErrorInvalidValue, nothing is launched.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current); make that first call outside any stream capture.  No call allocates or frees device memory.
 *   - All calls on a device share the one array: two calls that may overlap on the GPU (different streams, no
 *     dependency between them) race on it.  Serialise them, or use colinfer_processed_probs with separate scratch.
 *   - Nothing in the array needs clearing between calls: every entry a call reads it has written first. */
int colinfer_processed_probs_noalloc(const float* logits, const float* temperature, const int32_t* top_k,
                                     const float* top_p, const float* log_min_p, float* out, int R, int V, void* stream);
int colinfer_noalloc_max_rows(void);

/* Replaces inverse_cdf (engine/spec/accept.py:36-40): out[r] = #{ j : cumsum(P[r])_j < u[r] * sum(P[r]) }, clamped to
 * V - 1.  P [R, V] fp32, u [R], out [R] int64. */
int colinfer_inverse_cdf(const float* P, const float* u, int64_t* out, int R, int V, void* stream);

/* Replaces the accept / bonus / stop-cut lines of the speculative cycle (engine/spec/mtp.py:406-415, 422-423;
 * engine/spec/mtp4.py:538-547).  pred, tok: [B, k1] int64 (k1 = k + 1; tok[:, 1:] are the drafts); stop_ids [B, S]
 * int64 (-1 = unused) or NULL; active [B] int32 or NULL (= 1).  out_tok [B, k1] int64, n [B] int32. */
int colinfer_spec_accept(const int64_t* pred, const int64_t* tok, const int64_t* stop_ids, const int32_t* active,
                         int64_t* out_tok, int32_t* n, int B, int k1, int S, void* stream);

/* Keeps on the device what the reference's scheduler does on the host after every cycle (engine/runtime/scheduler.py:
 * 635-641: n and out_tok read back, `tokens.append(y); tokens += o[:-1]; y = o[-1]`).  For each slot with n[b] > 0: the
 * pending token y[b] and the accepted drafts out_tok[b, 0 .. n-2] are appended to history[b, :hist_len[b]] (int32 [B, H],
 * the history the penalties count in; NULL: no history; on overflow the most recent H ids are kept), y[b] becomes the
 * bonus token out_tok[b, n-1], hist_len[b] and pos[b] (int64, NULL: none) move on by n.  Slots with n[b] <= 0 keep
 * their state.  out_tok [B, k1] int64 and n [B] int32 as colinfer_spec_accept / colinfer_spec_verify write them. */
int colinfer_spec_advance(const int64_t* out_tok, const int32_t* n, int64_t* y, int32_t* history, int32_t* hist_len,
                          int64_t* pos, int B, int k1, int H, void* stream);

/* Rejection verify with the (p - q)+ residual resample (no counterpart in the reference, which accepts by exact match;
 * semantics: accept draft i iff p_i(d_i) > 0 and ua[i] * q_i(d_i) <= p_i(d_i); at the first rejection j emit a draw from
 * normalize(max(p_j - q_j, 0)) with us[j]; if none is rejected emit a draw from p_k with us[k]; temperature <= 0 uses
 * the argmax rule).  target_logits [B, k+1, V], draft_logits [B, k, V] (dtype), mask [B, k+1, W] or NULL (applies to
 * both), draft_ids [B, k] int64, ua [B, k], us [B, k+1].  Penalties in params (history, hist_len, the three factors)
 * apply to every row of both models with the slot's history, before mask and temperature; V <= 524,288.  scratch: B * (2k + 1) colinfer_row_stats and B * (k + 1)
 * int64 (device).  out_tok [B, k+1] int64 (accepted drafts, then the emitted token, then -1), n [B] int32 = accepted + 1. */
int colinfer_spec_verify(const void* target_logits, const void* draft_logits, int dtype, const int32_t* mask, int W,
                         const colinfer_sampler_params* params, const int64_t* draft_ids, const float* ua,
                         const float* us, int64_t* out_tok, int32_t* n, colinfer_row_stats* scratch_stats,
                         int64_t* scratch_ids, int B, int k, int V, void* stream);

/* Bytes of scratch_stats / scratch_ids that colinfer_spec_verify needs. */
int64_t colinfer_spec_verify_stats_bytes(int B, int k);
int64_t colinfer_spec_verify_ids_bytes(int B, int k);

/* Geometry the cluster-resident kernel would use for a vocabulary (for tests and benchmarks): CTAs per row (thread-block
 * cluster size; cluster = 0 picks the smallest that holds the row, else 1, 2, 4 or 8), elements per CTA slice, dynamic
 * shared memory per CTA, and whether the bulk-copy (TMA) load path applies. */
typedef struct colinfer_geometry {
    int32_t cluster;
    int32_t slice_elems;
    int32_t smem_bytes;
    int32_t bulk_copy;
} colinfer_geometry;
int colinfer_sample_geometry(int V, int dtype, const void* logits, int cluster, colinfer_geometry* out);

/* How many clusters of the sampler's geometry for this vocabulary the current device holds at once (occupancy query). */
int colinfer_max_active_clusters(int V, int dtype);

/* Replaces Scheduler._logprobs (engine/runtime/scheduler.py:714-722: log_softmax + gather + topk on the RAW logits of
 * the positions that produced the emitted tokens).  logits [rows, V] fp32 or bf16; toks [rows] int64 (NULL: no chosen
 * logprob); chosen [rows] fp32 = log_softmax(row)[tok]; top_ids / top_lp [rows, n_top]: the n_top (0 .. 32) most likely
 * tokens in descending order (equal logits: lower token first) with their logprobs.  One pass over each row. */
int colinfer_logprobs(const void* logits, int dtype, const int64_t* toks, int n_top, float* chosen, int64_t* top_ids,
                      float* top_lp, int rows, int V, void* stream);

/* Replace ops().rescore_bf16 / ops().rescore_nvfp4 (csrc/sampling.cu:36-115, csrc/bindings.cpp:547-572): exact logits of
 * candidate rows of the lm_head, out[b, j] = sum_k x[b, k] * W[cand[b, j], k] (NVFP4: E2M1 pairs [rows_w, K / 2], E4M3
 * scales sf [rows_w, K / 16], global scale gs).  x bf16 [B, K], cand int64 [B, NC], out fp32 [B, NC]; K a multiple of
 * 8 (16 for NVFP4), x and w 16-byte aligned.  Results are bit-identical to the reference's kernels (same fma order)
 * and independent of B and NC.  rows_w bounds the candidate ids: an id outside [0, rows_w) yields NaN, never a fault. */
int colinfer_rescore_bf16(const void* x, const void* w, const int64_t* cand, float* out, int B, int K, int NC,
                          int64_t rows_w, void* stream);
int colinfer_rescore_nvfp4(const void* x, const void* w, const void* sf, float gs, const int64_t* cand, float* out,
                           int B, int K, int NC, int64_t rows_w, void* stream);

/* Replaces the greedy draft() of the low-rank draft heads (engine/spec/mtp.py:301-309, engine/spec/mtp4.py:416-423: topk
 * over the approximate logits, gather of the candidates' lm_head rows, rescoring, argmax, two more gathers, logsumexp,
 * exp, clamp -- nine launches) with one.  ap fp32 [N, Vd] = the approximate logits over the draft vocabulary; x bf16
 * [N, K]; w = the lm_head, [rows_w, K] bf16 (w_format COLINFER_W_BF16) or NVFP4 as for colinfer_rescore_nvfp4 (sf, gs;
 * COLINFER_W_NVFP4); vocab_ids int64 [Vd] maps a draft-vocabulary index to its lm_head row and token id (NULL: identity).
 * Of the NC (<= 1024, <= Vd) largest entries of ap[n] (equal values: lower index first), the one with the largest exact
 * logit ex = x[n] . w[row] (accumulated as colinfer_rescore_* does; equal ex: larger ap, then lower index -- what argmax
 * over topk's sorted list gives) is chosen: out_ids[n] = its token id, out_p[n] = min(1, exp(ex - logsumexp(ap[n]))),
 * out_idx[n] (optional) = its draft-vocabulary index, out_ex[n] (optional) = ex.  A candidate whose row lies outside
 * [0, rows_w) is never chosen.  ctas_per_slot: 0 = by N, or 1, 2, 4, 8, 16.  scratch: colinfer_draft_pick_scratch_bytes(N)
 * bytes, 16-byte aligned, zero-filled by the caller once before its first use (every call leaves it ready for the next;
 * calls that may overlap in time need a scratch each); nothing in the launch waits for another launch or spins. */
enum { COLINFER_W_BF16 = 0, COLINFER_W_NVFP4 = 1 };
int64_t colinfer_draft_pick_scratch_bytes(int N);
int colinfer_draft_pick(const float* ap, const void* x, const void* w, const void* sf, float gs, int w_format,
                        const int64_t* vocab_ids, int64_t* out_ids, float* out_p, int32_t* out_idx, float* out_ex,
                        int N, int Vd, int K, int NC, int64_t rows_w, int ctas_per_slot, void* scratch, int64_t scratch_bytes,
                        void* stream);

/* The id gather of a row-sharded step over NVLink, in one launch of one CTA (no counterpart in the reference, which runs
 * on one GPU; it takes the place of an all-gather call behind the sampler).  Every rank calls it with its own ids
 * `local` [n_local] (the rows [row_offset, row_offset + n_local) of the step): they are stored into every rank's gather
 * buffer -- peer_bufs[p] is rank p's buffer of 2 * half_elems int64, mapped into this process (device array of n_ranks
 * pointers); steps alternate between its halves -- then this rank's flag is raised at every rank (peer_flags[p] is rank
 * p's array of n_ranks int64 flags) and the kernel waits until all n_ranks flags of this rank have reached the step.
 * step_counter: one int64 of this rank's device memory, zero before the first call; the kernel advances it, so a
 * captured launch can be replayed.  After the call, on the same stream, the ids of all half_elems rows of the step are
 * in out_all (this rank's memory).  The wait gives up after limit_cycles clock cycles (<= 0: about a second),
 * sets COLINFER_GATHER_TIMEOUT in *status (may be NULL) and returns.  Every rank must own its GPU: ranks that share
 * one would wait on kernels that cannot run. */
enum { COLINFER_GATHER_TIMEOUT = 1 };
int colinfer_gather_ids(const int64_t* local, int n_local, int64_t row_offset, int64_t* const* peer_bufs,
                        long long* const* peer_flags, int n_ranks, int rank, long long* step_counter, int64_t half_elems,
                        int64_t* out_all, int64_t limit_cycles, int32_t* status, void* stream);

/* Library version (major * 100 + minor). */
int colinfer_version(void);

#ifdef __cplusplus
}
#endif
#endif
