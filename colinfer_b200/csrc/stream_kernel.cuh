// stream_kernel.cuh -- the streaming form of the fused logits -> token kernel (sm_100a): one CTA per row.
//
// A persistent grid of one 1024-thread CTA per SM; each CTA owns one row at a time and streams it from global memory
// with 128-bit loads in two to three passes: the first pass comes from HBM, the later ones hit the 126 MB L2 (at most
// one row per SM is in flight: 148 x 608 KB = 90 MB).  No row is ever copied: penalties and the grammar mask are applied
// on the fly in every pass (a bitmap of the history's tokens in shared memory marks the few logits to penalise).  All
// reductions stay inside the CTA, so a row costs a handful of __syncthreads and no cluster traffic.
//
//   pass 1   maximum / argmax and four group maxima per thread
//   greedy   done
//   top_k <= 100   the k-th largest of the 4096 group maxima bounds the k-th largest logit from below; pass 2 collects
//            the logits above the bound (in token order) and the row is finished exactly on that list
//   larger top_k / top_p alone   pass 2 builds a 4096-bucket count histogram over the distance from the maximum (exact
//            bucket of the k-th largest; estimated bucket of the top-p pivot); pass 3 sums the exact masses (top-p:
//            above a narrow band, whose logits are gathered and resolved exactly); the draw rescans one warp's region
//   neither  pass 2 sums the masses; the draw rescans one warp's region
// Masses are exp(z - max) in integer units of 2^-30 and all sums are integer: results do not depend on the batch.
// If a list overflows or the estimated band misses, an exact radix select over the 32-bit keys runs (4 more passes).
#pragma once
#include "common.cuh"
#include "../../include/colinfer_b200.h"

namespace strm {

#ifdef COLINFER_PROFILE
#define FK_PROF_PARAMS , long long& prof_last, bool prof_on
#define FK_PROF_ARGS , prof_last, a.prof != nullptr
#define FK_PROF(slot) do { if (prof_on && threadIdx.x == 0) { const long long t_ = clock64(); sc->prof[slot] += t_ - prof_last; prof_last = t_; } } while (0)
#define ST_PROF(slot) do { if (a.prof && tid == 0) { const long long t_ = clock64(); sc->prof[slot] += t_ - prof_last; prof_last = t_; } } while (0)
#else
#define FK_PROF_PARAMS
#define FK_PROF_ARGS
#define FK_PROF(slot) do { } while (0)
#define ST_PROF(slot) do { } while (0)
#endif

constexpr int NT = 1024;             // threads per CTA
constexpr int CTAS_PER_SM = 1;       // (two CTAs of 512 threads per SM are slower: rows split unevenly over them and each keeps half the loads in flight)
constexpr int NW = NT / 32;
constexpr int NWA = 32;              // per-warp exchange arrays are sized (and reduced) for a full warp of warps
constexpr int NB1 = 8192;            // fine buckets over the distance from the row maximum (or from the sample's)
constexpr int HOFF = 4096;           // buckets kept above the sample's maximum when the histogram is built in pass 1
constexpr float RANGE = 50.0f;       // they cover distances up to RANGE * temperature (RANGE / 2 above a sample's maximum)
constexpr int FASTK = 100;           // largest top_k finished from the group-maxima bound
constexpr int BINS = 512;            // bins of the sample histogram and of the exact list selection
constexpr int BINS_PAD = BINS + BINS / 16;   // the count histograms keep one spare word per sixteen bins: a lane that reads its
                                              // sixteen consecutive bins then hits a bank of its own
__host__ __device__ __forceinline__ int padbin(int i) { return i + (i >> 4); }
constexpr float FAST_SCALE = 32.0f;  // sample-histogram bins per unit logit (16 units below the sample's maximum)
constexpr float FIN_SCALE = 64.0f;   // list-selection bins per unit logit (8 units below the maximum)
constexpr int WLIST = 2048 / (NT / 32);  // list entries per warp
constexpr int FCAP = 128;            // candidates of the one-warp finish
constexpr int GLIST = 1365;          // gathered list entries
constexpr int FIN_CAND = 64;         // entries of one bin compared pairwise
constexpr int FB_NB = 256;           // radix buckets per level of the fallback select
constexpr int PEN_TABLE = 2048;      // distinct history ids with an O(1) count
constexpr int XSTEPS = 128;           // 128-logit steps of one warp's region, at most (vocabularies up to 32 x 128 x 128)
constexpr int BAL_ROWS = 16384;      // launches up to this many rows deal their rows to the CTAs by cost class
constexpr int BAL_MINE = BAL_ROWS / 128 + 8;   // rows of one CTA then (the grid has at least 128 CTAs, or one row each)
#define ST_FLT_MAX 3.402823466e38f
#define ST_POS_INF (__int_as_float(0x7f800000))

struct Args {
    const void* logits; int dtype; int vec;
    const int32_t* mask; int mask_rows; int W;
    colinfer_sampler_params p;
    const void* pos; int pos_i64; const float* u;
    int64_t* out; colinfer_row_stats* stats; int32_t* status;
    int B, R, V; int flags;
    long long* prof; int prof_slots;   // optional cycles per phase (profiling hook)
};

template <bool B> struct BoolTag { static constexpr bool value = B; };
struct Cand { uint32_t idx; float l; };
struct Entry { uint32_t idx; float l; uint32_t q; };

struct Sc {
    u64 wsum[NWA], woff[NWA], wtotal;
    u64 wmass[NWA];
    float wf[NWA]; int wi[NWA];
    int found; u64 found_excl;
    int ncand; float cand_l[FIN_CAND]; u64 cand_w[FIN_CAND]; float res_f; int sel_ok;
    uint32_t cand_kmin, cand_kmax; // ordered keys: extremes of the pivot bin's entries (a crowded bin of equal logits)
    int hist_slow, overflow;
    int wcount[NWA], woffs[NWA + 1];
    u64 g_all[NWA], g_keep[NWA], g_tot_all, g_tot_keep;   // sums that ride on gather_lists
    float bc_f; int bc_i;
    float wtw[NWA], wmin[NWA];     // running top-k: each warp's threshold and smallest list entry
    int fin_ok;
    uint32_t fc_idx[FCAP]; float fc_l[FCAP];
    float fin_cut; u64 fin_total; int fin_token;
    long long prof[16];            // profiling hook: cycles per phase, summed over the CTA's rows
    int my_rows[BAL_MINE]; int my_count;
    u64 wsum2[NWA], woff2[NWA], wtotal2; int fb[3]; u64 fe[3];   // second scan and the three finds of fine_decide
    int x_warp; u64 x_off; u64 step_sum[XSTEPS];   // the draw's region, walked by all warps
    int glist_n;
};

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }

// Exclusive prefix of one value per thread (thread order) and the total.  Two __syncthreads.
__device__ __forceinline__ u64 block_excl_scan(u64 v, Sc* sc, u64& total) {
    const int lane = lane_id(), warp = warp_id();
    const u64 incl = warp_incl_scan_u64(v, lane);
    if (lane == 31) sc->wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const u64 w = sc->wsum[lane];
        const u64 wi = warp_incl_scan_u64(w, lane);
        sc->woff[lane] = wi - w;
        if (lane == 31) sc->wtotal = wi;
        if (lane == 0) sc->found = -1;
    }
    __syncthreads();
    total = sc->wtotal;
    return sc->woff[warp] + incl - v;
}

// Where the running sum of get(0..nbins-1) first reaches target: bin (-1 if never, or target 0), sum before it, total.
// Three __syncthreads.  All threads call.
template <class F>
__device__ void bins_find(F get, int nbins, u64 target, Sc* sc, int& bin, u64& before, u64& total) {
    const int per = (nbins + NT - 1) / NT;
    const int lo = min(threadIdx.x * per, nbins), hi = min(lo + per, nbins);
    u64 s = 0;
    for (int i = lo; i < hi; ++i) s += (u64)get(i);
    const u64 excl = block_excl_scan(s, sc, total);
    if (excl < target && target <= excl + s) {
        u64 run = excl;
        for (int i = lo; i < hi; ++i) {
            const u64 b = (u64)get(i);
            if (run + b >= target) { sc->found = i; sc->found_excl = run; break; }
            run += b;
        }
    }
    __syncthreads();
    bin = sc->found;
    before = sc->found_excl;
}

// Fine bucket of a logit: floor((href - x) * sc) + hoff clamped to [0, NB1), computed as a rounding float add (no
// conversion instruction: that pipe is the exponentials').  A logit exactly on an edge may land in either neighbour;
// every user keeps a whole bucket of margin.  One function for counting, corrections and thresholds.
__device__ __forceinline__ int fine_bucket(float x, float href, float sc1, float hoff_minus_half) {
    const float t = fminf(fmaxf(fmaf(href - x, sc1, hoff_minus_half), 0.0f), (float)(NB1 - 1));
    return __float_as_int(t + 8388608.0f) - 0x4B000000;
}

__device__ __forceinline__ u64 ceil_target(float frac, u64 total) {
    const double t = ceil((double)frac * (double)total);
    u64 q = t <= 1.0 ? 1ull : (u64)t;
    return q > total ? total : q;
}

// One pass over the fine histogram for everything the path decision needs: the bucket of the kk-th largest count, the
// bucket where the running count reaches cap, and the bucket where the running estimated mass reaches topp of its
// total.  Two prefix scans share the two block barriers.  Buckets beyond `last` count nothing.
struct FineDecision { int b_k; u64 before_k; u64 total_cnt; int b_cap; int b_p; u64 est_total; };
template <class W>
__device__ FineDecision fine_decide(const uint32_t* hist, W west, int last, u64 kk_target, u64 cap_target, float topp, bool want_p, Sc* sc) {
    constexpr int PER = NB1 / NT;
    const int lane = lane_id(), warp = warp_id();
    const int lo = threadIdx.x * PER;
    uint32_t c[PER];
#pragma unroll
    for (int t = 0; t < PER; t += 4) {
        const uint4 x = *reinterpret_cast<const uint4*>(hist + lo + t);
        c[t] = x.x; c[t + 1] = x.y; c[t + 2] = x.z; c[t + 3] = x.w;
    }
    u64 sc_c = 0, sc_e = 0;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
        if (lo + t <= last && c[t]) { sc_c += c[t]; if (want_p) sc_e += (u64)c[t] * west(lo + t); } else c[t] = 0;
    }
    const u64 in_c = warp_incl_scan_u64(sc_c, lane), in_e = warp_incl_scan_u64(sc_e, lane);
    if (lane == 31) { sc->wsum[warp] = in_c; sc->wsum2[warp] = in_e; }
    __syncthreads();
    if (warp == 0) {
        const u64 w1 = sc->wsum[lane], w2 = sc->wsum2[lane];
        const u64 i1 = warp_incl_scan_u64(w1, lane), i2 = warp_incl_scan_u64(w2, lane);
        sc->woff[lane] = i1 - w1; sc->woff2[lane] = i2 - w2;
        if (lane == 31) { sc->wtotal = i1; sc->wtotal2 = i2; }
        if (lane < 3) sc->fb[lane] = -1;
    }
    __syncthreads();
    FineDecision o;
    o.total_cnt = sc->wtotal; o.est_total = sc->wtotal2;
    const u64 ex_c = sc->woff[warp] + in_c - sc_c, ex_e = sc->woff2[warp] + in_e - sc_e;
    const u64 t_p = (want_p && o.est_total > 0) ? ceil_target(topp, o.est_total) : 0ull;
    if (kk_target && ex_c < kk_target && kk_target <= ex_c + sc_c) {
        u64 run = ex_c;
#pragma unroll
        for (int t = 0; t < PER; ++t) { if (run + c[t] >= kk_target) { sc->fb[0] = lo + t; sc->fe[0] = run; break; } run += c[t]; }
    }
    if (cap_target && ex_c < cap_target && cap_target <= ex_c + sc_c) {
        u64 run = ex_c;
#pragma unroll
        for (int t = 0; t < PER; ++t) { if (run + c[t] >= cap_target) { sc->fb[1] = lo + t; break; } run += c[t]; }
    }
    if (t_p && ex_e < t_p && t_p <= ex_e + sc_e) {
        u64 run = ex_e;
#pragma unroll
        for (int t = 0; t < PER; ++t) {
            const u64 b = c[t] ? (u64)c[t] * west(lo + t) : 0ull;
            if (run + b >= t_p) { sc->fb[2] = lo + t; break; }
            run += b;
        }
    }
    __syncthreads();
    o.b_k = sc->fb[0]; o.before_k = sc->fe[0]; o.b_cap = sc->fb[1]; o.b_p = sc->fb[2];
    return o;
}

__device__ __forceinline__ float row_uniform(const Args& a, int row, int b, int r) {
    if (a.u != nullptr) return a.u[row];
    if (a.pos != nullptr && a.p.seed != nullptr) {
        const long long p0 = a.pos_i64 ? reinterpret_cast<const long long*>(a.pos)[b]
                                       : (long long)reinterpret_cast<const int*>(a.pos)[b];
        return u32_to_uniform(philox_word(philox_key(a.p.seed[b]), (u64)p0 + (u64)r));
    }
    return 1.0f;
}


// Exact weighted selection among n list entries: the value v with W(l > v) < target <= W(l >= v).  BINS linear bins over
// (base - l) * scale, then the pivot bin's entries pairwise.  False when the pivot leaves the binned range or its bin
// is too crowded.  All threads call with the same arguments.
template <class GL, class W>
__device__ bool lean_select(GL getl, W wt, int n, float base, float scale, u64 target, u64* bins, Sc* sc, float& value) {
    const int tid = threadIdx.x;
    for (int i = tid; i < BINS; i += NT) bins[i] = 0;
    if (tid == 0) { sc->ncand = 0; sc->sel_ok = 0; sc->cand_kmin = 0xFFFFFFFFu; sc->cand_kmax = 0u; }
    __syncthreads();
    for (int i = tid; i < n; i += NT) {
        const u64 w = wt(i);
        if (w) atomicAdd(&bins[max(0, min(BINS - 1, __float2int_rz((base - getl(i)) * scale)))], w);
    }
    __syncthreads();
    int b_star; u64 before, total;
    bins_find([&](int i) { return bins[i]; }, BINS, target, sc, b_star, before, total);
    if (b_star < 0 || b_star >= BINS - 1) return false;
    for (int i = tid; i < n; i += NT) {
        const u64 w = wt(i);
        if (w && max(0, min(BINS - 1, __float2int_rz((base - getl(i)) * scale))) == b_star) {
            const int slot = atomicAdd(&sc->ncand, 1);
            if (slot < FIN_CAND) { sc->cand_l[slot] = getl(i); sc->cand_w[slot] = w; }
            else { const uint32_t k = f2key(getl(i)); atomicMin(&sc->cand_kmin, k); atomicMax(&sc->cand_kmax, k); }
        }
    }
    __syncthreads();
    const int nc = sc->ncand;
    if (nc > FIN_CAND) {
        // A crowded pivot bin.  When all of its entries are one value (bf16 logits: a hundred tokens share every value)
        // that value is the pivot: the weight above the bin is below the target, with the bin it reaches it.
        uint32_t kmin = sc->cand_kmin, kmax = sc->cand_kmax;
        for (int i = 0; i < FIN_CAND; ++i) { const uint32_t k = f2key(sc->cand_l[i]); kmin = min(kmin, k); kmax = max(kmax, k); }
        if (kmin != kmax) return false;
        value = key2f(kmin);
        return true;
    }
    if (tid < nc) {
        const float mine = sc->cand_l[tid];
        u64 gt = 0, eq = 0;
        for (int i = 0; i < nc; ++i) {
            const float o = sc->cand_l[i];
            if (o > mine) gt += sc->cand_w[i]; else if (o == mine) eq += sc->cand_w[i];
        }
        if (before + gt < target && target <= before + gt + eq) { sc->res_f = mine; sc->sel_ok = 1; }
    }
    __syncthreads();
    value = sc->res_f;
    return sc->sel_ok != 0;
}


// How long a row's lines should stay in L2: rows that are read twice (the wide ones: a pass for the histogram, a pass for
// the exact masses) ask to be evicted last on their first pass and first on their second; rows read once ask to be evicted
// first, so that the 126 MB keep the ~ 50 wide rows in flight (30 MB) instead of the last 90 MB streamed.
__device__ __forceinline__ unsigned long long l2_policy_keep() {
    unsigned long long p;
    asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ unsigned long long l2_policy_stream() {
    unsigned long long p;
    asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// One row as the passes see it: effective logits (penalties, then mask), four at a time.
struct Row {
    const float* p32; const __nv_bfloat16* p16; int V; bool vec, vec16;   // 128-bit fp32 loads / 64-bit bf16 loads of four logits
    unsigned long long pol;            // L2 eviction policy of the row's loads (l2_policy_keep / l2_policy_stream)
    const int32_t* mrow;
    bool has_pen; const uint32_t* pen_bits; const uint32_t* pen_prefix; const float* pen_val;
    bool pen_inline;                   // the passes apply the penalties element by element (else: raw logits, lists patched afterwards)
    const int32_t* hist; int hlen; float rp, pp, fp; int* hist_slow;

    // penalised value of a token beyond the table: count its occurrences by scanning the history
    __device__ float slow_penalty(float l, int tok) const {
        int cnt = 0;
        *hist_slow = 1;
        for (int h = 0; h < hlen; ++h) cnt += (hist[h] == tok);
        return apply_penalty(l, cnt, rp, pp, fp);
    }
    __device__ __forceinline__ float raw(int t) const { return p16 ? __bfloat162float(p16[t]) : __ldg(p32 + t); }

    // elements i .. i+3 (i a multiple of 4) as stored; positions >= V read as -inf.  A pure load: the passes issue
    // several of these before touching the values, so that their latencies overlap.
    __device__ __forceinline__ float4 raw4(int i) const {
        float4 v;
        if (vec) {
            if (i < V) asm("ld.global.cg.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
                           : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p32 + i), "l"(pol));
            else v = make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
        } else if (vec16) {
            if (i < V) {
                uint2 u;                                                            // four bf16: a float's upper halves
                asm("ld.global.cg.L2::cache_hint.v2.u32 {%0, %1}, [%2], %3;" : "=r"(u.x), "=r"(u.y) : "l"(p16 + i), "l"(pol));
                v = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u),
                                __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xFFFF0000u));
            } else {
                v = make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
            }
        } else {
            float e[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int t = i + j;
                e[j] = t < V ? (p16 ? __bfloat162float(p16[t]) : __ldg(p32 + t)) : CI_NEG_INF;
            }
            v = make_float4(e[0], e[1], e[2], e[3]);
        }
        return v;
    }
    __device__ __forceinline__ float4 load4(int i) const { return fix4(raw4(i), i, V); }
    __device__ __forceinline__ float4 fix4(float4 v, int i, int lim) const {
        return pen_inline ? fix4t<true>(v, i, lim) : fix4t<false>(v, i, lim);
    }
    // the effective logits of a loaded group: penalties, then mask.  Groups at or beyond lim (the end of the caller's
    // region; at most V) keep the caller's filler values.
    // PI: the row's penalties are applied here, element by element (the hot loops are compiled once for each case)
    template <bool PI>
    __device__ __forceinline__ float4 fix4t(float4 v, int i, int lim) const {
        if (PI && i < lim) {
            // the few penalised logits of the row were computed once (pen_val, by rank of the token in the history bitmap)
            const uint32_t word = pen_bits[i >> 5];
            const uint32_t nib = (word >> (i & 31)) & 0xFu;
            if (nib) {
                uint32_t rk = pen_prefix[i >> 5] + __popc(word & ((1u << (i & 31)) - 1u));
                if (nib & 1u) { if (rk < PEN_TABLE) v.x = pen_val[rk]; else v.x = slow_penalty(v.x, i); ++rk; }
                if (nib & 2u) { if (rk < PEN_TABLE) v.y = pen_val[rk]; else v.y = slow_penalty(v.y, i + 1); ++rk; }
                if (nib & 4u) { if (rk < PEN_TABLE) v.z = pen_val[rk]; else v.z = slow_penalty(v.z, i + 2); ++rk; }
                if (nib & 8u) { if (rk < PEN_TABLE) v.w = pen_val[rk]; else v.w = slow_penalty(v.w, i + 3); }
            }
        }
        if (mrow != nullptr && i < lim) {
            const uint32_t bits = ((uint32_t)__ldg(mrow + (i >> 5)) >> (i & 31)) & 0xFu;
            if (bits != 0xFu) {
                if (!(bits & 1u)) v.x = CI_NEG_INF;
                if (!(bits & 2u)) v.y = CI_NEG_INF;
                if (!(bits & 4u)) v.z = CI_NEG_INF;
                if (!(bits & 8u)) v.w = CI_NEG_INF;
            }
        }
        return v;
    }
};

// Pass 1 of rows that list nothing: maximum of the warp's region and the float4 group it was first seen in.  Its own
// function (and register allocation): the loop must keep four 128-bit loads per thread in flight.
static __device__ __noinline__ float2 pass1_lean(const Row rw, int r_lo, int r_hi, int lane) {
    float lmax = CI_NEG_INF;
    int lpos = -1;
    for (int i0 = r_lo; i0 < r_hi; i0 += 512) {
        float4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * 128 + lane * 4;
            v[k] = i < r_hi ? rw.raw4(i) : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = rw.fix4(v[k], i0 + k * 128 + lane * 4, r_hi);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float m4 = fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w));
            const bool up = m4 > lmax;                           // strict: the first (lowest) position of the maximum stays
            lmax = up ? m4 : lmax;
            lpos = up ? i0 + k * 128 + lane * 4 : lpos;
        }
    }
    return make_float2(lmax, __int_as_float(lpos));
}

// Appends the components of one float4 group selected by mk to the warp's list, in token order (lane, component).
template <int CAP = WLIST>
__device__ __forceinline__ void warp_append(Cand* mylist, int& wn, unsigned mk, const float* e4, uint32_t idx0, int lane) {
    const unsigned b0 = __ballot_sync(0xffffffffu, mk & 1u), b1 = __ballot_sync(0xffffffffu, mk & 2u);
    const unsigned b2 = __ballot_sync(0xffffffffu, mk & 4u), b3 = __ballot_sync(0xffffffffu, mk & 8u);
    if (!(b0 | b1 | b2 | b3)) return;
    const unsigned lt = (1u << lane) - 1u;
    int at = wn + __popc(b0 & lt) + __popc(b1 & lt) + __popc(b2 & lt) + __popc(b3 & lt);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (mk & (1u << j)) {
            if (at < CAP) { mylist[at].idx = idx0 + j; mylist[at].l = e4[j]; }
            ++at;
        }
    }
    wn += __popc(b0) + __popc(b1) + __popc(b2) + __popc(b3);
}

// Removes the entries of penalised tokens from a warp's list (token order kept); an overflowed list stays overflowed.
__device__ __forceinline__ int warp_drop_penalised(Cand* mylist, int wn, const uint32_t* pen_bits, int lane) {
    if (wn > WLIST) return wn;
    const unsigned lt = (1u << lane) - 1u;
    int out = 0;
    for (int j0 = 0; j0 < wn; j0 += 32) {
        const int j = j0 + lane;
        Cand c; c.idx = 0; c.l = 0.0f;
        bool keep = false;
        if (j < wn) { c = mylist[j]; keep = !((pen_bits[c.idx >> 5] >> (c.idx & 31)) & 1u); }
        const unsigned bal = __ballot_sync(0xffffffffu, keep);
        __syncwarp();
        if (keep) mylist[out + __popc(bal & lt)] = c;
        out += __popc(bal);
    }
    __syncwarp();
    return out;
}

// Concatenates the warps' lists (token order) into glist with masses; returns n, or -1 on overflow.  All threads call.
// wall / wkeep (one value per warp; s1 / s_above: their sums over the warps) ride on the same two barriers when given.
static __device__ int gather_lists(const Cand* ownlist, int wn, Entry* glist, const MassFn& mass, Sc* sc, u64 wall = 0, u64 wkeep = 0,
                                   u64* s1 = nullptr, u64* s_above = nullptr) {
    const int lane = lane_id(), warp = warp_id();
    if (lane == 0) { sc->wcount[warp] = wn; sc->g_all[warp] = wall; sc->g_keep[warp] = wkeep; }
    __syncthreads();
    if (warp == 0) {
        const u64 ta = warp_sum_u64(lane < NW ? sc->g_all[lane] : 0ull), tk = warp_sum_u64(lane < NW ? sc->g_keep[lane] : 0ull);
        if (lane == 0) { sc->g_tot_all = ta; sc->g_tot_keep = tk; }
        const int c = sc->wcount[lane];
        int incl = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
        sc->woffs[lane] = incl - c;
        if (lane == 31) sc->woffs[NWA] = incl;
        const unsigned over = __ballot_sync(0xffffffffu, c > WLIST);
        if (lane == 0) sc->overflow = over != 0u;
    }
    __syncthreads();
    if (s1) *s1 = sc->g_tot_all;
    if (s_above) *s_above = sc->g_tot_keep;
    const int n = sc->woffs[NWA];
    if (sc->overflow || n > GLIST) return -1;
    const int off = sc->woffs[warp];
    const Cand* src = ownlist + warp * WLIST;
    for (int j = lane; j < wn; j += 32) {
        Entry en;
        en.idx = src[j].idx; en.l = src[j].l; en.q = mass(src[j].l);
        glist[off + j] = en;
    }
    __syncthreads();
    return n;
}


// Appends the selected components (mk[k], bit j) of a batch of four float4 groups to the warp's list in token order
// (group, lane, component).  One packed shuffle scan gives every group's offsets.  The caller guarantees room.
template <int CAP>
__device__ __forceinline__ void warp_append_batch(Cand* mylist, int& wn, const unsigned (&mk)[4], const float4 (&v)[4], uint32_t idx0, int lane,
                                                  unsigned packed_incl, unsigned packed_cnt) {
    const unsigned tot = __shfl_sync(0xffffffffu, packed_incl, 31);
    const unsigned excl = packed_incl - packed_cnt;
    int base = wn;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (mk[k]) {
            int at = base + (int)((excl >> (8 * k)) & 0xFFu);
            const float e4[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (mk[k] & (1u << j)) {
                    if (at < CAP) { mylist[at].idx = idx0 + k * 128 + j; mylist[at].l = e4[j]; }
                    ++at;
                }
            }
        }
        base += (int)((tot >> (8 * k)) & 0xFFu);
    }
    wn = base;
}

// Bin of a BINS-bin count histogram in which the running count reaches kk, or -1; computed by the calling warp alone
// (every warp of the block gets the same answer, so no broadcast and no barrier follow).  `run`: count down to and
// including that bin.
__device__ __forceinline__ int warp_count_bin(const uint32_t* hist, uint32_t kk, int lane, uint32_t& run_out) {
    constexpr int PERB = BINS / 32;
    static_assert(PERB == 16, "padbin() pads after every sixteenth bin");
    uint32_t h[PERB]; uint32_t s = 0;
#pragma unroll
    for (int t = 0; t < PERB; ++t) { h[t] = hist[lane * (PERB + 1) + t]; s += h[t]; }
    uint32_t incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint32_t x = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += x; }
    const uint32_t all = __shfl_sync(0xffffffffu, incl, 31);
    if (all < kk) { run_out = all; return -1; }
    const unsigned hit = __ballot_sync(0xffffffffu, incl >= kk);
    const int hl = __ffs(hit) - 1;
    uint32_t run = incl - s; int b = lane * PERB;
#pragma unroll
    for (int t = 0; t < PERB; ++t) { if (run + h[t] >= kk) { b = lane * PERB + t; run += h[t]; break; } run += h[t]; }
    run_out = __shfl_sync(0xffffffffu, run, hl);
    return __shfl_sync(0xffffffffu, b, hl);
}

// Sorts 128 ordered keys held four per lane (element lane * 4 + t) into descending order across the warp: a bitonic
// network of 28 compare-exchange stages, the wide ones by shuffle.
__device__ __forceinline__ void warp_sort_desc4(uint32_t (&a)[4], int lane) {
#pragma unroll
    for (int k = 2; k <= 128; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            uint32_t b[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int i = lane * 4 + t;
                const uint32_t o = j >= 4 ? __shfl_xor_sync(0xffffffffu, a[t], j >> 2) : a[t ^ (j & 3)];
                const bool take_max = ((i & j) == 0) == ((i & k) == 0);
                b[t] = take_max ? max(a[t], o) : min(a[t], o);
            }
#pragma unroll
            for (int t = 0; t < 4; ++t) a[t] = b[t];
        }
    }
}

// Top-k (kk <= FASTK), then top-p and the draw, from the warps' running lists after the single pass over the row.
// The union of the lists holds every logit >= lo (lo: the largest warp threshold; the smallest listed value when no
// warp compacted).  BINS linear bins over [lo, L] find the bin of the kk-th largest; the entries down to that bin, at
// most FCAP and in token order, go to warp 0, which finishes exactly by bisection on the ordered keys.
// False: the caller takes the general path.  All threads call.
static __device__ bool finish_running_topk(const Cand* ownlist, int wn, float lo, float L, float lcut_in, float tc, const MassFn& mass,
                                    int kk, bool need_topp, float topp, float u, uint32_t* hist, Sc* sc,
                                    long long& token, float& lcut, u64& total FK_PROF_PARAMS) {
    const int tid = threadIdx.x, lane = lane_id(), warp = warp_id();
    const Cand* mine = ownlist + warp * WLIST;
    const float bound = lo;
    lo = fmaxf(lo, lcut_in);                                         // nothing below the min-p cut / the mass horizon matters
    if (!(lo <= L)) return false;
    const float scale = L > lo ? (float)(BINS - 2) / (L - lo) : 0.0f;
    auto bin_of = [&](float l) { return min(BINS - 1, __float2int_rz((L - l) * scale)); };
    for (int j = lane; j < wn; j += 32) { const float l = mine[j].l; if (l >= lo) atomicAdd(&hist[padbin(bin_of(l))], 1u); }
    if (tid == 0) sc->fin_ok = 0;
    __syncthreads();
    FK_PROF(8);
    uint32_t run_b;
    int bstar = warp_count_bin(hist, (uint32_t)kk, lane, run_b);     // every warp scans the bins itself
    bool complete;
    if (bstar < 0) {
        // fewer than kk listed logits reach lo.  If lo is the sample's bound, the bound did not hold; if it is the cut,
        // fewer than kk logits survive it and top-k removes nothing: all survivors are candidates
        if (!(lo > bound) || run_b == 0) return false;
        bstar = BINS - 1;
        complete = true;
    } else {
        // every row element in bins <= bstar is a candidate while bstar stays clear of the bins around lo
        complete = bstar <= BINS - 4;
    }
    const int nc = (int)run_b;                                       // entries down to and including bin bstar
    if (nc > FCAP) return false;
    // candidates in token order: warps in order, entries in list order
    {
        int cnt = 0;
        for (int j0 = 0; j0 < wn; j0 += 32) {
            const int j = j0 + lane;
            const bool is = j < wn && mine[j].l >= lo && bin_of(mine[j].l) <= bstar;
            cnt += __popc(__ballot_sync(0xffffffffu, is));
        }
        if (lane == 0) sc->wcount[warp] = cnt;
        __syncthreads();
        FK_PROF(9);
        int off = 0;
        for (int w2 = 0; w2 < warp; ++w2) off += sc->wcount[w2];
        const unsigned lt = (1u << lane) - 1u;
        for (int j0 = 0; j0 < wn; j0 += 32) {
            const int j = j0 + lane;
            const bool is = j < wn && mine[j].l >= lo && bin_of(mine[j].l) <= bstar;
            const unsigned bal = __ballot_sync(0xffffffffu, is);
            if (is) { const int at = off + __popc(bal & lt); if (at < FCAP) { sc->fc_idx[at] = mine[j].idx; sc->fc_l[at] = mine[j].l; } }
            off += __popc(bal);
        }
    }
    __syncthreads();
    FK_PROF(5);
    if (warp == 0) {
        constexpr int PERC = FCAP / 32;
        float l[PERC]; uint32_t key[PERC], q[PERC];
        static_assert(PERC == 4, "the warp sort holds four keys per lane");
        int surv = 0;
#pragma unroll
        for (int t = 0; t < PERC; ++t) {
            const int e = lane * PERC + t;
            l[t] = e < nc ? sc->fc_l[e] : CI_NEG_INF;
            key[t] = e < nc ? f2key(l[t]) : 0u;
            surv += (e < nc && l[t] >= lcut_in) ? 1 : 0;
        }
        surv = (int)__reduce_add_sync(0xffffffffu, (unsigned)surv);
        // the candidates' keys in descending order (absent entries, key 0, come last): the kk-th largest is read off,
        // the top-p pivot is where the running mass of the sorted candidates reaches its target
        uint32_t sk[PERC];
#pragma unroll
        for (int t = 0; t < PERC; ++t) sk[t] = key[t];
        warp_sort_desc4(sk, lane);
        auto sorted_at = [&](int pos) {                              // key at sorted position pos (warp-uniform pos)
            const int t = pos & 3;
            const uint32_t mine = t == 0 ? sk[0] : t == 1 ? sk[1] : t == 2 ? sk[2] : sk[3];
            return __shfl_sync(0xffffffffu, mine, pos >> 2);
        };
        float cut = lcut_in;
        bool ok = surv > 0;
        if (ok && kk <= surv) {                                      // else fewer than k survive min-p: top-k removes nothing
            const float lk = key2f(sorted_at(kk - 1));
            const float ck = lower_logit_for(scale_logit(lk, tc), tc, lk);
            ok = complete && ck >= lo && bin_of(ck) <= bstar;        // else a tie partner could lie outside the candidates
            cut = fmaxf(cut, ck);
        } else {
            ok = ok && complete;                                     // every logit >= the min-p cut is a candidate
        }
        FK_PROF(10);
#pragma unroll
        for (int t = 0; t < PERC; ++t) q[t] = l[t] >= cut ? mass(l[t]) : 0u;
        if (ok && need_topp) {
            // masses of the sorted candidates (the same function of the same logits), their running sum in sorted order
            u64 sq[PERC], s = 0;
#pragma unroll
            for (int t = 0; t < PERC; ++t) {
                const float sl = sk[t] ? key2f(sk[t]) : CI_NEG_INF;
                sq[t] = sl >= cut ? (u64)mass(sl) : 0ull;
                s += sq[t];
            }
            const u64 incl = warp_incl_scan_u64(s, lane);
            const u64 s1 = __shfl_sync(0xffffffffu, incl, 31);
            ok = s1 > 0;
            const u64 target = ceil_target(topp, s1);
            const unsigned hit = __ballot_sync(0xffffffffu, incl >= target);
            int pos = 0;
            if (hit) {
                const int hl = __ffs(hit) - 1;
                u64 run = incl - s; int tt = 0;
#pragma unroll
                for (int t = 0; t < PERC; ++t) { run += sq[t]; if (run >= target) { tt = t; break; } }
                pos = hl * PERC + __shfl_sync(0xffffffffu, tt, hl);
            }
            const float lp = key2f(sorted_at(pos));
            if (ok) cut = fmaxf(cut, lower_logit_for(scale_logit(lp, tc), tc, lp));
#pragma unroll
            for (int t = 0; t < PERC; ++t) q[t] = l[t] >= cut ? q[t] : 0u;
        }
        FK_PROF(11);
        u64 s = 0;
#pragma unroll
        for (int t = 0; t < PERC; ++t) s += q[t];
        const u64 incl = warp_incl_scan_u64(s, lane);
        const u64 tot = __shfl_sync(0xffffffffu, incl, 31);
        ok = ok && tot > 0;
        const u64 target = ceil_target(u, tot);
        const unsigned hit = __ballot_sync(0xffffffffu, incl >= target);
        if (ok && lane == __ffs(hit) - 1) {
            u64 run = incl - s; int e = lane * PERC;
#pragma unroll
            for (int t = 0; t < PERC; ++t) { run += q[t]; if (run >= target) { e = lane * PERC + t; break; } }
            sc->fin_token = (int)sc->fc_idx[e]; sc->fin_cut = cut; sc->fin_total = tot; sc->fin_ok = 1;
        }
    }
    __syncthreads();
    FK_PROF(6);
    if (!sc->fin_ok) return false;
    token = sc->fin_token; lcut = sc->fin_cut; total = sc->fin_total;
    return true;
}

}  // namespace strm

namespace strm {

// Top-k, top-p and the draw on a gathered list that holds every logit >= tl of the row (tl below the top-k pivot;
// -inf when the list is known to contain the row's whole top k).  False: the caller takes another path.
static __device__ bool finish_on_list(const Entry* gl, int n, float tl, float lcut_in, float tc, float L, bool use_topk, int kk,
                               bool need_topp, float topp, float u, u64* bins, Sc* sc, long long& token, float& lcut, u64& total) {
    const int tid = threadIdx.x;
    float cut = lcut_in;
    const float span = (tl > -1e30f) ? fmaxf(L - tl, 1e-30f) : 0.0f;
    const float scale = span > 0.0f ? (float)(BINS - 2) / span : FIN_SCALE;
    auto getl = [&](int i) { return gl[i].l; };
    u64 cnt = 0;
    for (int i = tid; i < n; i += NT) cnt += gl[i].l >= cut ? 1 : 0;
    u64 survivors;
    block_excl_scan(cnt, sc, survivors);
    if (survivors == 0) return false;
    if (use_topk && (u64)kk <= survivors) {                    // else fewer than k survive min-p: top-k removes nothing
        float lk;
        const float c0 = cut;
        if (!lean_select(getl, [&](int i) { return (u64)(gl[i].l >= c0 ? 1 : 0); }, n, L, scale, (u64)kk, bins, sc, lk)) return false;
        cut = fmaxf(cut, lower_logit_for(scale_logit(lk, tc), tc, lk));
        if (cut < tl) return false;                            // a tie partner could lie outside the list
    }
    if (need_topp) {
        const float c0 = cut;
        u64 part = 0;
        for (int i = tid; i < n; i += NT) part += gl[i].l >= c0 ? (u64)gl[i].q : 0ull;
        u64 s1;
        block_excl_scan(part, sc, s1);
        if (s1 == 0) return false;
        float lp;
        if (!lean_select(getl, [&](int i) { return gl[i].l >= c0 ? (u64)gl[i].q : 0ull; }, n, L, scale, ceil_target(topp, s1), bins, sc, lp))
            return false;
        cut = fmaxf(cut, lower_logit_for(scale_logit(lp, tc), tc, lp));
        if (cut < tl) return false;
    }
    // the draw: first entry (token order) whose running kept mass reaches u * total
    const int ept = (n + NT - 1) / NT;
    const int e_lo = tid * ept, e_hi = min(e_lo + ept, n);
    u64 mine = 0;
    for (int i = e_lo; i < e_hi; ++i) mine += gl[i].l >= cut ? (u64)gl[i].q : 0ull;
    const u64 excl = block_excl_scan(mine, sc, total);
    if (total == 0) return false;
    const u64 target = ceil_target(u, total);
    if (tid == 0) sc->bc_i = -1;
    __syncthreads();
    if (excl < target && target <= excl + mine) {
        u64 run = excl;
        for (int i = e_lo; i < e_hi; ++i) {
            run += gl[i].l >= cut ? (u64)gl[i].q : 0ull;
            if (run >= target) { sc->bc_i = (int)gl[i].idx; break; }
        }
    }
    __syncthreads();
    token = sc->bc_i;
    lcut = cut;
    return token >= 0;
}

// Exact radix select over the order-preserving keys of the effective logits >= lcut (four 8-bit levels, one streaming
// pass each).  by_mass: the top-p pivot; else the kk-th largest.  False when the filter removes nothing.
static __device__ bool radix_select(const Row& rw, int r_lo, int r_hi, const MassFn& mass, float lcut, bool by_mass, u64 kk, float topp,
                             u64* fb_hist, Sc* sc, float& pivot) {
    const int tid = threadIdx.x, lane = lane_id();
    const float lk = fmaxf(lcut, -ST_FLT_MAX);
    uint32_t prefix = 0;
    u64 target = by_mass ? 0 : kk;
    for (int lvl = 0; lvl < 4; ++lvl) {
        const int shift = 24 - 8 * lvl;
        for (int i = tid; i < FB_NB; i += NT) fb_hist[i] = 0;
        __syncthreads();
        for (int i0 = r_lo; i0 < r_hi; i0 += 128) {
            const float4 v = rw.load4(i0 + lane * 4);
            const float e4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float l = e4[j];
                int bin = -1;
                if (l >= lk) {
                    const uint32_t key = f2key(l);
                    if (lvl == 0 || (key >> (shift + 8)) == prefix) bin = FB_NB - 1 - (int)((key >> shift) & 0xFFu);
                }
                // lanes of one bin add once (most keys of a level share a few bins: plain atomics would serialise)
                const unsigned peers = __match_any_sync(0xffffffffu, bin);
                const uint32_t w = bin < 0 ? 0u : (by_mass ? mass(l) : 1u);
                const uint32_t lo = __reduce_add_sync(peers, w & 0xFFFFu), hi = __reduce_add_sync(peers, w >> 16);
                if (bin >= 0 && lane == __ffs(peers) - 1) atomicAdd(&fb_hist[bin], ((u64)hi << 16) + lo);
            }
        }
        __syncthreads();
        int b_star; u64 before, grand;
        if (lvl == 0) {
            bins_find([&](int i) { return fb_hist[i]; }, FB_NB, 0, sc, b_star, before, grand);
            if (by_mass) target = ceil_target(topp, grand);
            else if (target >= grand) return false;
            if (grand == 0) return false;
        }
        bins_find([&](int i) { return fb_hist[i]; }, FB_NB, target, sc, b_star, before, grand);
        if (b_star < 0) return false;
        target -= before;
        prefix = (prefix << 8) | (uint32_t)(FB_NB - 1 - b_star);
        __syncthreads();
    }
    pivot = key2f(prefix);
    return true;
}

}  // namespace strm

namespace strm {

// PEN: the launch has histories (penalties possible); MASK: it has a grammar mask; LOADER: 1 = fp32 rows that take
// 128-bit loads (16-byte aligned, V a multiple of 4), 2 = bf16 rows that take 64-bit loads (8-byte aligned, V a multiple
// of 4), 0 = the general loader.  Every launch runs the instantiation without the paths it cannot take.
template <bool PEN, bool MASK, int LOADER>
__global__ void __launch_bounds__(NT, CTAS_PER_SM) k_sample_stream(const __grid_constant__ Args a) {
    const int tid = threadIdx.x, lane = lane_id(), warp = warp_id();
    const int V = a.V;
    const int nw = (V + 31) >> 5;                                // bitmap words of a row

    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint32_t* hist1 = reinterpret_cast<uint32_t*>(smem_raw);                  // [NB1] counts; [BINS] group-maxima counts
    Entry* glist = reinterpret_cast<Entry*>(smem_raw);                        // gathered list, over hist1 (16 KB)
    u64* bins = reinterpret_cast<u64*>(smem_raw + NB1 * 4);                   // [BINS] list-selection bins
    u64* fb_hist = bins + BINS;                                               // [FB_NB] fallback radix
    Cand* ownlist = reinterpret_cast<Cand*>(fb_hist + FB_NB);                 // [NW][WLIST]
    Sc* sc = reinterpret_cast<Sc*>(ownlist + NW * WLIST);
    uint32_t* pen_bits = reinterpret_cast<uint32_t*>(sc + 1);                 // [nw] tokens of the history
    uint32_t* pen_prefix = pen_bits + nw;                                     // [nw] rank of each word's first set bit
    uint32_t* pen_cnt = pen_prefix + nw;                                      // [PEN_TABLE] occurrences per rank
    float* pen_val = reinterpret_cast<float*>(pen_cnt + PEN_TABLE);            // [PEN_TABLE] penalised logit per rank
    float* pen_raw = pen_val + PEN_TABLE;                                      // [PEN_TABLE] stored logit per rank
    int* pen_tok = reinterpret_cast<int*>(pen_raw + PEN_TABLE);                // [PEN_TABLE] token per rank (ascending)

    // warp w owns the contiguous region [r_lo, r_hi) of the row; lanes interleave float4 groups: token order inside a
    // region is (step, lane, component)
    const int reg = (((V + 127) / 128 + NW - 1) / NW) * 128;
    const int r_lo = min(warp * reg, V), r_hi = min(r_lo + reg, V);
    Cand* mylist = ownlist + warp * WLIST;
    const long long n_rows = (long long)a.B * a.R;
#ifdef COLINFER_PROFILE
    long long prof_last = clock64();
    if (a.prof && tid == 0) for (int i = 0; i < 16; ++i) sc->prof[i] = 0;
#endif
    if (tid < NWA) {                                             // neutral values for the warps a smaller CTA does not have
        sc->wsum[tid] = 0; sc->wsum2[tid] = 0; sc->wmass[tid] = 0; sc->wf[tid] = CI_NEG_INF; sc->wi[tid] = 0x7fffffff; sc->wcount[tid] = 0;
        sc->wtw[tid] = -ST_FLT_MAX; sc->wmin[tid] = ST_POS_INF;
    }
    __syncthreads();

    // ---------------------------------------------------------------------------------------- which rows are this CTA's
    // Rows differ in cost by a factor of ten (a wide top-p row takes several passes, a greedy row one), so dealing them
    // out by index would leave some CTAs with most of the expensive ones.  Every CTA orders the rows by cost class
    // (wide sampled, small top-k, greedy) -- the same order in all CTAs -- and takes every gridDim.x-th entry of it.  Launches with at most one row per CTA, or very many rows, keep the index order.
    long long my_n = n_rows > blockIdx.x ? (n_rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const bool dealt = n_rows > gridDim.x && n_rows <= BAL_ROWS && gridDim.x >= 128;
    if (dealt) {
        auto row_class = [&](int row) {
            const int b = row / a.R;
            const float T = a.p.temperature[b];
            const int k = a.p.top_k[b];
            if (!((T > 0.0f) || (a.flags & COLINFER_FORCE_DISTRIBUTION))) return 2;
            return (k > 0 && k <= FASTK && k < V) ? 1 : 0;
        };
        // one scan over the threads' per-class counts (three 21-bit counters in a word) orders the rows by (class, thread,
        // chunk): any order will do as long as every CTA computes the same one
        constexpr int CH = BAL_ROWS / NT;
        int cls[CH];
        u64 packed = 0;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int row = c * NT + tid;
            cls[c] = row < (int)n_rows ? row_class(row) : -1;
            if (cls[c] >= 0) packed += 1ull << (21 * cls[c]);
        }
        u64 tot;
        u64 ex = block_excl_scan(packed, sc, tot);
        // Wide rows go round the CTAs first.  Where that round ends, some CTAs hold one wide row fewer than the others: a
        // wide row costs about as much as two to three small-top-k rows, so those CTAs get two small-top-k rows each
        // before the rest of that class (and then the greedy rows) continue round the CTAs from there.
        const int G = (int)gridDim.x;
        const long long n0 = (long long)(tot & 0x1FFFFFull), n1 = (long long)((tot >> 21) & 0x1FFFFFull);
        const int r0 = (int)(n0 % G), n_short = r0 ? G - r0 : 0;
        const long long extra = min(2ll * n_short, n1);
        if (tid == 0) sc->my_count = 0;
        __syncthreads();
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            if (cls[c] >= 0) {
                const int j = cls[c];
                const long long q = (long long)((ex >> (21 * j)) & 0x1FFFFFull);     // position inside the class
                ex += 1ull << (21 * j);
                int cta;
                if (j == 0) cta = (int)(q % G);
                else if (j == 1) cta = q < extra ? r0 + (int)(q % n_short) : (int)((r0 + q - extra) % G);
                else cta = (int)((r0 + n1 - extra + q) % G);
                if (cta == (int)blockIdx.x) sc->my_rows[atomicAdd(&sc->my_count, 1)] = c * NT + tid;   // any order
            }
        }
        __syncthreads();
        my_n = sc->my_count;
    }
    for (long long it = 0; it < my_n; ++it) {
        __syncthreads();                                         // the previous row's shared tables are free
        const long long row = dealt ? (long long)sc->my_rows[it] : blockIdx.x + it * gridDim.x;
        ST_PROF(0);
        const int b = (int)(row / a.R), r = (int)(row % a.R);
        // ------------------------------------------------------------------------------------ parameters of the slot
        const float T = a.p.temperature[b];
        const bool sampled = (T > 0.0f) || (a.flags & COLINFER_FORCE_DISTRIBUTION);
        const float tc = fmaxf(T, 1e-6f);
        const int kk = a.p.top_k[b];
        const float topp = a.p.top_p[b];
        const float log_min_p = a.p.log_min_p[b];
        Row rw;
        rw.V = V; rw.vec = LOADER == 1; rw.vec16 = LOADER == 2;
        rw.p32 = a.dtype == COLINFER_F32 ? reinterpret_cast<const float*>(a.logits) + (size_t)row * V : nullptr;
        rw.p16 = a.dtype == COLINFER_BF16 ? reinterpret_cast<const __nv_bfloat16*>(a.logits) + (size_t)row * V : nullptr;
        rw.mrow = (MASK && a.mask) ? a.mask + ((size_t)b * a.mask_rows + r) * a.W : nullptr;
        rw.rp = a.p.repetition_penalty ? a.p.repetition_penalty[b] : 1.0f;
        rw.pp = a.p.presence_penalty ? a.p.presence_penalty[b] : 0.0f;
        rw.fp = a.p.frequency_penalty ? a.p.frequency_penalty[b] : 0.0f;
        rw.hist = a.p.history ? a.p.history + (size_t)b * a.p.hist_stride : nullptr;
        int hlen = rw.hist ? (a.p.hist_len ? a.p.hist_len[b] : a.p.hist_stride) : 0;
        hlen = max(0, min(hlen, a.p.hist_stride));
        rw.hlen = hlen;
        rw.has_pen = PEN && hlen > 0 && !(rw.rp == 1.0f && rw.pp == 0.0f && rw.fp == 0.0f);
        rw.pen_bits = pen_bits; rw.pen_prefix = pen_prefix; rw.pen_val = pen_val; rw.hist_slow = &sc->hist_slow;
        if (tid == 0) sc->hist_slow = 0;
        const bool fastk = sampled && kk > 0 && kk <= FASTK && kk < V;
        rw.pol = (sampled && !fastk) ? l2_policy_keep() : l2_policy_stream();
        // Rows that are finished from their candidate lists alone -- greedy and small-top-k rows -- need the penalties of
        // the listed tokens only.  When the penalties can only lower a logit (the usual setting) such a row builds no
        // tables: after the pass every history entry looks itself up in the lists (they are ordered by token) and the
        // entries found take their penalised value.  If the row then turns out to need more than its lists (a list
        // overflowed, too few candidates stay above the bound, the finish leaves the lists), it starts again with tables.
        const bool lowering = rw.rp >= 1.0f && rw.pp >= 0.0f && rw.fp >= 0.0f;
      for (int redo = 0; redo < 2; ++redo) {
        if (redo) __syncthreads();
        const bool lazy = PEN && rw.has_pen && lowering && (fastk || !sampled) && redo == 0;
        int* hist_s = reinterpret_cast<int*>(pen_raw);               // lazy rows: the first PEN_TABLE history entries, staged
        if (lazy) {
            for (int i = tid; i < PEN_TABLE; i += NT) pen_cnt[i] = 0u;   // occurrences per list entry (NW * WLIST = PEN_TABLE)
            for (int i = tid; i < min(hlen, PEN_TABLE); i += NT)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(hist_s + i)), "l"(rw.hist + i) : "memory");
            asm volatile("cp.async.commit_group;" ::: "memory");
        }

        // ------------------------------------------------------------------------------------ penalty tables (whole row)
        int pen_distinct = 0;
        rw.pen_inline = rw.has_pen;
        if (rw.has_pen && !lazy) {
            // Each thread keeps its first HP history entries and their stored logits in registers: the two dependent loads
            // (id, then logit) run under the bitmap and rank steps.  Longer histories re-read the rest.
            constexpr int HP = 2048 / NT;
            int ht[HP]; float hx[HP];
            for (int i = tid; i < nw; i += NT) pen_bits[i] = 0u;
            for (int i = tid; i < PEN_TABLE; i += NT) pen_cnt[i] = 0u;
#pragma unroll
            for (int j = 0; j < HP; ++j) {
                const int i = tid + j * NT;
                ht[j] = i < hlen ? __ldg(rw.hist + i) : -1;
                if (ht[j] >= V) ht[j] = -1;
            }
#pragma unroll
            for (int j = 0; j < HP; ++j) {
                hx[j] = CI_NEG_INF;
                if (ht[j] >= 0) {
                    const bool masked = rw.mrow != nullptr && !((__ldg(rw.mrow + (ht[j] >> 5)) >> (ht[j] & 31)) & 1);
                    if (!masked) hx[j] = rw.raw(ht[j]);
                }
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < HP; ++j) if (ht[j] >= 0) atomicOr(&pen_bits[ht[j] >> 5], 1u << (ht[j] & 31));
            for (int i = tid + HP * NT; i < hlen; i += NT) {
                const int v = __ldg(rw.hist + i);
                if (v >= 0 && v < V) atomicOr(&pen_bits[v >> 5], 1u << (v & 31));
            }
            __syncthreads();
            {
                // ranks of the set bits (exclusive prefix of popcounts over the bitmap words)
                const int ipt = (nw + NT - 1) / NT;
                const int lo = min(tid * ipt, nw), hi = min(lo + ipt, nw);
                u64 local = 0;
                for (int i = lo; i < hi; ++i) local += __popc(pen_bits[i]);
                u64 total_bits;
                uint32_t run = (uint32_t)block_excl_scan(local, sc, total_bits);
                pen_distinct = (int)total_bits;
                for (int i = lo; i < hi; ++i) { pen_prefix[i] = run; run += __popc(pen_bits[i]); }
                __syncthreads();
                auto rank_of = [&](int v) { return pen_prefix[v >> 5] + __popc(pen_bits[v >> 5] & ((1u << (v & 31)) - 1u)); };
                uint32_t hr[HP];
#pragma unroll
                for (int j = 0; j < HP; ++j) hr[j] = ht[j] >= 0 ? rank_of(ht[j]) : 0xFFFFFFFFu;
                if (rw.fp != 0.0f) {                              // occurrences per rank
#pragma unroll
                    for (int j = 0; j < HP; ++j) if (hr[j] < PEN_TABLE) atomicAdd(&pen_cnt[hr[j]], 1u);
                    for (int i = tid + HP * NT; i < hlen; i += NT) {
                        const int v = __ldg(rw.hist + i);
                        if (v >= 0 && v < V) { const uint32_t rk = rank_of(v); if (rk < PEN_TABLE) atomicAdd(&pen_cnt[rk], 1u); }
                    }
                    __syncthreads();
                }
                // the stored and the penalised logit of every marked token (equal tokens write equal values)
                auto put = [&](uint32_t rk, float x, int tok) {
                    if (rk < PEN_TABLE) {
                        const int cnt = rw.fp != 0.0f ? (int)pen_cnt[rk] : 1;
                        pen_raw[rk] = x;
                        pen_tok[rk] = tok;
                        pen_val[rk] = x > CI_NEG_INF ? apply_penalty(x, cnt, rw.rp, rw.pp, rw.fp) : CI_NEG_INF;
                    }
                };
#pragma unroll
                for (int j = 0; j < HP; ++j) put(hr[j], hx[j], ht[j]);
                for (int i = tid + HP * NT; i < hlen; i += NT) {
                    const int v = __ldg(rw.hist + i);
                    if (v >= 0 && v < V) {
                        const bool masked = rw.mrow != nullptr && !((__ldg(rw.mrow + (v >> 5)) >> (v & 31)) & 1);
                        put(rank_of(v), masked ? CI_NEG_INF : rw.raw(v), v);
                    }
                }
            }
            __syncthreads();
        }
        ST_PROF(1);

        // ------------------------------------------------------------------------------------ pass 1: maximum, argmax; running top-k lists
        // Small top_k: each warp lists the logits of its region that are >= its own threshold -- the kk-th largest it
        // has seen, raised whenever the list fills -- so that the lists together always hold the row's top kk.
        // Penalised rows read the logits as stored -- no per-element test of the history bitmap -- and patch afterwards:
        // the listed candidates (which give the penalised maximum, and decide small-top-k and greedy rows), and for
        // wide rows every count and sum, by the difference the few penalised tokens make.
        const bool patch = PEN && rw.has_pen && pen_distinct <= PEN_TABLE;
        // rows with a top-p (or a small top-k) list their top logits: a row whose listed logits hold all of its mass (a
        // dominant token, everything unlisted below the mass horizon) is finished from the list alone
        const bool do_lists = fastk || patch || (sampled && topp < 1.0f);   // (plain rows keep the lean pass)
        // Wide rows that need a pivot (large top_k, top_p) count the fine histogram in this pass too, in buckets laid
        // out from the sample's maximum (the row's is not known yet), HOFF of them above it.
        const bool wide_hist = sampled && !fastk && ((kk > 0 && kk < V) || topp < 1.0f);
        const bool listpass = do_lists || wide_hist;
        const int kq = fastk ? kk : 8;
        const float SCW = (float)NB1 / (RANGE * tc);
        float lref = CI_NEG_INF;
        if (patch) rw.pen_inline = false;
        float lmax = CI_NEG_INF;
        int lpos = -1, lidx = 0x7fffffff;
        float tw = -ST_FLT_MAX;
        int wn1 = 0, fk_bad = 0;
#define ST_LOAD_BATCH(v, i0)                                                                                              \
    _Pragma("unroll") for (int k = 0; k < 4; ++k) {                                                                       \
        const int i = (i0) + k * 128 + lane * 4;                                                                          \
        v[k] = i < r_hi ? rw.raw4(i) : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);                       \
    }                                                                                                                     \
    _Pragma("unroll") for (int k = 0; k < 4; ++k) v[k] = rw.fix4(v[k], (i0) + k * 128 + lane * 4, r_hi);
#define ST_LOAD_BATCH_T(v, i0, PI)                                                                                       \
    _Pragma("unroll") for (int k = 0; k < 4; ++k) {                                                                       \
        const int i = (i0) + k * 128 + lane * 4;                                                                          \
        v[k] = i < r_hi ? rw.raw4(i) : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);                       \
    }                                                                                                                     \
    _Pragma("unroll") for (int k = 0; k < 4; ++k) v[k] = rw.template fix4t<PI>(v[k], (i0) + k * 128 + lane * 4, r_hi);
#define ST_TRACK_MAX(v, i0)                                                                                               \
    _Pragma("unroll") for (int k = 0; k < 4; ++k) {                                                                       \
        const float m4 = fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w));                                             \
        const bool up = m4 > lmax;               /* strict: the first (lowest) position of the maximum stays */            \
        lmax = up ? m4 : lmax;                                                                                            \
        lpos = up ? (i0) + k * 128 + lane * 4 : lpos;                                                                     \
    }
        if (!listpass) {
            if constexpr (PEN) {
                const float2 mp = pass1_lean(rw, r_lo, r_hi, lane);
                lmax = mp.x; lpos = __float_as_int(mp.y);
            } else {
                for (int i0 = r_lo; i0 < r_hi; i0 += 512) {
                    float4 v[4];
                    ST_LOAD_BATCH(v, i0)
                    ST_TRACK_MAX(v, i0)
                }
            }
        } else {
            // The first batch of every warp (a tenth of the row at 151,936 logits) bounds the row's kk-th largest logit
            // from below: the kk-th largest of the sample's float4 maxima.  The pass then lists what reaches the bound.
            constexpr int NSB = 32 / NW;                             // sample batches per warp: 16,384 logits per row in all
            float gm[4 * NSB];
#pragma unroll
            for (int sb = 0; sb < NSB; ++sb) {
                float4 v[4];
                ST_LOAD_BATCH(v, r_lo + sb * 512)
                ST_TRACK_MAX(v, r_lo + sb * 512)
#pragma unroll
                for (int k = 0; k < 4; ++k) gm[sb * 4 + k] = fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w));
            }
            float sm = lmax;
#pragma unroll
            for (int o = 16; o; o >>= 1) sm = fmaxf(sm, __shfl_xor_sync(0xffffffffu, sm, o));
            if (lane == 0) sc->wf[warp] = sm;
            for (int i = tid; i < BINS_PAD; i += NT) hist1[i] = 0u;
            __syncthreads();
            lref = sc->wf[lane];
            // the bins of the bound hang from the smallest finite warp maximum plus 4: a few dominant tokens in the
            // sample (far above everything else) must not stretch them beyond the bulk
            float lbulk = lref > CI_NEG_INF ? lref : ST_POS_INF;
#pragma unroll
            for (int o = 16; o; o >>= 1) {
                lref = fmaxf(lref, __shfl_xor_sync(0xffffffffu, lref, o));
                lbulk = fminf(lbulk, __shfl_xor_sync(0xffffffffu, lbulk, o));
            }
            if (do_lists) {
                const float top = fminf(lbulk + 4.0f, lref);         // +inf when no warp saw a finite logit
#pragma unroll
                for (int k = 0; k < 4 * NSB; ++k)
                    if (gm[k] > CI_NEG_INF && top < ST_POS_INF)
                        atomicAdd(&hist1[padbin(max(0, min(BINS - 1, __float2int_rz((top - gm[k]) * FAST_SCALE))))], 1u);
                __syncthreads();
                uint32_t have;
                const int bk = warp_count_bin(hist1, (uint32_t)kq, lane, have);
                if (bk >= 0 && bk < BINS - 1) tw = top - ((float)(bk + 1) + 0.01f) / FAST_SCALE - fabsf(top) * 1e-6f;
            } else {
                tw = ST_POS_INF;                                 // nothing to list
            }
            const bool count_hist = wide_hist && lref > CI_NEG_INF && lref < ST_POS_INF;
            if (count_hist) {
                __syncthreads();
                for (int i = tid; i < NB1; i += NT) hist1[i] = 0u;
                __syncthreads();
            } else {
                lref = CI_NEG_INF;                               // marks: no histogram from this pass
            }
            auto listing_pass = [&](auto pi_tag) {
                constexpr bool PI = decltype(pi_tag)::value;
                for (int i0 = r_lo; i0 < r_hi; i0 += 512) {
                    float4 v[4];
                    ST_LOAD_BATCH_T(v, i0, PI)
                    float bmax = CI_NEG_INF;                         // the batch's largest logit of this lane
    #pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float m4 = fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w));
                        const bool up = m4 > lmax;                   // strict: the first (lowest) position of the maximum stays
                        lmax = up ? m4 : lmax;
                        lpos = up ? i0 + k * 128 + lane * 4 : lpos;
                        bmax = fmaxf(bmax, m4);
                    }
                    if (count_hist) {
    #pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float e[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
    #pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (e[j] > CI_NEG_INF) atomicAdd(&hist1[fine_bucket(e[j], lref, SCW, (float)HOFF - 0.5f)], 1u);
                        }
                    }
                    if (__ballot_sync(0xffffffffu, bmax >= tw)) {    // some lane has a logit for its list
                        unsigned mk[4];
    #pragma unroll
                        for (int k = 0; k < 4; ++k)
                            mk[k] = (v[k].x >= tw ? 1u : 0u) | (v[k].y >= tw ? 2u : 0u) | (v[k].z >= tw ? 4u : 0u) | (v[k].w >= tw ? 8u : 0u);
                        // per-lane counts of the four groups, one byte each (a group holds at most 128: no carry)
                        const unsigned cnt = __popc(mk[0]) | (__popc(mk[1]) << 8) | (__popc(mk[2]) << 16) | (__popc(mk[3]) << 24);
                        unsigned incl = cnt;
    #pragma unroll
                        for (int o = 1; o < 32; o <<= 1) { const unsigned t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
                        warp_append_batch<WLIST>(mylist, wn1, mk, v, (uint32_t)(i0 + lane * 4), lane, incl, cnt);
                    }
                }
            };
            if (PEN && rw.pen_inline) listing_pass(BoolTag<PEN>{}); else listing_pass(BoolTag<false>{});
            if (wn1 > WLIST) fk_bad = 1;                         // a list overflowed (its tail was dropped): general path
            if (!do_lists) { tw = -ST_FLT_MAX; wn1 = 0; }
        }
        ST_PROF(2);
        bool from_lists = false;                                 // the maximum comes from the patched lists
        if (patch) {
            // penalised values for the listed tokens; the maximum and argmax of the row are then among the listed ones --
            // provided no penalised token rose from below the bound to above it, and enough candidates remain
            int bad = fk_bad;
            float pm = CI_NEG_INF; int pi = 0x7fffffff, cnt_ok = 0;
            if (lazy) {
                // every history entry finds its token in the list of the warp that owns it and counts itself there
                if (lane == 0) sc->wcount[warp] = min(wn1, WLIST);
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                __syncthreads();
                for (int i = tid; i < hlen; i += NT) {
                    const int v = i < PEN_TABLE ? hist_s[i] : __ldg(rw.hist + i);
                    if (v < 0 || v >= V) continue;
                    const int w = v / reg;
                    const Cand* lst = ownlist + w * WLIST;
                    int lo = 0, hi = sc->wcount[w];
                    while (lo < hi) { const int mid = (lo + hi) >> 1; if (lst[mid].idx < (uint32_t)v) lo = mid + 1; else hi = mid; }
                    if (lo < sc->wcount[w] && lst[lo].idx == (uint32_t)v) atomicAdd(&pen_cnt[w * WLIST + lo], 1u);
                }
                __syncthreads();
                for (int j = lane; j < min(wn1, WLIST); j += 32) {
                    const uint32_t c = pen_cnt[warp * WLIST + j];
                    float l = mylist[j].l;
                    if (c) { l = apply_penalty(l, rw.fp != 0.0f ? (int)c : 1, rw.rp, rw.pp, rw.fp); mylist[j].l = l; }
                    if (l >= tw) { ++cnt_ok; if (l > pm) { pm = l; pi = (int)mylist[j].idx; } }   // token order: the first maximum stays
                }
            } else {
                for (int j = lane; j < min(wn1, WLIST); j += 32) {
                    const uint32_t idx = mylist[j].idx;
                    const uint32_t word = pen_bits[idx >> 5];
                    float l = mylist[j].l;
                    if ((word >> (idx & 31)) & 1u) {
                        l = pen_val[pen_prefix[idx >> 5] + __popc(word & ((1u << (idx & 31)) - 1u))];
                        mylist[j].l = l;
                    }
                    if (l >= tw) { ++cnt_ok; if (l > pm) { pm = l; pi = (int)idx; } }   // token order: the first maximum stays
                }
                for (int rk = tid; rk < pen_distinct; rk += NT)
                    if (pen_val[rk] >= tw && !(pen_raw[rk] >= tw)) bad = 1;
            }
            cnt_ok = (int)__reduce_add_sync(0xffffffffu, (unsigned)cnt_ok);
            if (lane == 0) sc->wcount[warp] = cnt_ok;
            bad = __syncthreads_or(bad);
            int have_ok = sc->wcount[lane];
            have_ok = (int)__reduce_add_sync(0xffffffffu, (unsigned)have_ok);
            if (!bad && have_ok >= kq && tw > -ST_FLT_MAX) {
                from_lists = true;
                lmax = pm; lidx = pi;
            } else if (lazy) {
                continue;                                        // the lists do not decide this row: again, with tables
            } else {
                // the bound does not hold for the penalised values: the element-wise pass after all
                __syncthreads();
                fk_bad = 1;
                rw.pen_inline = true;
                lmax = CI_NEG_INF; lpos = -1;
                for (int i0 = r_lo; i0 < r_hi; i0 += 512) {
                    float4 v[4];
                    ST_LOAD_BATCH(v, i0)
                    ST_TRACK_MAX(v, i0)
                }
            }
        }
        if (patch && !from_lists) lref = CI_NEG_INF;             // the histogram of this pass counted stored logits: void
        uint32_t* fin_bins = fastk ? hist1 : reinterpret_cast<uint32_t*>(bins);   // wide rows keep their histogram in hist1
        if (sampled) {                                           // bins of the finish (the reduce below has the barriers after)
            if (fastk) __syncthreads();                          // every warp has read the sample's bins
            for (int i = tid; i < BINS_PAD; i += NT) fin_bins[i] = 0u;
        }
        if (!from_lists && lpos >= 0) {
            const float4 v = rw.load4(lpos);
            lidx = lpos + (v.x == lmax ? 0 : v.y == lmax ? 1 : v.z == lmax ? 2 : 3);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, lmax, o);
            const int oi = __shfl_xor_sync(0xffffffffu, lidx, o);
            if (om > lmax || (om == lmax && oi < lidx)) { lmax = om; lidx = oi; }
        }
        if (lane == 0) { sc->wf[warp] = lmax; sc->wi[warp] = lidx; }
        __syncthreads();
        if (warp == 0) {
            float bm = sc->wf[lane]; int bi = sc->wi[lane];
#pragma unroll
            for (int o = 16; o; o >>= 1) {
                const float om = __shfl_xor_sync(0xffffffffu, bm, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (om > bm || (om == bm && oi < bi)) { bm = om; bi = oi; }
            }
            if (lane == 0) { sc->bc_f = bm; sc->bc_i = bi; }
        }
        __syncthreads();
        const float L = sc->bc_f;
        int aidx = sc->bc_i;
        if (aidx == 0x7fffffff) aidx = 0;
        __syncthreads();
        ST_PROF(3);

        int status = 0;
        const bool finite_max = (L > CI_NEG_INF) && (L < ST_POS_INF);
        if (sampled && !finite_max) status |= COLINFER_ROW_DEGENERATE;
        float lcut = CI_NEG_INF;
        u64 total_mass = 0;
        long long token = aidx;

        if (sampled && finite_max) {
            const float m = scale_logit(L, tc);
            MassFn mass;
            mass.init(tc, m);
            const float thr = __fadd_rn(m, log_min_p);
            lcut = lower_logit_for(thr, tc, __fmul_rn(thr, tc));
            // Logits more than 22 temperatures below the maximum have integer mass 0 (2^30 exp(-22) < 1/2): they can never
            // be drawn and add nothing to any sum, so every selection works above that horizon.  (A top-k whose k-th
            // largest lies below it removes nothing that could be drawn.)  Rows with a dominant token -- everything else
            // tens of logits below -- then stay on the fast paths instead of searching the massless bulk.
            lcut = fmaxf(lcut, L - 22.0f * tc - fabsf(L) * 1e-6f);
            bool need_topk = kk > 0 && kk < V;
            const bool need_topp = topp < 1.0f;
            const float u = row_uniform(a, (int)row, b, r);
            bool done = false;

            // -------------------------------------------------------------------------------- small top-k: finish from the running lists
            // Small top-k rows; and any other row whose bound lies below the mass horizon: every logit that carries mass is
            // listed (top-k, if any, then removes nothing: kk beyond the list).
            const bool all_listed = !fastk && tw > -ST_FLT_MAX && tw < lcut;
            if (fastk || all_listed) {
                ST_PROF(4);
                if (!__syncthreads_or(fk_bad || !(tw > -ST_FLT_MAX)) &&
                    finish_running_topk(ownlist, wn1, tw, L, lcut, tc, mass, fastk ? kk : (need_topk ? kk : 0x7fffffff), need_topp, topp, u,
                                        fin_bins, sc, token, lcut, total_mass FK_PROF_ARGS))
                    done = true;
                __syncthreads();
                ST_PROF(7);
                if (!done && lazy) continue;                     // the general path needs the tables: again, with them
            }
            // Wide rows of a penalised slot keep reading the stored logits: every count and sum is corrected afterwards by
            // the difference the (at most PEN_TABLE) penalised tokens make.  Without the patched maximum: element by element.
            bool corr = !done && from_lists;
            rw.pen_inline = rw.has_pen && !corr;
            // the penalised tokens of this warp's own region (corrections of the warp's own sums need no atomics)
            // (dense loops over the ranks: the tables hold the tokens in ascending order, a region's are consecutive)
            auto for_my_pen = [&](auto f) {
                if (r_lo < r_hi) {
                    const int rk_hi = r_hi < V ? (int)pen_prefix[r_hi >> 5] : pen_distinct;
                    for (int rk = (int)pen_prefix[r_lo >> 5] + lane; rk < rk_hi; rk += 32) f(pen_tok[rk], pen_raw[rk], pen_val[rk]);
                }
            };
            auto for_each_pen = [&](auto f) {
                for (int rk = tid; rk < pen_distinct; rk += NT) f(pen_tok[rk], pen_raw[rk], pen_val[rk]);
            };

            if (!done) {
                enum { PATH_PURE = 0, PATH_LIST = 1, PATH_BAND = 2, PATH_FALLBACK = 3 };
                int path = PATH_PURE;
                float t_hi = CI_NEG_INF, t_lo = ST_POS_INF;
                int band_top = 0, band_bot = 0;                  // fine buckets the band covers (from, to)
                const float SC1 = SCW;
                // The fine buckets: from pass 1 (laid out from the sample's maximum, HOFF of them above it) or counted now
                // (from the row's maximum).  Bucket b holds the logits in (edge(b + 1), edge(b)].  A stored logit of a
                // penalised token may lie above every bucket: bucket 0.
                const bool hist_ready = lref > CI_NEG_INF && (L - lref) * SC1 < (float)(HOFF - 2);   // the maximum lies inside the buckets laid out from the sample
                const float href = hist_ready ? lref : L;
                const int hoff = hist_ready ? HOFF : 0;
                auto bucket1 = [&](float x) { return fine_bucket(x, href, SC1, (float)hoff - 0.5f); };
                auto edge = [&](int b) { return href - (float)(b - hoff) / SC1; };
                if (need_topk || need_topp) {
                    if (!hist_ready) {
                        // -------------------------------------------------------------------- pass 2: fine count histogram
                        for (int i = tid; i < NB1; i += NT) hist1[i] = 0u;
                        __syncthreads();
                        for (int i0 = r_lo; i0 < r_hi; i0 += 512) {
                            float4 v[4];
                            ST_LOAD_BATCH(v, i0)
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const float e[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
                                for (int j = 0; j < 4; ++j) if (e[j] > CI_NEG_INF) atomicAdd(&hist1[bucket1(e[j])], 1u);
                            }
                        }
                    }
                    __syncthreads();
                    if (corr) {
                        for_each_pen([&](int, float r, float e) {
                            if (r > CI_NEG_INF) atomicSub(&hist1[bucket1(r)], 1u);
                            if (e > CI_NEG_INF) atomicAdd(&hist1[bucket1(e)], 1u);
                        });
                        __syncthreads();
                    }
                    ST_PROF(8);
                    // the histogram counts every finite logit; buckets wholly below the min-p cut are left out of the scans
                    const int b_cut = lcut > CI_NEG_INF ? bucket1(lcut) : NB1 - 1;
                    const float dL = (L - href) / tc;
                    auto mass_est = [&](int i) {
                        return (u64)__float2uint_rn(exp2f(fminf(0.0f, -(((float)(i - hoff) + 0.5f) * (RANGE / (float)NB1) + dL) * CI_LOG2E)) * CI_MASS_SCALE);
                    };
                    // 768: how far down the list capacity reaches (~24 per warp list of 64)
                    const FineDecision fd = fine_decide(hist1, mass_est, b_cut, need_topk ? (u64)kk : 0ull, 768ull, topp, need_topp, sc);
                    const int bsel = fd.b_k;
                    if (need_topk && (u64)kk >= fd.total_cnt) need_topk = false;   // at most k reach the min-p cut's bucket: top-k removes nothing
                    if (need_topk) {
                        const u64 n_upto = bsel >= 0 ? fd.before_k + hist1[bsel] : (u64)GLIST + 1;
                        if (bsel < (hist_ready ? 1 : 0) || bsel >= NB1 - 3 || n_upto > GLIST - 64) path = PATH_FALLBACK;   // bucket 0 of a pass-1 histogram may mix logits from far above the sample's maximum
                        else {
                            path = PATH_LIST;
                            t_lo = edge(bsel + 2) - 0.01f / SC1 - fabsf(href) * 1e-6f;
                        }
                    } else if (need_topp) {
                        const int bp = fd.b_p, bcap = fd.b_cap;
                        if (fd.est_total == 0) path = PATH_FALLBACK;
                        else {
                            const int up = a.dtype == COLINFER_BF16 ? 3 : 1, dn = a.dtype == COLINFER_BF16 ? 4 : 2;
                            if (bp < (hist_ready ? 1 : 0)) path = PATH_FALLBACK;
                            else if (bcap < 0 || bcap > bp + dn + 1) {
                                // small nucleus: gather everything down to well below the estimated pivot; nothing is "above"
                                path = PATH_BAND;
                                t_hi = ST_POS_INF;
                                t_lo = bcap < 0 ? -ST_FLT_MAX : edge(bcap);
                                band_top = 0; band_bot = bcap < 0 ? NB1 - 1 : bcap;
                            } else if (bp + dn + 2 >= NB1) path = PATH_FALLBACK;
                            else {
                                path = PATH_BAND;
                                t_hi = bp - up <= 0 ? ST_POS_INF : edge(bp - up);
                                t_lo = edge(bp + dn + 1);
                                band_top = max(0, bp - up); band_bot = bp + dn;
                                if (a.flags & COLINFER_TEST_MISS_BAND) {     // test hook: a band eight buckets off (above or below by row parity)
                                    const int sh = (row & 1) ? 8 : -8;
                                    if (bp - up + sh > 0 && bp + dn + sh + 2 < NB1) {
                                        t_hi = edge(bp - up + sh); t_lo = edge(bp + dn + 1 + sh);
                                        band_top = bp - up + sh; band_bot = bp + dn + sh;
                                    }
                                }
                            }
                        }
                    }
                    __syncthreads();
                    ST_PROF(9);
                }

                // ---------------------------------------------------------------------------- large top-k (then top-p) on a gathered list
                if (path == PATH_LIST) {
                    const float tl = fmaxf(fmaxf(t_lo, lcut), -ST_FLT_MAX);
                    int wn = 0;
                    for (int i0 = r_lo; i0 < r_hi; i0 += 512) {
                        float4 v[4];
                        unsigned mk[4], anym = 0;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int i = i0 + k * 128 + lane * 4;
                            v[k] = i < r_hi ? rw.raw4(i) : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
                            }
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                            v[k] = rw.fix4(v[k], i0 + k * 128 + lane * 4, r_hi);
                            mk[k] = (v[k].x >= tl ? 1u : 0u) | (v[k].y >= tl ? 2u : 0u) | (v[k].z >= tl ? 4u : 0u) | (v[k].w >= tl ? 8u : 0u);
                            anym |= mk[k];
                        }
                        if (__ballot_sync(0xffffffffu, anym != 0u)) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const float e4[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
                                warp_append(mylist, wn, mk[k], e4, (uint32_t)(i0 + k * 128 + lane * 4), lane);
                            }
                        }
                    }
                    int raised = 0;
                    if (corr) {
                        // listed penalised tokens take their penalised value in place (below tl: -inf, never kept); one
                        // that rises from below tl to above it is not listed: the element-wise fallback
                        for (int j = lane; j < min(wn, WLIST); j += 32) {
                            const uint32_t idx = mylist[j].idx, word = pen_bits[idx >> 5];
                            if ((word >> (idx & 31)) & 1u) {
                                const float e = pen_val[pen_prefix[idx >> 5] + __popc(word & ((1u << (idx & 31)) - 1u))];
                                mylist[j].l = e >= tl ? e : CI_NEG_INF;
                            }
                        }
                        for_each_pen([&](int, float r, float e) { if (e >= tl && !(r >= tl)) raised = 1; });
                    }
                    raised = __syncthreads_or(raised);
                    const int n = raised ? -1 : gather_lists(ownlist, wn, glist, mass, sc);
                    if (n > 0 && finish_on_list(glist, n, tl, fmaxf(lcut, -ST_FLT_MAX), tc, L, true, kk, need_topp, topp, u, bins, sc, token, lcut, total_mass)) done = true;
                    else path = PATH_FALLBACK;
                    __syncthreads();
                    ST_PROF(10);
                }

                // ---------------------------------------------------------------------------- fallback: exact radix select over the keys
                if (path == PATH_FALLBACK) {
                    status |= COLINFER_ROW_SELECT_SLOW;
                    corr = false; rw.pen_inline = rw.has_pen;
                    float lpiv;
                    if (kk > 0 && kk < V && radix_select(rw, r_lo, r_hi, mass, lcut, false, (u64)kk, topp, fb_hist, sc, lpiv))
                        lcut = fmaxf(lcut, lower_logit_for(scale_logit(lpiv, tc), tc, lpiv));
                    if (need_topp && radix_select(rw, r_lo, r_hi, mass, lcut, true, 0, topp, fb_hist, sc, lpiv))
                        lcut = fmaxf(lcut, lower_logit_for(scale_logit(lpiv, tc), tc, lpiv));
                    path = PATH_PURE;
                    t_hi = CI_NEG_INF; t_lo = ST_POS_INF;
                }

                // ---------------------------------------------------------------------------- mass pass and inverse CDF over the row
                if (!done) {
                    const bool band = path == PATH_BAND;
                    const float lk = fmaxf(lcut, -ST_FLT_MAX);
                    u64 wkeep = 0;
                    for (int attempt = 0; attempt < 2; ++attempt) {
                    u64 acc_all = 0, acc_above = 0;
                    int wn = 0;
                    auto mass_pass = [&](auto pi_tag, auto band_tag) {
                        constexpr bool PI = decltype(pi_tag)::value;
                        constexpr bool BAND = decltype(band_tag)::value;
                        for (int i0 = r_lo; i0 < r_hi; i0 += 512) {
                            float4 v[4];
                            ST_LOAD_BATCH_T(v, i0, PI)
                            unsigned mk[4], anym = 0;
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const float e[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
                                uint32_t q[4];
                                mass.four(e, lk, q);
                                acc_all += ((u64)q[0] + q[1]) + ((u64)q[2] + q[3]);   // 64-bit adds: a stored logit of a penalised token may exceed the maximum
                                mk[k] = 0;
                                if (BAND) {
#pragma unroll
                                    for (int j = 0; j < 4; ++j) {
                                        if (e[j] > t_hi) acc_above += q[j];
                                        else if (e[j] >= t_lo && e[j] >= lk) mk[k] |= 1u << j;
                                    }
                                }
                                anym |= mk[k];
                            }
                            if (BAND && __ballot_sync(0xffffffffu, anym != 0u)) {
                                const unsigned cnt = __popc(mk[0]) | (__popc(mk[1]) << 8) | (__popc(mk[2]) << 16) | (__popc(mk[3]) << 24);
                                unsigned incl = cnt;
#pragma unroll
                                for (int o = 1; o < 32; o <<= 1) { const unsigned t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
                                warp_append_batch<WLIST>(mylist, wn, mk, v, (uint32_t)(i0 + lane * 4), lane, incl, cnt);
                            }
                        }
                    };
                    rw.pol = l2_policy_stream();                 // the row's last full read
                    if (PEN && rw.pen_inline) { if (band) mass_pass(BoolTag<PEN>{}, BoolTag<true>{}); else mass_pass(BoolTag<PEN>{}, BoolTag<false>{}); }
                    else { if (band) mass_pass(BoolTag<false>{}, BoolTag<true>{}); else mass_pass(BoolTag<false>{}, BoolTag<false>{}); }
                    ST_PROF(11);
                    wkeep = warp_sum_u64(band ? acc_above : acc_all);       // kept mass of the region known so far
                    u64 wall_corr = 0;
                    if (corr) {
                        // what the penalised tokens change: their stored logits were summed, their penalised ones count
                        u64 d_all = 0, d_ab = 0;
                        for_my_pen([&](int, float r, float e) {
                            const u64 qr = r >= lk ? mass(r) : 0u, qe = e >= lk ? mass(e) : 0u;
                            d_all += qe - qr;
                            if (band) d_ab += (e > t_hi ? qe : 0ull) - (r > t_hi ? qr : 0ull);
                        });
                        wall_corr = warp_sum_u64(d_all);
                        wkeep += band ? warp_sum_u64(d_ab) : wall_corr;
                        if (band) wn = warp_drop_penalised(mylist, wn, pen_bits, lane);   // their penalised values join the band below
                    }
                    if (band) {
                        const u64 wall = warp_sum_u64(acc_all) + wall_corr;
                        u64 s1, s_above;
                        int n = gather_lists(ownlist, wn, glist, mass, sc, wall, wkeep, &s1, &s_above);
                        if (corr && n >= 0) {
                            if (tid == 0) sc->glist_n = n;
                            __syncthreads();
                            for_each_pen([&](int tok, float, float e) {
                                if (e >= lk && e >= t_lo && !(e > t_hi)) {
                                    const int slot = atomicAdd(&sc->glist_n, 1);
                                    if (slot < GLIST) { Entry en; en.idx = (uint32_t)tok; en.l = e; en.q = mass(e); glist[slot] = en; }
                                }
                            });
                            __syncthreads();
                            n = sc->glist_n <= GLIST ? sc->glist_n : -1;
                        }
                        bool ok = n >= 0 && s1 > 0;
                        float cut2 = lcut;
                        if (ok) {
                            u64 part = 0;
                            for (int i = tid; i < n; i += NT) part += glist[i].q;
                            u64 s_band;
                            block_excl_scan(part, sc, s_band);
                            const u64 target = ceil_target(topp, s1);
                            ok = s_above < target && target <= s_above + s_band;   // the pivot lies inside the band
                            if (ok) {
                                const float base = t_hi < ST_POS_INF ? t_hi : L;
                                // (a small nucleus gathers everything above the cut: the bins span [cut, base], not [-max, base])
                                const float scale = (float)(BINS - 2) / fmaxf(base - fmaxf(t_lo, lk), 1e-30f);
                                float lp;
                                ok = lean_select([&](int i) { return glist[i].l; }, [&](int i) { return (u64)glist[i].q; }, n, base, scale,
                                                 target - s_above, bins, sc, lp);
                                if (ok) {
                                    cut2 = fmaxf(lcut, lower_logit_for(scale_logit(lp, tc), tc, lp));
                                    if (cut2 < t_lo) ok = false;          // a tie partner could lie below the band
                                }
                            }
                        }
                        if (ok) {
                            lcut = cut2;
                            u64 add = 0;
                            const int mine = min(wn, WLIST);
                            for (int j = lane; j < mine; j += 32) if (mylist[j].l >= lcut) add += mass(mylist[j].l);
                            wkeep += warp_sum_u64(add);
                            if (corr) {
                                // penalised tokens whose penalised value lies in the band (those above it are in wkeep already)
                                u64 d = 0;
                                for_my_pen([&](int, float, float e) { if (e >= lcut && e >= lk && !(e > t_hi)) d += mass(e); });
                                wkeep += warp_sum_u64(d);
                            }
                        } else {
                            status |= COLINFER_ROW_SELECT_SLOW;
                            if (attempt == 0 && n >= 0 && s1 > 0) {
                                // The estimated band missed the pivot.  Exact masses of the WIN fine buckets next to the band,
                                // on the side the pivot lies, give its bucket; the mass pass then runs again around it.
                                constexpr int WIN = BINS + FB_NB;
                                u64* win = bins;                             // bins and fb_hist are contiguous
                                const u64 target = ceil_target(topp, s1);
                                const int w0 = target <= s_above ? max(0, band_top - WIN + 1) : max(0, band_bot);
                                for (int i = tid; i < WIN; i += NT) win[i] = 0;
                                __syncthreads();
                                u64 hi = 0;
                                auto put = [&](float x, bool add) {
                                    if (x >= lk) {
                                        const u64 q = add ? (u64)mass(x) : 0ull - (u64)mass(x);
                                        const int b = bucket1(x);
                                        if (b < w0) hi += q;
                                        else if (b < w0 + WIN) atomicAdd(reinterpret_cast<unsigned long long*>(&win[b - w0]), (unsigned long long)q);
                                    }
                                };
                                for (int i0 = r_lo; i0 < r_hi; i0 += 128) {
                                    const float4 v = rw.load4(i0 + lane * 4);
                                    put(v.x, true); put(v.y, true); put(v.z, true); put(v.w, true);
                                }
                                if (corr) for_each_pen([&](int, float r, float e) { put(r, false); put(e, true); });
                                u64 s_hi;
                                block_excl_scan(hi, sc, s_hi);
                                int bw = -1; u64 bef_w = 0, tot_w = 0;
                                if (target > s_hi) bins_find([&](int i) { return win[i]; }, WIN, target - s_hi, sc, bw, bef_w, tot_w);
                                __syncthreads();
                                if (bw >= 0) {
                                    const int bstar = w0 + bw;
                                    t_hi = bstar - 1 <= 0 ? ST_POS_INF : edge(bstar - 1);
                                    t_lo = edge(bstar + 2);
                                    continue;                                // the mass pass again, around the pivot's bucket
                                }
                            }
                            // a list overflowed, or the pivot lies far from the estimate: exact radix select by mass, then the
                            // regions' kept masses again
                            float lpiv;
                            corr = false; rw.pen_inline = rw.has_pen;
                            if (radix_select(rw, r_lo, r_hi, mass, lcut, true, 0, topp, fb_hist, sc, lpiv))
                                lcut = fmaxf(lcut, lower_logit_for(scale_logit(lpiv, tc), tc, lpiv));
                            const float lk3 = fmaxf(lcut, -ST_FLT_MAX);
                            u64 acc = 0;
                            for (int i0 = r_lo; i0 < r_hi; i0 += 128) {
                                const float4 v = rw.load4(i0 + lane * 4);
                                acc += (u64)(v.x >= lk3 ? mass(v.x) : 0u) + (v.y >= lk3 ? mass(v.y) : 0u);
                                acc += (u64)(v.z >= lk3 ? mass(v.z) : 0u) + (v.w >= lk3 ? mass(v.w) : 0u);
                            }
                            wkeep = warp_sum_u64(acc);
                        }
                    }
                    break;
                    }
                    rw.pen_inline = rw.has_pen;                 // the rescan of one region applies penalties in place
                    ST_PROF(12);
                    const u64 woff = __shfl_sync(0xffffffffu, block_excl_scan(lane == 0 ? wkeep : 0ull, sc, total_mass), 0);
                    const u64 target = ceil_target(u, total_mass);
                    token = -1;
                    // The draw falls into one warp's region; all warps walk that region together, one 128-logit step each.
                    if (lane == 0 && total_mass > 0 && woff < target && target <= woff + wkeep) { sc->x_warp = warp; sc->x_off = woff; }
                    __syncthreads();
                    if (total_mass > 0) {
                        const float lkf = fmaxf(lcut, -ST_FLT_MAX);
                        const int x_lo = min(sc->x_warp * reg, V), x_hi = min(x_lo + reg, V);
                        const int nsteps = (x_hi - x_lo + 127) >> 7;        // at most XSTEPS
                        const u64 t2 = target - sc->x_off;                  // the crossing inside the region
                        auto step_masses = [&](int st, u64 (&q4)[4]) {
                            const int i = x_lo + st * 128 + lane * 4;
                            const float4 v = i < x_hi ? rw.load4(i) : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
                            q4[0] = v.x >= lkf ? mass(v.x) : 0u; q4[1] = v.y >= lkf ? mass(v.y) : 0u;
                            q4[2] = v.z >= lkf ? mass(v.z) : 0u; q4[3] = v.w >= lkf ? mass(v.w) : 0u;
                        };
                        for (int st = warp; st < nsteps; st += NW) {
                            u64 q4[4];
                            step_masses(st, q4);
                            const u64 ws = warp_sum_u64(q4[0] + q4[1] + q4[2] + q4[3]);
                            if (lane == 0) sc->step_sum[st] = ws;
                        }
                        __syncthreads();
                        if (warp == 0) {
                            // the step in which the running kept mass reaches t2 (four steps per lane), then its lane and logit
                            constexpr int PS = XSTEPS / 32;
                            u64 mine[PS], s = 0;
#pragma unroll
                            for (int t = 0; t < PS; ++t) { const int st = lane * PS + t; mine[t] = st < nsteps ? sc->step_sum[st] : 0ull; s += mine[t]; }
                            const u64 incl = warp_incl_scan_u64(s, lane);
                            const unsigned hit = __ballot_sync(0xffffffffu, incl >= t2);
                            int sx = -1; u64 before = 0;
                            if (hit) {
                                const int hl = __ffs(hit) - 1;
                                u64 run = incl - s; int st = lane * PS;
#pragma unroll
                                for (int t = 0; t < PS; ++t) { if (run + mine[t] >= t2) { st = lane * PS + t; break; } run += mine[t]; }
                                sx = __shfl_sync(0xffffffffu, st, hl);
                                before = __shfl_sync(0xffffffffu, run, hl);
                            }
                            if (sx >= 0) {
                                u64 q4[4];
                                step_masses(sx, q4);
                                const u64 s4 = q4[0] + q4[1] + q4[2] + q4[3];
                                const u64 inc2 = warp_incl_scan_u64(s4, lane);
                                const unsigned h2 = __ballot_sync(0xffffffffu, before + inc2 >= t2);
                                if (h2 && lane == __ffs(h2) - 1) {
                                    u64 c = before + inc2 - s4;
                                    int j = 0;
                                    for (; j < 3; ++j) { c += q4[j]; if (c >= t2) break; }
                                    if (a.out) a.out[row] = (long long)(x_lo + sx * 128 + lane * 4 + j);
                                }
                            }
                        }
                    }
                    if (total_mass == 0) { status |= COLINFER_ROW_DEGENERATE; token = aidx; }
                }
            }
        }
        __syncthreads();
        ST_PROF(13);
        if (tid == 0) {
            if (sc->hist_slow) status |= COLINFER_ROW_HIST_SLOW;
            if (token >= 0 && a.out) a.out[row] = token;          // greedy, list-path or degenerate rows
            if (a.status) a.status[row] = status;
            if (a.stats) {
                colinfer_row_stats st;
                st.lmax = L; st.lcut = lcut; st.tc = tc; st.status = status; st.argmax = aidx; st.mass_q = total_mass;
                a.stats[row] = st;
            }
        }
        break;
      }
    }
#ifdef COLINFER_PROFILE
    if (a.prof && tid == 0 && (int)blockIdx.x < a.prof_slots)
        for (int i = 0; i < 16; ++i) a.prof[(size_t)blockIdx.x * 16 + i] = sc->prof[i];
#endif
}

}  // namespace strm

