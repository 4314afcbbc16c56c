// The greedy draft of the low-rank draft heads in one launch: top-NC candidates of the approximate logits, their exact
// logits against the rows of the lm_head, the argmax and the drafter's probability of it.  The reference does this with
// nine launches (engine/spec/mtp.py:301-309, engine/spec/mtp4.py:416-423):
//
//     cand = ap.topk(NC, -1).indices;  ex = rescore(x, w, vocab_ids[cand]);  best = ex.argmax(-1)
//     ids  = vocab_ids[cand.gather(-1, best)];  p = exp(ex[best] - logsumexp(ap, -1)).clamp_max(1)
//
// Here G CTAs work on a slot.  Each of them finds the candidate set of the whole row by itself (the row is 0.28 MB and
// sits in L2 behind the GEMM that wrote it; one SM reads it at some 30 bytes per clock, so every pass over it costs about
// 5 us and there is one).  Over the head of the row first: a floor that at least NC values reach (from the threads' own
// maxima), so that nothing below it can be a candidate.  Then the pass: a running maximum and sum of exp per thread for
// the log-sum-exp; a value that reaches the floor (a few percent do; the others cost one compare) is listed in shared
// memory and counted in a 4096-bin histogram of the top 12 bits of its order-preserving key.  The histogram gives the bin
// that holds the NC-th largest value; listed values above that bin are candidates, those inside it (a few hundred) are
// ranked among themselves.  When slots are few, the G CTAs of a slot form a thread-block cluster and share even that
// pass: each keeps an interleaved 1/G of the row in registers (one round of loads), the CTAs agree on the floor through
// distributed shared memory, and every warp stores what it lists into its own stretch of the list of every CTA (a
// couple of thousand entries in all), so that each CTA runs the same selection on the same list; the log-sum-exp travels as per-CTA partial sums with the posted results.  Rows on which too much reaches the floor (values that crowd into one bin, many equal values)
// take the general route: the bin is narrowed with the next 12 and the last 8 bits of the keys, a pass each, values equal
// to the NC-th largest are taken in index order, and a last pass collects.  Each CTA then rescores the candidates whose
// index is congruent to its number modulo G (the exact logit of a row costs 5 KB of the matrix: this is where the bytes
// are), one warp per candidate with the accumulation order of colinfer_rescore_*, and posts its best.  The CTA that
// posts last picks the slot's best and writes the outputs; nobody waits for anybody.  Between candidates with the same
// exact logit the larger approximate logit wins, then the lower index: what argmax over the sorted candidate list of
// the reference gives.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cooperative_groups.h>
#include <stdint.h>
#include <limits.h>
#include <mutex>

#include "../../include/colinfer_b200.h"
#include "rescore_row.cuh"

namespace cg = cooperative_groups;

namespace dpk {

constexpr int NT = 512, NW = NT / 32;
constexpr int BINS = 4096;            // bins of one level (12 bits; the last level has 256)
constexpr int LCAP = 4096;            // listed entries (what reaches the floor; or sure ones from the front, the pivot bin's from the back)
constexpr int WCAP = LCAP / NW;       // a warp's own stretch of the list on the one-CTA fast route
constexpr int PCAP = BINS / 2;        // the pivot bin's entries, in the histogram's memory
constexpr int MAXC = 1024;            // candidates per slot at most
constexpr int RMAX = 9;               // split route: 128-bit loads a thread keeps in registers
constexpr int GSPLIT = 8;             // split route: CTAs per cluster at most (the portable cluster size)
constexpr float L2E = 1.4426950408889634f;

struct Partial { float ex; uint32_t key; int idx; float m; float s; int pad[3]; };   // m, s: this CTA's share of the log-sum-exp

struct Args {
    const float* ap; const __nv_bfloat16* x; const void* w; const uint8_t* sf; float gs; const int64_t* vocab_ids;
    int64_t* out_ids; float* out_p; int32_t* out_idx; float* out_ex;
    Partial* partials; unsigned* counters;
    int Vd, K, NC, G; long long rows_w;
};

struct Sc {
    float wf[NW]; float wsum[NW]; int wi[NW]; int wcnt[NW]; Partial wbest[NW];
    int allcnt[GSPLIT * NW];                        // split route: how much every warp of the cluster listed
    float cta_floor;
    int pivot, above, h, n_sure, n_piv, n_mine, istar;
};

struct Ctx {
    uint32_t* hist; uint32_t* pkey; int* pidx;      // BINS counters; later the pivot bin's entries (PCAP keys, PCAP indices)
    uint32_t* lkey; int* lidx;                      // LCAP
    int* mine; uint32_t* mkey;                      // MAXC: this CTA's candidates
    Sc* sc; uint4* xs;
};
constexpr size_t SMEM_FIXED = (size_t)BINS * 4 + (size_t)LCAP * 8 + (size_t)MAXC * 8 + ((sizeof(Sc) + 15) & ~size_t(15));

__device__ __forceinline__ uint32_t fkey(float x) {                  // larger value <=> larger key; NaN above everything
    const uint32_t u = __float_as_uint(x);
    if (x != x) return 0xFFFFFFFFu;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {             // the value whose key is k (a NaN for keys beyond +inf's)
    return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}
__device__ __forceinline__ float ex2_fast(float x) {                 // 2^x, 2 ulp, flushes to zero below 2^-126
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ bool better(float ex, uint32_t key, int idx, const Partial& b) {
    return ex > b.ex || (ex == b.ex && (key > b.key || (key == b.key && idx < b.idx)));
}
// (m, s) <- the log-sum-exp state of two disjoint sets: maxima m, mo and sums of exp(v - maximum) s, so
__device__ __forceinline__ void lse_merge(float& m, float& s, float mo, float so) {
    const float mm = fmaxf(m, mo);
    s = s * ex2_fast((m - mm) * L2E) + so * ex2_fast((mo - mm) * L2E);
    m = mm;
}

// f(value, index) over the row, or over its first `limit` elements: 128-bit loads when the row allows them.  Whole batches
// issue their U loads back to back, without a guard between them, before the first value is used.
constexpr int U = 8;
template <class F>
__device__ __forceinline__ void for_row(const float* row, int limit, bool vec, F f) {
    if (vec) {
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int n4 = limit >> 2;
        int i0 = threadIdx.x;
        for (; i0 + (U - 1) * NT < n4; i0 += NT * U) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = __ldg(r4 + i0 + u * NT);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = 4 * (i0 + u * NT);
                f(v[u].x, i); f(v[u].y, i + 1); f(v[u].z, i + 2); f(v[u].w, i + 3);
            }
        }
        float4 v[U];                                                 // the ragged end: clamped addresses, guarded use
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = __ldg(r4 + min(i0 + u * NT, n4 - 1));
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (i0 + u * NT < n4) {
                const int i = 4 * (i0 + u * NT);
                f(v[u].x, i); f(v[u].y, i + 1); f(v[u].z, i + 2); f(v[u].w, i + 3);
            }
    } else {
        int i0 = threadIdx.x;
        for (; i0 + (U - 1) * NT < limit; i0 += NT * U) {
            float v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = __ldg(row + i0 + u * NT);
#pragma unroll
            for (int u = 0; u < U; ++u) f(v[u], i0 + u * NT);
        }
        for (; i0 < limit; i0 += NT) f(__ldg(row + i0), i0);
    }
}

__device__ __forceinline__ int block_excl_scan(int v, Sc* sc) {      // two barriers
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += t; }
    if (lane == 31) sc->wi[warp] = inc;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += sc->wi[w];
    __syncthreads();
    return base + inc - v;
}

// The bin that holds the need-th largest of the keys counted in hist[0 .. nb): sc->pivot, with sc->above keys in the bins
// above it and sc->h in it.  Thread t owns the bins [nb - (t + 1) * per, nb - t * per), highest first.  Three barriers.
__device__ __forceinline__ void find_pivot(const uint32_t* hist, int nb, int need, Sc* sc) {
    const int tid = threadIdx.x, per = nb / NT > 0 ? nb / NT : 1;
    int tsum = 0;
    if (tid * per < nb) for (int j = 0; j < per; ++j) tsum += (int)hist[nb - 1 - (tid * per + j)];
    const int pre = block_excl_scan(tsum, sc);
    if (tid * per < nb && pre < need && need <= pre + tsum) {
        int acc = pre;
        for (int j = 0; j < per; ++j) {
            const int b = nb - 1 - (tid * per + j), c = (int)hist[b];
            if (acc + c >= need) { sc->pivot = b; sc->above = acc; sc->h = c; break; }
            acc += c;
        }
    }
    __syncthreads();
}

// The r-th largest of the warp's 32 values (every lane gets it); -inf when r > 32 or NaNs break the ranking.
__device__ __forceinline__ float warp_rth_largest(float m, int r, int lane) {
    int rank = 0;                                                    // how many lanes come before this one, largest first
#pragma unroll
    for (int l = 0; l < 32; ++l) {
        const float o = __shfl_sync(0xffffffffu, m, l);
        rank += (o > m || (o == m && l < lane)) ? 1 : 0;
    }
    const unsigned who = __ballot_sync(0xffffffffu, rank == r - 1);
    const float rth = __shfl_sync(0xffffffffu, m, who ? __ffs(who) - 1 : 0);
    return (r <= 32 && who) ? rth : -__int_as_float(0x7f800000);
}

// The selection on listed values (lkey holds their bits, lidx their indices; slot e counts when valid(e)): histogram of
// the top 12 bits of the keys, the bin of the NC-th largest, candidates above it, ranking inside it.  Fills this CTA's
// candidates (index congruent to g modulo gmask + 1).  False (nothing filled) when the pivot bin is too full.
template <class Valid>
__device__ __forceinline__ bool select_listed(const Ctx& c, int nslots, Valid valid, int NC, int g, int gmask) {
    Sc* sc = c.sc;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int e = tid; e < nslots; e += NT)
        if (valid(e)) {
            const uint32_t k = fkey(__uint_as_float(c.lkey[e]));
            c.lkey[e] = k;
            atomicAdd(&c.hist[k >> 20], 1u);
        }
    __syncthreads();
    find_pivot(c.hist, BINS, NC, sc);
    if (sc->h > PCAP) return false;
    __syncthreads();                                                 // the histogram is dead: its memory takes the pivot bin's entries
    const uint32_t pivot = (uint32_t)sc->pivot;
    const int need = NC - sc->above;
    {   // a warp counts what it will store, reserves both ranges with one atomic each, then stores by ballot
        const unsigned lt = (1u << lane) - 1u;
        int n_up = 0, n_in = 0;
        for (int e0 = warp * 32; e0 < nslots; e0 += NT) {
            const int e = e0 + lane;
            const bool ok = e < nslots && valid(e);
            const uint32_t b = ok ? c.lkey[e] >> 20 : 0u;
            n_up += __popc(__ballot_sync(0xffffffffu, ok && b > pivot && (c.lidx[e] & gmask) == g));
            n_in += __popc(__ballot_sync(0xffffffffu, ok && b == pivot));
        }
        int base_up = 0, base_in = 0;
        if (lane == 0) { base_up = n_up ? atomicAdd(&sc->n_mine, n_up) : 0; base_in = n_in ? atomicAdd(&sc->n_piv, n_in) : 0; }
        base_up = __shfl_sync(0xffffffffu, base_up, 0); base_in = __shfl_sync(0xffffffffu, base_in, 0);
        for (int e0 = warp * 32; e0 < nslots; e0 += NT) {
            const int e = e0 + lane;
            const bool ok = e < nslots && valid(e);
            const uint32_t k = ok ? c.lkey[e] : 0u; const int i = ok ? c.lidx[e] : 0;
            const bool up = ok && (k >> 20) > pivot && (i & gmask) == g, in = ok && (k >> 20) == pivot;
            const unsigned bu = __ballot_sync(0xffffffffu, up), bi = __ballot_sync(0xffffffffu, in);
            if (up) { const int p = base_up + __popc(bu & lt); c.mine[p] = i; c.mkey[p] = k; }
            if (in) { const int p = base_in + __popc(bi & lt); c.pkey[p] = k; c.pidx[p] = i; }
            base_up += __popc(bu); base_in += __popc(bi);
        }
    }
    __syncthreads();
    const int n_piv = sc->n_piv;
    for (int e = warp; e < n_piv; e += NW) {                         // one warp per entry, the lanes share the count
        const uint32_t k = c.pkey[e]; const int i = c.pidx[e];
        if ((i & gmask) != g) continue;
        int r = 0;
        if (n_piv > need) {
            for (int f = lane; f < n_piv; f += 32) r += (c.pkey[f] > k || (c.pkey[f] == k && c.pidx[f] < i)) ? 1 : 0;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        }
        if (lane == 0 && r < need) { const int p = atomicAdd(&sc->n_mine, 1); c.mine[p] = i; c.mkey[p] = k; }
    }
    return true;
}

// The general route (rows without 128-bit loads; too much reaches the floor: values crowd together, or many are equal):
// the bin of the NC-th largest key from histograms of the top 12, the next 12 and the last 8 bits of the keys, a pass
// over the row each, until what is left fits the list; values equal to the NC-th largest are taken in index order; a last
// pass collects.  Fills this CTA's candidates and returns the row's maximum and sum of exp(v - maximum).
__device__ __noinline__ void general_route(const Ctx& c, const float* row, int Vd, bool vec, float floor_v, int NC, int g, int gmask,
                                           float& mx, float& ssum) {
    Sc* sc = c.sc;
    uint32_t* hist = c.hist; uint32_t* lkey = c.lkey; int* lidx = c.lidx;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t floor_k = fkey(floor_v);
    __syncthreads();
    if (tid == 0) { sc->n_mine = 0; sc->n_piv = 0; sc->n_sure = 0; sc->istar = INT_MAX; }
    uint32_t pmask = 0, pval = 0;
    int above_total = 0, h = 0;
    for (int level = 0; level < 3 && (level == 0 || above_total + h > LCAP); ++level) {
        const int shift = level == 0 ? 20 : level == 1 ? 8 : 0, nb = level == 2 ? 256 : BINS;
        __syncthreads();
        for (int i = tid; i < nb; i += NT) hist[i] = 0;
        __syncthreads();
        const float edge = key_value(pval > floor_k ? pval : floor_k);
        float m = -3.0e38f, s = 0.f;
        for_row(row, Vd, vec, [&](float v, int) {
            if (level == 0) {                                        // the log-sum-exp rides on the first pass
                if (v > m) { s = s * ex2_fast((m - v) * L2E) + 1.0f; m = v; }
                else s += ex2_fast((v - m) * L2E);
            }
            if (!(v < edge)) {
                const uint32_t k = fkey(v);
                if (k >= floor_k && (k & pmask) == pval) atomicAdd(&hist[(k >> shift) & (uint32_t)(nb - 1)], 1u);
            }
        });
        if (level == 0) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) lse_merge(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
            if (lane == 0) { sc->wf[warp] = m; sc->wsum[warp] = s; }
        }
        __syncthreads();
        if (level == 0) {
            mx = sc->wf[0]; ssum = 0.f;
            for (int w = 1; w < NW; ++w) mx = fmaxf(mx, sc->wf[w]);
            for (int w = 0; w < NW; ++w) ssum += sc->wsum[w] * ex2_fast((sc->wf[w] - mx) * L2E);
        }
        find_pivot(hist, nb, NC - above_total, sc);
        above_total += sc->above; h = sc->h;
        pval |= (uint32_t)sc->pivot << shift; pmask |= (uint32_t)(nb - 1) << shift;
    }
    __syncthreads();
    const int need = NC - above_total;                               // how many of the pivot bin's entries are taken

    // more keys equal to the NC-th largest than fit: they are taken in index order, up to sc->istar
    if (above_total + h > LCAP) {
        const int seg = (((Vd + NW - 1) / NW) + 31) & ~31, lo = warp * seg, hi = min(Vd, lo + seg);
        int cnt = 0;
        for (int base = lo; base < hi; base += 32) {
            const int i = base + lane;
            const bool eq = i < hi && fkey(__ldg(row + i)) == pval;
            cnt += __popc(__ballot_sync(0xffffffffu, eq));
        }
        if (lane == 0) sc->wi[warp] = cnt;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += sc->wi[w];
        if (before < need && need <= before + cnt) {                 // the need-th equal key lies in this warp's segment
            int running = before;
            for (int base = lo; base < hi; base += 32) {
                const int i = base + lane;
                const bool eq = i < hi && fkey(__ldg(row + i)) == pval;
                const unsigned bal = __ballot_sync(0xffffffffu, eq);
                const int pc = __popc(bal);
                if (running + pc >= need) {
                    const int kth = need - running;                  // 1-based among this chunk's set bits
                    if (eq && __popc(bal & ((2u << lane) - 1u)) == kth) sc->istar = i;
                    break;
                }
                running += pc;
            }
        }
        __syncthreads();
    }
    const int istar = sc->istar;

    // collect: above the pivot bin from the front of the list, inside it from the back
    const float edge = key_value(pval > floor_k ? pval : floor_k);
    for_row(row, Vd, vec, [&](float v, int i) {
        if (!(v < edge)) {
            const uint32_t k = fkey(v), pre = k & pmask;
            if (pre > pval) { const int p = atomicAdd(&sc->n_sure, 1); lkey[p] = k; lidx[p] = i; }
            else if (pre == pval && k >= floor_k && i <= istar) { const int p = atomicAdd(&sc->n_piv, 1); lkey[LCAP - 1 - p] = k; lidx[LCAP - 1 - p] = i; }
        }
    });
    __syncthreads();
    const int n_sure = sc->n_sure, n_piv = sc->n_piv;
    for (int e = tid; e < n_sure; e += NT)
        if ((lidx[e] & gmask) == g) { const int p = atomicAdd(&sc->n_mine, 1); c.mine[p] = lidx[e]; c.mkey[p] = lkey[e]; }
    for (int e = warp; e < n_piv; e += NW) {
        const uint32_t k = lkey[LCAP - 1 - e]; const int i = lidx[LCAP - 1 - e];
        if ((i & gmask) != g) continue;
        int r = 0;
        if (n_piv > need) {
            for (int f = lane; f < n_piv; f += 32) {
                const uint32_t kf = lkey[LCAP - 1 - f]; const int jf = lidx[LCAP - 1 - f];
                r += (kf > k || (kf == k && jf < i)) ? 1 : 0;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        }
        if (lane == 0 && r < need) { const int p = atomicAdd(&sc->n_mine, 1); c.mine[p] = i; c.mkey[p] = k; }
    }
}

template <bool FP4, bool SPLIT>
__global__ void __launch_bounds__(NT, SPLIT ? 1 : 2) k_draft_pick(const Args a) {
    extern __shared__ __align__(16) unsigned char smem[];
    Ctx c;
    c.hist = reinterpret_cast<uint32_t*>(smem);
    c.pkey = c.hist; c.pidx = reinterpret_cast<int*>(c.hist + PCAP);
    c.lkey = c.hist + BINS; c.lidx = reinterpret_cast<int*>(c.lkey + LCAP);
    c.mine = c.lidx + LCAP; c.mkey = reinterpret_cast<uint32_t*>(c.mine + MAXC);
    c.sc = reinterpret_cast<Sc*>(c.mkey + MAXC);
    c.xs = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(c.sc) + ((sizeof(Sc) + 15) & ~size_t(15)));
    Sc* sc = c.sc;

    const int n = blockIdx.y, g = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Vd = a.Vd, NC = a.NC, G = a.G, gmask = G - 1;
    const float* row = a.ap + (size_t)n * Vd;
    const bool vec = (Vd & 3) == 0 && ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
    const float ninf = -__int_as_float(0x7f800000);

    if (tid == 0) { sc->n_sure = 0; sc->n_piv = 0; sc->n_mine = 0; sc->istar = INT_MAX; sc->pivot = 0; sc->above = 0; sc->h = 0; }
    for (int i = tid; i < BINS; i += NT) c.hist[i] = 0;

    auto stage_x = [&]() {                                           // the slot's activations, once per CTA
        const uint4* xg = reinterpret_cast<const uint4*>(a.x + (size_t)n * a.K);
        for (int i = tid; i < (a.K >> 3); i += NT) c.xs[i] = __ldg(xg + i);
    };
    float floor_v = ninf;
    float m_part = -3.0e38f, s_part = 0.f;                           // this CTA's share of the slot's log-sum-exp
    bool fast = vec;

    if (SPLIT) {
        // ---- the slot's G CTAs are a cluster: an interleaved 1/G of the row in this CTA's registers, one round of loads
        // (the host launches this route only for rows with 128-bit loads that fit: ceil(Vd / 4 / (G * NT)) <= RMAX)
        cg::cluster_group cluster = cg::this_cluster();
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int n4 = Vd >> 2;
        float4 v[RMAX];
#pragma unroll
        for (int j = 0; j < RMAX; ++j) v[j] = __ldg(r4 + min((j * G + g) * NT + tid, n4 - 1));
        stage_x();                                                   // while those loads are in flight
        float m = ninf;
#pragma unroll
        for (int j = 0; j < RMAX; ++j)
            if ((j * G + g) * NT + tid < n4) m = fmaxf(m, fmaxf(fmaxf(v[j].x, v[j].y), fmaxf(v[j].z, v[j].w)));
        // the floor: with r = ceil(NC / (NW * G)), the r-th largest of a warp's 32 thread maxima has r values at or above
        // it; the smallest such value over the cluster's G * NW warps has at least NC
        const float rth = warp_rth_largest(m, (NC + NW * G - 1) / (NW * G), lane);
        m = fmaxf(m, -3.0e38f);                                      // finite from here on, so that -inf values add exp(-inf) = 0
        if (lane == 0) sc->wf[warp] = rth;
        __syncthreads();
        if (tid == 0) { float f = sc->wf[0]; for (int w = 1; w < NW; ++w) f = fminf(f, sc->wf[w]); sc->cta_floor = f; }
        cluster.sync();
        {
            float f = *cluster.map_shared_rank(&sc->cta_floor, 0);
            for (int q = 1; q < G; ++q) f = fminf(f, *cluster.map_shared_rank(&sc->cta_floor, q));
            if (f == f) floor_v = f;
        }
        // this CTA's share of the log-sum-exp, and its list of what reaches the floor: warp w of CTA g owns the stretch
        // (g * NW + w) * SW of the list, in every CTA of the cluster (a ballot and a count per warp)
        const int SW = LCAP / (G * NW), sbase = (g * NW + warp) * SW;
        float* lval = reinterpret_cast<float*>(c.lkey);
        float s = 0.f;
        int cnt = 0;
        const unsigned lt = (1u << lane) - 1u;
#pragma unroll
        for (int j = 0; j < RMAX; ++j) {
            const int i4 = (j * G + g) * NT + tid;
            const bool valid = i4 < n4;
            const float q = (ex2_fast((v[j].x - m) * L2E) + ex2_fast((v[j].y - m) * L2E)) + (ex2_fast((v[j].z - m) * L2E) + ex2_fast((v[j].w - m) * L2E));
            s += valid ? q : 0.f;
            const float c4[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const bool pass = valid && !(c4[e] < floor_v);
                const unsigned bal = __ballot_sync(0xffffffffu, pass);
                if (bal) {
                    const int pos = cnt + __popc(bal & lt);
                    if (pass && pos < SW) { lval[sbase + pos] = c4[e]; c.lidx[sbase + pos] = 4 * i4 + e; }
                    cnt += __popc(bal);
                }
            }
        }
        __syncwarp();
        for (int q = 1; q < G; ++q) {                                // the stretch and its count go to the other CTAs
            const int peer = (g + q) & gmask;
            float* pv = cluster.map_shared_rank(lval, peer); int* pi = cluster.map_shared_rank(c.lidx, peer);
            for (int e = lane; e < min(cnt, SW); e += 32) { pv[sbase + e] = lval[sbase + e]; pi[sbase + e] = c.lidx[sbase + e]; }
        }
        if (lane < G) cluster.map_shared_rank(sc, lane)->allcnt[g * NW + warp] = cnt;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lse_merge(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
        if (lane == 0) { sc->wf[warp] = m; sc->wsum[warp] = s; }
        cluster.sync();                                              // the last touch of another CTA's memory lies before this
        m_part = sc->wf[0]; s_part = 0.f;
        for (int w = 1; w < NW; ++w) m_part = fmaxf(m_part, sc->wf[w]);
        for (int w = 0; w < NW; ++w) s_part += sc->wsum[w] * ex2_fast((sc->wf[w] - m_part) * L2E);
        int over = tid < G * NW && sc->allcnt[tid] > SW;
        fast = !__syncthreads_or(over);
        const int sh = 31 - __clz(SW);
        if (fast) fast = select_listed(c, LCAP, [&](int e) { return (e & (SW - 1)) < sc->allcnt[e >> sh]; }, NC, g, gmask);
    } else {
        stage_x();
        // ---- one CTA reads the whole row.  A floor from the head of the row first (each thread's first batch of loads):
        // with r = ceil(NC / NW), the smallest over the warps of the r-th largest thread maximum has at least NC values
        // at or above it
        {
            float m = ninf;
            for_row(row, min(Vd, NT * U * 4), vec, [&](float v, int) { m = fmaxf(m, v); });
            const float rth = warp_rth_largest(m, (NC + NW - 1) / NW, lane);
            if (lane == 0) sc->wf[warp] = rth;
            __syncthreads();
            float l2 = sc->wf[0];
            for (int w = 1; w < NW; ++w) l2 = fminf(l2, sc->wf[w]);
            if (l2 == l2) floor_v = l2;
            __syncthreads();
        }
        // the fast route, one pass over the whole row (rows read with 128-bit loads).  Per batch of U loads: the running
        // maximum and sum of exp of the thread (no branch: one rescale per batch); and each value that reaches the floor
        // is listed in the warp's own stretch of the list (a ballot and a count per warp: no atomics)
        if (fast) {
            const float4* r4 = reinterpret_cast<const float4*>(row);
            const int n4 = Vd >> 2, wbase = warp * WCAP;
            const unsigned lt = (1u << lane) - 1u;
            float* lval = reinterpret_cast<float*>(c.lkey);          // values first; their keys take their place later
            float m = -3.0e38f, s = 0.f;                             // finite, so that -inf values add exp(-inf) = 0
            int cnt = 0;                                             // the same in every lane
            for (int b0 = 0; b0 < n4; b0 += NT * U) {
                const int i0 = b0 + tid;
                const bool full = b0 + NT * U <= n4;                 // the same for the whole CTA
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) v[u] = __ldg(r4 + (full ? i0 + u * NT : min(i0 + u * NT, n4 - 1)));
                float bm = ninf;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float q = fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w));
                    bm = (full || i0 + u * NT < n4) ? fmaxf(bm, q) : bm;
                }
                const float nm = fmaxf(m, bm);
                s *= ex2_fast((m - nm) * L2E);
                m = nm;
                float t = 0.f;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float q = (ex2_fast((v[u].x - m) * L2E) + ex2_fast((v[u].y - m) * L2E)) +
                                    (ex2_fast((v[u].z - m) * L2E) + ex2_fast((v[u].w - m) * L2E));
                    t += (full || i0 + u * NT < n4) ? q : 0.f;
                }
                s += t;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const bool valid = full || i0 + u * NT < n4;
                    const float c4[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const bool pass = valid && !(c4[e] < floor_v);
                        const unsigned bal = __ballot_sync(0xffffffffu, pass);
                        if (bal) {
                            const int pos = cnt + __popc(bal & lt);
                            if (pass && pos < WCAP) { lval[wbase + pos] = c4[e]; c.lidx[wbase + pos] = 4 * (i0 + u * NT) + e; }
                            cnt += __popc(bal);
                        }
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) lse_merge(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
            if (lane == 0) { sc->wf[warp] = m; sc->wsum[warp] = s; sc->wcnt[warp] = cnt; }
            __syncthreads();
            float mx = sc->wf[0], ssum = 0.f;
            for (int w = 1; w < NW; ++w) mx = fmaxf(mx, sc->wf[w]);
            for (int w = 0; w < NW; ++w) { ssum += sc->wsum[w] * ex2_fast((sc->wf[w] - mx) * L2E); fast = fast && sc->wcnt[w] <= WCAP; }
            if (g == 0) { m_part = mx; s_part = ssum; }              // every CTA has the whole sum: the first one posts it
            if (fast) fast = select_listed(c, LCAP, [&](int e) { return (e & (WCAP - 1)) < sc->wcnt[e / WCAP]; }, NC, g, gmask);
        }
    }
    if (!fast) {
        float mx, ssum;
        general_route(c, row, Vd, vec, floor_v, NC, g, gmask, mx, ssum);
        m_part = g == 0 ? mx : -3.0e38f;                             // every CTA has the whole sum: the first one posts it
        s_part = g == 0 ? ssum : 0.f;
    }
    __syncthreads();
    const int n_mine = sc->n_mine;

    // ---- exact logits of this CTA's candidates, one warp each (the loads of a whole row of the matrix in flight at once
    // where the registers allow it); the warp's best
    Partial best; best.ex = ninf; best.key = 0; best.idx = INT_MAX; best.m = m_part; best.s = s_part;
    long long my_row = -1;
    for (int j = warp, t = 0; j < n_mine; j += NW, ++t) {
        if ((t & 31) == 0) {                                         // the lm_head rows of this warp's next 32 candidates, one per
            const int jj = j + lane * NW;                            // lane: looked up at once, not one per round trip
            my_row = -1;
            if (jj < n_mine) { const int id = c.mine[jj]; my_row = a.vocab_ids ? (long long)__ldg(a.vocab_ids + id) : (long long)id; }
        }
        const int idx = c.mine[j];
        const long long r = __shfl_sync(0xffffffffu, my_row, t & 31);
        float ex = __int_as_float(0x7fc00000);                        // a row outside the matrix: NaN, never chosen
        if (r >= 0 && r < a.rows_w) {
            if (FP4) ex = rsc::dot_row_nvfp4<(SPLIT ? 10 : 4)>(c.xs, reinterpret_cast<const uint8_t*>(a.w), a.sf, r, a.K, lane) * a.gs;
            else     ex = rsc::dot_row_bf16<(SPLIT ? 10 : 4)>(c.xs, reinterpret_cast<const __nv_bfloat16*>(a.w), r, a.K, lane);
        }
        if (better(ex, c.mkey[j], idx, best)) { best.ex = ex; best.key = c.mkey[j]; best.idx = idx; }
    }
    if (lane == 0) sc->wbest[warp] = best;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < NW; ++w) { const Partial o = sc->wbest[w]; if (better(o.ex, o.key, o.idx, best)) { best.ex = o.ex; best.key = o.key; best.idx = o.idx; } }
        a.partials[(size_t)n * G + g] = best;
        __threadfence();
        const unsigned ticket = atomicAdd(&a.counters[n], 1u);
        if (ticket == (unsigned)(G - 1)) {                           // every CTA of the slot has posted
            __threadfence();
            const volatile Partial* ps = a.partials + (size_t)n * G;
            Partial top; top.ex = ps[0].ex; top.key = ps[0].key; top.idx = ps[0].idx;
            float m = ps[0].m, s = ps[0].s;
            for (int q = 1; q < G; ++q) {
                Partial o; o.ex = ps[q].ex; o.key = ps[q].key; o.idx = ps[q].idx;
                if (better(o.ex, o.key, o.idx, top)) { top.ex = o.ex; top.key = o.key; top.idx = o.idx; }
                lse_merge(m, s, ps[q].m, ps[q].s);
            }
            const bool found = top.idx != INT_MAX;
            const int idx = found ? top.idx : -1;
            a.out_ids[n] = !found ? -1 : a.vocab_ids ? __ldg(a.vocab_ids + idx) : (int64_t)idx;
            const float lse = m + logf(s);
            if (a.out_p) a.out_p[n] = fminf(expf(top.ex - lse), 1.0f);
            if (a.out_idx) a.out_idx[n] = idx;
            if (a.out_ex) a.out_ex[n] = top.ex;
            // the scratch is left zero-filled, as found: a later call may lay it out for another number of slots
            uint4* z = reinterpret_cast<uint4*>(a.partials + (size_t)n * G);
            for (int q = 0; q < G * (int)(sizeof(Partial) / sizeof(uint4)); ++q) z[q] = make_uint4(0, 0, 0, 0);
            a.counters[n] = 0;
        }
    }
}

// The kernels' dynamic shared memory (up to about 110 KB with K = 16384) goes beyond the default limit: opted in once per device.
static cudaError_t opt_in() {
    static std::mutex mu;
    static bool done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
    const int bytes = (int)(SMEM_FIXED + 16 * 1024 * 2);
    e = cudaFuncSetAttribute(k_draft_pick<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_draft_pick<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_draft_pick<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_draft_pick<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
    return e;
}

}  // namespace dpk

extern "C" int64_t colinfer_draft_pick_scratch_bytes(int N) {
    return (int64_t)(N > 0 ? N : 0) * (int64_t)(16 * sizeof(dpk::Partial) + 16);
}

// Replaces the draft() block of the low-rank heads (engine/spec/mtp.py:301-309, engine/spec/mtp4.py:416-423).
extern "C" int colinfer_draft_pick(const float* ap, const void* x, const void* w, const void* sf, float gs, int w_format,
                                   const int64_t* vocab_ids, int64_t* out_ids, float* out_p, int32_t* out_idx, float* out_ex,
                                   int N, int Vd, int K, int NC, int64_t rows_w, int ctas_per_slot, void* scratch, int64_t scratch_bytes,
                                   void* stream) {
    const bool fp4 = w_format == COLINFER_W_NVFP4;
    if (N < 0 || Vd < 1 || NC < 1 || NC > dpk::MAXC || NC > Vd || rows_w < 1 || K < (fp4 ? 16 : 8) || (K % (fp4 ? 16 : 8)) != 0 ||
        K > 16 * 1024 || (w_format != COLINFER_W_BF16 && !fp4) ||
        (ctas_per_slot != 0 && ctas_per_slot != 1 && ctas_per_slot != 2 && ctas_per_slot != 4 && ctas_per_slot != 8 && ctas_per_slot != 16))
        return (int)cudaErrorInvalidValue;
    if (N == 0) return (int)cudaSuccess;
    if (!ap || !x || !w || !out_ids || !scratch || (fp4 && !sf) || N > 65535 || (((uintptr_t)x) & 15) || (((uintptr_t)w) & 15) ||
        (((uintptr_t)scratch) & 15) || scratch_bytes < colinfer_draft_pick_scratch_bytes(N))
        return (int)cudaErrorInvalidValue;
    // CTAs per slot: as many as fill the part once when slots are few.  4 or 8 of them share the reading of the row as a
    // cluster when the row allows it (128-bit loads, a share that fits the registers); otherwise every CTA reads all of it.
    const int G = ctas_per_slot ? ctas_per_slot : N <= 9 ? 8 : N <= 37 ? 4 : N <= 74 ? 2 : 1;
    const bool split = (G == 4 || G == 8) && (Vd & 3) == 0 && (((uintptr_t)ap) & 15) == 0 &&
                       ((Vd >> 2) + G * dpk::NT - 1) / (G * dpk::NT) <= dpk::RMAX;
    dpk::Args a;
    a.ap = ap; a.x = (const __nv_bfloat16*)x; a.w = w; a.sf = (const uint8_t*)sf; a.gs = gs; a.vocab_ids = vocab_ids;
    a.out_ids = out_ids; a.out_p = out_p; a.out_idx = out_idx; a.out_ex = out_ex;
    a.partials = reinterpret_cast<dpk::Partial*>(scratch);
    a.counters = reinterpret_cast<unsigned*>(reinterpret_cast<unsigned char*>(scratch) + (size_t)N * 16 * sizeof(dpk::Partial));
    a.Vd = Vd; a.K = K; a.NC = NC; a.G = G; a.rows_w = (long long)rows_w;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = dpk::opt_in();
    if (e != cudaSuccess) return (int)e;
    const size_t smem = dpk::SMEM_FIXED + (size_t)K * 2;
    if (split) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(G, N); cfg.blockDim = dim3(dpk::NT); cfg.dynamicSmemBytes = smem; cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = G; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        e = fp4 ? cudaLaunchKernelEx(&cfg, dpk::k_draft_pick<true, true>, a) : cudaLaunchKernelEx(&cfg, dpk::k_draft_pick<false, true>, a);
        return (int)(e != cudaSuccess ? e : cudaGetLastError());
    }
    if (fp4) dpk::k_draft_pick<true, false><<<dim3(G, N), dpk::NT, smem, st>>>(a);
    else     dpk::k_draft_pick<false, false><<<dim3(G, N), dpk::NT, smem, st>>>(a);
    return (int)cudaGetLastError();
}
