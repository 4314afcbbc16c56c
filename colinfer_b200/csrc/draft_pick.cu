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
// ranked among themselves.  Rows on which too much reaches the floor (values that crowd into one bin, many equal values)
// take the general route: the bin is narrowed with the next 12 and the last 8 bits of the keys, a pass each, values equal
// to the NC-th largest are taken in index order, and a last pass collects.  Each CTA then rescores the candidates whose
// index is congruent to its number modulo G (the exact logit of a row costs 5 KB of the matrix: this is where the bytes
// are), one warp per candidate with the accumulation order of colinfer_rescore_*, and posts its best.  The CTA that
// posts last picks the slot's best and writes the outputs; nobody waits for anybody.  Between candidates with the same
// exact logit the larger approximate logit wins, then the lower index: what argmax over the sorted candidate list of
// the reference gives.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <limits.h>
#include <mutex>

#include "../../include/colinfer_b200.h"
#include "rescore_row.cuh"

namespace dpk {

constexpr int NT = 512, NW = NT / 32;
constexpr int BINS = 4096;            // bins of one level (12 bits; the last level has 256)
constexpr int LCAP = 4096;            // listed entries (what reaches the floor; or sure ones from the front, the pivot bin's from the back)
constexpr int WCAP = LCAP / NW;        // a warp's own stretch of the list on the fast route
constexpr int PCAP = BINS / 2;        // the pivot bin's entries, in the histogram's memory
constexpr int MAXC = 1024;            // candidates per slot at most

struct Partial { float ex; uint32_t key; int idx; int pad; };

struct Args {
    const float* ap; const __nv_bfloat16* x; const void* w; const uint8_t* sf; float gs; const int64_t* vocab_ids;
    int64_t* out_ids; float* out_p; int32_t* out_idx; float* out_ex;
    Partial* partials; unsigned* counters;
    int Vd, K, NC, G; long long rows_w;
};

struct Sc {
    float wf[NW]; float wsum[NW]; int wi[NW]; int wcnt[NW]; Partial wbest[NW];
    int pivot, above, h, n_sure, n_piv, n_mine, istar;
};

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

template <bool FP4>
__global__ void __launch_bounds__(NT) k_draft_pick(const Args a) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint32_t* hist = reinterpret_cast<uint32_t*>(smem);                                 // BINS; later the pivot bin's entries:
    uint32_t* pkey = hist;                                                              //   PCAP keys
    int* pidx = reinterpret_cast<int*>(hist + PCAP);                                    //   PCAP indices
    uint32_t* lkey = hist + BINS;                                                       // LCAP
    int* lidx = reinterpret_cast<int*>(lkey + LCAP);                                    // LCAP
    int* mine = lidx + LCAP;                                                            // MAXC
    uint32_t* mkey = reinterpret_cast<uint32_t*>(mine + MAXC);                          // MAXC
    Sc* sc = reinterpret_cast<Sc*>(mkey + MAXC);
    uint4* xs = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(sc) + ((sizeof(Sc) + 15) & ~size_t(15)));

    const int n = blockIdx.y, g = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Vd = a.Vd, NC = a.NC, gmask = a.G - 1;
    const float* row = a.ap + (size_t)n * Vd;
    const bool vec = (Vd & 3) == 0 && ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
    const float ninf = -__int_as_float(0x7f800000), L2E = 1.4426950408889634f;

    {   // the slot's activations, once per CTA
        const uint4* xg = reinterpret_cast<const uint4*>(a.x + (size_t)n * a.K);
        for (int c = tid; c < (a.K >> 3); c += NT) xs[c] = __ldg(xg + c);
    }
    if (tid == 0) { sc->n_sure = 0; sc->n_piv = 0; sc->n_mine = 0; sc->istar = INT_MAX; sc->pivot = 0; sc->above = 0; sc->h = 0; }
    for (int i = tid; i < BINS; i += NT) hist[i] = 0;

    // ---- a floor under the candidates, from the head of the row (each thread's first batch of loads): with r = ceil(NC / NW),
    // the r-th largest of a warp's 32 thread maxima has r values at or above it, so the smallest such value over the NW
    // warps has at least NC: nothing below it can be a candidate
    float floor_v = ninf;
    {
        float m = ninf;
        for_row(row, min(Vd, NT * U * 4), vec, [&](float v, int) { m = fmaxf(m, v); });
        const int r = (NC + NW - 1) / NW;
        int rank = 0;                                                // how many lanes come before this one, largest first
#pragma unroll
        for (int l = 0; l < 32; ++l) {
            const float o = __shfl_sync(0xffffffffu, m, l);
            rank += (o > m || (o == m && l < lane)) ? 1 : 0;
        }
        const unsigned who = __ballot_sync(0xffffffffu, rank == r - 1);
        const float rth = __shfl_sync(0xffffffffu, m, who ? __ffs(who) - 1 : 0);
        if (lane == 0) sc->wf[warp] = (r <= 32 && who) ? rth : ninf;  // NaN maxima break the ranks: no floor then
        __syncthreads();
        float l2 = sc->wf[0];
        for (int w = 1; w < NW; ++w) l2 = fminf(l2, sc->wf[w]);
        if (l2 == l2) floor_v = l2;
        __syncthreads();
    }
    const uint32_t floor_k = fkey(floor_v);

    // ---- the fast route, one pass over the whole row (rows read with 128-bit loads).  Per batch of U loads: the running
    // maximum and sum of exp of the thread (the log-sum-exp; no branch: one rescale per batch); and each value that reaches
    // the floor is listed in the warp's own stretch of the list (a ballot and a count per warp: no atomics)
    float mx = ninf, ssum = 0.f;
    bool fast = vec;
    if (fast) {
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int n4 = Vd >> 2, wbase = warp * WCAP;
        const unsigned lt = (1u << lane) - 1u;
        float* lval = reinterpret_cast<float*>(lkey);                // values first; their keys take their place below
        float m = -3.0e38f, s = 0.f;                                 // finite, so that -inf values add exp(-inf) = 0
        int cnt = 0;                                                 // the same in every lane
        for (int b0 = 0; b0 < n4; b0 += NT * U) {
            const int i0 = b0 + tid;
            const bool full = b0 + NT * U <= n4;                     // the same for the whole CTA
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
                for (int c = 0; c < 4; ++c) {
                    const bool pass = valid && !(c4[c] < floor_v);
                    const unsigned bal = __ballot_sync(0xffffffffu, pass);
                    if (bal) {
                        const int pos = cnt + __popc(bal & lt);
                        if (pass && pos < WCAP) { lval[wbase + pos] = c4[c]; lidx[wbase + pos] = 4 * (i0 + u * NT) + c; }
                        cnt += __popc(bal);
                    }
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m, o), so = __shfl_xor_sync(0xffffffffu, s, o);
            const float mm = fmaxf(m, mo);
            s = s * ex2_fast((m - mm) * L2E) + so * ex2_fast((mo - mm) * L2E);
            m = mm;
        }
        if (lane == 0) { sc->wf[warp] = m; sc->wsum[warp] = s; sc->wcnt[warp] = cnt; }
        __syncthreads();
        mx = sc->wf[0];
        for (int w = 1; w < NW; ++w) mx = fmaxf(mx, sc->wf[w]);
        for (int w = 0; w < NW; ++w) { ssum += sc->wsum[w] * ex2_fast((sc->wf[w] - mx) * L2E); fast = fast && sc->wcnt[w] <= WCAP; }
    }
    if (fast) {
        // the histogram of the top 12 bits of the listed values' keys, and the bin that holds the NC-th largest of them
        for (int e = tid; e < LCAP; e += NT)
            if ((e & (WCAP - 1)) < sc->wcnt[e / WCAP]) {
                const uint32_t k = fkey(__uint_as_float(lkey[e]));
                lkey[e] = k;
                atomicAdd(&hist[k >> 20], 1u);
            }
        __syncthreads();
        find_pivot(hist, BINS, NC, sc);
        fast = sc->h <= PCAP;
        __syncthreads();                                             // the histogram is dead: its memory takes the pivot bin's entries
    }
    if (fast) {
        // ---- listed values above the pivot bin are candidates; those inside it are ranked among themselves
        const uint32_t pivot = (uint32_t)sc->pivot;
        const int need = NC - sc->above;
        for (int e = tid; e < LCAP; e += NT)
            if ((e & (WCAP - 1)) < sc->wcnt[e / WCAP]) {
                const uint32_t k = lkey[e]; const int i = lidx[e];
                if ((k >> 20) > pivot) { if ((i & gmask) == g) { const int p = atomicAdd(&sc->n_mine, 1); mine[p] = i; mkey[p] = k; } }
                else if ((k >> 20) == pivot) { const int p = atomicAdd(&sc->n_piv, 1); pkey[p] = k; pidx[p] = i; }
            }
        __syncthreads();
        const int n_piv = sc->n_piv;
        for (int e = warp; e < n_piv; e += NW) {                     // one warp per entry, the lanes share the count
            const uint32_t k = pkey[e]; const int i = pidx[e];
            if ((i & gmask) != g) continue;
            int r = 0;
            if (n_piv > need) {
                for (int f = lane; f < n_piv; f += 32) r += (pkey[f] > k || (pkey[f] == k && pidx[f] < i)) ? 1 : 0;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
            }
            if (lane == 0 && r < need) { const int p = atomicAdd(&sc->n_mine, 1); mine[p] = i; mkey[p] = k; }
        }
    } else {
        // ---- the general route (rows without 128-bit loads; too much reaches the floor: values crowd together, or many
        // are equal): the bin of the NC-th largest key from histograms of the top 12, the next 12 and the last 8 bits of
        // the keys, a pass over the row each, until what is left fits the list
        if (tid == 0) { sc->n_mine = 0; sc->n_piv = 0; sc->n_sure = 0; }
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
                if (level == 0) {                                    // the log-sum-exp rides on the first pass
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
                for (int o = 16; o > 0; o >>= 1) {
                    const float mo = __shfl_xor_sync(0xffffffffu, m, o), so = __shfl_xor_sync(0xffffffffu, s, o);
                    const float mm = fmaxf(m, mo);
                    s = s * ex2_fast((m - mm) * L2E) + so * ex2_fast((mo - mm) * L2E);
                    m = mm;
                }
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
        const int need = NC - above_total;                           // how many of the pivot bin's entries are taken

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
            if (before < need && need <= before + cnt) {             // the need-th equal key lies in this warp's segment
                int running = before;
                for (int base = lo; base < hi; base += 32) {
                    const int i = base + lane;
                    const bool eq = i < hi && fkey(__ldg(row + i)) == pval;
                    const unsigned bal = __ballot_sync(0xffffffffu, eq);
                    const int pc = __popc(bal);
                    if (running + pc >= need) {
                        const int kth = need - running;              // 1-based among this chunk's set bits
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
            if ((lidx[e] & gmask) == g) { const int p = atomicAdd(&sc->n_mine, 1); mine[p] = lidx[e]; mkey[p] = lkey[e]; }
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
            if (lane == 0 && r < need) { const int p = atomicAdd(&sc->n_mine, 1); mine[p] = i; mkey[p] = k; }
        }
    }
    __syncthreads();
    const int n_mine = sc->n_mine;

    // ---- exact logits of this CTA's candidates, one warp each; the warp's best
    Partial best; best.ex = -__int_as_float(0x7f800000); best.key = 0; best.idx = INT_MAX; best.pad = 0;
    for (int j = warp; j < n_mine; j += NW) {
        const int idx = mine[j];
        const long long r = a.vocab_ids ? (long long)__ldg(a.vocab_ids + idx) : (long long)idx;
        float ex = __int_as_float(0x7fc00000);                        // a row outside the matrix: NaN, never chosen
        if (r >= 0 && r < a.rows_w) {
            if (FP4) ex = rsc::dot_row_nvfp4(xs, reinterpret_cast<const uint8_t*>(a.w), a.sf, r, a.K, lane) * a.gs;
            else     ex = rsc::dot_row_bf16(xs, reinterpret_cast<const __nv_bfloat16*>(a.w), r, a.K, lane);
        }
        if (better(ex, mkey[j], idx, best)) { best.ex = ex; best.key = mkey[j]; best.idx = idx; }
    }
    if (lane == 0) sc->wbest[warp] = best;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < NW; ++w) { const Partial o = sc->wbest[w]; if (better(o.ex, o.key, o.idx, best)) best = o; }
        a.partials[(size_t)n * a.G + g] = best;
        __threadfence();
        const unsigned ticket = atomicAdd(&a.counters[n], 1u);
        if (ticket == (unsigned)(a.G - 1)) {                         // every CTA of the slot has posted
            __threadfence();
            const volatile Partial* ps = a.partials + (size_t)n * a.G;
            Partial top; top.ex = ps[0].ex; top.key = ps[0].key; top.idx = ps[0].idx; top.pad = 0;
            for (int q = 1; q < a.G; ++q) {
                Partial o; o.ex = ps[q].ex; o.key = ps[q].key; o.idx = ps[q].idx;
                if (better(o.ex, o.key, o.idx, top)) top = o;
            }
            const bool found = top.idx != INT_MAX;
            const int idx = found ? top.idx : -1;
            a.out_ids[n] = !found ? -1 : a.vocab_ids ? __ldg(a.vocab_ids + idx) : (int64_t)idx;
            const float lse = mx + logf(ssum);
            if (a.out_p) a.out_p[n] = fminf(expf(top.ex - lse), 1.0f);
            if (a.out_idx) a.out_idx[n] = idx;
            if (a.out_ex) a.out_ex[n] = top.ex;
        }
    }
}

// The kernels' dynamic shared memory (up to 96 KB with K = 16384) goes beyond the default limit: opted in once per device.
static cudaError_t opt_in(bool fp4) {
    static std::mutex mu;
    static bool done[2][64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && done[fp4][dev]) return cudaSuccess;
    e = fp4 ? cudaFuncSetAttribute(k_draft_pick<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)
            : cudaFuncSetAttribute(k_draft_pick<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e == cudaSuccess && dev >= 0 && dev < 64) done[fp4][dev] = true;
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
    // CTAs per slot: every one of them reads the whole row of approximate logits, so no more than fill the part once
    const int G = ctas_per_slot ? ctas_per_slot : N <= 9 ? 16 : N <= 18 ? 8 : N <= 37 ? 4 : N <= 74 ? 2 : 1;
    dpk::Args a;
    a.ap = ap; a.x = (const __nv_bfloat16*)x; a.w = w; a.sf = (const uint8_t*)sf; a.gs = gs; a.vocab_ids = vocab_ids;
    a.out_ids = out_ids; a.out_p = out_p; a.out_idx = out_idx; a.out_ex = out_ex;
    a.partials = reinterpret_cast<dpk::Partial*>(scratch);
    a.counters = reinterpret_cast<unsigned*>(reinterpret_cast<unsigned char*>(scratch) + (size_t)N * 16 * sizeof(dpk::Partial));
    a.Vd = Vd; a.K = K; a.NC = NC; a.G = G; a.rows_w = (long long)rows_w;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(a.counters, 0, (size_t)N * sizeof(unsigned), st);
    if (e != cudaSuccess) return (int)e;
    const size_t smem = (size_t)dpk::BINS * 4 + (size_t)dpk::LCAP * 8 + (size_t)dpk::MAXC * 8 + ((sizeof(dpk::Sc) + 15) & ~size_t(15)) + (size_t)K * 2;
    e = dpk::opt_in(fp4);
    if (e != cudaSuccess) return (int)e;
    if (fp4) dpk::k_draft_pick<true><<<dim3(G, N), dpk::NT, smem, st>>>(a);
    else     dpk::k_draft_pick<false><<<dim3(G, N), dpk::NT, smem, st>>>(a);
    return (int)cudaGetLastError();
}
