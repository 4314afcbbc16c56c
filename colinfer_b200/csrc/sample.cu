// sample.cu -- the fused logits -> token kernel (sm_100a).
//
// One thread-block cluster per row.  Each CTA of the cluster copies its slice of the row from HBM into its own shared
// memory exactly once (1-D bulk copies completed on mbarriers when the row is 16-byte aligned fp32, plain loads
// otherwise) and the whole row stays resident in the cluster's distributed shared memory.  Everything after that --
// penalties, grammar mask, row maximum / argmax, the min-p / top-k / top-p threshold selects and the inverse-CDF draw --
// works on shared memory, so HBM is read once per row whatever the sampling parameters are.
//
// Selection is exact.  The kept set is always {logit >= threshold}.  Masses are exp(z - max) rounded to integers in
// units of 2^-30 and summed as integers, so every sum, every cumulative-mass crossing and the CDF crossing are
// independent of thread, CTA and cluster geometry and of the other rows in the launch (the reference's row-invariance
// property).  How the threshold is found depends on the row's parameters:
//   top_k <= 128   each CTA bounds its slice's k-th largest logit from below with a histogram of its threads' maxima,
//                  collects the few logits above that bound in token order, and the cluster's first CTA finishes
//                  top-k, top-p and the draw exactly on the gathered list (two cluster barriers in all);
//   larger top_k   a fine count histogram over the distance from the row maximum (4096 buckets, reduced across the
//                  cluster) gives the bucket of the k-th largest logit; the logits down to it are gathered as above;
//   top_p alone    the same histogram with per-bucket mass estimates gives the bucket of the top-p pivot approximately;
//                  one pass sums the exact mass above a narrow band around it and gathers the band, the pivot is found
//                  exactly on the list, and the draw walks the row once more only inside one warp's region;
//   neither        one mass pass and the draw.
// If a list would overflow, or the estimated band misses the true pivot, an exact 4-level radix select over the
// order-preserving 32-bit keys runs instead (slower, same result).
//
// What the reference does in ~25 torch / FlashInfer launches per slot (engine/spec/accept.py:23-52 after
// engine/runtime/sampler.py:50-56) is one launch here.
#include <mutex>

#include "common.cuh"
#include "../../include/colinfer_b200.h"

#define CI_THREADS 256
#define CI_WARPS (CI_THREADS / 32)
#define CI_CHUNK 4096            // elements per bulk copy
#define CI_MAX_CHUNKS 16
#define CI_NB1 4096              // fine buckets over the distance from the row maximum
#define CI_RANGE 25.0f           // the buckets cover distances up to CI_RANGE * temperature
#define CI_FASTK 100             // largest top_k handled by the per-slice candidate lists
#define CI_FAST_BINS 512         // bins of the thread-maxima histogram and of the exact finish
#define CI_TGROUPS 4              // maxima each thread keeps (interleaved groups of its elements) for the top-k bound
#define CI_FIN_MAX 1024          // candidates of one row at the CTA that finishes it (8 x CI_PCAP)
#define CI_FAST_SCALE 32.0f      // its bins per unit logit (covers 16 units below the slice maximum)
#define CI_PCAP 128              // candidates one CTA may push to the CTA that finishes the row
#define CI_FIN_SCALE 64.0f       // bins per unit logit of the exact selection on the pushed candidates (8 units)
#define CI_FIN_CAND 64           // candidates of one bin examined pairwise
#define CI_RETRY 8               // rows a CTA may set aside for the generic path before the fast path is switched off
#define CI_WLIST 48              // list entries per warp
#define CI_GLIST 1365            // gathered list entries (16 KB)
#define CI_SEL_BINS 512          // coarse bins of the exact selection on a gathered list
#define CI_FB_NB 256             // radix buckets per level of the fallback select (8 bits)
#define CI_MAX_CAND 128          // tied / neighbouring candidates examined one by one in the final list step
#define CI_PEN_TABLE 2048        // distinct history ids per slice with an O(1) count
#define CI_WAIT_CYCLES 400000000LL
#define CI_FLT_MAX 3.402823466e38f
#define CI_POS_INF (__int_as_float(0x7f800000))

struct SampleArgs {
    const void* logits; int dtype; int use_bulk;
    const int32_t* mask; int mask_rows; int W;
    colinfer_sampler_params p;
    const void* pos; int pos_i64; const float* u;
    int64_t* out; colinfer_row_stats* stats; int32_t* status;
    int B, R, V; int slice_elems; int flags;
    long long* prof; int prof_slots;   // optional per-CTA phase timestamps (profiling hook)
};
// Profiling hook: thread 0 adds the cycles since its previous marker to the slot's total (summed over the CTA's rows).
#define CI_PROF(slot) do { if (a.prof && tid == 0) { const long long t_ = clock64(); sc->prof[slot] += t_ - prof_last; prof_last = t_; } } while (0)

struct ListEntry { uint32_t idx; float l; uint32_t q; };   // gathered list: token, logit, mass
struct Cand { uint32_t idx; float l; };                      // a warp's list / pushed candidates: token, logit

// A row whose candidates have been pushed to this CTA and that waits for its exact finish.
struct Pending { int row; float L; int aidx; int status; int count[8]; };

// What every CTA writes into each peer's shared memory before the first cluster barrier.
struct Hello { float lmax; int lidx; int flags; int pad; };   // flags: 1 = a bounded wait gave up, 4 = slow history path, 8 = stop using the fast path; pad: candidates pushed

// Values one CTA publishes in its own shared memory for its peers to read after a later barrier.
struct Xch {
    u64 seg_cnt, seg_est;          // totals of this CTA's reduced bucket segment: counts, estimated mass
    u64 fb_segtot;                 // the same for the fallback radix select
    u64 s_all, s_above;            // band pass: kept mass of the slice, and of its part above the band
    u64 cta_mass;                  // kept mass of the slice under the final threshold
    unsigned short wcount[CI_WARPS];   // entries in each warp's list
    int list_overflow;
};

struct Scratch {
    Hello hello[2][8];             // written by the peers, one set per row parity
    u64 warp_tot[CI_WARPS];
    u64 warp_aux[CI_WARPS];
    float warp_f[CI_WARPS]; int warp_i[CI_WARPS];
    uint32_t warp_u[CI_WARPS], warp_v[CI_WARPS];
    unsigned short pcount[8 * CI_WARPS]; unsigned short poff[8 * CI_WARPS + 1];
    int found_idx; u64 found_before;
    int ncand; float sel_value; int sel_ok;
    int fail;
    int hist_slow;
    u64 wsum[CI_WARPS], woff[CI_WARPS], wtotal;   // block scan
    int found_tid; u64 found_excl;
    float cand_l[CI_FIN_CAND]; u64 cand_w[CI_FIN_CAND]; float res_f;
    Pending pend;
    int n_retry_common, n_retry_mine, want_fast_off;
    int retry_common[CI_RETRY], retry_mine[CI_RETRY], retry_all[CI_RETRY * 9];
    long long prof[12];            // profiling hook: cycles per phase, summed over the CTA's rows
    int bcast_i[2];                // written by the cluster's first CTA, per row parity
    u64 mass_in[2][8];             // kept mass of every CTA's slice, written by the peers, per row parity
};

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }

// Block-wide: index of the first entry (ascending) at which the running sum of get(0..n-1) reaches `target`
// (1 <= target <= total), and the sum before it.  All threads call; all threads get the result.
template <class F>
__device__ void block_find(F get, int n, u64 target, Scratch* s, int& idx, u64& before) {
    const int ipt = (n + CI_THREADS - 1) / CI_THREADS;
    const int lo = threadIdx.x * ipt;
    u64 local = 0;
    for (int i = lo; i < lo + ipt && i < n; ++i) local += get(i);
    const u64 incl = warp_incl_scan_u64(local, lane_id());
    if (threadIdx.x == 0) { s->found_idx = n - 1; s->found_before = 0; }
    if (lane_id() == 31) s->warp_tot[warp_id()] = incl;
    __syncthreads();
    u64 off = 0;
    for (int w = 0; w < warp_id(); ++w) off += s->warp_tot[w];
    u64 excl = off + incl - local;
    if (excl < target && target <= excl + local) {
        for (int i = lo; i < lo + ipt && i < n; ++i) {
            const u64 v = get(i);
            if (excl + v >= target) { s->found_idx = i; s->found_before = excl; break; }
            excl += v;
        }
    }
    __syncthreads();
    idx = s->found_idx;
    before = s->found_before;
    __syncthreads();
}

__device__ u64 block_sum_u64(u64 v, Scratch* s) {
    v = warp_sum_u64(v);
    if (lane_id() == 0) s->warp_tot[warp_id()] = v;
    __syncthreads();
    u64 t = 0;
    for (int w = 0; w < CI_WARPS; ++w) t += s->warp_tot[w];
    __syncthreads();
    return t;
}


// Estimated mass (units of 2^-30) of one element in distance bucket b: exp(-(b + 0.5) * CI_RANGE / CI_NB1).
__device__ __forceinline__ u64 bucket_mass_est(int b) {
    return (u64)__float2uint_rn(exp2f(-((float)b + 0.5f) * (CI_RANGE * CI_LOG2E / (float)CI_NB1)) * CI_MASS_SCALE);
}

__device__ __forceinline__ u64 ceil_target(float frac, u64 total) {
    const double t = ceil((double)frac * (double)total);
    u64 q = t <= 1.0 ? 1ull : (u64)t;
    return q > total ? total : q;
}

// The row's uniform in (0, 1]: explicit, or Philox keyed by (seed, position + row of the slot), or 1 when no draw is asked.
__device__ __forceinline__ float row_uniform(const SampleArgs& a, int row, int b, int r) {
    if (a.u != nullptr) return a.u[row];
    if (a.pos != nullptr && a.p.seed != nullptr) {
        const long long p0 = a.pos_i64 ? reinterpret_cast<const long long*>(a.pos)[b]
                                       : (long long)reinterpret_cast<const int*>(a.pos)[b];
        return u32_to_uniform(philox_word(philox_key(a.p.seed[b]), (u64)p0 + (u64)r));
    }
    return 1.0f;
}

// Exact weighted selection on a gathered list: the value v among the entries with wt > 0 such that
// W(l > v) < target <= W(l >= v).  Up to 512 coarse bins over the entries' key range (a shift, so monotone), then the
// entries of the pivot bin one by one (a warp each).  Returns false when the pivot bin holds more than CI_MAX_CAND
// entries.  All threads of the CTA call; 1 <= target <= total weight.
template <class W>
__device__ bool list_select(const ListEntry* gl, int n, W wt, u64 target, u64* bins, uint32_t* cand, Scratch* sc, float& value) {
    const int tid = threadIdx.x, lane = lane_id(), warp = warp_id();
    uint32_t kmin = 0xFFFFFFFFu, kmax = 0u;
    for (int i = tid; i < n; i += CI_THREADS) {
        if (wt(i) > 0) { const uint32_t k = f2key(gl[i].l); kmin = min(kmin, k); kmax = max(kmax, k); }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, o));
        kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    }
    if (lane == 0) { sc->warp_u[warp] = kmin; sc->warp_v[warp] = kmax; }
    for (int i = tid; i < CI_SEL_BINS; i += CI_THREADS) bins[i] = 0;
    if (tid == 0) { sc->ncand = 0; sc->sel_ok = 0; sc->sel_value = 0.0f; }
    __syncthreads();
    for (int w = 0; w < CI_WARPS; ++w) { kmin = min(kmin, sc->warp_u[w]); kmax = max(kmax, sc->warp_v[w]); }
    const uint32_t span = kmax - kmin;                                   // bins cover [0, span] >> sh, at most 512
    const int sh = max(0, 32 - __clz(span) - 9);
    for (int i = tid; i < n; i += CI_THREADS) {
        const u64 w = wt(i);
        if (w > 0) atomicAdd(&bins[(kmax - f2key(gl[i].l)) >> sh], w);
    }
    __syncthreads();
    int b_star; u64 before;
    block_find([&](int i) { return bins[i]; }, CI_SEL_BINS, target, sc, b_star, before);
    for (int i = tid; i < n; i += CI_THREADS) {
        if (wt(i) > 0 && (int)((kmax - f2key(gl[i].l)) >> sh) == b_star) {
            const int slot = atomicAdd(&sc->ncand, 1);
            if (slot < CI_MAX_CAND) cand[slot] = (uint32_t)i;
        }
    }
    __syncthreads();
    const int nc = sc->ncand;
    if (nc > CI_MAX_CAND) { __syncthreads(); return false; }
    for (int c = warp; c < nc; c += CI_WARPS) {
        const uint32_t kc = f2key(gl[cand[c]].l);
        u64 gt = 0, eq = 0;
        for (int j = lane; j < nc; j += 32) {                            // only the pivot bin's entries matter
            const uint32_t k = f2key(gl[cand[j]].l);
            const u64 w = wt((int)cand[j]);
            if (k > kc) gt += w; else if (k == kc) eq += w;
        }
        gt = warp_sum_u64(gt); eq = warp_sum_u64(eq);
        if (lane == 0 && before + gt < target && target <= before + gt + eq) { sc->sel_value = gl[cand[c]].l; sc->sel_ok = 1; }
    }
    __syncthreads();
    value = sc->sel_value;
    const bool ok = sc->sel_ok != 0;
    __syncthreads();
    return ok;
}

// Exact radix select over the order-preserving 32-bit keys of the logits >= lcut, four levels of 8 bits, across the
// cluster.  by_mass: the pivot where the descending cumulative mass first reaches top_p of the total; else the kk-th
// largest.  Returns false when the filter removes nothing (fewer survivors than kk); else pivot holds the pivot logit.
// Every CTA of the cluster calls it with identical arguments and takes identical decisions.
struct RadixCtx {
    const float* rowbuf; int n_pad; u64* fb_hist; u64* fb_seg; Xch* xch; Scratch* sc; int rank, CS;
};
__device__ bool radix_select(cg::cluster_group& cluster, const RadixCtx& c, const MassFn& mass, float lcut, bool by_mass,
                             u64 kk, float topp, float& pivot) {
    const int tid = threadIdx.x;
    const float lk = fmaxf(lcut, -CI_FLT_MAX);
    uint32_t prefix = 0;
    u64 target = by_mass ? 0 : kk;
    for (int lvl = 0; lvl < 4; ++lvl) {
        const int shift = 24 - 8 * lvl;
        for (int i = tid; i < CI_FB_NB; i += CI_THREADS) c.fb_hist[i] = 0;
        __syncthreads();
        const float4* row4 = reinterpret_cast<const float4*>(c.rowbuf);
        for (int i = tid; i * 4 < c.n_pad; i += CI_THREADS) {
            const float4 v = row4[i];
            const float e4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float l = e4[j];
                if (l >= lk) {
                    const uint32_t key = f2key(l);
                    if (lvl == 0 || (key >> (shift + 8)) == prefix)
                        atomicAdd(&c.fb_hist[CI_FB_NB - 1 - (int)((key >> shift) & 0xFFu)], by_mass ? (u64)mass(l) : 1ull);
                }
            }
        }
        __syncthreads();
        cluster.sync();                                                    // local histograms complete
        const int G = CI_FB_NB / c.CS;
        u64 part = 0;
        for (int g = tid; g < G; g += CI_THREADS) {
            u64 sum = 0;
            for (int q = 0; q < c.CS; ++q) sum += cluster.map_shared_rank(c.fb_hist, q)[c.rank * G + g];
            c.fb_seg[g] = sum;
            part += sum;
        }
        const u64 tot = block_sum_u64(part, c.sc);
        if (tid == 0) c.xch->fb_segtot = tot;
        __syncthreads();
        cluster.sync();                                                    // reduced segments published
        u64 grand = 0, segtots[8];
        for (int q = 0; q < c.CS; ++q) { segtots[q] = cluster.map_shared_rank(c.xch, q)->fb_segtot; grand += segtots[q]; }
        if (lvl == 0) {
            if (by_mass) target = ceil_target(topp, grand);
            else if (target >= grand) return false;
        }
        if (grand == 0) return false;
        int s_star = c.CS - 1; u64 before_seg = 0, run = 0;
        for (int q = 0; q < c.CS; ++q) {
            if (run + segtots[q] >= target) { s_star = q; before_seg = run; break; }
            run += segtots[q];
        }
        const u64* pseg = cluster.map_shared_rank(c.fb_seg, s_star);
        int g_star; u64 before;
        block_find([&](int i) { return pseg[i]; }, G, target - before_seg, c.sc, g_star, before);
        target -= before_seg + before;
        prefix = (prefix << 8) | (uint32_t)(CI_FB_NB - 1 - (s_star * G + g_star));
    }
    pivot = key2f(prefix);
    return true;
}

// Gathers the per-warp lists of every CTA of the cluster into glist, in token order (CTA rank, warp, position).
// Returns the number of entries, or -1 when a list overflowed or the total exceeds the capacity.  The entries' masses
// are computed here (the warps' lists hold token and logit only).  All threads call.
__device__ int gather_lists(cg::cluster_group& cluster, int CS, Xch* xch, Cand* ownlist, ListEntry* glist, Scratch* sc,
                            const MassFn& mass) {
    const int tid = threadIdx.x, lane = lane_id(), warp = warp_id();
    const int np = CS * CI_WARPS;                                          // (CTA, warp) pairs, at most 128
    int overflow = 0;
    if (tid < CS) overflow = cluster.map_shared_rank(xch, tid)->list_overflow;
    if (tid < np) sc->pcount[tid] = cluster.map_shared_rank(xch, tid / CI_WARPS)->wcount[tid % CI_WARPS];
    overflow = __syncthreads_or(overflow);
    if (warp == 0) {                                                       // exclusive prefix of up to 128 counts
        int c4[4], s = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) { c4[j] = lane * 4 + j < np ? sc->pcount[lane * 4 + j] : 0; s += c4[j]; }
        int incl = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
        int run = incl - s;
#pragma unroll
        for (int j = 0; j < 4; ++j) { if (lane * 4 + j < np) sc->poff[lane * 4 + j] = (unsigned short)run; run += c4[j]; }
        if (lane == 31) sc->poff[np] = (unsigned short)min(incl, 65535);
    }
    __syncthreads();
    const int n = sc->poff[np];
    if (overflow || n > CI_GLIST) return -1;
    for (int e = tid; e < n; e += CI_THREADS) {
        int lo = 0, hi = np - 1;                                           // last pair p with poff[p] <= e
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (sc->poff[mid] <= e) lo = mid; else hi = mid - 1; }
        const Cand c = *(cluster.map_shared_rank(ownlist, lo / CI_WARPS) + (lo % CI_WARPS) * CI_WLIST + (e - sc->poff[lo]));
        ListEntry en;
        en.idx = c.idx; en.l = c.l; en.q = mass(c.l);
        glist[e] = en;
    }
    __syncthreads();
    return n;
}

// Top-k, top-p and the draw on a gathered list that is known to hold every logit >= tl of the row (tl below the
// top-k pivot).  Returns false when the result cannot be trusted from the list alone (the caller falls back).
// On success: token, lcut (final threshold) and total (kept mass).  All threads of the CTA call.
__device__ bool finish_on_list(const ListEntry* glist, int n, float tl, float lcut_in, float tc, int kk, bool need_topp,
                               float topp, float u, u64* bins, uint32_t* cand, Scratch* sc,
                               long long& token, float& lcut, u64& total) {
    const int tid = threadIdx.x;
    float cut = lcut_in;
    u64 cnt = 0;
    for (int i = tid; i < n; i += CI_THREADS) cnt += glist[i].l >= cut ? 1 : 0;
    const u64 survivors = block_sum_u64(cnt, sc);
    if (survivors == 0) return false;
    if ((u64)kk <= survivors) {                                            // else fewer than k survive min-p: top-k removes nothing
        float lk_val;
        if (!list_select(glist, n, [&](int i) { return (u64)(glist[i].l >= cut ? 1 : 0); }, (u64)kk, bins, cand, sc, lk_val))
            return false;
        cut = fmaxf(cut, lower_logit_for(scale_logit(lk_val, tc), tc, lk_val));
        if (cut < tl) return false;                                        // a tie partner could lie outside the list
    }
    if (need_topp) {
        u64 part = 0;
        for (int i = tid; i < n; i += CI_THREADS) if (glist[i].l >= cut) part += glist[i].q;
        const u64 s1 = block_sum_u64(part, sc);
        if (s1 == 0) return false;
        float lp_val;
        const float c0 = cut;
        if (!list_select(glist, n, [&](int i) { return (u64)(glist[i].l >= c0 ? glist[i].q : 0u); }, ceil_target(topp, s1), bins,
                         cand, sc, lp_val))
            return false;
        cut = fmaxf(cut, lower_logit_for(scale_logit(lp_val, tc), tc, lp_val));
        if (cut < tl) return false;
    }
    u64 part = 0;
    for (int i = tid; i < n; i += CI_THREADS) if (glist[i].l >= cut) part += glist[i].q;
    total = block_sum_u64(part, sc);
    if (total == 0) return false;
    int at; u64 before;
    block_find([&](int i) { return (u64)(glist[i].l >= cut ? glist[i].q : 0u); }, n, ceil_target(u, total), sc, at, before);
    token = (long long)glist[at].idx;
    lcut = cut;
    return true;
}

// Appends the components of one float4 group selected by the 4-bit mask mk to the warp's list, in token order
// (lane, then component).  Positions come from four ballots, no scan.  wn is the warp's running count (uniform over
// the warp); entries beyond CI_WLIST are dropped and counted.
__device__ __forceinline__ void warp_append(Cand* mylist, int& wn, unsigned mk, const float* e4, uint32_t idx0, int lane) {
    const unsigned b0 = __ballot_sync(0xffffffffu, mk & 1u), b1 = __ballot_sync(0xffffffffu, mk & 2u);
    const unsigned b2 = __ballot_sync(0xffffffffu, mk & 4u), b3 = __ballot_sync(0xffffffffu, mk & 8u);
    if (!(b0 | b1 | b2 | b3)) return;
    const unsigned lt = (1u << lane) - 1u;
    int at = wn + __popc(b0 & lt) + __popc(b1 & lt) + __popc(b2 & lt) + __popc(b3 & lt);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (mk & (1u << j)) {
            if (at < CI_WLIST) { mylist[at].idx = idx0 + j; mylist[at].l = e4[j]; }
            ++at;
        }
    }
    wn += __popc(b0) + __popc(b1) + __popc(b2) + __popc(b3);
}

// Collects, in token order, the logits >= tl of one warp's region [r_lo, r_hi) of the slice into the warp's list.
// Four float4 groups per lane and step are loaded together (their latencies overlap); appends are rare.
__device__ __forceinline__ void collect_region(const float* rowbuf, int r_lo, int r_hi, float tl, Cand* mylist, int& wn,
                                               uint32_t slice_lo, int lane) {
    for (int i0 = r_lo; i0 < r_hi; i0 += 512) {
        float4 v[4];
        unsigned mk[4], anym = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * 128 + lane * 4;
            v[k] = i < r_hi ? *reinterpret_cast<const float4*>(rowbuf + i) : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
            mk[k] = (v[k].x >= tl ? 1u : 0u) | (v[k].y >= tl ? 2u : 0u) | (v[k].z >= tl ? 4u : 0u) | (v[k].w >= tl ? 8u : 0u);
            anym |= mk[k];
        }
        if (__ballot_sync(0xffffffffu, anym != 0u)) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float e4[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
                warp_append(mylist, wn, mk[k], e4, slice_lo + (uint32_t)(i0 + k * 128 + lane * 4), lane);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ lean block primitives
// Exclusive prefix of one value per thread over the CTA (thread order), and the total.  Two __syncthreads.
__device__ __forceinline__ u64 block_excl_scan(u64 v, Scratch* sc, u64& total) {
    const int lane = lane_id(), warp = warp_id();
    const u64 incl = warp_incl_scan_u64(v, lane);
    if (lane == 31) sc->wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const u64 w = lane < CI_WARPS ? sc->wsum[lane] : 0ull;
        const u64 wi = warp_incl_scan_u64(w, lane);
        if (lane < CI_WARPS) sc->woff[lane] = wi - w;
        if (lane == CI_WARPS - 1) sc->wtotal = wi;
        if (lane == 0) sc->found_tid = -1;
    }
    __syncthreads();
    total = sc->wtotal;
    return sc->woff[warp] + incl - v;
}

// Where the running sum of CI_FAST_BINS bins (ascending index) first reaches `target`: the bin, the sum before it, and
// the total.  bin = -1 when target exceeds the total (or is 0).  Three __syncthreads.  All threads call.
template <class T>
__device__ void bins_find(const T* bins, u64 target, Scratch* sc, int& bin, u64& before, u64& total) {
    constexpr int PER = CI_FAST_BINS / CI_THREADS;
    const int tid = threadIdx.x;
    u64 loc[PER], s = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) { loc[j] = (u64)bins[tid * PER + j]; s += loc[j]; }
    const u64 excl = block_excl_scan(s, sc, total);
    if (excl < target && target <= excl + s) {
        u64 run = excl;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            if (run + loc[j] >= target) { sc->found_tid = tid * PER + j; sc->found_excl = run; break; }
            run += loc[j];
        }
    }
    __syncthreads();
    bin = sc->found_tid;
    before = sc->found_excl;
}

// Exact weighted selection among n entries (logits fl[0..n) in shared memory, weight wt(i)): the value v such that
// W(l > v) < target <= W(l >= v).  CI_FAST_BINS bins over the distance from the row maximum, then the pivot bin's
// entries pairwise.  Returns false when the pivot falls outside the binned range or its bin is too crowded.
// All threads call with the same arguments.
template <class W>
__device__ bool lean_select(const float* fl, int n, W wt, float L, u64 target, u64* bins, Scratch* sc, float& value) {
    const int tid = threadIdx.x;
    for (int i = tid; i < CI_FAST_BINS; i += CI_THREADS) bins[i] = 0;
    if (tid == 0) { sc->ncand = 0; sc->sel_ok = 0; }
    __syncthreads();
    for (int i = tid; i < n; i += CI_THREADS) {
        const u64 w = wt(i);
        if (w) atomicAdd(&bins[min(CI_FAST_BINS - 1, __float2int_rz((L - fl[i]) * CI_FIN_SCALE))], w);
    }
    __syncthreads();
    int b_star; u64 before, total;
    bins_find(bins, target, sc, b_star, before, total);
    if (b_star < 0 || b_star >= CI_FAST_BINS - 1) return false;
    for (int i = tid; i < n; i += CI_THREADS) {
        const u64 w = wt(i);
        if (w && min(CI_FAST_BINS - 1, __float2int_rz((L - fl[i]) * CI_FIN_SCALE)) == b_star) {
            const int slot = atomicAdd(&sc->ncand, 1);
            if (slot < CI_FIN_CAND) { sc->cand_l[slot] = fl[i]; sc->cand_w[slot] = w; }
        }
    }
    __syncthreads();
    const int nc = sc->ncand;
    if (nc > CI_FIN_CAND) return false;
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

// Exact finish of a row from the candidates its CTAs pushed into this CTA's shared memory: min-p, top-k, top-p and
// the draw, all inside this CTA (no cluster traffic).  The candidates contain the row's top k logits (and possibly
// more), in token order: CTA by CTA, each CTA's in token order.  Writes the row's outputs and returns true, or returns
// false when the row has to take the generic path.  `work` is CI_FAST_BINS * 8 + CI_FIN_MAX * 8 bytes of scratch.
// All threads of the CTA call.
__device__ bool finish_pending(const SampleArgs& a, const Pending& pd, const Cand* plist, int CS, unsigned char* work, Scratch* sc) {
    const int tid = threadIdx.x;
    u64* bins = reinterpret_cast<u64*>(work);
    float* fl = reinterpret_cast<float*>(work + CI_FAST_BINS * 8);
    uint32_t* fi = reinterpret_cast<uint32_t*>(fl + CI_FIN_MAX);
    const int row = pd.row, b = row / a.R, r = row % a.R;
    const float tc = fmaxf(a.p.temperature[b], 1e-6f);
    const int kk = a.p.top_k[b];
    const float topp = a.p.top_p[b];
    const float L = pd.L;
    const float m = scale_logit(L, tc);
    MassFn mass;
    mass.init(tc, m);
    const float thr = __fadd_rn(m, a.p.log_min_p[b]);
    float cut = lower_logit_for(thr, tc, __fmul_rn(thr, tc));
    cut = fmaxf(cut, L - 22.0f * tc - fabsf(L) * 1e-6f);           // the mass horizon (see the generic path)
    const float u = row_uniform(a, row, b, r);
    int pre[9];
    pre[0] = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) pre[q + 1] = pre[q] + (q < CS ? pd.count[q] : 0);
    const int n = pre[8];
    if (n > CI_FIN_MAX || n <= 0) return false;
    // the concatenated lists, contiguous and in token order
    for (int e = tid; e < n; e += CI_THREADS) {
        int q = 0;
#pragma unroll
        for (int t = 1; t < 8; ++t) q += (pre[t] <= e) ? 1 : 0;
        const Cand c = plist[q * CI_PCAP + (e - pre[q])];
        fl[e] = c.l; fi[e] = c.idx;
    }
    __syncthreads();
    // ---- top-k: the k-th largest of the candidates that survive min-p
    u64 cnt = 0;
    for (int i = tid; i < n; i += CI_THREADS) cnt += (fl[i] >= cut && fl[i] > CI_NEG_INF) ? 1 : 0;
    u64 survivors;
    block_excl_scan(cnt, sc, survivors);
    if (survivors == 0) return false;
    if ((u64)kk <= survivors) {                               // else fewer than k survive min-p: top-k removes nothing
        float lk;
        const float c0 = cut;
        if (!lean_select(fl, n, [&](int i) { return (u64)((fl[i] >= c0 && fl[i] > CI_NEG_INF) ? 1 : 0); }, L, (u64)kk, bins, sc, lk))
            return false;
        cut = fmaxf(cut, lower_logit_for(scale_logit(lk, tc), tc, lk));
    }
    // ---- top-p over the kept candidates
    if (topp < 1.0f) {
        const float c0 = cut;
        u64 part = 0;
        for (int i = tid; i < n; i += CI_THREADS) part += (fl[i] >= c0 && fl[i] > CI_NEG_INF) ? (u64)mass(fl[i]) : 0ull;
        u64 s1;
        block_excl_scan(part, sc, s1);
        if (s1 == 0) return false;
        float lp;
        if (!lean_select(fl, n, [&](int i) { return (fl[i] >= c0 && fl[i] > CI_NEG_INF) ? (u64)mass(fl[i]) : 0ull; }, L,
                         ceil_target(topp, s1), bins, sc, lp))
            return false;
        cut = fmaxf(cut, lower_logit_for(scale_logit(lp, tc), tc, lp));
    }
    // ---- the draw: first candidate (token order) whose running kept mass reaches u * total
    const int ept = (n + CI_THREADS - 1) / CI_THREADS;
    const int e_lo = tid * ept, e_hi = min(e_lo + ept, n);
    u64 mine = 0;
    for (int i = e_lo; i < e_hi; ++i) mine += (fl[i] >= cut && fl[i] > CI_NEG_INF) ? (u64)mass(fl[i]) : 0ull;
    u64 total;
    const u64 excl = block_excl_scan(mine, sc, total);
    if (total == 0) return false;
    const u64 target = ceil_target(u, total);
    if (excl < target && target <= excl + mine) {
        u64 run = excl;
        long long token = -1;
        for (int i = e_lo; i < e_hi; ++i) {
            run += (fl[i] >= cut && fl[i] > CI_NEG_INF) ? (u64)mass(fl[i]) : 0ull;
            if (run >= target) { token = (long long)fi[i]; break; }
        }
        if (a.out) a.out[row] = token;
        if (a.status) a.status[row] = pd.status;
        if (a.stats) {
            colinfer_row_stats st;
            st.lmax = L; st.lcut = cut; st.tc = tc; st.status = pd.status; st.argmax = pd.aidx; st.mass_q = total;
            a.stats[row] = st;
        }
    }
    __syncthreads();
    return true;
}

extern "C" __global__ void __launch_bounds__(CI_THREADS, 2) k_sample(const __grid_constant__ SampleArgs a) {
    cg::cluster_group cluster = cg::this_cluster();
    // Every CTA announces that it runs; the matching wait comes just before the first write into a peer's shared memory.
    cluster.barrier_arrive();
    const int CS = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = lane_id(), warp = warp_id();
    const int V = a.V;

    const int slice_cap = a.slice_elems;                      // multiple of 128
    const int slice_lo = rank * slice_cap;
    const int slice_len = max(0, min(slice_cap, V - slice_lo));
    const int n_pad = (slice_len + 127) & ~127;               // processed elements (tail holds -inf)
    const int nchunks = (slice_len + CI_CHUNK - 1) / CI_CHUNK;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* rowbuf = reinterpret_cast<float*>(smem_raw);
    unsigned char* hreg = smem_raw + (size_t)slice_cap * 4;                 // 24 KB work area
    uint32_t* hist1 = reinterpret_cast<uint32_t*>(hreg);                      // [CI_NB1] fine counts
    uint32_t* segcnt = reinterpret_cast<uint32_t*>(hreg + CI_NB1 * 4);        // [<= 2048] reduced segment
    ListEntry* glist = reinterpret_cast<ListEntry*>(hreg);                    // gathered list, over hist1
    u64* bins = reinterpret_cast<u64*>(hreg + CI_NB1 * 4);                    // [512] selection bins, over segcnt
    uint32_t* cand = reinterpret_cast<uint32_t*>(hreg + CI_NB1 * 4 + CI_SEL_BINS * 8);
    u64* fb_hist = reinterpret_cast<u64*>(hreg);                              // fallback radix, over hist1
    u64* fb_seg = fb_hist + CI_FB_NB;
    Cand* ownlist = reinterpret_cast<Cand*>(hreg + 24 * 1024);                // [CI_WARPS][CI_WLIST] this CTA's lists
    Cand* plist = ownlist + CI_WARPS * CI_WLIST;                              // [8][CI_PCAP] candidates pushed by the cluster
    u64* mbar = reinterpret_cast<u64*>(plist + 8 * CI_PCAP);
    Xch* xch = reinterpret_cast<Xch*>(mbar + CI_MAX_CHUNKS);
    Scratch* sc = reinterpret_cast<Scratch*>(xch + 1);
    // penalty tables alias the work area (used before the first histogram)
    uint32_t* pen_bits = reinterpret_cast<uint32_t*>(hreg);
    const int nw = slice_cap >> 5;
    uint32_t* pen_prefix = pen_bits + nw;
    uint32_t* pen_cnt = pen_prefix + nw;

    // The mbarriers of the bulk copies are set up once; each row completes one phase of each.
    if (tid == 0 && a.use_bulk) {
        for (int c = 0; c < nchunks; ++c) mbar_init(&mbar[c], 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    const int n_clusters = (int)gridDim.x / CS;
    const long long n_rows = (long long)a.B * a.R;
    long long prof_last = clock64();
    const long long prof_t0 = prof_last;
    if (a.prof && tid == 0) for (int i = 0; i < 12; ++i) sc->prof[i] = 0;

    // Starts the bulk copies of one row's slice (thread 0 only; every thread must be done reading the buffer).
    auto issue_row = [&](const long long rw) {
        fence_proxy_async();                                   // earlier reads of the buffer precede these writes
        const float* src = reinterpret_cast<const float*>(a.logits) + (size_t)rw * V + slice_lo;
        if (a.flags & COLINFER_TEST_DROP_COPY) return;        // test flag: nothing is armed, nothing is in flight; the waits run out
        for (int c = 0; c < nchunks; ++c) {
            const int len = min(CI_CHUNK, slice_len - c * CI_CHUNK);
            mbar_expect_tx(&mbar[c], (uint32_t)len * 4u);
            bulk_g2s(rowbuf + c * CI_CHUNK, src + c * CI_CHUNK, (uint32_t)len * 4u, &mbar[c]);
        }
    };
    bool prefetched = false;          // the next row's copies are already in flight
    bool fast_enabled = true;         // small top-k rows may take the deferred path (identical in every CTA)
    int fast_seq = 0;                 // deferred rows so far: row j is finished by CTA j % CS
    int n_set_aside = 0;              // rows set aside for the generic path by every CTA alike
    if (tid == 0) { sc->pend.row = -1; sc->n_retry_common = 0; sc->n_retry_mine = 0; sc->want_fast_off = 0; }

    // Every CTA that holds a deferred row finishes it; then the cluster meets so that candidates may be pushed again.
    auto flush = [&]() {
        __syncthreads();
        if (sc->pend.row >= 0) {
            const bool ok = finish_pending(a, sc->pend, plist, CS, hreg, sc);
            if (tid == 0) {
                if (!ok) {
                    if (sc->n_retry_mine < CI_RETRY) sc->retry_mine[sc->n_retry_mine++] = sc->pend.row;
                    if (sc->n_retry_mine >= CI_RETRY - 1) sc->want_fast_off = 1;
                }
                sc->pend.row = -1;
            }
        }
        cluster.sync();
    };

    // One row of the batch.  `it` counts this cluster's rows: its parity selects the mbarrier phase and the exchange slots.
    auto process_row = [&](const int row, const int it, const bool allow_fast, const long long next_row) {
    const int par = it & 1;
    const int b = row / a.R, r = row % a.R;
    // ---------------------------------------------------------------------------------------- start the HBM read
    // One thread issues every bulk copy of the slice at once, before anything else (unless the previous row already
    // started this row's copies because it no longer needed the buffer).
    if (tid == 0) {
        sc->fail = 0; sc->hist_slow = 0; xch->list_overflow = 0;
        if (a.use_bulk && !prefetched) issue_row(row);
    }
    prefetched = false;
    CI_PROF(0);

    // ---------------------------------------------------------------------------------------- parameters of the slot
    const float T = a.p.temperature[b];
    const bool sampled = (T > 0.0f) || (a.flags & COLINFER_FORCE_DISTRIBUTION);
    const float tc = fmaxf(T, 1e-6f);
    const float rp = a.p.repetition_penalty ? a.p.repetition_penalty[b] : 1.0f;
    const float pp = a.p.presence_penalty ? a.p.presence_penalty[b] : 0.0f;
    const float fp = a.p.frequency_penalty ? a.p.frequency_penalty[b] : 0.0f;
    const int32_t* hist = a.p.history ? a.p.history + (size_t)b * a.p.hist_stride : nullptr;
    int hlen = hist ? (a.p.hist_len ? a.p.hist_len[b] : a.p.hist_stride) : 0;
    hlen = max(0, min(hlen, a.p.hist_stride));
    const bool has_pen = hlen > 0 && !(rp == 1.0f && pp == 0.0f && fp == 0.0f);
    const int32_t* mrow = a.mask ? a.mask + ((size_t)b * a.mask_rows + r) * a.W : nullptr;
    const int kk = a.p.top_k[b];
    const float topp = a.p.top_p[b];
    const float log_min_p = a.p.log_min_p[b];
    const bool fastk = allow_fast && fast_enabled && sampled && kk >= 1 && kk <= CI_FASTK && kk < V &&
                       !(a.flags & COLINFER_FORCE_DISTRIBUTION);         // identical in every CTA of the cluster

    // tail of the slice buffer: -inf (never selected, zero mass); disjoint from the bulk-copy destinations
    for (int i = slice_len + tid; i < n_pad; i += CI_THREADS) rowbuf[i] = CI_NEG_INF;
    __syncthreads();                                           // mbarriers initialised, tail filled

    // ---------------------------------------------------------------------------------------- penalty tables
    // bitmap of the slice's tokens that occur in the history, their ranks, and the occurrence count per rank
    if (has_pen) {
        // this thread's share of the history, loaded once (8 ids per thread cover 2,048 ids; longer histories loop)
        constexpr int HREG = 8;
        int hv[HREG];
#pragma unroll
        for (int j = 0; j < HREG; ++j) { const int i = tid + j * CI_THREADS; hv[j] = i < hlen ? __ldg(hist + i) - slice_lo : -1; }
        for (int i = tid; i < nw; i += CI_THREADS) pen_bits[i] = 0u;
        for (int i = tid; i < CI_PEN_TABLE; i += CI_THREADS) pen_cnt[i] = 0u;
        __syncthreads();
#pragma unroll
        for (int j = 0; j < HREG; ++j) if (hv[j] >= 0 && hv[j] < slice_len) atomicOr(&pen_bits[hv[j] >> 5], 1u << (hv[j] & 31));
        for (int i = tid + HREG * CI_THREADS; i < hlen; i += CI_THREADS) {
            const int v = __ldg(hist + i) - slice_lo;
            if (v >= 0 && v < slice_len) atomicOr(&pen_bits[v >> 5], 1u << (v & 31));
        }
        __syncthreads();
        if (fp != 0.0f) {
            // ranks of the set bits (exclusive prefix of popcounts over the bitmap words), then the count per rank
            const int ipt = (nw + CI_THREADS - 1) / CI_THREADS;
            const int lo = tid * ipt;
            u64 local = 0;
            for (int i = lo; i < lo + ipt && i < nw; ++i) local += __popc(pen_bits[i]);
            u64 total_bits;
            uint32_t run = (uint32_t)block_excl_scan(local, sc, total_bits);
            for (int i = lo; i < lo + ipt && i < nw; ++i) { pen_prefix[i] = run; run += __popc(pen_bits[i]); }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < HREG; ++j) {
                const int v = hv[j];
                if (v >= 0 && v < slice_len) {
                    const uint32_t rk = pen_prefix[v >> 5] + __popc(pen_bits[v >> 5] & ((1u << (v & 31)) - 1u));
                    if (rk < CI_PEN_TABLE) atomicAdd(&pen_cnt[rk], 1u);
                }
            }
            for (int i = tid + HREG * CI_THREADS; i < hlen; i += CI_THREADS) {
                const int v = __ldg(hist + i) - slice_lo;
                if (v >= 0 && v < slice_len) {
                    const uint32_t rk = pen_prefix[v >> 5] + __popc(pen_bits[v >> 5] & ((1u << (v & 31)) - 1u));
                    if (rk < CI_PEN_TABLE) atomicAdd(&pen_cnt[rk], 1u);
                }
            }
            __syncthreads();
        }
    }

    CI_PROF(1);
    // ---------------------------------------------------------------------------------------- pass A: land, penalise, mask, maximum
    float lmax = CI_NEG_INF;
    int lidx = 0x7fffffff;
    int lpos = -1;                                              // float4 group of the slice that holds this thread's maximum
    float tg[CI_TGROUPS];                                       // maxima of this thread's interleaved element groups
#pragma unroll
    for (int j = 0; j < CI_TGROUPS; ++j) tg[j] = CI_NEG_INF;
    // (1) the slice lands: wait for the bulk copies, or load it with plain loads (unaligned fp32 rows, bf16)
    if (a.use_bulk) {
        const bool drop = (a.flags & COLINFER_TEST_DROP_COPY) != 0;
        if (drop) for (int i = tid; i < slice_len; i += CI_THREADS) rowbuf[i] = 0.0f;   // (the test reads a defined buffer)
        for (int c = 0; c < nchunks; ++c)
            if (!mbar_wait_bounded(&mbar[c], (uint32_t)par, drop ? 20000LL : CI_WAIT_CYCLES)) sc->fail = 1;
    } else {
        const size_t g0 = (size_t)row * V + slice_lo;
        if (a.dtype == COLINFER_BF16) {
            const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(a.logits) + g0;
            if ((((uintptr_t)src) & 15) == 0) {
                const uint4* s4 = reinterpret_cast<const uint4*>(src);
                for (int i = tid; i * 8 < slice_len; i += CI_THREADS) {
                    if (i * 8 + 8 <= slice_len) {
                        const uint4 q = __ldg(s4 + i);
                        const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
                        float* d = rowbuf + i * 8;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            d[2 * j] = __uint_as_float(ww[j] << 16);
                            d[2 * j + 1] = __uint_as_float(ww[j] & 0xFFFF0000u);
                        }
                    } else {
                        for (int j = i * 8; j < slice_len; ++j) rowbuf[j] = __bfloat162float(src[j]);
                    }
                }
            } else {
                for (int i = tid; i < slice_len; i += CI_THREADS) rowbuf[i] = __bfloat162float(src[i]);
            }
        } else {
            const float* src = reinterpret_cast<const float*>(a.logits) + g0;
            for (int i = tid; i < slice_len; i += CI_THREADS) rowbuf[i] = __ldg(src + i);
        }
        __syncthreads();
    }
    CI_PROF(5);
    // (2) penalties: one bitmap word (32 tokens) per thread and step
    if (has_pen) {
        const int wn = n_pad >> 5;
        for (int wi = tid; wi < wn; wi += CI_THREADS) {
            const uint32_t word = pen_bits[wi];
            uint32_t rest = word;
            while (rest) {
                const int bit = __ffs(rest) - 1;
                rest &= rest - 1;
                const int v = (wi << 5) + bit;
                int cnt = 1;
                if (fp != 0.0f) {
                    const uint32_t rk = pen_prefix[wi] + __popc(word & ((1u << bit) - 1u));
                    if (rk < CI_PEN_TABLE) cnt = (int)pen_cnt[rk];
                    else {
                        cnt = 0; sc->hist_slow = 1;
                        for (int i = 0; i < hlen; ++i) cnt += (hist[i] == v + slice_lo);
                    }
                }
                rowbuf[v] = apply_penalty(rowbuf[v], cnt, rp, pp, fp);
            }
        }
        __syncthreads();
    }
    // (3) mask and maximum: four float4 groups per thread and step, loaded together so that their latencies overlap
    {
        float4* row4 = reinterpret_cast<float4*>(rowbuf);
        const int n4 = n_pad >> 2;
        for (int i0 = tid; i0 < n4; i0 += CI_TGROUPS * CI_THREADS) {
            float4 v[CI_TGROUPS];
#pragma unroll
            for (int k = 0; k < CI_TGROUPS; ++k) {
                const int i = i0 + k * CI_THREADS;
                v[k] = i < n4 ? row4[i] : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
            }
            if (mrow != nullptr) {
#pragma unroll
                for (int k = 0; k < CI_TGROUPS; ++k) {
                    const int i = i0 + k * CI_THREADS;
                    const int g = slice_lo + i * 4;             // global token index of v[k].x
                    if (i < n4 && g < V) {
                        const uint32_t bits = ((uint32_t)__ldg(mrow + (g >> 5)) >> (g & 31)) & 0xFu;
                        if (bits != 0xFu) {
                            if (!(bits & 1u)) v[k].x = CI_NEG_INF;
                            if (!(bits & 2u)) v[k].y = CI_NEG_INF;
                            if (!(bits & 4u)) v[k].z = CI_NEG_INF;
                            if (!(bits & 8u)) v[k].w = CI_NEG_INF;
                            row4[i] = v[k];
                        }
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < CI_TGROUPS; ++k) {
                const float m4 = fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w));
                tg[k] = fmaxf(tg[k], m4);
                const bool up = m4 > lmax;                      // strict: the first (lowest) position of the maximum stays
                lmax = up ? m4 : lmax;
                lpos = up ? i0 + k * CI_THREADS : lpos;
            }
        }
    }
    CI_PROF(2);
    if (lpos >= 0) {
        const float4 v = reinterpret_cast<const float4*>(rowbuf)[lpos];
        lidx = slice_lo + lpos * 4 + (v.x == lmax ? 0 : v.y == lmax ? 1 : v.z == lmax ? 2 : 3);
    }
    // block reduce (largest value, lowest index among equals)
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, lmax, o);
        const int oi = __shfl_xor_sync(0xffffffffu, lidx, o);
        if (om > lmax || (om == lmax && oi < lidx)) { lmax = om; lidx = oi; }
    }
    if (lane == 0) { sc->warp_f[warp] = lmax; sc->warp_i[warp] = lidx; }
    if (fastk) for (int i = tid; i < CI_FAST_BINS; i += CI_THREADS) hist1[i] = 0u;   // (the penalty tables are done with)
    __syncthreads();
    {
        float bm = sc->warp_f[0]; int bi = sc->warp_i[0];
#pragma unroll
        for (int w = 1; w < CI_WARPS; ++w) {
            const float om = sc->warp_f[w]; const int oi = sc->warp_i[w];
            if (om > bm || (om == bm && oi < bi)) { bm = om; bi = oi; }
        }
        lmax = bm; lidx = bi;                                   // the slice maximum, in every thread
    }

    // warp w owns the contiguous region [r_lo, r_hi) of the slice; lanes interleave float4 groups, so the token
    // order inside a region is (step, lane, component).
    const int reg = ((n_pad / 128 + CI_WARPS - 1) / CI_WARPS) * 128;
    const int r_lo = min(warp * reg, n_pad), r_hi = min(r_lo + reg, n_pad);
    Cand* mylist = ownlist + warp * CI_WLIST;

    // ---------------------------------------------------------------------------------------- small top-k: candidates of the slice
    // The k-th largest of the threads' group maxima (CI_TGROUPS disjoint groups per thread) bounds the slice's k-th largest logit from below, and every logit of the
    // row's top k is among its own slice's top k: the logits >= that bound, over all slices, contain the row's top k.
    float tl_fast = CI_NEG_INF;
    int my_count = 0;
    if (it == 0) cluster.barrier_wait();                        // every CTA of the cluster runs: peers' memory may be written
    if (fastk) {
#pragma unroll
        for (int j = 0; j < CI_TGROUPS; ++j)
            if (tg[j] > CI_NEG_INF) atomicAdd(&hist1[min(CI_FAST_BINS - 1, __float2int_rz((lmax - tg[j]) * CI_FAST_SCALE))], 1u);
        __syncthreads();
        int bk; u64 before, have;
        bins_find(hist1, (u64)kk, sc, bk, before, have);
        if (have >= (u64)kk && bk >= 0 && bk < CI_FAST_BINS - 1)
            tl_fast = lmax - ((float)(bk + 1) + 0.01f) / CI_FAST_SCALE - fabsf(lmax) * 1e-6f;
        else tl_fast = -CI_FLT_MAX;                             // fewer than k threads saw a finite logit: take them all
        CI_PROF(10);
        int wn = 0;
        collect_region(rowbuf, r_lo, r_hi, tl_fast, mylist, wn, (uint32_t)slice_lo, lane);
        CI_PROF(11);
        if (lane == 0) sc->warp_i[warp] = wn;
        __syncthreads();                                        // every thread is done with the row buffer
        int woff = 0;
        bool over = false;
#pragma unroll
        for (int w = 0; w < CI_WARPS; ++w) {
            const int c = sc->warp_i[w];
            if (w < warp) woff += c;
            my_count += c;
            over |= c > CI_WLIST;
        }
        if (over || my_count > CI_PCAP) my_count = 0xFFFF;      // overflow marker: the row takes the generic path later
        else {
            // push this CTA's candidates, in token order, to the CTA that will finish the row
            Cand* dst = cluster.map_shared_rank(plist, fast_seq % CS) + rank * CI_PCAP + woff;
            for (int j = lane; j < wn; j += 32) dst[j] = mylist[j];
        }
        // the row buffer is free: start the next row's copies now
        if (a.use_bulk && next_row >= 0) {
            if (tid == 0) issue_row(next_row);
            prefetched = true;
        }
    } else if (!sampled && a.use_bulk && next_row >= 0) {
        // greedy row: only the maximum is needed from here on
        if (tid == 0) issue_row(next_row);
        prefetched = true;
    }

    // ---------------------------------------------------------------------------------------- first exchange
    CI_PROF(3);
    if (tid < CS) {
        Hello h;
        h.lmax = lmax; h.lidx = lidx;
        h.flags = (sc->fail ? 1 : 0) | (sc->hist_slow ? 4 : 0) | (sc->want_fast_off ? 8 : 0);
        h.pad = my_count;
        cluster.map_shared_rank(sc, tid)->hello[par][rank] = h;
    }
    cluster.sync();                                                                    // (1) slice maxima (and list sizes) exchanged
    CI_PROF(4);
    float L = CI_NEG_INF; int aidx = 0x7fffffff; int hflags = 0; int fast_total = 0; bool fast_overflow = false;
    for (int q = 0; q < CS; ++q) {
        const Hello h = sc->hello[par][q];
        if (h.lmax > L || (h.lmax == L && h.lidx < aidx)) { L = h.lmax; aidx = h.lidx; }
        hflags |= h.flags;
        fast_total += h.pad;
        if (h.pad >= 0xFFFF) fast_overflow = true;
    }
    if (aidx == 0x7fffffff) aidx = 0;
    if (hflags & 8) fast_enabled = false;                       // a CTA ran out of room for set-aside rows

    int status = ((hflags & 1) ? COLINFER_ROW_TIMEOUT : 0) | ((hflags & 4) ? COLINFER_ROW_HIST_SLOW : 0);
    const bool finite_max = (L > CI_NEG_INF) && (L < CI_POS_INF);
    if (sampled && !finite_max) status |= COLINFER_ROW_DEGENERATE;
    const bool do_dist = sampled && finite_max && !(hflags & 1);   // identical in every CTA of the cluster

    float lcut = CI_NEG_INF;
    u64 total_mass = 0;
    long long token = aidx;

    if (!do_dist) {
        // greedy, degenerate or failed row: the argmax.  Nobody reads a peer's memory after the barrier: leave at once.
        if (rank == 0 && tid == 0) {
            if (a.out) a.out[row] = token;
            if (a.status) a.status[row] = status;
            if (a.stats) {
                colinfer_row_stats st;
                st.lmax = L; st.lcut = lcut; st.tc = tc; st.status = status; st.argmax = aidx; st.mass_q = 0;
                a.stats[row] = st;
            }
        }
        return;
    }

    // ---------------------------------------------------------------------------------------- small top-k: defer the exact finish
    if (fastk) {
        // The candidates of every CTA sit in the shared memory of CTA fast_seq % CS, which finishes the row later, on its
        // own, while the cluster moves on.  A row whose lists overflowed is set aside for the generic path instead.
        const bool deferred = !fast_overflow && fast_total >= 1;
        if (deferred) {
            if (rank == fast_seq % CS && tid == 0) {
                Pending pd;
                pd.row = row; pd.L = L; pd.aidx = aidx; pd.status = status;
                for (int q = 0; q < 8; ++q) pd.count[q] = q < CS ? sc->hello[par][q].pad : 0;
                sc->pend = pd;
            }
            ++fast_seq;
            if (fast_seq % CS == 0) flush();                    // every CTA holds a row now
        } else {
            if (tid == 0 && sc->n_retry_common < CI_RETRY) sc->retry_common[sc->n_retry_common++] = row;
            if (++n_set_aside >= CI_RETRY) fast_enabled = false;
        }
        return;
    }

    const float m = scale_logit(L, tc);
    MassFn mass;
    mass.init(tc, m);
    // ---------------------------------------------------------------------------------------- min-p threshold
    const float thr = __fadd_rn(m, log_min_p);
    lcut = lower_logit_for(thr, tc, __fmul_rn(thr, tc));
    // Mass horizon: a logit more than 22 temperatures below the maximum has integer mass 0 (2^30 exp(-22) < 1/2); it can
    // never be drawn and adds nothing to any sum, so every selection works above it.
    lcut = fmaxf(lcut, L - 22.0f * tc - fabsf(L) * 1e-6f);
    bool need_topk = kk > 0 && kk < V;
    const bool need_topp = topp < 1.0f;
    const float u = row_uniform(a, row, b, r);

    // (generic path from here on: the whole cluster works on the row until its token is out)
    enum { PATH_PURE = 0, PATH_LIST = 1, PATH_BAND = 2, PATH_FALLBACK = 3 };
    int path = PATH_PURE;
    float t_hi = CI_NEG_INF, t_lo = CI_POS_INF;                 // band thresholds (PATH_BAND), list threshold (PATH_LIST: t_lo)

    if (need_topk || need_topp) {
        // ------------------------------------------------------------------------------------ fine count histogram
        const float SC = (float)CI_NB1 / (CI_RANGE * tc);
        const float lk = fmaxf(lcut, -CI_FLT_MAX);             // excludes -inf (masked / padding) as well
        for (int i = tid; i < CI_NB1; i += CI_THREADS) hist1[i] = 0u;
        if (tid == 0) xch->list_overflow = 0;
        __syncthreads();
        {
            const float4* row4 = reinterpret_cast<const float4*>(rowbuf);
            const int n4 = n_pad >> 2;
            for (int i0 = tid; i0 < n4; i0 += 4 * CI_THREADS) {
                float e[16];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int i = i0 + k * CI_THREADS;
                    const float4 v = i < n4 ? row4[i] : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
                    e[4 * k] = v.x; e[4 * k + 1] = v.y; e[4 * k + 2] = v.z; e[4 * k + 3] = v.w;
                }
                int bkt[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) bkt[j] = min(CI_NB1 - 1, __float2int_rz((L - e[j]) * SC));
#pragma unroll
                for (int j = 0; j < 16; ++j) if (e[j] >= lk) atomicAdd(&hist1[bkt[j]], 1u);
            }
        }
        __syncthreads();
        CI_PROF(10);
        cluster.sync();                                                                // (A) local histograms complete
        CI_PROF(11);
        // each CTA reduces its segment of the buckets over the cluster
        const int G = CI_NB1 / CS;
        uint32_t* myseg = (CS == 1) ? hist1 : segcnt;
        u64 pc = 0, pe = 0;
        for (int g = tid; g < G; g += CI_THREADS) {
            uint32_t sum = 0;
            if (CS == 1) sum = hist1[g];
            else {
                for (int q = 0; q < CS; ++q) sum += cluster.map_shared_rank(hist1, q)[rank * G + g];
                segcnt[g] = sum;
            }
            pc += sum;
            pe += (u64)sum * bucket_mass_est(rank * G + g);
        }
        const u64 totc = block_sum_u64(pc, sc);
        const u64 tote = block_sum_u64(pe, sc);
        if (tid == 0) { xch->seg_cnt = totc; xch->seg_est = tote; }
        __syncthreads();
        cluster.sync();                                                                // (B) reduced segments published
        u64 segc[8], sege[8], survivors = 0, est_total = 0;
        for (int q = 0; q < CS; ++q) {
            const Xch* px = cluster.map_shared_rank(xch, q);
            segc[q] = px->seg_cnt; sege[q] = px->seg_est;
            survivors += segc[q]; est_total += sege[q];
        }
        if (need_topk && (u64)kk >= survivors) need_topk = false;   // fewer survivors than k: top-k removes nothing
        if (need_topk) {
            // bucket of the k-th largest logit, exactly
            int s_star = CS - 1; u64 before_seg = 0, run = 0;
            for (int q = 0; q < CS; ++q) {
                if (run + segc[q] >= (u64)kk) { s_star = q; before_seg = run; break; }
                run += segc[q];
            }
            const uint32_t* pseg = cluster.map_shared_rank(myseg, s_star);
            int g_star; u64 before;
            block_find([&](int i) { return (u64)pseg[i]; }, G, (u64)kk - before_seg, sc, g_star, before);
            const int bk = s_star * G + g_star;
            const u64 n_upto = before_seg + before + pseg[g_star];
            if (bk >= CI_NB1 - 3 || n_upto > CI_GLIST - 64) path = PATH_FALLBACK;
            else {
                path = PATH_LIST;
                // every element of buckets <= bk + 1 satisfies l >= t_lo (a slightly wider set is harmless)
                t_lo = L - ((float)(bk + 2) + 0.01f) / SC - fabsf(L) * 1e-6f;
            }
        } else if (need_topp) {
            // bucket where the descending cumulative estimated mass reaches top_p of the estimated total
            if (est_total == 0) path = PATH_FALLBACK;
            else {
                const u64 target = ceil_target(topp, est_total);
                int s_star = CS - 1; u64 before_seg = 0, run = 0;
                for (int q = 0; q < CS; ++q) {
                    if (run + sege[q] >= target) { s_star = q; before_seg = run; break; }
                    run += sege[q];
                }
                const uint32_t* pseg = cluster.map_shared_rank(myseg, s_star);
                int g_star; u64 before;
                block_find([&](int i) { return (u64)pseg[i] * bucket_mass_est(s_star * G + i); }, G, target - before_seg, sc, g_star, before);
                const int bp = s_star * G + g_star;
                const int up = a.dtype == COLINFER_BF16 ? 3 : 1, dn = a.dtype == COLINFER_BF16 ? 4 : 2;
                if (bp + dn + 2 >= CI_NB1) path = PATH_FALLBACK;
                else {
                    path = PATH_BAND;
                    t_hi = bp - up <= 0 ? CI_POS_INF : L - (float)(bp - up) / SC;
                    t_lo = L - (float)(bp + dn + 1) / SC;
                }
            }
        }
    }
    CI_PROF(5);

    // ---------------------------------------------------------------------------------------- large top-k (then top-p) on a gathered list
    bool done = false;
    if (path == PATH_LIST) {
        const float tl = fmaxf(fmaxf(t_lo, lcut), -CI_FLT_MAX);
        int wn = 0;
        collect_region(rowbuf, r_lo, r_hi, tl, mylist, wn, (uint32_t)slice_lo, lane);
        if (lane == 0) {
            xch->wcount[warp] = (unsigned short)min(wn, CI_WLIST);
            if (wn > CI_WLIST) xch->list_overflow = 1;
        }
        __syncthreads();
        CI_PROF(6);
        cluster.sync();                                                                // (L) lists published
        // every CTA gathers the lists and finishes alike (identical inputs, identical decisions)
        const int n = gather_lists(cluster, CS, xch, ownlist, glist, sc, mass);
        if (n > 0 && finish_on_list(glist, n, tl, lcut, tc, kk, need_topp, topp, u, bins, cand, sc, token, lcut, total_mass)) done = true;
        else path = PATH_FALLBACK;
    }

    // ---------------------------------------------------------------------------------------- fallback: exact radix select over the 32-bit keys
    if (path == PATH_FALLBACK) {
        // (a CTA reaches this point only after every peer finished reading its reduced segment and its lists: those
        // reads precede the peers' next cluster barrier, and the first write below follows this CTA's next barrier)
        const RadixCtx rc = {rowbuf, n_pad, fb_hist, fb_seg, xch, sc, rank, CS};
        float lpiv;
        if (kk > 0 && kk < V && radix_select(cluster, rc, mass, lcut, false, (u64)kk, topp, lpiv))
            lcut = fmaxf(lcut, lower_logit_for(scale_logit(lpiv, tc), tc, lpiv));
        if (need_topp && radix_select(cluster, rc, mass, lcut, true, 0, topp, lpiv))
            lcut = fmaxf(lcut, lower_logit_for(scale_logit(lpiv, tc), tc, lpiv));
        path = PATH_PURE;
        t_hi = CI_NEG_INF; t_lo = CI_POS_INF;
    }

    // ---------------------------------------------------------------------------------------- mass pass and inverse CDF over the row
    if (!done) {
        const bool band = path == PATH_BAND;
        const float lk = fmaxf(lcut, -CI_FLT_MAX);
        u64 acc_all = 0, acc_above = 0;
        int wn = 0;
        for (int i0 = r_lo; i0 < r_hi; i0 += 512) {
            float e[16];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + k * 128 + lane * 4;
                const float4 v = i < r_hi ? *reinterpret_cast<const float4*>(rowbuf + i) : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
                e[4 * k] = v.x; e[4 * k + 1] = v.y; e[4 * k + 2] = v.z; e[4 * k + 3] = v.w;
            }
            uint32_t q[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) q[j] = e[j] >= lk ? mass(e[j]) : 0u;
#pragma unroll
            for (int j = 0; j < 16; j += 2) acc_all += (u64)q[j] + q[j + 1];
            if (band) {
                unsigned mk[4], anym = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    mk[k] = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float x = e[4 * k + j];
                        if (x > t_hi) acc_above += q[4 * k + j];
                        else if (x >= t_lo && x >= lk) mk[k] |= 1u << j;
                    }
                    anym |= mk[k];
                }
                if (__ballot_sync(0xffffffffu, anym != 0u)) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        warp_append(mylist, wn, mk[k], &e[4 * k], (uint32_t)(slice_lo + i0 + k * 128 + lane * 4), lane);
                }
            }
        }
        u64 wkeep = warp_sum_u64(band ? acc_above : acc_all);   // kept mass of the region known so far
        if (band) {
            const u64 wall = warp_sum_u64(acc_all);
            if (lane == 0) {
                sc->warp_tot[warp] = wkeep; sc->warp_aux[warp] = wall;
                xch->wcount[warp] = (unsigned short)min(wn, CI_WLIST);
                if (wn > CI_WLIST) xch->list_overflow = 1;
            }
            __syncthreads();
            if (tid == 0) {
                u64 ta = 0, tb = 0;
                for (int w = 0; w < CI_WARPS; ++w) { ta += sc->warp_aux[w]; tb += sc->warp_tot[w]; }
                xch->s_all = ta; xch->s_above = tb;
            }
            __syncthreads();
            CI_PROF(11);
            cluster.sync();                                                            // (L) band lists and sums published
            u64 s1 = 0, s_above = 0;
            for (int q = 0; q < CS; ++q) {
                const Xch* px = cluster.map_shared_rank(xch, q);
                s1 += px->s_all; s_above += px->s_above;
            }
            const int n = gather_lists(cluster, CS, xch, ownlist, glist, sc, mass);
            bool ok = n >= 0 && s1 > 0;
            float cut2 = lcut;
            if (ok) {
                u64 part = 0;
                for (int i = tid; i < n; i += CI_THREADS) part += glist[i].q;
                const u64 s_band = block_sum_u64(part, sc);
                const u64 target = ceil_target(topp, s1);
                ok = s_above < target && target <= s_above + s_band;           // the pivot lies inside the band
                if (ok) {
                    float lp_val;
                    ok = list_select(glist, n, [&](int i) { return (u64)glist[i].q; }, target - s_above, bins, cand, sc, lp_val);
                    if (ok) {
                        cut2 = fmaxf(lcut, lower_logit_for(scale_logit(lp_val, tc), tc, lp_val));
                        if (cut2 < t_lo) ok = false;                           // a tie partner could lie below the band
                    }
                }
            }
            if (ok) {
                lcut = cut2;
                // add the kept band entries of this warp's own list to its region's kept mass
                u64 add = 0;
                const int mine = min(wn, CI_WLIST);
                for (int j = lane; j < mine; j += 32) if (mylist[j].l >= lcut) add += mass(mylist[j].l);
                wkeep += warp_sum_u64(add);
            } else {
                // The estimated band missed the pivot (or a list overflowed): every CTA takes the exact radix select
                // by mass, then recomputes its regions' kept mass.  Rare; same result, more time.
                const RadixCtx rc = {rowbuf, n_pad, fb_hist, fb_seg, xch, sc, rank, CS};
                float lpiv;
                if (radix_select(cluster, rc, mass, lcut, true, 0, topp, lpiv))
                    lcut = fmaxf(lcut, lower_logit_for(scale_logit(lpiv, tc), tc, lpiv));
                const float lk3 = fmaxf(lcut, -CI_FLT_MAX);
                u64 acc = 0;
                for (int i0 = r_lo; i0 < r_hi; i0 += 128) {
                    const float4 v = *reinterpret_cast<const float4*>(rowbuf + i0 + lane * 4);
                    acc += (u64)(v.x >= lk3 ? mass(v.x) : 0u) + (v.y >= lk3 ? mass(v.y) : 0u);
                    acc += (u64)(v.z >= lk3 ? mass(v.z) : 0u) + (v.w >= lk3 ? mass(v.w) : 0u);
                }
                wkeep = warp_sum_u64(acc);
            }
        }
        __syncthreads();
        if (lane == 0) sc->warp_tot[warp] = wkeep;
        __syncthreads();
        u64 my_mass = 0;
        for (int w = 0; w < CI_WARPS; ++w) my_mass += sc->warp_tot[w];
        if (tid < CS) cluster.map_shared_rank(sc, tid)->mass_in[par][rank] = my_mass;
        CI_PROF(6);
        cluster.sync();                                                                // (C) slice masses exchanged
        CI_PROF(7);
        u64 my_off = 0;
        for (int q = 0; q < CS; ++q) {
            const u64 cm = sc->mass_in[par][q];
            if (q < rank) my_off += cm;
            total_mass += cm;
        }
        const u64 target = ceil_target(u, total_mass);
        token = -1;
        if (total_mass > 0 && my_off < target && target <= my_off + my_mass) {
            // the crossing lies in this CTA: find the warp region, then the element
            u64 woff = my_off;
            for (int w = 0; w < warp; ++w) woff += sc->warp_tot[w];
            if (woff < target && target <= woff + wkeep) {
                const float lkf = fmaxf(lcut, -CI_FLT_MAX);
                u64 run = woff;
                for (int i0 = r_lo; i0 < r_hi; i0 += 128) {
                    const int i = i0 + lane * 4;
                    const float4 v = *reinterpret_cast<const float4*>(rowbuf + i);
                    u64 q4[4];
                    q4[0] = v.x >= lkf ? mass(v.x) : 0u; q4[1] = v.y >= lkf ? mass(v.y) : 0u;
                    q4[2] = v.z >= lkf ? mass(v.z) : 0u; q4[3] = v.w >= lkf ? mass(v.w) : 0u;
                    const u64 s4 = q4[0] + q4[1] + q4[2] + q4[3];
                    const u64 incl = warp_incl_scan_u64(s4, lane);
                    const u64 grp = __shfl_sync(0xffffffffu, incl, 31);
                    if (run + grp >= target) {
                        const unsigned hit = __ballot_sync(0xffffffffu, run + incl >= target);
                        const int first = __ffs(hit) - 1;
                        if (lane == first) {
                            u64 c = run + incl - s4;
                            int j = 0;
                            for (; j < 3; ++j) { c += q4[j]; if (c >= target) break; }
                            if (a.out) a.out[row] = (long long)(slice_lo + i + j);
                        }
                        break;
                    }
                    run += grp;
                }
            }
        }
        if (total_mass == 0) { status |= COLINFER_ROW_DEGENERATE; token = aidx; }
    }

    if (rank == 0 && tid == 0) {
        if (token >= 0 && a.out) a.out[row] = token;           // list-path or degenerate rows (else the crossing lane stored it)
        if (a.status) a.status[row] = status;
        if (a.stats) {
            colinfer_row_stats st;
            st.lmax = L; st.lcut = lcut; st.tc = tc; st.status = status; st.argmax = aidx; st.mass_q = total_mass;
            a.stats[row] = st;
        }
    }
    CI_PROF(8);
    // After the mass exchange nobody reads a peer's memory; after a list path peers may still be gathering: wait for them.
    if (done) cluster.sync();
    CI_PROF(9);
    };  // process_row

    if (a.prof && tid == 0 && (int)blockIdx.x < a.prof_slots) {
        unsigned long long gt; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
        unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        a.prof[(size_t)blockIdx.x * 16 + 15] = (long long)gt; a.prof[(size_t)blockIdx.x * 16 + 14] = smid;
    }
    int it = 0;
    for (long long row = blockIdx.x / CS; row < n_rows; row += n_clusters, ++it) {
        if (it) __syncthreads();                               // every thread is done with the previous row's buffers
        const long long nxt = row + n_clusters < n_rows ? row + n_clusters : -1;
        process_row((int)row, it, true, nxt);
    }
    // Deferred rows still waiting; then the rows that were set aside take the generic path.
    if (it == 0) cluster.barrier_wait();                       // (a cluster without rows still completes the opening barrier)
    flush();
    {
        int n_all = 0;
        if (tid == 0) {
            for (int i = 0; i < sc->n_retry_common; ++i) sc->retry_all[n_all++] = sc->retry_common[i];
            for (int q = 0; q < CS; ++q) {
                const Scratch* ps = cluster.map_shared_rank(sc, q);
                const int nq = ps->n_retry_mine;
                for (int i = 0; i < nq && i < CI_RETRY; ++i) sc->retry_all[n_all++] = ps->retry_mine[i];
            }
            sc->bcast_i[0] = n_all;
        }
        cluster.sync();                                        // every CTA has read the peers' lists
        n_all = sc->bcast_i[0];
        for (int i = 0; i < n_all; ++i, ++it) {
            __syncthreads();
            process_row(sc->retry_all[i], it, false, -1);
        }
    }
    if (a.prof && tid == 0 && (int)blockIdx.x < a.prof_slots) {
        unsigned long long gt; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
        a.prof[(size_t)blockIdx.x * 16 + 13] = (long long)gt;
        a.prof[(size_t)blockIdx.x * 16 + 12] = clock64() - prof_t0;
        for (int i = 0; i < 12; ++i) a.prof[(size_t)blockIdx.x * 16 + i] = sc->prof[i];
    }
}

// ------------------------------------------------------------------------------------------------ host side
int colinfer_launch_stream(const void*, int, const int32_t*, int, int, const colinfer_sampler_params*, const void*, int, const float*,
                           int64_t*, colinfer_row_stats*, int32_t*, int, int, int, int, cudaStream_t);

#ifdef COLINFER_PROFILE
static long long* g_prof = nullptr;                        // profiling builds only: cycles per phase of later launches
static int g_prof_slots = 0;
#endif
static const int kFixedSmem = 24 * 1024 + (CI_WARPS * CI_WLIST + 8 * CI_PCAP) * (int)sizeof(Cand) + CI_MAX_CHUNKS * 8 +
                              (int)sizeof(Xch) + (int)sizeof(Scratch) + 64;

// forced: 0 = the smallest cluster that holds the row; 1, 2, 4, 8 = that cluster size
static int pick_geometry(int V, int dtype, const void* logits, int forced, colinfer_geometry* g) {
    if (V <= 0) return 1;
    const int cap2 = (113 * 1024 - kFixedSmem) / 4;           // slice elements that allow two CTAs per SM
    const int cap1 = (226 * 1024 - kFixedSmem) / 4;           // one CTA per SM
    const int max_slice = CI_CHUNK * CI_MAX_CHUNKS;
    int cs = 0, slice = 0;
    auto slice_for = [&](int c) { return (((V + c - 1) / c) + 127) & ~127; };
    if (forced > 0) {
        cs = forced; slice = slice_for(cs);
        if (slice > cap1 || slice > max_slice) return 1;
    } else {
        for (int c = 1; c <= 8 && !cs; c *= 2) if (slice_for(c) <= cap2 && slice_for(c) <= max_slice) { cs = c; slice = slice_for(c); }
        for (int c = 1; c <= 8 && !cs; c *= 2) if (slice_for(c) <= cap1 && slice_for(c) <= max_slice) { cs = c; slice = slice_for(c); }
        if (!cs) return 1;
    }
    g->cluster = cs;
    g->slice_elems = slice;
    g->smem_bytes = slice * 4 + kFixedSmem;
    g->bulk_copy = (dtype == COLINFER_F32 && (V % 4) == 0 && (((uintptr_t)logits) & 15) == 0) ? 1 : 0;
    return 0;
}

extern "C" int colinfer_sample_geometry(int V, int dtype, const void* logits, int cluster, colinfer_geometry* out) {
    if (cluster != 0 && cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return (int)cudaErrorInvalidValue;
    return pick_geometry(V, dtype, logits, cluster, out) ? (int)cudaErrorInvalidValue : 0;
}

#ifdef COLINFER_PROFILE
void colinfer_profile_buffer(long long** buf, int* slots) { *buf = g_prof; *slots = g_prof_slots; }
// (profiling builds) the first `ctas` CTAs of later launches add their cycles per phase into dev[ctas * 16]
extern "C" int colinfer_set_profile_buffer(void* dev, int ctas) {
    g_prof = reinterpret_cast<long long*>(dev);
    g_prof_slots = dev ? ctas : 0;
    return 0;
}
#else
void colinfer_profile_buffer(long long** buf, int* slots) { *buf = nullptr; *slots = 0; }
#endif

static void fill_launch(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, const colinfer_geometry& g, long long clusters, cudaStream_t st) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3((unsigned)(clusters * g.cluster), 1, 1);
    cfg.blockDim = dim3(CI_THREADS, 1, 1);
    cfg.dynamicSmemBytes = (size_t)g.smem_bytes;
    cfg.stream = st;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)g.cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
}

// Clusters of this geometry that the current device holds at once (cached per device and geometry): the kernel is
// persistent, each cluster walks over rows, so the grid never exceeds this.
static int active_clusters(const colinfer_geometry& g) {
    struct Entry { int dev, smem, cs, n; };
    static Entry cache[16];
    static int used = 0;
    static std::mutex guard;
    std::lock_guard<std::mutex> lock(guard);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    for (int i = 0; i < used; ++i)
        if (cache[i].dev == dev && cache[i].smem == g.smem_bytes && cache[i].cs == g.cluster) return cache[i].n;
    if (cudaFuncSetAttribute(k_sample, cudaFuncAttributeMaxDynamicSharedMemorySize, g.smem_bytes) != cudaSuccess) return -2;
    cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[1];
    fill_launch(cfg, attr, g, 1024, nullptr);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, k_sample, &cfg) != cudaSuccess || n <= 0) return -3;
    if (used < 16) cache[used++] = Entry{dev, g.smem_bytes, g.cluster, n};
    return n;
}

extern "C" int colinfer_max_active_clusters(int V, int dtype) {
    colinfer_geometry g;
    if (pick_geometry(V, dtype, nullptr, 0, &g)) return -1;
    return active_clusters(g);
}

extern "C" int colinfer_sample(const void* logits, int dtype, const int32_t* mask, int mask_rows, int W,
                               const colinfer_sampler_params* params, const void* pos, int pos_is_i64, const float* u,
                               int64_t* out_ids, colinfer_row_stats* stats, int32_t* status,
                               int B, int R, int V, int flags, void* stream) {
    if (B < 0 || R < 0 || V <= 0) return (int)cudaErrorInvalidValue;
    if ((long long)B * R == 0) return 0;
    if (!logits || !params || (!out_ids && !stats)) return (int)cudaErrorInvalidValue;
    if (dtype != COLINFER_F32 && dtype != COLINFER_BF16) return (int)cudaErrorInvalidValue;
    if (!params->temperature || !params->top_k || !params->top_p || !params->log_min_p) return (int)cudaErrorInvalidValue;
    if (out_ids && u == nullptr && (pos == nullptr || params->seed == nullptr)) return (int)cudaErrorInvalidValue;
    if (mask && (W < (V + 31) / 32 || mask_rows < R)) return (int)cudaErrorInvalidValue;
    if ((long long)B * R > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
    // Which kernel: the caller's choice (bits COLINFER_KERNEL_* of flags), else automatic.  Few rows -- at most as many
    // as the device holds clusters at once -- are a latency problem: one CTA per row would leave most SMs idle, so each
    // row gets a whole 8-CTA cluster of the cluster-resident kernel.  More rows are a throughput problem: the streaming
    // kernel (one CTA per row, later passes over L2).  The cluster-resident kernel also runs when a row's tables do not
    // fit the streaming kernel.
    const int choice = (flags >> 8) & 7;                   // 0 auto, 1 streaming, 2 .. 5: clusters of 1, 2, 4, 8
    if (choice > 5) return (int)cudaErrorInvalidValue;
    const int forced = choice >= 2 ? (1 << (choice - 2)) : 0;
    if (choice <= 1) {
        bool use_stream = true;
        if (choice == 0) {
            colinfer_geometry g0;
            if (!pick_geometry(V, dtype, logits, 0, &g0)) {
                const int res0 = active_clusters(g0);
                if (res0 > 0 && (long long)B * R <= res0) use_stream = false;
            }
        }
        if (use_stream) {
            const int rc = colinfer_launch_stream(logits, dtype, mask, mask_rows, W, params, pos, pos_is_i64, u, out_ids, stats, status,
                                                  B, R, V, flags, (cudaStream_t)stream);
            if (rc != (int)cudaErrorInvalidValue) return rc;
        }
    }
    colinfer_geometry g;
    if (pick_geometry(V, dtype, logits, forced, &g)) return (int)cudaErrorInvalidValue;
    const int resident = active_clusters(g);
    if (resident <= 0) return (int)cudaErrorInvalidConfiguration;
    const long long clusters = (long long)B * R < resident ? (long long)B * R : resident;

    SampleArgs a;
    a.logits = logits; a.dtype = dtype; a.use_bulk = g.bulk_copy;
    a.mask = mask; a.mask_rows = mask_rows; a.W = W;
    a.p = *params;
    a.pos = pos; a.pos_i64 = pos_is_i64; a.u = u;
    a.out = out_ids; a.stats = stats; a.status = status;
    a.B = B; a.R = R; a.V = V; a.slice_elems = g.slice_elems; a.flags = flags;
    colinfer_profile_buffer(&a.prof, &a.prof_slots);

    cudaError_t e = cudaFuncSetAttribute(k_sample, cudaFuncAttributeMaxDynamicSharedMemorySize, g.smem_bytes);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[1];
    fill_launch(cfg, attr, g, clusters, (cudaStream_t)stream);
    e = cudaLaunchKernelEx(&cfg, k_sample, a);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}
