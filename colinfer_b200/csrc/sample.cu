// sample.cu -- the fused logits -> token kernel (sm_100a).
//
// One thread-block cluster per row.  Each CTA of the cluster copies its slice of the row from HBM into its own shared
// memory exactly once (1-D bulk copies completed on mbarriers when the row is 16-byte aligned fp32, plain loads
// otherwise) and the whole row stays resident in the cluster's distributed shared memory.  Everything after that --
// penalties, grammar mask, row maximum / argmax, the min-p / top-k / top-p threshold selects and the inverse-CDF draw --
// works on shared memory, so HBM is read once per row whatever the sampling parameters are.
//
// Selection is exact and order independent.  The kept set is always {logit >= threshold}; thresholds are found by a
// three-level radix select over the order-preserving 32-bit key of the logit, with count histograms for top-k and
// mass histograms for top-p.  Masses are exp(z - max) rounded to integers in units of 2^-40 and summed as integers:
// every histogram, every prefix sum and the CDF crossing are therefore independent of thread, CTA and cluster geometry
// and of the other rows in the launch (the reference's row-invariance property).
//
// What the reference does in ~25 torch / FlashInfer launches per slot (engine/spec/accept.py:23-52 after
// engine/runtime/sampler.py:50-56) is one launch here.
#include "common.cuh"
#include "../../include/colinfer_b200.h"

#define CI_THREADS 512
#define CI_WARPS (CI_THREADS / 32)
#define CI_CHUNK 4096            // elements per bulk copy
#define CI_MAX_CHUNKS 16
#define CI_NB 2048               // radix buckets per level (11 bits)
#define CI_PEN_TABLE 2048        // distinct history ids per slice with an O(1) count
#define CI_WAIT_CYCLES 400000000LL

struct SampleArgs {
    const void* logits; int dtype; int use_bulk;
    const int32_t* mask; int mask_rows; int W;
    colinfer_sampler_params p;
    const void* pos; int pos_i64; const float* u;
    int64_t* out; colinfer_row_stats* stats; int32_t* status;
    int B, R, V; int slice_elems; int flags;
};

// Values one CTA publishes to its cluster peers.
struct Xch {
    float lmax; int lidx;          // slice maximum and its lowest global index
    u64 segtot;                    // total of this CTA's reduced histogram segment
    u64 cta_mass;                  // kept mass of this CTA's slice
};

struct Scratch {
    u64 warp_tot[CI_WARPS];
    float warp_f[CI_WARPS]; int warp_i[CI_WARPS];
    int found_idx; u64 found_before;
    int fail;
    int hist_slow;
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

// Effective logit of one token outside the resident row: penalties (by scanning the history) and mask.  Used by the
// verify finish kernel; one thread.
__device__ float effective_logit(float l, int tok, int V, const int32_t* hist, int hlen, float rp, float pp, float fp,
                                 const int32_t* mask_row) {
    if (hist != nullptr && hlen > 0 && !(rp == 1.0f && pp == 0.0f && fp == 0.0f)) {
        int cnt = 0;
        for (int i = 0; i < hlen; ++i) cnt += (hist[i] == tok);
        if (cnt > 0) {
            l = l > 0.0f ? __fdiv_rn(l, rp) : __fmul_rn(l, rp);
            l = __fsub_rn(l, __fmul_rn(fp, (float)cnt));
            l = __fsub_rn(l, pp);
        }
    }
    if (mask_row != nullptr && !((mask_row[tok >> 5] >> (tok & 31)) & 1)) l = CI_NEG_INF;
    return l;
}

__device__ __forceinline__ float apply_penalty(float l, int cnt, float rp, float pp, float fp) {
    l = l > 0.0f ? __fdiv_rn(l, rp) : __fmul_rn(l, rp);
    l = __fsub_rn(l, __fmul_rn(fp, (float)cnt));
    return __fsub_rn(l, pp);
}

extern "C" __global__ void __launch_bounds__(CI_THREADS, 2) k_sample(const __grid_constant__ SampleArgs a) {
    cg::cluster_group cluster = cg::this_cluster();
    const int CS = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int row = blockIdx.x / CS;
    const int b = row / a.R, r = row % a.R;
    const int tid = threadIdx.x, lane = lane_id(), warp = warp_id();
    const int V = a.V;

    const int slice_cap = a.slice_elems;                      // multiple of 128
    const int slice_lo = rank * slice_cap;
    const int slice_len = max(0, min(slice_cap, V - slice_lo));
    const int n_pad = (slice_len + 127) & ~127;               // processed elements (tail holds -inf)

    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* rowbuf = reinterpret_cast<float*>(smem_raw);
    u64* hist64 = reinterpret_cast<u64*>(smem_raw + (size_t)slice_cap * 4);
    uint32_t* hist32 = reinterpret_cast<uint32_t*>(hist64);
    u64* seg = hist64 + CI_NB;
    u64* mbar = seg + CI_NB;
    Xch* xch = reinterpret_cast<Xch*>(mbar + CI_MAX_CHUNKS);
    Scratch* sc = reinterpret_cast<Scratch*>(xch + 1);
    // penalty tables alias the histogram area (used before the first histogram)
    uint32_t* pen_bits = hist32;
    const int nw = slice_cap >> 5;
    uint32_t* pen_prefix = pen_bits + nw;
    uint32_t* pen_cnt = pen_prefix + nw;

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
    const int nchunks = (slice_len + CI_CHUNK - 1) / CI_CHUNK;

    // ---------------------------------------------------------------------------------------- start the HBM read
    if (tid == 0) {
        sc->fail = 0; sc->hist_slow = 0;
        if (a.use_bulk) {
            for (int c = 0; c < nchunks; ++c) mbar_init(&mbar[c], 1);
            fence_mbar_init();
            fence_proxy_async();
        }
    }
    __syncthreads();
    if (a.use_bulk && tid == 0) {
        const float* src = reinterpret_cast<const float*>(a.logits) + (size_t)row * V + slice_lo;
        for (int c = 0; c < nchunks; ++c) {
            const int len = min(CI_CHUNK, slice_len - c * CI_CHUNK);
            mbar_expect_tx(&mbar[c], (uint32_t)len * 4u);
            bulk_g2s(rowbuf + c * CI_CHUNK, src + c * CI_CHUNK, (uint32_t)len * 4u, &mbar[c]);
        }
    }
    // tail of the slice buffer: -inf (never selected, zero mass); disjoint from the bulk-copy destinations
    for (int i = slice_len + tid; i < n_pad; i += CI_THREADS) rowbuf[i] = CI_NEG_INF;
    __syncthreads();

    // ---------------------------------------------------------------------------------------- penalty tables
    // bitmap of the slice's tokens that occur in the history, their ranks, and the occurrence count per rank
    if (has_pen) {
        for (int i = tid; i < nw; i += CI_THREADS) pen_bits[i] = 0u;
        for (int i = tid; i < CI_PEN_TABLE; i += CI_THREADS) pen_cnt[i] = 0u;
        __syncthreads();
        for (int i = tid; i < hlen; i += CI_THREADS) {
            const int v = hist[i] - slice_lo;
            if (v >= 0 && v < slice_len) atomicOr(&pen_bits[v >> 5], 1u << (v & 31));
        }
        __syncthreads();
        // exclusive prefix of popcounts over the bitmap words (block scan, contiguous words per thread)
        {
            const int ipt = (nw + CI_THREADS - 1) / CI_THREADS;
            const int lo = tid * ipt;
            u64 local = 0;
            for (int i = lo; i < lo + ipt && i < nw; ++i) local += __popc(pen_bits[i]);
            const u64 incl = warp_incl_scan_u64(local, lane);
            if (lane == 31) sc->warp_tot[warp] = incl;
            __syncthreads();
            u64 off = 0;
            for (int w = 0; w < warp; ++w) off += sc->warp_tot[w];
            uint32_t run = (uint32_t)(off + incl - local);
            for (int i = lo; i < lo + ipt && i < nw; ++i) { pen_prefix[i] = run; run += __popc(pen_bits[i]); }
            __syncthreads();
        }
        for (int i = tid; i < hlen; i += CI_THREADS) {
            const int v = hist[i] - slice_lo;
            if (v >= 0 && v < slice_len) {
                const uint32_t w = pen_bits[v >> 5];
                const uint32_t rk = pen_prefix[v >> 5] + __popc(w & ((1u << (v & 31)) - 1u));
                if (rk < CI_PEN_TABLE) atomicAdd(&pen_cnt[rk], 1u);
            }
        }
        __syncthreads();
    }

    // ---------------------------------------------------------------------------------------- pass A: land, penalise, mask, maximum
    float lmax = CI_NEG_INF;
    int lidx = 0x7fffffff;
    const int n_pass_chunks = (n_pad + CI_CHUNK - 1) / CI_CHUNK;
    for (int c = 0; c < n_pass_chunks; ++c) {
        const int c_lo = c * CI_CHUNK;
        const int c_len = min(CI_CHUNK, n_pad - c_lo);          // multiple of 128
        if (c < nchunks) {
            if (a.use_bulk) {
                if (!mbar_wait_bounded(&mbar[c], 0, CI_WAIT_CYCLES)) sc->fail = 1;
            } else {
                const int valid = min(CI_CHUNK, slice_len - c_lo);
                const size_t g0 = (size_t)row * V + slice_lo + c_lo;
                if (a.dtype == COLINFER_BF16) {
                    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(a.logits) + g0;
                    if ((((uintptr_t)src) & 15) == 0) {
                        const uint4* s4 = reinterpret_cast<const uint4*>(src);
                        for (int i = tid; i * 8 < valid; i += CI_THREADS) {
                            if (i * 8 + 8 <= valid) {
                                const uint4 q = __ldg(s4 + i);
                                const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
                                float* d = rowbuf + c_lo + i * 8;
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    d[2 * j] = __uint_as_float(ww[j] << 16);
                                    d[2 * j + 1] = __uint_as_float(ww[j] & 0xFFFF0000u);
                                }
                            } else {
                                for (int j = i * 8; j < valid; ++j) rowbuf[c_lo + j] = __bfloat162float(src[j]);
                            }
                        }
                    } else {
                        for (int i = tid; i < valid; i += CI_THREADS) rowbuf[c_lo + i] = __bfloat162float(src[i]);
                    }
                } else {
                    const float* src = reinterpret_cast<const float*>(a.logits) + g0;
                    for (int i = tid; i < valid; i += CI_THREADS) rowbuf[c_lo + i] = __ldg(src + i);
                }
                __syncthreads();
            }
        }
        if (has_pen) {
            // one bitmap word (32 tokens) per thread
            const int w0 = c_lo >> 5, wn = c_len >> 5;
            for (int wi = tid; wi < wn; wi += CI_THREADS) {
                const uint32_t word = pen_bits[w0 + wi];
                uint32_t rest = word;
                while (rest) {
                    const int bit = __ffs(rest) - 1;
                    rest &= rest - 1;
                    const int v = ((w0 + wi) << 5) + bit;
                    const uint32_t rk = pen_prefix[w0 + wi] + __popc(word & ((1u << bit) - 1u));
                    int cnt;
                    if (rk < CI_PEN_TABLE) cnt = (int)pen_cnt[rk];
                    else {
                        cnt = 0; sc->hist_slow = 1;
                        for (int i = 0; i < hlen; ++i) cnt += (hist[i] == v + slice_lo);
                    }
                    rowbuf[v] = apply_penalty(rowbuf[v], cnt, rp, pp, fp);
                }
            }
            __syncthreads();
        }
        float4* row4 = reinterpret_cast<float4*>(rowbuf + c_lo);
        for (int i = tid; i * 4 < c_len; i += CI_THREADS) {
            float4 v = row4[i];
            const int g = slice_lo + c_lo + i * 4;              // global token index of v.x
            if (mrow != nullptr && g < V) {
                const uint32_t bits = ((uint32_t)__ldg(mrow + (g >> 5)) >> (g & 31)) & 0xFu;
                if (bits != 0xFu) {
                    if (!(bits & 1u)) v.x = CI_NEG_INF;
                    if (!(bits & 2u)) v.y = CI_NEG_INF;
                    if (!(bits & 4u)) v.z = CI_NEG_INF;
                    if (!(bits & 8u)) v.w = CI_NEG_INF;
                    row4[i] = v;
                }
            }
            const float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
            if (m4 > lmax) {
                lmax = m4;
                lidx = g + (v.x == m4 ? 0 : v.y == m4 ? 1 : v.z == m4 ? 2 : 3);
            }
        }
    }
    // block reduce (largest value, lowest index among equals)
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, lmax, o);
        const int oi = __shfl_xor_sync(0xffffffffu, lidx, o);
        if (om > lmax || (om == lmax && oi < lidx)) { lmax = om; lidx = oi; }
    }
    if (lane == 0) { sc->warp_f[warp] = lmax; sc->warp_i[warp] = lidx; }
    __syncthreads();
    if (tid == 0) {
        float bm = sc->warp_f[0]; int bi = sc->warp_i[0];
        for (int w = 1; w < CI_WARPS; ++w) {
            const float om = sc->warp_f[w]; const int oi = sc->warp_i[w];
            if (om > bm || (om == bm && oi < bi)) { bm = om; bi = oi; }
        }
        xch->lmax = bm; xch->lidx = bi;
    }
    __syncthreads();
    cluster.sync();                                                                    // (1) slice maxima published
    float L = CI_NEG_INF; int aidx = 0x7fffffff; int any_fail = 0;
    for (int q = 0; q < CS; ++q) {
        const Xch* px = cluster.map_shared_rank(xch, q);
        const Scratch* ps = cluster.map_shared_rank(sc, q);
        const float om = px->lmax; const int oi = px->lidx;
        if (om > L || (om == L && oi < aidx)) { L = om; aidx = oi; }
        any_fail |= ps->fail;
    }
    if (aidx == 0x7fffffff) aidx = 0;

    int status = any_fail ? COLINFER_ROW_TIMEOUT : 0;
    const bool finite_max = (L > CI_NEG_INF) && (L < __int_as_float(0x7f800000));
    if (sampled && !finite_max) status |= COLINFER_ROW_DEGENERATE;
    const bool do_dist = sampled && finite_max && !any_fail;   // identical in every CTA of the cluster

    float lcut = CI_NEG_INF;
    u64 total_mass = 0;
    long long token = aidx;

    if (do_dist) {
        const float m = scale_logit(L, tc);
        // ------------------------------------------------------------------------------------ min-p threshold
        const float lmp = a.p.log_min_p[b];
        const float thr = __fadd_rn(m, lmp);
        lcut = lower_logit_for(thr, tc, __fmul_rn(thr, tc));
        int kk = a.p.top_k[b];
        const bool do_topk = kk > 0 && kk < V;
        const float topp = a.p.top_p[b];
        const bool do_topp = topp < 1.0f;

        // ------------------------------------------------------------------------------------ radix selects
        // stage 0: k-th largest by count; stage 1: top-p pivot by mass.  Three levels each (11 + 11 + 10 key bits).
        for (int stage = 0; stage < 2; ++stage) {
            if (stage == 0 && !do_topk) continue;
            if (stage == 1 && !do_topp) continue;
            const bool by_mass = stage == 1;
            uint32_t prefix = 0;
            u64 target = by_mass ? 0 : (u64)kk;
            bool skip = false;
            for (int lvl = 0; lvl < 3; ++lvl) {
                const int shift = lvl == 0 ? 21 : lvl == 1 ? 10 : 0;
                const int nbits = lvl == 2 ? 10 : 11;
                const int nb = 1 << nbits;
                for (int i = tid; i < nb; i += CI_THREADS) hist64[i] = 0;
                __syncthreads();
                const float4* row4 = reinterpret_cast<const float4*>(rowbuf);
                for (int i = tid; i * 4 < n_pad; i += CI_THREADS) {
                    const float4 v = row4[i];
                    const float e4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float l = e4[j];
                        if (l >= lcut && l > CI_NEG_INF) {
                            const uint32_t key = f2key(l);
                            if (lvl == 0 || (key >> (shift + nbits)) == prefix) {
                                const int bk = nb - 1 - (int)((key >> shift) & (uint32_t)(nb - 1));
                                if (by_mass) atomicAdd(&hist64[bk], mass_q(l, tc, m));
                                else atomicAdd(&hist32[bk * 2], 1u);   // low word of the 64-bit slot
                            }
                        }
                    }
                }
                __syncthreads();
                cluster.sync();                                                        // (A) local histograms complete
                const int G = nb / CS;
                u64 part = 0;
                for (int g = tid; g < G; g += CI_THREADS) {
                    u64 sum = 0;
                    for (int q = 0; q < CS; ++q) {
                        const u64* ph = cluster.map_shared_rank(hist64, q);
                        u64 x = ph[rank * G + g];
                        if (!by_mass) x &= 0xFFFFFFFFull;
                        sum += x;
                    }
                    seg[g] = sum;
                    part += sum;
                }
                const u64 tot = block_sum_u64(part, sc);
                if (tid == 0) xch->segtot = tot;
                __syncthreads();
                cluster.sync();                                                        // (B) reduced segments published
                u64 grand = 0;
                u64 segtots[8];
                for (int q = 0; q < CS; ++q) { segtots[q] = cluster.map_shared_rank(xch, q)->segtot; grand += segtots[q]; }
                if (lvl == 0) {
                    if (by_mass) {
                        // target = smallest integer >= top_p * mass, at least 1
                        double t = ceil((double)topp * (double)grand);
                        u64 tq = t <= 1.0 ? 1ull : (u64)t;
                        if (tq > grand) tq = grand;
                        target = tq;
                    } else if (target >= grand) {
                        skip = true;                          // fewer survivors than k: top-k removes nothing
                    }
                }
                if (grand == 0) skip = true;
                if (skip) break;                              // identical decision in every CTA
                int s_star = CS - 1; u64 before_seg = 0;
                {
                    u64 run = 0;
                    for (int q = 0; q < CS; ++q) {
                        if (run + segtots[q] >= target) { s_star = q; before_seg = run; break; }
                        run += segtots[q];
                    }
                }
                const u64* pseg = cluster.map_shared_rank(seg, s_star);
                int g_star; u64 before;
                block_find([&](int i) { return pseg[i]; }, G, target - before_seg, sc, g_star, before);
                const int b_star = s_star * G + g_star;
                target -= before_seg + before;
                prefix = (prefix << nbits) | (uint32_t)(nb - 1 - b_star);
            }
            if (!skip) {
                const float lpiv = key2f(prefix);
                const float zc = scale_logit(lpiv, tc);
                lcut = fmaxf(lcut, lower_logit_for(zc, tc, lpiv));
            }
            // make sure no peer still reads this CTA's segment when the next stage rewrites it: the next stage's
            // sync (A) orders that; after the last stage the CDF sync below does.
        }

        // ------------------------------------------------------------------------------------ inverse CDF over the kept set
        // warp w owns the contiguous region [w * reg, (w + 1) * reg) of the slice; lanes interleave float4 groups.
        const int reg = ((n_pad / 128 + CI_WARPS - 1) / CI_WARPS) * 128;
        const int r_lo = min(warp * reg, n_pad), r_hi = min(r_lo + reg, n_pad);
        u64 lane_mass = 0;
        for (int i = r_lo + lane * 4; i < r_hi; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(rowbuf + i);
            if (v.x >= lcut) lane_mass += mass_q(v.x, tc, m);
            if (v.y >= lcut) lane_mass += mass_q(v.y, tc, m);
            if (v.z >= lcut) lane_mass += mass_q(v.z, tc, m);
            if (v.w >= lcut) lane_mass += mass_q(v.w, tc, m);
        }
        const u64 wtot = warp_sum_u64(lane_mass);
        if (lane == 0) sc->warp_tot[warp] = wtot;
        __syncthreads();
        if (tid == 0) {
            u64 t = 0;
            for (int w = 0; w < CI_WARPS; ++w) t += sc->warp_tot[w];
            xch->cta_mass = t;
        }
        __syncthreads();
        cluster.sync();                                                                // (C) slice masses published
        u64 my_off = 0;
        for (int q = 0; q < CS; ++q) {
            const u64 cm = cluster.map_shared_rank(xch, q)->cta_mass;
            if (q < rank) my_off += cm;
            total_mass += cm;
        }
        // the uniform of this row
        float u = 1.0f;
        if (a.u != nullptr) u = a.u[row];
        else if (a.pos != nullptr && a.p.seed != nullptr) {
            const long long p0 = a.pos_i64 ? reinterpret_cast<const long long*>(a.pos)[b]
                                           : (long long)reinterpret_cast<const int*>(a.pos)[b];
            u = u32_to_uniform(philox_word(philox_key(a.p.seed[b]), (u64)p0 + (u64)r));
        }
        u64 target;
        {
            double t = ceil((double)u * (double)total_mass);
            target = t <= 1.0 ? 1ull : (u64)t;
            if (target > total_mass) target = total_mass;
        }
        const u64 my_mass = xch->cta_mass;
        token = -1;
        if (total_mass > 0 && my_off < target && target <= my_off + my_mass) {
            // the crossing lies in this CTA: find the warp region, then the element
            u64 woff = my_off;
            for (int w = 0; w < warp; ++w) woff += sc->warp_tot[w];
            if (woff < target && target <= woff + wtot) {
                u64 run = woff;
                for (int i0 = r_lo; i0 < r_hi; i0 += 128) {
                    const int i = i0 + lane * 4;
                    u64 q4[4] = {0, 0, 0, 0};
                    if (i < r_hi) {
                        const float4 v = *reinterpret_cast<const float4*>(rowbuf + i);
                        if (v.x >= lcut) q4[0] = mass_q(v.x, tc, m);
                        if (v.y >= lcut) q4[1] = mass_q(v.y, tc, m);
                        if (v.z >= lcut) q4[2] = mass_q(v.z, tc, m);
                        if (v.w >= lcut) q4[3] = mass_q(v.w, tc, m);
                    }
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
        if (token >= 0 && a.out) a.out[row] = token;                   // greedy, degenerate or failed rows
        int hs = 0;
        for (int q = 0; q < CS; ++q) hs |= cluster.map_shared_rank(sc, q)->hist_slow;
        if (hs) status |= COLINFER_ROW_HIST_SLOW;
        if (a.status) a.status[row] = status;
        if (a.stats) {
            colinfer_row_stats st;
            st.lmax = L; st.lcut = lcut; st.tc = tc; st.status = status; st.argmax = aidx; st.mass_q = total_mass;
            a.stats[row] = st;
        }
    }
    cluster.sync();                                            // no CTA leaves while a peer may still read its shared memory
}

// ------------------------------------------------------------------------------------------------ host side
static int g_cluster_override = 0;
static const int kFixedSmem = CI_NB * 8 * 2 + CI_MAX_CHUNKS * 8 + (int)sizeof(Xch) + (int)sizeof(Scratch) + 64;

static int pick_geometry(int V, int dtype, const void* logits, colinfer_geometry* g) {
    if (V <= 0) return 1;
    const int cap2 = (113 * 1024 - kFixedSmem) / 4;           // slice elements that allow two CTAs per SM
    const int cap1 = (226 * 1024 - kFixedSmem) / 4;           // one CTA per SM
    const int max_slice = CI_CHUNK * CI_MAX_CHUNKS;
    int cs = 0, slice = 0;
    auto slice_for = [&](int c) { return (((V + c - 1) / c) + 127) & ~127; };
    if (g_cluster_override) {
        cs = g_cluster_override; slice = slice_for(cs);
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

extern "C" int colinfer_sample_geometry(int V, int dtype, const void* logits, colinfer_geometry* out) {
    return pick_geometry(V, dtype, logits, out) ? (int)cudaErrorInvalidValue : 0;
}

extern "C" int colinfer_set_cluster_override(int cluster) {
    if (cluster != 0 && cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return (int)cudaErrorInvalidValue;
    g_cluster_override = cluster;
    return 0;
}

extern "C" int colinfer_sample(const void* logits, int dtype, const int32_t* mask, int mask_rows, int W,
                               const colinfer_sampler_params* params, const void* pos, int pos_is_i64, const float* u,
                               int64_t* out_ids, colinfer_row_stats* stats, int32_t* status,
                               int B, int R, int V, int flags, void* stream) {
    if (!logits || !params || (!out_ids && !stats) || B < 0 || R < 0 || V <= 0) return (int)cudaErrorInvalidValue;
    if (dtype != COLINFER_F32 && dtype != COLINFER_BF16) return (int)cudaErrorInvalidValue;
    if (!params->temperature || !params->top_k || !params->top_p || !params->log_min_p) return (int)cudaErrorInvalidValue;
    if (out_ids && u == nullptr && (pos == nullptr || params->seed == nullptr)) return (int)cudaErrorInvalidValue;
    if (mask && (W < (V + 31) / 32 || mask_rows < R)) return (int)cudaErrorInvalidValue;
    if ((long long)B * R == 0) return 0;
    colinfer_geometry g;
    if (pick_geometry(V, dtype, logits, &g)) return (int)cudaErrorInvalidValue;
    if ((long long)B * R * g.cluster > 0x7fffffffLL) return (int)cudaErrorInvalidValue;

    SampleArgs a;
    a.logits = logits; a.dtype = dtype; a.use_bulk = g.bulk_copy;
    a.mask = mask; a.mask_rows = mask_rows; a.W = W;
    a.p = *params;
    a.pos = pos; a.pos_i64 = pos_is_i64; a.u = u;
    a.out = out_ids; a.stats = stats; a.status = status;
    a.B = B; a.R = R; a.V = V; a.slice_elems = g.slice_elems; a.flags = flags;

    cudaError_t e = cudaFuncSetAttribute(k_sample, cudaFuncAttributeMaxDynamicSharedMemorySize, g.smem_bytes);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((long long)B * R * g.cluster), 1, 1);
    cfg.blockDim = dim3(CI_THREADS, 1, 1);
    cfg.dynamicSmemBytes = (size_t)g.smem_bytes;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)g.cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, k_sample, a);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}
