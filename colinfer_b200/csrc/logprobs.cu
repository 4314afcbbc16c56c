// Logprobs of emitted tokens: for every row of RAW logits, log_softmax at the emitted token and the n_top most likely
// alternatives -- what engine/runtime/scheduler.py:714-722 computes with log_softmax + gather + topk (three full-vocabulary
// passes and a [r, V] temporary) -- in ONE pass over the row.
//
// Two 512-thread CTAs per SM walk over rows (persistent): every row costs the same, so the SM's rows split evenly, and
// while one CTA is in its short block-wide steps (the sample's bound, the selection of the alternatives) the other one
// streams.  Warp w owns a contiguous region of the row; lanes read 128-bit groups, four in flight per thread.  Each thread keeps an online (maximum, sum of exp) pair; the first batch
// of every warp (a tenth of the row at 151,936 logits) bounds the n_top-th largest logit from below, and the pass lists
// what reaches the bound (a few hundred logits), from which one warp takes the exact top n_top in descending order
// (equal logits: lower token first).  A row whose lists overflow (long runs of equal logits) takes n_top extra passes.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include <mutex>

#include "common.cuh"
#include "../../include/colinfer_b200.h"

namespace lpk {

constexpr int NT = 512, NW = NT / 32;
constexpr int CTAS_PER_SM = 2;
constexpr int BINS = 512;            // bins of the sample histogram and of the candidate selection
constexpr float SAMPLE_SCALE = 32.0f;
constexpr int WLIST = 128;           // list entries per warp
constexpr int FCAP = 128;            // candidates of the one-warp selection
constexpr int MAX_TOP = 32;          // n_top <= MAX_TOP
#define LP_FLT_MAX 3.402823466e38f
#define LP_POS_INF (__int_as_float(0x7f800000))

struct Cand { uint32_t idx; float l; };

struct Sc {
    float wm[32], ws[32];            // per-warp (maximum, sum)
    float wf[32];
    int wcount[32];
    int overflow;
    uint32_t fc_idx[FCAP]; float fc_l[FCAP];
    float sel_l; int sel_i;          // slow path: the previous pick
};

struct Row {
    const float* p32; const __nv_bfloat16* p16; int V; bool vec, vec16;
    __device__ __forceinline__ float4 load4(int i) const {
        if (vec) return i < V ? __ldcg(reinterpret_cast<const float4*>(p32 + i)) : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
        if (vec16) {
            if (i >= V) return make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
            const uint2 u = __ldcg(reinterpret_cast<const uint2*>(p16 + i));        // four bf16: a float's upper halves
            return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u),
                               __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xFFFF0000u));
        }
        float e[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int t = i + j;
            e[j] = t < V ? (p16 ? __bfloat162float(p16[t]) : __ldg(p32 + t)) : CI_NEG_INF;
        }
        return make_float4(e[0], e[1], e[2], e[3]);
    }
    __device__ __forceinline__ float at(int t) const { return p16 ? __bfloat162float(p16[t]) : __ldg(p32 + t); }
};

// (m, s) <- (m, s) + (m2, s2): sums of exp relative to their maxima
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
    const float M = fmaxf(m, m2);
    if (M == CI_NEG_INF) { s = 0.0f; return; }                      // both empty
    s = s * __expf(m - M) + s2 * __expf(m2 - M);                    // exp(-inf) = 0 for an empty side
    m = M;
}

// value descending, then token ascending
__device__ __forceinline__ bool before(float l1, uint32_t i1, float l2, uint32_t i2) { return l1 > l2 || (l1 == l2 && i1 < i2); }

__device__ __forceinline__ int warp_count_bin(const uint32_t* hist, uint32_t kk, int lane, uint32_t& run_out) {
    constexpr int PERB = BINS / 32;
    uint32_t h[PERB]; uint32_t s = 0;
#pragma unroll
    for (int t = 0; t < PERB; t += 4) {
        const uint4 x = *reinterpret_cast<const uint4*>(hist + lane * PERB + t);
        h[t] = x.x; h[t + 1] = x.y; h[t + 2] = x.z; h[t + 3] = x.w;
        s += x.x + x.y + x.z + x.w;
    }
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

struct Args {
    const void* logits; int dtype; int vec;
    const int64_t* toks; int n_top;
    float* chosen; int64_t* top_ids; float* top_lp;
    int rows, V;
};

// LOADER: 1 = fp32 rows that take 128-bit loads, 2 = bf16 rows that take 64-bit loads of four logits, 0 = the general
// loader (unaligned rows, vocabularies that are not a multiple of 4).
template <int LOADER>
__global__ void __launch_bounds__(NT, CTAS_PER_SM) k_logprobs(const __grid_constant__ Args a) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int V = a.V, n_top = a.n_top;
    __shared__ __align__(16) uint32_t hist[BINS];
    __shared__ Cand ownlist[NW * WLIST];
    __shared__ Sc sc;
    const int reg = (((V + 127) / 128 + NW - 1) / NW) * 128;
    const int r_lo = min(warp * reg, V), r_hi = min(r_lo + reg, V);
    Cand* mylist = ownlist + warp * WLIST;
    if (tid >= NW && tid < 32) {                                    // neutral entries for the warps this CTA does not have
        sc.wm[tid] = CI_NEG_INF; sc.ws[tid] = 0.0f; sc.wf[tid] = CI_NEG_INF; sc.wcount[tid] = -1;
    }

    for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
        __syncthreads();
        Row rw;
        rw.V = V; rw.vec = LOADER == 1; rw.vec16 = LOADER == 2;
        rw.p32 = a.dtype == COLINFER_F32 ? reinterpret_cast<const float*>(a.logits) + (size_t)row * V : nullptr;
        rw.p16 = a.dtype == COLINFER_BF16 ? reinterpret_cast<const __nv_bfloat16*>(a.logits) + (size_t)row * V : nullptr;

        // ------------------------------------------------------------------------------------ the sample's bound
        float tw = LP_POS_INF;                                      // n_top == 0: nothing to list
        if (n_top > 0) {
            float gm[4], sm = CI_NEG_INF;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = r_lo + k * 128 + lane * 4;
                const float4 v = i < r_hi ? rw.load4(i) : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
                gm[k] = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
                sm = fmaxf(sm, gm[k]);
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) sm = fmaxf(sm, __shfl_xor_sync(0xffffffffu, sm, o));
            if (lane == 0) sc.wf[warp] = sm;
            for (int i = tid; i < BINS; i += NT) hist[i] = 0u;
            __syncthreads();
            // the bins hang from the smallest finite warp maximum plus 4: a dominant token in the sample (far above
            // everything else) must not stretch them beyond the bulk
            float lref = sc.wf[lane];
            float lbulk = lref > CI_NEG_INF ? lref : LP_POS_INF;
#pragma unroll
            for (int o = 16; o; o >>= 1) {
                lref = fmaxf(lref, __shfl_xor_sync(0xffffffffu, lref, o));
                lbulk = fminf(lbulk, __shfl_xor_sync(0xffffffffu, lbulk, o));
            }
            const float top = fminf(lbulk + 4.0f, lref);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (gm[k] > CI_NEG_INF && top < LP_POS_INF)
                    atomicAdd(&hist[max(0, min(BINS - 1, __float2int_rz((top - gm[k]) * SAMPLE_SCALE)))], 1u);
            __syncthreads();
            uint32_t have;
            const int bk = warp_count_bin(hist, (uint32_t)n_top, lane, have);
            tw = (bk >= 0 && bk < BINS - 1) ? top - ((float)(bk + 1) + 0.01f) / SAMPLE_SCALE - fabsf(top) * 1e-6f : -LP_FLT_MAX;
            __syncthreads();                                        // every warp has read the sample's bins
        }

        // ------------------------------------------------------------------------------------ the pass
        float m = CI_NEG_INF, s = 0.0f;
        int wn = 0;
        for (int i0 = r_lo; i0 < r_hi; i0 += 512) {
            float4 v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + k * 128 + lane * 4;
                v[k] = i < r_hi ? rw.load4(i) : make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF);
            }
            float bm = CI_NEG_INF;
#pragma unroll
            for (int k = 0; k < 4; ++k) bm = fmaxf(bm, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
            if (bm > m) { s = m > CI_NEG_INF ? s * __expf(m - bm) : 0.0f; m = bm; }
            if (m > CI_NEG_INF) {
                float add = 0.0f;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    add += (__expf(v[k].x - m) + __expf(v[k].y - m)) + (__expf(v[k].z - m) + __expf(v[k].w - m));
                s += add;
            }
            unsigned mk[4], anym = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                mk[k] = (v[k].x >= tw ? 1u : 0u) | (v[k].y >= tw ? 2u : 0u) | (v[k].z >= tw ? 4u : 0u) | (v[k].w >= tw ? 8u : 0u);
                anym |= mk[k];
            }
            if (__ballot_sync(0xffffffffu, anym != 0u)) {
                // per-lane counts of the four groups, one byte each; one packed scan gives every group's offsets
                const unsigned cnt = __popc(mk[0]) | (__popc(mk[1]) << 8) | (__popc(mk[2]) << 16) | (__popc(mk[3]) << 24);
                unsigned incl = cnt;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) { const unsigned t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
                const unsigned tot = __shfl_sync(0xffffffffu, incl, 31), excl = incl - cnt;
                int base = wn;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (mk[k]) {
                        int at = base + (int)((excl >> (8 * k)) & 0xFFu);
                        const float e4[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (mk[k] & (1u << j)) {
                                if (at < WLIST) { mylist[at].idx = (uint32_t)(i0 + k * 128 + lane * 4 + j); mylist[at].l = e4[j]; }
                                ++at;
                            }
                        }
                    }
                    base += (int)((tot >> (8 * k)) & 0xFFu);
                }
                wn = base;
            }
        }

        // ------------------------------------------------------------------------------------ log-sum-exp of the row
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
            lse_merge(m, s, m2, s2);
        }
        if (lane == 0) { sc.wm[warp] = m; sc.ws[warp] = s; }
        for (int i = tid; i < BINS; i += NT) hist[i] = 0u;
        const int over = __syncthreads_or(wn > WLIST);
        float M = sc.wm[lane], S = sc.ws[lane];
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, M, o), s2 = __shfl_xor_sync(0xffffffffu, S, o);
            lse_merge(M, S, m2, s2);
        }
        const float lse = M + logf(S);                              // -inf + log(0) = NaN for a row without finite logits
        if (tid == 0 && a.chosen) {
            const long long t = a.toks ? a.toks[row] : -1;
            a.chosen[row] = (t >= 0 && t < V) ? rw.at((int)t) - lse : __int_as_float(0x7fc00000);
        }
        if (n_top <= 0) continue;

        // ------------------------------------------------------------------------------------ the top n_top
        bool done = false;
        if (!over && tw > -LP_FLT_MAX && tw <= M) {
            const float scale = M > tw ? (float)(BINS - 2) / (M - tw) : 0.0f;
            auto bin_of = [&](float l) { return min(BINS - 1, __float2int_rz((M - l) * scale)); };
            for (int j = lane; j < wn; j += 32) atomicAdd(&hist[bin_of(mylist[j].l)], 1u);
            __syncthreads();
            uint32_t nc;
            const int bstar = warp_count_bin(hist, (uint32_t)n_top, lane, nc);
            if (bstar >= 0 && (int)nc <= FCAP) {
                int cnt = 0;
                for (int j0 = 0; j0 < wn; j0 += 32) {
                    const int j = j0 + lane;
                    cnt += __popc(__ballot_sync(0xffffffffu, j < wn && bin_of(mylist[j].l) <= bstar));
                }
                if (lane == 0) sc.wcount[warp] = cnt;
                __syncthreads();
                int off = 0;
                for (int w2 = 0; w2 < warp; ++w2) off += sc.wcount[w2];
                const unsigned lt = (1u << lane) - 1u;
                for (int j0 = 0; j0 < wn; j0 += 32) {
                    const int j = j0 + lane;
                    const bool is = j < wn && bin_of(mylist[j].l) <= bstar;
                    const unsigned bal = __ballot_sync(0xffffffffu, is);
                    if (is) { const int at = off + __popc(bal & lt); if (at < FCAP) { sc.fc_idx[at] = mylist[j].idx; sc.fc_l[at] = mylist[j].l; } }
                    off += __popc(bal);
                }
                __syncthreads();
                {
                    // rank of every candidate among the candidates (value descending, then token ascending): a few threads
                    // per candidate compare it with a share of the others each; a candidate of rank < n_top is that alternative
                    constexpr int TPC = NT / FCAP;                  // threads per candidate
                    static_assert(TPC == 4 || TPC == 8, "four or eight threads per candidate");
                    const int c = tid / TPC, part = tid % TPC;
                    int rank = 0;
                    if (c < (int)nc) {
                        const float lc = sc.fc_l[c]; const uint32_t ic = sc.fc_idx[c];
#pragma unroll
                        for (int t = 0; t < FCAP / TPC; ++t) {
                            const int o = part * (FCAP / TPC) + t;
                            if (o < (int)nc && before(sc.fc_l[o], sc.fc_idx[o], lc, ic)) ++rank;
                        }
                    }
                    rank += __shfl_xor_sync(0xffffffffu, rank, 1);
                    rank += __shfl_xor_sync(0xffffffffu, rank, 2);
                    if (TPC == 8) rank += __shfl_xor_sync(0xffffffffu, rank, 4);
                    if (part == 0 && c < (int)nc && rank < n_top) {
                        a.top_ids[(size_t)row * n_top + rank] = (long long)sc.fc_idx[c];
                        a.top_lp[(size_t)row * n_top + rank] = sc.fc_l[c] - lse;
                    }
                }
                done = true;
            }
        }
        if (!done) {
            // lists overflowed (long runs of equal logits) or the bound did not hold: n_top passes, each taking the
            // best logit after the previous pick in (value descending, token ascending) order
            if (tid == 0) { sc.sel_l = LP_POS_INF; sc.sel_i = -1; }
            __syncthreads();
            for (int r = 0; r < n_top; ++r) {
                const float pl = sc.sel_l; const uint32_t pi = (uint32_t)sc.sel_i;
                const bool first = sc.sel_i < 0;
                float bl = CI_NEG_INF; uint32_t bi = 0xFFFFFFFFu;
                for (int i0 = r_lo; i0 < r_hi; i0 += 128) {
                    const int i = i0 + lane * 4;
                    const float4 v = rw.load4(i);
                    const float e4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t id = (uint32_t)(i + j);
                        if (i + j < V && (first || before(pl, pi, e4[j], id)) && (bi == 0xFFFFFFFFu || before(e4[j], id, bl, bi))) { bl = e4[j]; bi = id; }
                    }
                }
#pragma unroll
                for (int o = 16; o; o >>= 1) {
                    const float ol = __shfl_xor_sync(0xffffffffu, bl, o);
                    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (oi != 0xFFFFFFFFu && (bi == 0xFFFFFFFFu || before(ol, oi, bl, bi))) { bl = ol; bi = oi; }
                }
                __syncthreads();
                if (lane == 0) { sc.wf[warp] = bl; sc.wcount[warp] = (int)bi; }
                __syncthreads();
                if (warp == 0) {
                    float cl = sc.wf[lane]; uint32_t ci = (uint32_t)sc.wcount[lane];
#pragma unroll
                    for (int o = 16; o; o >>= 1) {
                        const float ol = __shfl_xor_sync(0xffffffffu, cl, o);
                        const uint32_t oi = __shfl_xor_sync(0xffffffffu, ci, o);
                        if (oi != 0xFFFFFFFFu && (ci == 0xFFFFFFFFu || before(ol, oi, cl, ci))) { cl = ol; ci = oi; }
                    }
                    if (lane == 0) {
                        sc.sel_l = cl; sc.sel_i = (int)ci;
                        a.top_ids[(size_t)row * n_top + r] = ci == 0xFFFFFFFFu ? -1ll : (long long)ci;
                        a.top_lp[(size_t)row * n_top + r] = cl - lse;
                    }
                }
                __syncthreads();
            }
        }
    }
}

}  // namespace lpk

// Replaces Scheduler._logprobs (engine/runtime/scheduler.py:714-722).
extern "C" int colinfer_logprobs(const void* logits, int dtype, const int64_t* toks, int n_top, float* chosen,
                                 int64_t* top_ids, float* top_lp, int rows, int V, void* stream) {
    if (rows == 0) return (int)cudaSuccess;
    if (logits == nullptr || rows < 0 || V < 1 || n_top < 0 || n_top > lpk::MAX_TOP || n_top > V ||
        (dtype != COLINFER_F32 && dtype != COLINFER_BF16) || (n_top > 0 && (top_ids == nullptr || top_lp == nullptr)))
        return (int)cudaErrorInvalidValue;
    static int sm_count[64] = {};
    static std::mutex guard;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lock(guard);
        if (sm_count[dev] == 0) {
            int n = 0;
            e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return (int)e;
            sm_count[dev] = n > 0 ? n : 1;
        }
    }
    lpk::Args a;
    a.logits = logits; a.dtype = dtype;
    a.vec = (dtype == COLINFER_F32 && (V % 4) == 0 && (((uintptr_t)logits) & 15) == 0) ? 1 : 0;
    a.toks = toks; a.n_top = n_top; a.chosen = chosen; a.top_ids = top_ids; a.top_lp = top_lp;
    a.rows = rows; a.V = V;
    const int slots = sm_count[dev] * lpk::CTAS_PER_SM;
    const int grid = rows < slots ? rows : slots;
    const bool vec16 = dtype == COLINFER_BF16 && (V % 4) == 0 && (((uintptr_t)logits) & 7) == 0;
    if (a.vec) lpk::k_logprobs<1><<<grid, lpk::NT, 0, (cudaStream_t)stream>>>(a);
    else if (vec16) lpk::k_logprobs<2><<<grid, lpk::NT, 0, (cudaStream_t)stream>>>(a);
    else lpk::k_logprobs<0><<<grid, lpk::NT, 0, (cudaStream_t)stream>>>(a);
    return (int)cudaGetLastError();
}
