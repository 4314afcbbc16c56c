// ops.cu -- the small kernels of the logits -> token path (sm_100a): Philox uniforms, the stand-alone grammar mask, the
// full-probability writer behind processed_probs, inverse_cdf, and the speculative accept / verify steps.
#include <mutex>

#include "common.cuh"
#include "../../include/colinfer_b200.h"

// ------------------------------------------------------------------------------------------------ philox_uniform
// Replaces k_philox_uniform (csrc/sampling.cu:25-35 of the reference).  One thread per output; the grid covers B * n.
__global__ void k_philox_uniform(const int64_t* __restrict__ seed, const int64_t* __restrict__ offset,
                                 float* __restrict__ out, int B, int n) {
    const long long total = (long long)B * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int b = (int)(i / n), j = (int)(i % n);
        out[i] = u32_to_uniform(philox_word(philox_key(seed[b]), (u64)offset[b] + (u64)j));
    }
}

extern "C" int colinfer_philox_uniform(const int64_t* seed, const int64_t* offset, float* out, int B, int n, void* stream) {
    if (!seed || !offset || !out || B < 0 || n < 0) return (int)cudaErrorInvalidValue;
    const long long total = (long long)B * n;
    if (total == 0) return 0;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 8 ? (total + threads - 1) / threads : 148 * 8);
    k_philox_uniform<<<blocks, threads, 0, (cudaStream_t)stream>>>(seed, offset, out, B, n);
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ apply_mask
// Replaces apply_mask (engine/runtime/sampler.py:50-56): pure streaming, 4 tokens per thread share one mask nibble.
__global__ void k_apply_mask(const float* __restrict__ logits, const int32_t* __restrict__ mask, float* __restrict__ out,
                             long long rows, int V, int W, int vec) {
    const long long row = blockIdx.y;
    const float* src = logits + row * V;
    float* dst = out + row * V;
    const int32_t* m = mask + row * W;
    if (vec) {
        const int n4 = V >> 2;
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) {
            float4 v = __ldg(reinterpret_cast<const float4*>(src) + i);
            const int g = i << 2;
            const uint32_t bits = ((uint32_t)__ldg(m + (g >> 5)) >> (g & 31)) & 0xFu;
            if (!(bits & 1u)) v.x = CI_NEG_INF;
            if (!(bits & 2u)) v.y = CI_NEG_INF;
            if (!(bits & 4u)) v.z = CI_NEG_INF;
            if (!(bits & 8u)) v.w = CI_NEG_INF;
            reinterpret_cast<float4*>(dst)[i] = v;
        }
    } else {
        for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < V; g += gridDim.x * blockDim.x) {
            const float v = __ldg(src + g);
            dst[g] = (((uint32_t)__ldg(m + (g >> 5)) >> (g & 31)) & 1u) ? v : CI_NEG_INF;
        }
    }
}

extern "C" int colinfer_apply_mask(const float* logits, const int32_t* mask, float* out, int64_t rows, int V, int W, void* stream) {
    if (!logits || !mask || !out || rows < 0 || V <= 0 || W < (V + 31) / 32) return (int)cudaErrorInvalidValue;
    if (rows == 0) return 0;
    if (rows > 65535) {
        // the row index rides in gridDim.y; split very tall inputs
        for (int64_t r0 = 0; r0 < rows; r0 += 65535) {
            const int64_t nr = rows - r0 < 65535 ? rows - r0 : 65535;
            const int e = colinfer_apply_mask(logits + r0 * V, mask + r0 * W, out + r0 * V, nr, V, W, stream);
            if (e) return e;
        }
        return 0;
    }
    const int vec = ((V & 3) == 0 && ((((uintptr_t)logits) | ((uintptr_t)out)) & 15) == 0) ? 1 : 0;
    const int threads = 256;
    const int work = vec ? V / 4 : V;
    int bx = (work + threads - 1) / threads;
    if (bx > 1024) bx = 1024;
    k_apply_mask<<<dim3(bx, (unsigned)rows), threads, 0, (cudaStream_t)stream>>>(logits, mask, out, rows, V, W, vec);
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ processed_probs
// P(t) = exp(z_t - m) / S on the kept set of the row (described by the row statistics of the fused kernel), else 0.
__global__ void k_write_probs(const float* __restrict__ logits, const colinfer_row_stats* __restrict__ stats,
                              float* __restrict__ out, int V) {
    const int row = blockIdx.y;
    const colinfer_row_stats st = stats[row];
    const float* src = logits + (size_t)row * V;
    float* dst = out + (size_t)row * V;
    const bool bad = (st.status & (COLINFER_ROW_DEGENERATE | COLINFER_ROW_TIMEOUT)) != 0 || st.mass_q == 0;
    const float m = scale_logit(st.lmax, st.tc);
    const float S = (float)((double)st.mass_q * CI_MASS_INV);
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < V; g += gridDim.x * blockDim.x) {
        const float l = __ldg(src + g);
        float p;
        if (bad) p = __int_as_float(0x7fc00000);               // NaN, as a softmax without a finite maximum gives
        else if (l >= st.lcut && l > CI_NEG_INF) p = __fdiv_rn(expf(scale_logit(l, st.tc) - m), S);
        else p = 0.0f;
        dst[g] = p;
    }
}

extern "C" int colinfer_processed_probs(const float* logits, const float* temperature, const int32_t* top_k,
                                        const float* top_p, const float* log_min_p, float* out,
                                        colinfer_row_stats* scratch, int R, int V, void* stream) {
    if (!logits || !temperature || !top_k || !top_p || !log_min_p || !out || !scratch || R < 0 || V <= 0)
        return (int)cudaErrorInvalidValue;
    if (R == 0) return 0;
    colinfer_sampler_params p = {};
    p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.log_min_p = log_min_p;
    int e = colinfer_sample(logits, COLINFER_F32, nullptr, 0, 0, &p, nullptr, 0, nullptr, nullptr, scratch, nullptr,
                            1, R, V, COLINFER_FORCE_DISTRIBUTION, stream);
    if (e) return e;
    const int threads = 256;
    int bx = (V + threads - 1) / threads;
    if (bx > 296) bx = 296;
    for (int r0 = 0; r0 < R; r0 += 65535) {
        const int nr = R - r0 < 65535 ? R - r0 : 65535;
        k_write_probs<<<dim3(bx, nr), threads, 0, (cudaStream_t)stream>>>(logits + (size_t)r0 * V, scratch + r0,
                                                                           out + (size_t)r0 * V, V);
    }
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ processed_probs without caller scratch
// For callers that cannot hand over scratch memory: a host that binds this C ABI directly (no torch caching allocator
// behind it) and replays the call inside a captured CUDA graph, or runs under a fixed memory budget, has nowhere to
// take the per-row statistics buffer from -- cudaMalloc is illegal during capture and forbidden by such hosts.  This
// variant keeps the statistics in a fixed array that lives in the library's device image instead.
#define COLINFER_NOALLOC_MAX_ROWS 4096
static __device__ __align__(256) colinfer_row_stats g_noalloc_stats[COLINFER_NOALLOC_MAX_ROWS];   // 128 KB per device

// Device address of g_noalloc_stats on the current device.  In host code the array's name is only a handle, never an
// address a kernel may dereference: the address is asked for once per device, with that device current.
static int noalloc_stats_ptr(colinfer_row_stats** out) {
    static colinfer_row_stats* cached[64] = {};
    static std::mutex guard;                               // (first calls of two host threads may coincide)
    std::lock_guard<std::mutex> lock(guard);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_stats);
        if (e != cudaSuccess) return (int)e;
        cached[dev] = reinterpret_cast<colinfer_row_stats*>(p);
    }
    *out = cached[dev];
    return 0;
}

extern "C" int colinfer_processed_probs_noalloc(const float* logits, const float* temperature, const int32_t* top_k,
                                                const float* top_p, const float* log_min_p, float* out, int R, int V,
                                                void* stream) {
    if (R > COLINFER_NOALLOC_MAX_ROWS) return (int)cudaErrorInvalidValue;   // more rows than the fixed array holds
    colinfer_row_stats* stats = nullptr;
    const int e = noalloc_stats_ptr(&stats);
    if (e) return e;
    // Every row's entry is written by the statistics pass before the probability pass reads it: nothing in the array has
    // to start at zero, and what an earlier call left behind is never read.
    return colinfer_processed_probs(logits, temperature, top_k, top_p, log_min_p, out, stats, R, V, stream);
}

extern "C" int colinfer_noalloc_max_rows(void) { return COLINFER_NOALLOC_MAX_ROWS; }

// ------------------------------------------------------------------------------------------------ inverse_cdf
// One CTA per row.  Sums are float64 (the reference's fp32 scan order is device dependent; float64 is what its CPU
// cumsum accumulates in).  Warp w owns a contiguous region, lanes interleave, so the index order is (warp, step, lane).
#define ICDF_THREADS 1024
__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_incl_scan_f64(double v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    return v;
}

__global__ void __launch_bounds__(ICDF_THREADS) k_inverse_cdf(const float* __restrict__ P, const float* __restrict__ u,
                                                              int64_t* __restrict__ out, int V) {
    __shared__ double wtot[ICDF_THREADS / 32];
    __shared__ long long result;
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* src = P + (size_t)row * V;
    const int nwarps = ICDF_THREADS / 32;
    const int reg = (((V + 31) / 32 + nwarps - 1) / nwarps) * 32;
    const int lo = min(warp * reg, V), hi = min(lo + reg, V);
    double acc = 0.0;
    for (int i = lo + lane; i < hi; i += 32) acc += (double)__ldg(src + i);
    const double wt = warp_sum_f64(acc);
    if (lane == 0) wtot[warp] = wt;
    if (threadIdx.x == 0) result = V - 1;
    __syncthreads();
    double total = 0.0, woff = 0.0;
    for (int w = 0; w < nwarps; ++w) { if (w < warp) woff += wtot[w]; total += wtot[w]; }
    if (threadIdx.x == 0 && !(total > 0.0)) result = 0;          // a row without mass: no prefix lies below u * 0 (the reference counts none)
    const double t = (double)u[row] * total;
    // first index whose inclusive prefix reaches t; the owning warp is the first whose inclusive total reaches it
    if (woff < t && woff + wt >= t) {
        double run = woff;
        for (int i0 = lo; i0 < hi; i0 += 32) {
            const int i = i0 + lane;
            const double v = i < hi ? (double)__ldg(src + i) : 0.0;
            const double incl = warp_incl_scan_f64(v, lane);
            const unsigned hit = __ballot_sync(0xffffffffu, run + incl >= t);
            if (hit) {
                if (lane == __ffs(hit) - 1) result = i;
                break;
            }
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) out[row] = result;
}

extern "C" int colinfer_inverse_cdf(const float* P, const float* u, int64_t* out, int R, int V, void* stream) {
    if (!P || !u || !out || R < 0 || V <= 0) return (int)cudaErrorInvalidValue;
    if (R == 0) return 0;
    k_inverse_cdf<<<R, ICDF_THREADS, 0, (cudaStream_t)stream>>>(P, u, out, V);
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ spec_accept
// The accept / bonus / stop-cut lines of the reference's speculative cycle (engine/spec/mtp.py:406-415, 422-423),
// one thread per slot instead of ~20 tiny launches.
__global__ void k_spec_accept(const int64_t* __restrict__ pred, const int64_t* __restrict__ tok,
                              const int64_t* __restrict__ stop_ids, const int32_t* __restrict__ active,
                              int64_t* __restrict__ out_tok, int32_t* __restrict__ n_out, int B, int k1, int S) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int k = k1 - 1;
    const int64_t* pr = pred + (size_t)b * k1;
    const int64_t* d = tok + (size_t)b * k1 + 1;
    int n = 1;
    while (n - 1 < k && pr[n - 1] == d[n - 1]) ++n;
    int64_t bonus = pr[n - 1];
    if (stop_ids != nullptr) {
        const int64_t* st = stop_ids + (size_t)b * S;
        bool cut = false;
        for (int i = 0; i < n - 1 && i < k && !cut; ++i) {
            for (int s = 0; s < S; ++s) {
                if (d[i] == st[s]) { n = i + 1; bonus = d[i]; cut = true; break; }
            }
        }
    }
    if (active != nullptr) n *= active[b];
    int64_t* o = out_tok + (size_t)b * k1;
    for (int i = 0; i < k; ++i) o[i] = d[i];
    o[k] = bonus;
    if (n >= 1) o[n - 1] = bonus;
    n_out[b] = n;
}

extern "C" int colinfer_spec_accept(const int64_t* pred, const int64_t* tok, const int64_t* stop_ids,
                                    const int32_t* active, int64_t* out_tok, int32_t* n, int B, int k1, int S, void* stream) {
    if (!pred || !tok || !out_tok || !n || B < 0 || k1 < 1 || S < 0) return (int)cudaErrorInvalidValue;
    if (B == 0) return 0;
    k_spec_accept<<<(B + 127) / 128, 128, 0, (cudaStream_t)stream>>>(pred, tok, S > 0 ? stop_ids : nullptr, active, out_tok, n, B, k1, S);
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ spec_advance
// The bookkeeping the reference's scheduler does on the host after every cycle (engine/runtime/scheduler.py:635-641:
// n and out_tok read back with .tolist(), `tokens.append(y); tokens += o[:-1]; y = o[-1]`), kept on the device: the
// slot's pending token and the cycle's accepted drafts are appended to its token history (the one the penalties count
// in), the bonus token becomes the pending token, the position moves on by n.  One CTA per slot.  A history that
// would overflow keeps its most recent H ids.
#define ADV_THREADS 256
__global__ void __launch_bounds__(ADV_THREADS) k_spec_advance(const int64_t* __restrict__ out_tok, const int32_t* __restrict__ n_in,
                                                              int64_t* __restrict__ y, int32_t* __restrict__ history,
                                                              int32_t* __restrict__ hist_len, int64_t* __restrict__ pos, int k1, int H) {
    const int b = blockIdx.x, tid = threadIdx.x;
    const int n = n_in[b];
    if (n <= 0) return;                                              // an inactive slot keeps its state
    const int64_t* o = out_tok + (size_t)b * k1;
    const int nn = n < k1 ? n : k1;
    int32_t* h = history ? history + (size_t)b * H : nullptr;
    if (h != nullptr && H > 0) {
        int len = hist_len[b];
        len = len < 0 ? 0 : len > H ? H : len;
        const int add = nn < H ? nn : H;                             // the last `add` of [y, o[0 .. nn-2]]
        const int keep = len + add > H ? H - add : len;              // the most recent `keep` of the old ids stay
        const int drop = len - keep;
        if (drop > 0) {                                              // move left: every id is read before any is written
            int32_t buf[8];
            for (int base = 0; base < keep; base += ADV_THREADS * 8) {
#pragma unroll
                for (int u = 0; u < 8; ++u) { const int i = base + u * ADV_THREADS + tid; buf[u] = i < keep ? h[i + drop] : 0; }
                __syncthreads();
#pragma unroll
                for (int u = 0; u < 8; ++u) { const int i = base + u * ADV_THREADS + tid; if (i < keep) h[i] = buf[u]; }
                __syncthreads();
            }
        }
        for (int i = tid; i < add; i += ADV_THREADS) {
            const int src = nn - add + i;                            // index into [y, o[0], ..., o[nn-2]]
            h[keep + i] = (int32_t)(src == 0 ? y[b] : o[src - 1]);
        }
        __syncthreads();
        if (tid == 0) hist_len[b] = keep + add;
    } else {
        __syncthreads();
    }
    if (tid == 0) {
        y[b] = o[nn - 1];
        if (pos != nullptr) pos[b] += nn;
    }
}

extern "C" int colinfer_spec_advance(const int64_t* out_tok, const int32_t* n, int64_t* y, int32_t* history, int32_t* hist_len,
                                     int64_t* pos, int B, int k1, int H, void* stream) {
    if (!out_tok || !n || !y || B < 0 || k1 < 1 || H < 0 || (history && !hist_len)) return (int)cudaErrorInvalidValue;
    if (B == 0) return 0;
    k_spec_advance<<<B, ADV_THREADS, 0, (cudaStream_t)stream>>>(out_tok, n, y, H > 0 ? history : nullptr, hist_len, pos, k1, H);
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ spec_verify (rejection)
// Finish step: per slot, decide the accepted prefix from the row statistics of the target and draft rows, then, at a
// rejection, stream the two rows of that position once to draw from the residual max(p - q, 0).
#define VF_THREADS 256
#define VF_NSEG 32                     // segments a slot's rejected position is summed in (one CTA each)
struct VerifyArgs {
    const void* tl; const void* dl; int dtype;
    const int32_t* mask; int W;
    const float* temperature;
    const int64_t* draft_ids; const float* ua; const float* us;
    const colinfer_row_stats* st_t; const colinfer_row_stats* st_d; const int64_t* samp_t;
    int64_t* out_tok; int32_t* n;
    int2* slot;                        // [B] (first rejected position j, mode: 0 = token known, 1 = residual draw)
    u64* seg_sums;                     // [B, VF_NSEG] residual mass per segment of the rejected position
    int seg;                           // elements per segment (a multiple of 128)
    int vec;                           // fp32 rows that take 128-bit loads
    int B, k, V;
    const int32_t* history; const int32_t* hist_len; int hist_stride;   // the slots' penalties (NULL: none)
    const float* rp; const float* pp; const float* fp;
};

// A slot's penalties as the verify's kernels see them: every row of the slot, target and draft, is penalised with the
// slot's history before mask and temperature, as the two sampler launches did when they took the rows' statistics.
#define VF_BM_WORDS 512                // bitmap of one segment's tokens that occur in the history (segments up to 16,384 logits)
struct PenSlot {
    const int32_t* h; int len; float rp, pp, fp; bool on;
    __device__ void init(const VerifyArgs& a, int b) {
        h = a.history ? a.history + (size_t)b * a.hist_stride : nullptr;
        len = h ? (a.hist_len ? min(max(a.hist_len[b], 0), a.hist_stride) : a.hist_stride) : 0;
        rp = a.rp ? a.rp[b] : 1.0f; pp = a.pp ? a.pp[b] : 0.0f; fp = a.fp ? a.fp[b] : 0.0f;
        on = len > 0 && !(rp == 1.0f && pp == 0.0f && fp == 0.0f);
    }
    __device__ int count(int tok) const {                            // one thread scans the history
        int c = 0;
        for (int i = 0; i < len; ++i) c += (__ldg(h + i) == tok) ? 1 : 0;
        return c;
    }
    __device__ int count_warp(int tok, int lane) const {             // a warp shares the scan
        int c = 0;
        for (int i = lane; i < len; i += 32) c += (__ldg(h + i) == tok) ? 1 : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        return c;
    }
    // marks in bm (zeroed here) the tokens of [lo, hi) that occur in the history; all threads of the CTA call it
    __device__ void mark(uint32_t* bm, int lo, int hi) const {
        for (int i = threadIdx.x; i < VF_BM_WORDS; i += blockDim.x) bm[i] = 0;
        __syncthreads();
        if (on)
            for (int i = threadIdx.x; i < len; i += blockDim.x) {
                const int v = __ldg(h + i);
                if (v >= lo && v < hi) atomicOr(&bm[(v - lo) >> 5], 1u << ((v - lo) & 31));
            }
        __syncthreads();
    }
    // the two logits of token i as the distributions see them
    __device__ __forceinline__ void fix(const uint32_t* bm, int lo, int i, float& lt, float& ld) const {
        if (on && ((bm[(i - lo) >> 5] >> ((i - lo) & 31)) & 1u)) {
            const int c = count(i);
            lt = apply_penalty(lt, c, rp, pp, fp); ld = apply_penalty(ld, c, rp, pp, fp);
        }
    }
};

__device__ __forceinline__ float load_logit(const void* base, int dtype, size_t idx) {
    return dtype == COLINFER_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx])
                                  : __ldg(reinterpret_cast<const float*>(base) + idx);
}
__device__ __forceinline__ bool mask_allows(const int32_t* mrow, int t) {
    return mrow == nullptr || (((uint32_t)__ldg(mrow + (t >> 5)) >> (t & 31)) & 1u);
}
// probability of one token under a row's processed distribution, in float64
__device__ double token_prob(const colinfer_row_stats& st, float l, long long tok) {
    if (st.status & COLINFER_ROW_DEGENERATE) return tok == st.argmax ? 1.0 : 0.0;
    if (!(l >= st.lcut) || !(l > CI_NEG_INF) || st.mass_q == 0) return 0.0;
    const float d = scale_logit(l, st.tc) - scale_logit(st.lmax, st.tc);
    return exp((double)d) / ((double)st.mass_q * CI_MASS_INV);
}
// residual mass of one token in units of 2^-40 (fp32 arithmetic, integer result: order-independent sums)
struct Residual {
    colinfer_row_stats st, sd; float mt, md, inv_t, inv_d;
    __device__ void init(const colinfer_row_stats& st_, const colinfer_row_stats& sd_) {
        st = st_; sd = sd_;
        mt = scale_logit(st.lmax, st.tc); md = scale_logit(sd.lmax, sd.tc);
        inv_t = (float)(1.0 / ((double)st.mass_q * CI_MASS_INV)); inv_d = (float)(1.0 / ((double)sd.mass_q * CI_MASS_INV));
    }
    __device__ __forceinline__ u64 operator()(float lt, float ld) const {
        float p = 0.0f, q = 0.0f;
        if (lt >= st.lcut && lt > CI_NEG_INF) p = exp2f((scale_logit(lt, st.tc) - mt) * CI_LOG2E) * inv_t;
        if (ld >= sd.lcut && ld > CI_NEG_INF) q = exp2f((scale_logit(ld, sd.tc) - md) * CI_LOG2E) * inv_d;
        const float rres = p - q;
        return rres > 0.0f ? __float2ull_rn(rres * 1099511627776.0f) : 0ull;   // units of 2^-40
    }
};

// Step 1, one warp per slot: the accepted prefix from the row statistics of the target and draft rows (the lanes share
// the count of a draft token in the slot's history; everything else every lane does alike).
__global__ void k_verify_decide(const __grid_constant__ VerifyArgs a) {
    const int b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (b >= a.B) return;
    const int k = a.k, V = a.V;
    const colinfer_row_stats* st_t = a.st_t + (size_t)b * (k + 1);
    const colinfer_row_stats* st_d = a.st_d + (size_t)b * k;
    const bool greedy = !(a.temperature[b] > 0.0f);
    PenSlot pen;
    pen.init(a, b);
    int j = 0;
    for (; j < k; ++j) {
        const long long d = a.draft_ids[(size_t)b * k + j];
        bool ok;
        if (greedy) ok = (d == st_t[j].argmax);
        else if (d < 0 || d >= V) ok = false;
        else {
            const int32_t* mrow = a.mask ? a.mask + ((size_t)b * (k + 1) + j) * a.W : nullptr;
            float lt = load_logit(a.tl, a.dtype, ((size_t)b * (k + 1) + j) * V + d);
            float ld = load_logit(a.dl, a.dtype, ((size_t)b * k + j) * V + d);
            if (pen.on) {
                const int c = pen.count_warp((int)d, lane);
                if (c > 0) { lt = apply_penalty(lt, c, pen.rp, pen.pp, pen.fp); ld = apply_penalty(ld, c, pen.rp, pen.pp, pen.fp); }
            }
            if (!mask_allows(mrow, (int)d)) { lt = CI_NEG_INF; ld = CI_NEG_INF; }
            const double p = token_prob(st_t[j], lt, d), q = token_prob(st_d[j], ld, d);
            // (a draft token the target gives no probability -- masked, or outside its kept set -- is never accepted,
            // whatever the draft thought of it: 0 <= 0 must not pass)
            ok = p > 0.0 && (double)a.ua[(size_t)b * k + j] * q <= p;
        }
        if (!ok) break;
    }
    int mode = 1;
    if (greedy || j == k) mode = 0;
    else if ((st_t[j].status | st_d[j].status) & (COLINFER_ROW_DEGENERATE | COLINFER_ROW_TIMEOUT)) mode = 0;
    if (lane == 0) a.slot[b] = make_int2(j, mode);
}

// Step 2, VF_NSEG CTAs per slot: the residual mass max(p - q, 0) of one segment of the rejected position's two rows,
// streamed once with 128-bit loads where the rows allow it.
__global__ void __launch_bounds__(VF_THREADS) k_verify_residual(const __grid_constant__ VerifyArgs a) {
    __shared__ u64 wsum[VF_THREADS / 32];
    __shared__ uint32_t bm[VF_BM_WORDS];
    const int b = blockIdx.x / VF_NSEG, sgi = blockIdx.x % VF_NSEG;
    const int2 sl = a.slot[b];
    if (sl.y != 1) return;
    const int j = sl.x, k = a.k, V = a.V, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    Residual res;
    res.init(a.st_t[(size_t)b * (k + 1) + j], a.st_d[(size_t)b * k + j]);
    const int32_t* mrow = a.mask ? a.mask + ((size_t)b * (k + 1) + j) * a.W : nullptr;
    const size_t bt = ((size_t)b * (k + 1) + j) * V, bd = ((size_t)b * k + j) * V;
    const int lo = min(sgi * a.seg, V), hi = min(lo + a.seg, V);
    PenSlot pen;
    pen.init(a, b);
    if (pen.on) pen.mark(bm, lo, hi);                                // (the same for every thread of the CTA)
    u64 acc = 0;
    if (a.vec) {
        const float* pt = reinterpret_cast<const float*>(a.tl) + bt;
        const float* pd = reinterpret_cast<const float*>(a.dl) + bd;
        for (int i0 = lo + threadIdx.x * 4; i0 < hi; i0 += 2 * VF_THREADS * 4) {
            const int i1 = i0 + VF_THREADS * 4;
            const float4 t0 = __ldcg(reinterpret_cast<const float4*>(pt + i0)), d0 = __ldcg(reinterpret_cast<const float4*>(pd + i0));
            float4 t1 = make_float4(CI_NEG_INF, CI_NEG_INF, CI_NEG_INF, CI_NEG_INF), d1 = t1;
            if (i1 < hi) { t1 = __ldcg(reinterpret_cast<const float4*>(pt + i1)); d1 = __ldcg(reinterpret_cast<const float4*>(pd + i1)); }
            const float tt[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w}, dd[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int i = (e < 4 ? i0 : i1 - 4) + e;
                if (i < hi && mask_allows(mrow, i)) { float lt = tt[e], ld = dd[e]; pen.fix(bm, lo, i, lt, ld); acc += res(lt, ld); }
            }
        }
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += VF_THREADS)
            if (mask_allows(mrow, i)) {
                float lt = load_logit(a.tl, a.dtype, bt + i), ld = load_logit(a.dl, a.dtype, bd + i);
                pen.fix(bm, lo, i, lt, ld);
                acc += res(lt, ld);
            }
    }
    const u64 wt = warp_sum_u64(acc);
    if (lane == 0) wsum[warp] = wt;
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 t = 0;
        for (int w = 0; w < VF_THREADS / 32; ++w) t += wsum[w];
        a.seg_sums[(size_t)b * VF_NSEG + sgi] = t;
    }
}

// Step 3, one CTA per slot: the segment in which the running residual mass reaches us * total, then the token inside it
// (threads own consecutive chunks of the segment: token order); and the slot's outputs.
__global__ void __launch_bounds__(VF_THREADS) k_verify_pick(const __grid_constant__ VerifyArgs a) {
    __shared__ u64 tsum[VF_THREADS];
    __shared__ uint32_t bm[VF_BM_WORDS];
    __shared__ long long s_token;
    const int b = blockIdx.x, k = a.k, V = a.V, tid = threadIdx.x;
    const int2 sl = a.slot[b];
    const int j = sl.x;
    if (tid == 0) {
        if (sl.y == 0) {
            const bool greedy = !(a.temperature[b] > 0.0f);
            s_token = greedy ? a.st_t[(size_t)b * (k + 1) + j].argmax : a.samp_t[(size_t)b * (k + 1) + j];
        } else s_token = -1;
    }
    __syncthreads();
    if (sl.y == 1) {
        u64 total = 0;
        for (int s = 0; s < VF_NSEG; ++s) total += a.seg_sums[(size_t)b * VF_NSEG + s];
        if (total == 0) {
            if (tid == 0) s_token = a.samp_t[(size_t)b * (k + 1) + j];   // no residual mass: draw from p_j
        } else {
            double t = ceil((double)a.us[(size_t)b * (k + 1) + j] * (double)total);
            u64 target = t <= 1.0 ? 1ull : (u64)t;
            if (target > total) target = total;
            int sx = 0; u64 before = 0;
            for (; sx < VF_NSEG - 1; ++sx) {
                const u64 v = a.seg_sums[(size_t)b * VF_NSEG + sx];
                if (before + v >= target) break;
                before += v;
            }
            Residual res;
            res.init(a.st_t[(size_t)b * (k + 1) + j], a.st_d[(size_t)b * k + j]);
            const int32_t* mrow = a.mask ? a.mask + ((size_t)b * (k + 1) + j) * a.W : nullptr;
            const size_t bt = ((size_t)b * (k + 1) + j) * V, bd = ((size_t)b * k + j) * V;
            const int lo = min(sx * a.seg, V), hi = min(lo + a.seg, V);
            const int per = (hi - lo + VF_THREADS - 1) / VF_THREADS;
            const int c_lo = min(lo + tid * per, hi), c_hi = min(c_lo + per, hi);
            PenSlot pen;
            pen.init(a, b);
            if (pen.on) pen.mark(bm, lo, hi);                        // (sx, and so this branch, is the same for every thread)
            u64 mine = 0;
            for (int i = c_lo; i < c_hi; ++i)
                if (mask_allows(mrow, i)) {
                    float lt = load_logit(a.tl, a.dtype, bt + i), ld = load_logit(a.dl, a.dtype, bd + i);
                    pen.fix(bm, lo, i, lt, ld);
                    mine += res(lt, ld);
                }
            tsum[tid] = mine;
            __syncthreads();
            if (tid == 0) {
                u64 run = before;
                int tx = VF_THREADS - 1;
                for (int t2 = 0; t2 < VF_THREADS; ++t2) { if (run + tsum[t2] >= target) { tx = t2; break; } run += tsum[t2]; }
                tsum[0] = run; s_token = -2 - tx;                 // (thread tx walks its chunk from the running sum `run`)
            }
            __syncthreads();
            if (s_token == -2 - tid) {
                u64 run = tsum[0];
                long long tok = c_hi > c_lo ? c_hi - 1 : lo;
                for (int i = c_lo; i < c_hi; ++i) {
                    if (mask_allows(mrow, i)) {
                        float lt = load_logit(a.tl, a.dtype, bt + i), ld = load_logit(a.dl, a.dtype, bd + i);
                        pen.fix(bm, lo, i, lt, ld);
                        run += res(lt, ld);
                    }
                    if (run >= target) { tok = i; break; }
                }
                s_token = tok;
            }
        }
        __syncthreads();
    }
    if (tid == 0) {
        int64_t* o = a.out_tok + (size_t)b * (k + 1);
        for (int i = 0; i <= k; ++i) o[i] = i < j ? a.draft_ids[(size_t)b * k + i] : -1;
        o[j] = s_token;
        a.n[b] = j + 1;
    }
}

// scratch_stats holds, after the 2k + 1 row statistics of every slot, the per-slot decision and the segment sums
extern "C" int64_t colinfer_spec_verify_stats_bytes(int B, int k) {
    return (int64_t)B * (2 * k + 1) * (int64_t)sizeof(colinfer_row_stats) + (int64_t)B * 8 + (int64_t)B * VF_NSEG * 8;
}
extern "C" int64_t colinfer_spec_verify_ids_bytes(int B, int k) { return (int64_t)B * (k + 1) * 8; }

extern "C" int colinfer_spec_verify(const void* target_logits, const void* draft_logits, int dtype, const int32_t* mask,
                                    int W, const colinfer_sampler_params* params, const int64_t* draft_ids,
                                    const float* ua, const float* us, int64_t* out_tok, int32_t* n,
                                    colinfer_row_stats* scratch_stats, int64_t* scratch_ids, int B, int k, int V,
                                    void* stream) {
    if (!target_logits || !draft_logits || !params || !draft_ids || !ua || !us || !out_tok || !n || !scratch_stats ||
        !scratch_ids || B < 0 || k < 1 || V <= 0)
        return (int)cudaErrorInvalidValue;
    if (B == 0) return 0;
    if ((((V + VF_NSEG - 1) / VF_NSEG + 127) / 128) * 128 > VF_BM_WORDS * 32) return (int)cudaErrorInvalidValue;
    colinfer_row_stats* st_t = scratch_stats;
    colinfer_row_stats* st_d = scratch_stats + (size_t)B * (k + 1);
    // target rows: statistics and the plain draw of every row with its sampling uniform
    int e = colinfer_sample(target_logits, dtype, mask, k + 1, W, params, nullptr, 0, us, scratch_ids, st_t, nullptr,
                            B, k + 1, V, 0, stream);
    if (e) return e;
    // draft rows: statistics only (the first k mask rows of each slot apply)
    e = colinfer_sample(draft_logits, dtype, mask, k + 1, W, params, nullptr, 0, nullptr, nullptr, st_d, nullptr,
                        B, k, V, 0, stream);
    if (e) return e;
    VerifyArgs a;
    a.tl = target_logits; a.dl = draft_logits; a.dtype = dtype; a.mask = mask; a.W = W;
    a.temperature = params->temperature; a.draft_ids = draft_ids; a.ua = ua; a.us = us;
    a.st_t = st_t; a.st_d = st_d; a.samp_t = scratch_ids; a.out_tok = out_tok; a.n = n; a.B = B; a.k = k; a.V = V;
    a.slot = reinterpret_cast<int2*>(st_d + (size_t)B * k);
    a.seg_sums = reinterpret_cast<u64*>(a.slot + B);
    a.seg = (((V + VF_NSEG - 1) / VF_NSEG + 127) / 128) * 128;
    a.history = params->history; a.hist_len = params->hist_len; a.hist_stride = params->history ? params->hist_stride : 0;
    a.rp = params->repetition_penalty; a.pp = params->presence_penalty; a.fp = params->frequency_penalty;
    a.vec = (dtype == COLINFER_F32 && (V % 4) == 0 && (((uintptr_t)target_logits) & 15) == 0 && (((uintptr_t)draft_logits) & 15) == 0) ? 1 : 0;
    cudaStream_t st = (cudaStream_t)stream;
    k_verify_decide<<<(B + 3) / 4, 128, 0, st>>>(a);
    k_verify_residual<<<B * VF_NSEG, VF_THREADS, 0, st>>>(a);
    k_verify_pick<<<B, VF_THREADS, 0, st>>>(a);
    return (int)cudaGetLastError();
}

extern "C" int colinfer_version(void) { return 100; }
