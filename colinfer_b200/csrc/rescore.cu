// Exact logits of candidate rows of the lm_head (the rescoring step of the low-rank draft heads, the step just before
// verify): out[b, j] = sum_k x[b, k] * W[cand[b, j], k], for a BF16 matrix (csrc/sampling.cu:84-115 of the reference)
// and for an NVFP4 matrix with E4M3 block scales (csrc/sampling.cu:36-82).  A gather of NC rows per slot: HBM-bound.
//
// The accumulation order is the reference's, so results are bit-identical to its kernels and a row's logit does not
// depend on B or NC: one warp per candidate; lane l takes the chunks l, l + 32, ... in order, one fp32 fma per element
// in element order; then the lanes are summed with xor-shuffles 16, 8, 4, 2, 1.  What differs is how the bytes move:
// the slot's activation row is staged once per CTA in shared memory (the reference re-reads it from L1/L2 for every
// candidate), sixteen candidates share a CTA, every lane issues the loads of two chunks before the first fma, and the
// matrix rows are read with the streaming (evict-first) policy.  The step is a gather of matrix rows and runs at the
// copy rate of the part, as the reference's kernel does: what is left to win is fusing it with its neighbours.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <stdint.h>

#include "../../include/colinfer_b200.h"

namespace rsc {

constexpr int WARPS = 16;            // candidates per CTA
constexpr int UNROLL = 2;            // chunks per lane in flight

// ------------------------------------------------------------------------------------------------ BF16 rows
__global__ void __launch_bounds__(WARPS * 32) k_rescore_bf16(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                            const int64_t* __restrict__ cand, float* __restrict__ out, int K, int NC,
                                                            long long n_rows_w) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint4* xs = reinterpret_cast<uint4*>(smem);                      // the slot's activations: K bf16 = K / 8 chunks
    const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = K >> 3;
    const uint4* xg = reinterpret_cast<const uint4*>(x + (size_t)b * K);
    for (int c = threadIdx.x; c < chunks; c += WARPS * 32) xs[c] = __ldg(xg + c);
    __syncthreads();
    const int j = blockIdx.x * WARPS + warp;
    if (j >= NC) return;
    const int64_t row = cand[(size_t)b * NC + j];
    if (row < 0 || row >= n_rows_w) { if (lane == 0) out[(size_t)b * NC + j] = __int_as_float(0x7fc00000); return; }   // NaN, never a fault
    const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)row * K);
    float acc = 0.f;
    int c = lane;
    for (; c + 32 * (UNROLL - 1) < chunks; c += 32 * UNROLL) {
        uint4 wv[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) wv[u] = __ldcs(wr + c + 32 * u);   // streamed: the row is read once by this warp
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const uint4 xv = xs[c + 32 * u];
            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv[u]);
            const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 wf = __bfloat1622float2(w2[i]), xf = __bfloat1622float2(x2[i]);
                acc = fmaf(wf.x, xf.x, acc);
                acc = fmaf(wf.y, xf.y, acc);
            }
        }
    }
    for (; c < chunks; c += 32) {
        const uint4 wv = __ldcs(wr + c), xv = xs[c];
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 wf = __bfloat1622float2(w2[i]), xf = __bfloat1622float2(x2[i]);
            acc = fmaf(wf.x, xf.x, acc);
            acc = fmaf(wf.y, xf.y, acc);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[(size_t)b * NC + j] = acc;
}

// ------------------------------------------------------------------------------------------------ NVFP4 rows
// Row layout: K / 2 bytes of E2M1 pairs (byte i: elements 2i in the low nibble, 2i + 1 in the high one) and K / 16 E4M3
// scales, one per 16 elements.  out = gs * sum over blocks of (sum over the block's 16 elements of w * x) * scale.
__device__ __forceinline__ float2 e2m1_pair(uint32_t byte) {        // low nibble -> .x, high nibble -> .y
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
    return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
// 16 consecutive elements: the two words of packed weights against 16 bf16 activations, one fma per element in order
__device__ __forceinline__ float block16(uint2 pw, const uint4& x0, const uint4& x1) {
    const uint32_t word[2] = {pw.x, pw.y};
    const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};   // bf16 pairs, element order
    float s = 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 wf = e2m1_pair((word[h] >> (8 * q)) & 0xFFu);
            const float2 xf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[4 * h + q]));
            s = fmaf(wf.x, xf.x, s);
            s = fmaf(wf.y, xf.y, s);
        }
    }
    return s;
}
__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
    const __half_raw sc = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&sc));
}

__global__ void __launch_bounds__(WARPS * 32) k_rescore_nvfp4(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ w,
                                                             const uint8_t* __restrict__ sf, float gs, const int64_t* __restrict__ cand,
                                                             float* __restrict__ out, int K, int NC, long long n_rows_w) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint4* xs = reinterpret_cast<uint4*>(smem);
    const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint4* xg = reinterpret_cast<const uint4*>(x + (size_t)b * K);
    for (int c = threadIdx.x; c < (K >> 3); c += WARPS * 32) xs[c] = __ldg(xg + c);
    __syncthreads();
    const int j = blockIdx.x * WARPS + warp;
    if (j >= NC) return;
    const int64_t row = cand[(size_t)b * NC + j];
    if (row < 0 || row >= n_rows_w) { if (lane == 0) out[(size_t)b * NC + j] = __int_as_float(0x7fc00000); return; }
    const uint2* wr = reinterpret_cast<const uint2*>(w + (size_t)row * (K / 2));
    const uint8_t* sr = sf + (size_t)row * (K / 16);
    const int blocks = K >> 4;
    float acc = 0.f;
    int blk = lane;
    for (; blk + 32 * (UNROLL - 1) < blocks; blk += 32 * UNROLL) {
        uint2 pw[UNROLL]; uint8_t sv[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) { pw[u] = __ldg(wr + blk + 32 * u); sv[u] = __ldg(sr + blk + 32 * u); }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int bb = blk + 32 * u;
            acc = fmaf(block16(pw[u], xs[2 * bb], xs[2 * bb + 1]), e4m3_to_float(sv[u]), acc);
        }
    }
    for (; blk < blocks; blk += 32)
        acc = fmaf(block16(__ldg(wr + blk), xs[2 * blk], xs[2 * blk + 1]), e4m3_to_float(__ldg(sr + blk)), acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[(size_t)b * NC + j] = acc * gs;
}

}  // namespace rsc

static int rescore_check(const void* x, const void* w, const void* cand, const void* out, int B, int K, int NC, long long rows_w, int kmul) {
    if (B < 0 || NC < 0 || K < kmul || (K % kmul) != 0 || rows_w < 1 || K > 48 * 1024) return (int)cudaErrorInvalidValue;
    if (B == 0 || NC == 0) return -1;                               // nothing to do
    if (!x || !w || !cand || !out || (((uintptr_t)x) & 15) || (((uintptr_t)w) & 15) || B > 65535) return (int)cudaErrorInvalidValue;
    return 0;
}

// Replaces ops().rescore_bf16 (csrc/sampling.cu:84-115, csrc/bindings.cpp:561-572).
extern "C" int colinfer_rescore_bf16(const void* x, const void* w, const int64_t* cand, float* out, int B, int K, int NC,
                                     int64_t rows_w, void* stream) {
    const int chk = rescore_check(x, w, cand, out, B, K, NC, rows_w, 8);
    if (chk) return chk < 0 ? (int)cudaSuccess : chk;
    const int smem = K * 2;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(rsc::k_rescore_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
    }
    rsc::k_rescore_bf16<<<dim3((NC + rsc::WARPS - 1) / rsc::WARPS, B), rsc::WARPS * 32, smem, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, cand, out, K, NC, (long long)rows_w);
    return (int)cudaGetLastError();
}

// Replaces ops().rescore_nvfp4 (csrc/sampling.cu:36-82, csrc/bindings.cpp:547-558).
extern "C" int colinfer_rescore_nvfp4(const void* x, const void* w, const void* sf, float gs, const int64_t* cand, float* out,
                                      int B, int K, int NC, int64_t rows_w, void* stream) {
    const int chk = rescore_check(x, w, cand, out, B, K, NC, rows_w, 16);
    if (chk) return chk < 0 ? (int)cudaSuccess : chk;
    if (!sf || (((uintptr_t)w) & 7)) return (int)cudaErrorInvalidValue;
    const int smem = K * 2;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(rsc::k_rescore_nvfp4, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
    }
    rsc::k_rescore_nvfp4<<<dim3((NC + rsc::WARPS - 1) / rsc::WARPS, B), rsc::WARPS * 32, smem, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (const uint8_t*)w, (const uint8_t*)sf, gs, cand, out, K, NC, (long long)rows_w);
    return (int)cudaGetLastError();
}
