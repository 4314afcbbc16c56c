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
#include <stdint.h>

#include "../../include/colinfer_b200.h"
#include "rescore_row.cuh"

namespace rsc {

constexpr int WARPS = 16;            // candidates per CTA

// ------------------------------------------------------------------------------------------------ BF16 rows
__global__ void __launch_bounds__(WARPS * 32) k_rescore_bf16(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                            const int64_t* __restrict__ cand, float* __restrict__ out, int K, int NC,
                                                            long long n_rows_w) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint4* xs = reinterpret_cast<uint4*>(smem);                      // the slot's activations: K bf16 = K / 8 chunks
    const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint4* xg = reinterpret_cast<const uint4*>(x + (size_t)b * K);
    for (int c = threadIdx.x; c < (K >> 3); c += WARPS * 32) xs[c] = __ldg(xg + c);
    __syncthreads();
    const int j = blockIdx.x * WARPS + warp;
    if (j >= NC) return;
    const int64_t row = cand[(size_t)b * NC + j];
    if (row < 0 || row >= n_rows_w) { if (lane == 0) out[(size_t)b * NC + j] = __int_as_float(0x7fc00000); return; }   // NaN, never a fault
    const float acc = dot_row_bf16(xs, w, row, K, lane);
    if (lane == 0) out[(size_t)b * NC + j] = acc;
}

// ------------------------------------------------------------------------------------------------ NVFP4 rows
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
    const float acc = dot_row_nvfp4(xs, w, sf, row, K, lane);
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
