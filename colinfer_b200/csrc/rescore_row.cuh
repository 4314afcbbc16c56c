// One warp's exact logit of one matrix row: the dot products shared by the rescoring kernels and the fused draft pick.
//
// The accumulation order is that of the reference's rescoring kernels (csrc/sampling.cu:36-115), so a row's logit is the
// same bit for bit wherever it is computed: lane l takes the chunks l, l + 32, ... in order, one fp32 fma per element in
// element order; then the lanes are summed with xor-shuffles 16, 8, 4, 2, 1 (every lane ends with the sum).  Every lane
// issues the loads of two chunks before the first fma; BF16 rows are read with the streaming (evict-first) policy.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <stdint.h>

namespace rsc {

constexpr int UNROLL = 2;            // chunks per lane in flight

__device__ __forceinline__ float dot8_bf16(const uint4& wv, const uint4& xv, float acc) {
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 wf = __bfloat1622float2(w2[i]), xf = __bfloat1622float2(x2[i]);
        acc = fmaf(wf.x, xf.x, acc);
        acc = fmaf(wf.y, xf.y, acc);
    }
    return acc;
}

// xs: the slot's K bf16 activations in shared memory; w: the matrix [rows, K] bf16; row: which row.  UN loads of a lane are
// in flight before the first fma (the order of the fmas does not depend on it).
template <int UN = UNROLL>
__device__ __forceinline__ float dot_row_bf16(const uint4* xs, const __nv_bfloat16* w, long long row, int K, int lane) {
    const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)row * K);
    const int chunks = K >> 3;
    float acc = 0.f;
    int c = lane;
    for (; c + 32 * (UN - 1) < chunks; c += 32 * UN) {
        uint4 wv[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) wv[u] = __ldcs(wr + c + 32 * u);   // streamed: the row is read once by this warp
#pragma unroll
        for (int u = 0; u < UN; ++u) acc = dot8_bf16(wv[u], xs[c + 32 * u], acc);
    }
    for (; c < chunks; c += 32) acc = dot8_bf16(__ldcs(wr + c), xs[c], acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    return acc;
}

// NVFP4 row layout: K / 2 bytes of E2M1 pairs (byte i: elements 2i in the low nibble, 2i + 1 in the high one) and K / 16
// E4M3 scales, one per 16 elements.  The sum over blocks of (sum over the block's 16 elements of w * x) * scale; the
// caller multiplies by the global scale.
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

template <int UN = UNROLL>
__device__ __forceinline__ float dot_row_nvfp4(const uint4* xs, const uint8_t* w, const uint8_t* sf, long long row, int K, int lane) {
    const uint2* wr = reinterpret_cast<const uint2*>(w + (size_t)row * (K / 2));
    const uint8_t* sr = sf + (size_t)row * (K / 16);
    const int blocks = K >> 4;
    float acc = 0.f;
    int blk = lane;
    for (; blk + 32 * (UN - 1) < blocks; blk += 32 * UN) {
        uint2 pw[UN]; uint8_t sv[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) { pw[u] = __ldg(wr + blk + 32 * u); sv[u] = __ldg(sr + blk + 32 * u); }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int bb = blk + 32 * u;
            acc = fmaf(block16(pw[u], xs[2 * bb], xs[2 * bb + 1]), e4m3_to_float(sv[u]), acc);
        }
    }
    for (; blk < blocks; blk += 32)
        acc = fmaf(block16(__ldg(wr + blk), xs[2 * blk], xs[2 * blk + 1]), e4m3_to_float(__ldg(sr + blk)), acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    return acc;
}

}  // namespace rsc
