// common.cuh -- device helpers shared by the logits -> token kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <cooperative_groups.h>

namespace cg = cooperative_groups;
typedef unsigned long long u64;

#define CI_NEG_INF (__int_as_float(0xff800000))
#define CI_LOG2E 1.4426950408889634f
#define CI_MASS_BITS 30
#define CI_MASS_SCALE 1073741824.0f     // 2^30: kept masses are summed as integers in units of 2^-30
#define CI_MASS_INV (1.0 / 1073741824.0)

// ------------------------------------------------------------------------------------------------ ordered float keys
// Order-preserving map float -> uint32 (ascending).  -0 is folded onto +0 so that equal floats get equal keys.
__device__ __forceinline__ uint32_t f2key(float f) {
    f = f + 0.0f;
    const uint32_t b = __float_as_uint(f);
    return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}
__device__ __forceinline__ float key2f(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}
#define CI_KEY_NEG_INF 0x007FFFFFu  // f2key(-inf)

// z = l / tc exactly as the reference computes it (one IEEE division); tc == 1 needs no division.
// Repetition / presence / frequency penalties of one logit whose token occurs cnt > 0 times in the slot's history (not in
// the reference; this project's definition): l > 0 ? l / rp : l * rp, then - fp * cnt, then - pp, each rounded to fp32.
__device__ __forceinline__ float apply_penalty(float l, int cnt, float rp, float pp, float fp) {
    l = l > 0.0f ? __fdiv_rn(l, rp) : __fmul_rn(l, rp);
    l = __fsub_rn(l, __fmul_rn(fp, (float)cnt));
    return __fsub_rn(l, pp);
}

__device__ __forceinline__ float scale_logit(float l, float tc) { return __fdiv_rn(l, tc); }

// Smallest float c with c / tc >= zt (division rounded to nearest, monotone in c).  `start` must be within a few
// units in the last place of the answer (it is zt * tc, or a value whose quotient is zt).
__device__ __forceinline__ float lower_logit_for(float zt, float tc, float start) {
    if (!(zt > CI_NEG_INF)) return CI_NEG_INF;
    uint32_t k = f2key(start);
    for (int it = 0; it < 64 && k > CI_KEY_NEG_INF + 1; ++it) {
        if (scale_logit(key2f(k - 1), tc) >= zt) --k; else break;
    }
    for (int it = 0; it < 64 && k < 0xFF800000u; ++it) {  // f2key(+inf) = 0xFF800000
        if (scale_logit(key2f(k), tc) >= zt) break;
        ++k;
    }
    return key2f(k);
}

// Kept mass of one element in units of 2^-30: exp(z - m), z = l / tc.  The same function feeds every histogram and
// every prefix sum, so all sums are exact integer sums of the same addends (order independent, reproducible).
// The division is the two-FMA sequence q = l * r, q += fma(-q, tc, l) * r with r = 1 / tc rounded to nearest, which
// gives the IEEE quotient for every operand in range (it can be one unit off only when tc's significand is all ones);
// it only feeds masses -- thresholds and ties always use the exact division.  The exponential is the hardware
// ex2.approx (relative error ~2^-22); results below 2^-31 round to zero mass.
struct MassFn {
    float tc, rinv, m;
    __device__ __forceinline__ void init(float tc_, float m_) { tc = tc_; rinv = __frcp_rn(tc_); m = m_; }
    __device__ __forceinline__ uint32_t operator()(float l) const {
        const float q0 = l * rinv;
        const float z = fmaf(fmaf(-q0, tc, l), rinv, q0);
        float e;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"((z - m) * CI_LOG2E));
        return __float2uint_rn(e * CI_MASS_SCALE);
    }
    // Four masses at once (0 for logits below lk); the same values as operator().
    __device__ __forceinline__ void four(const float (&l)[4], float lk, uint32_t (&q)[4]) const {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float q0 = l[j] * rinv;
            const float z = fmaf(fmaf(-q0, tc, l[j]), rinv, q0);
            float e;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"((z - m) * CI_LOG2E));
            q[j] = l[j] >= lk ? __float2uint_rn(e * CI_MASS_SCALE) : 0u;
        }
    }
};

// ------------------------------------------------------------------------------------------------ Philox4x32-10
// Salmon et al. 2011; keyed and indexed as the reference's csrc/sampling.cu:11-30 (counter (n / 4, 0), word n % 4).
__device__ __forceinline__ uint32_t philox_word(u64 key, u64 n) {
    uint32_t c0 = (uint32_t)(n >> 2), c1 = (uint32_t)(n >> 34), c2 = 0u, c3 = 0u;
    uint32_t k0 = (uint32_t)key, k1 = (uint32_t)(key >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        if (r) { k0 += 0x9E3779B9u; k1 += 0xBB67AE85u; }
        const uint32_t lo0 = 0xD2511F53u * c0, hi0 = __umulhi(0xD2511F53u, c0);
        const uint32_t lo1 = 0xCD9E8D57u * c2, hi1 = __umulhi(0xCD9E8D57u, c2);
        const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    }
    const uint32_t sel = (uint32_t)(n & 3);
    return sel == 0 ? c0 : sel == 1 ? c1 : sel == 2 ? c2 : c3;
}
__device__ __forceinline__ u64 philox_key(int64_t seed) {
    return (u64)seed * 6364136223846793005ULL + 1442695040888963407ULL;
}
// (0, 1]: two separate fp32 operations (no fused multiply-add), as the reference builds with --fmad=false.
__device__ __forceinline__ float u32_to_uniform(uint32_t x) {
    return __fadd_rn(__fmul_rn((float)x, 2.3283064e-10f), 2.3283064e-10f / 2.0f);
}

// ------------------------------------------------------------------------------------------------ warp helpers
__device__ __forceinline__ u64 warp_sum_u64(u64 v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ u64 warp_incl_scan_u64(u64 v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    return v;
}

// ------------------------------------------------------------------------------------------------ bulk copy (TMA)
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(void* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(20000u) : "memory");   // may suspend the thread up to ~20 us
    return ok != 0;
}
// Bounded wait for a phase of an mbarrier, for a whole warp: one lane waits (suspended by the hardware between tries,
// so the other warps of the SM keep their issue slots), then the warp reconverges.  Gives up after `limit` clock
// cycles and returns false (the caller records a status and carries on).
__device__ __forceinline__ bool mbar_wait_bounded(void* bar, uint32_t parity, long long limit) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) {
        if (!mbar_test(bar, parity)) {
            const long long t0 = clock64();
            while (!mbar_test(bar, parity)) {
                if (clock64() - t0 > limit) { ok = 0; break; }
                __nanosleep(64);
            }
        }
    }
    __syncwarp();
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted on an mbarrier.  dst, src 16-byte aligned,
// bytes a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, void* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
