// gather.cu -- the id gather of the row-sharded sampler over NVLink, as one small kernel (sm_100a).
//
// Rows are sharded over the GPUs of a node; after the sampler every rank holds the ids of its own rows and every rank
// needs all of them (8 bytes per row).  Instead of a collective call behind the kernel, each rank's GPU stores its ids
// straight into every rank's gather buffer -- plain peer stores through pointers exchanged once at set-up -- then raises
// its flag at every rank and waits until every rank's flag has reached the same step.  One launch of one CTA; no
// multicast objects, no library kernel is handed a peer's memory.
//
// Protocol (buffers are double: steps alternate between two halves, flags hold the step number).
//   step s of rank r:  ids -> bufs[p][s & 1][offset_r ...] for every rank p;  __threadfence_system;  flags[p][r] = s
//   then wait until flags[r][q] >= s for every rank q (its ids of step s have landed in this rank's buffer).
// A rank can run step s + 2 (which reuses half s & 1) only after its own wait of step s + 1, i.e. after every other rank
// has launched its step s + 1 -- stream-ordered behind whatever consumed step s there.
// The wait is bounded: after `limit_cycles` it gives up, records COLINFER_GATHER_TIMEOUT in *status and the kernel
// returns (the context stays usable; the ids of the late ranks are whatever the buffer held).
#include "common.cuh"
#include "../../include/colinfer_b200.h"

namespace {

__device__ __forceinline__ long long ld_acquire_sys(const long long* p) {
    long long v;
    asm volatile("ld.acquire.sys.global.s64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(long long* p, long long v) {
    asm volatile("st.release.sys.global.s64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__global__ void __launch_bounds__(1024) k_gather_ids(const int64_t* __restrict__ local, int n_local, int64_t row_offset,
                                                     int64_t* const* __restrict__ peer_bufs, long long* const* __restrict__ peer_flags,
                                                     int n_ranks, int rank, long long* step_counter, int64_t half_elems,
                                                     int64_t* __restrict__ out_all, long long limit_cycles, int32_t* status) {
    __shared__ long long s_step;
    if (threadIdx.x == 0) s_step = *step_counter + 1;          // this call's step (kept on the device: replays of a captured launch advance it)
    __syncthreads();
    const long long step = s_step;
    const int64_t half = (step & 1) * half_elems;
    // my ids into every rank's buffer (this rank's own included)
    for (int p = 0; p < n_ranks; ++p) {
        int64_t* dst = peer_bufs[p] + half + row_offset;
        for (int i = threadIdx.x; i < n_local; i += blockDim.x) dst[i] = local[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < n_ranks) st_release_sys(peer_flags[threadIdx.x] + rank, step);
    // every rank's ids of this step have landed here
    if (threadIdx.x < n_ranks) {
        const long long* mine = peer_flags[rank] + threadIdx.x;
        const long long t0 = clock64();
        bool ok = true;
        while (ld_acquire_sys(mine) < step) {
            if (clock64() - t0 > limit_cycles) { ok = false; break; }
            __nanosleep(200);
        }
        if (!ok && status) atomicOr(status, COLINFER_GATHER_TIMEOUT);
    }
    __threadfence_system();
    __syncthreads();
    // the step's ids of all rows, in row order, where the caller wants them (the double buffer stays the kernel's own)
    const int64_t* src = peer_bufs[rank] + half;
    for (int64_t i = threadIdx.x; i < half_elems; i += blockDim.x) out_all[i] = __ldcg(src + i);   // (L2: where the peers' stores arrive)
    if (threadIdx.x == 0) *step_counter = step;
}

}  // namespace

extern "C" int colinfer_gather_ids(const int64_t* local, int n_local, int64_t row_offset, int64_t* const* peer_bufs,
                                   long long* const* peer_flags, int n_ranks, int rank, long long* step_counter,
                                   int64_t half_elems, int64_t* out_all, int64_t limit_cycles, int32_t* status, void* stream) {
    if (!local || !peer_bufs || !peer_flags || !step_counter || !out_all || n_local < 0 || n_ranks < 1 || n_ranks > 1024 || rank < 0 ||
        rank >= n_ranks || row_offset < 0 || row_offset + n_local > half_elems)
        return (int)cudaErrorInvalidValue;
    k_gather_ids<<<1, 1024, 0, (cudaStream_t)stream>>>(local, n_local, row_offset, peer_bufs, peer_flags, n_ranks, rank, step_counter,
                                                       half_elems, out_all, limit_cycles > 0 ? limit_cycles : 2000000000LL, status);
    return (int)cudaGetLastError();
}
