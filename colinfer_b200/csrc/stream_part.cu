// stream_part.cu -- one instantiation of the streaming kernel per translation unit (the build compiles this file once
// per COLINFER_STREAM_PART = 0 .. 8, side by side): parts 0-3 fp32 rows with 128-bit loads, 4-7 bf16 rows with 64-bit
// loads (bit 1: histories / penalties, bit 0: grammar mask), part 8 the general loader in its fullest form.
#include <mutex>

#include "stream_kernel.cuh"

#ifndef COLINFER_STREAM_PART
#error "compile with -DCOLINFER_STREAM_PART=<0..8>"
#endif

#define ST_CAT2(a, b) a##b
#define ST_CAT(a, b) ST_CAT2(a, b)

namespace {
constexpr int kPart = COLINFER_STREAM_PART;
constexpr int kLoader = kPart == 8 ? 0 : 1 + kPart / 4;
constexpr bool kPen = kPart == 8 ? true : ((kPart >> 1) & 1) != 0;
constexpr bool kMask = kPart == 8 ? true : (kPart & 1) != 0;
}  // namespace

// Launches this part's kernel.  The opt-in to large dynamic shared memory is per kernel and device: done once.
int ST_CAT(colinfer_stream_part_, COLINFER_STREAM_PART)(const strm::Args* a, int grid, int block, int smem, cudaStream_t stream, int dev) {
    static unsigned char opted[64] = {};
    static std::mutex guard;
    auto kernel = strm::k_sample_stream<kPen, kMask, kLoader>;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lock(guard);
        if (!opted[dev]) {
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
            if (e != cudaSuccess) return (int)e;
            opted[dev] = 1;
        }
    }
    kernel<<<grid, block, smem, stream>>>(*a);
    return (int)cudaGetLastError();
}
