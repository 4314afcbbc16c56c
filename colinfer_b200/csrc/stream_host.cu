// stream_host.cu -- host side of the streaming kernel: geometry of a launch and the choice of its instantiation.
#include <mutex>

#include "stream_kernel.cuh"

void colinfer_profile_buffer(long long** buf, int* slots);   // sample.cu: the buffer colinfer_set_profile_buffer registered

#define ST_DECL(n) int colinfer_stream_part_##n(const strm::Args*, int, int, int, cudaStream_t, int);
ST_DECL(0) ST_DECL(1) ST_DECL(2) ST_DECL(3) ST_DECL(4) ST_DECL(5) ST_DECL(6) ST_DECL(7) ST_DECL(8)

namespace {
using PartFn = int (*)(const strm::Args*, int, int, int, cudaStream_t, int);
const PartFn kParts[9] = {colinfer_stream_part_0, colinfer_stream_part_1, colinfer_stream_part_2, colinfer_stream_part_3,
                          colinfer_stream_part_4, colinfer_stream_part_5, colinfer_stream_part_6, colinfer_stream_part_7,
                          colinfer_stream_part_8};

int stream_smem_bytes(int V) {
    const int nw = (V + 31) / 32;
    return strm::NB1 * 4 + strm::BINS * 8 + strm::FB_NB * 8 + strm::NW * strm::WLIST * (int)sizeof(strm::Cand) +
           (int)sizeof(strm::Sc) + 2 * nw * 4 + strm::PEN_TABLE * 16 + 256;
}

// Multiprocessors of a device, looked up once.
int sm_count_of(int dev, int* out) {
    static int sm_count[64] = {};
    static std::mutex guard;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(guard);
    if (sm_count[dev] == 0) {
        int n = 0;
        const cudaError_t e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        sm_count[dev] = n > 0 ? n : 1;
    }
    *out = sm_count[dev];
    return 0;
}
}  // namespace

// Launches the streaming kernel; returns cudaErrorInvalidValue when the vocabulary's penalty bitmap does not fit.
int colinfer_launch_stream(const void* logits, int dtype, const int32_t* mask, int mask_rows, int W,
                           const colinfer_sampler_params* params, const void* pos, int pos_is_i64, const float* u,
                           int64_t* out_ids, colinfer_row_stats* stats, int32_t* status, int B, int R, int V, int flags,
                           cudaStream_t stream) {
    const int smem = stream_smem_bytes(V);
    if (smem > 226 * 1024 || V > strm::NW * 128 * strm::XSTEPS) return (int)cudaErrorInvalidValue;
    const bool vec = dtype == COLINFER_F32 && (V % 4) == 0 && (((uintptr_t)logits) & 15) == 0;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    const int rc = sm_count_of(dev, &sms);
    if (rc) return rc;
    strm::Args a;
    a.logits = logits; a.dtype = dtype;
    a.vec = vec ? 1 : 0;
    a.mask = mask; a.mask_rows = mask_rows; a.W = W;
    a.p = *params;
    a.pos = pos; a.pos_i64 = pos_is_i64; a.u = u;
    a.out = out_ids; a.stats = stats; a.status = status;
    a.B = B; a.R = R; a.V = V; a.flags = flags;
    colinfer_profile_buffer(&a.prof, &a.prof_slots);
    // one instantiation per loader (general, fp32 x 4, bf16 x 4), histories (penalties) or not, grammar mask or not; the
    // general loader (unaligned rows, odd vocabularies) only in its fullest form
    const bool vec16 = dtype == COLINFER_BF16 && (V % 4) == 0 && (((uintptr_t)logits) & 7) == 0;
    const int variant = (params->history != nullptr ? 2 : 0) + (mask != nullptr ? 1 : 0);
    const int part = vec ? variant : vec16 ? 4 + variant : 8;
    const long long rows = (long long)B * R;
    const int slots = sms * strm::CTAS_PER_SM;
    const int grid = (int)(rows < slots ? rows : slots);
    return kParts[part](&a, grid, strm::NT, smem, stream, dev);
}
