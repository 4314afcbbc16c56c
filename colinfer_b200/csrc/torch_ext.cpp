// torch_ext.cpp -- the thin PyTorch C++ extension over the C ABI of libcolinfer_b200.so.
//
// What the reference's csrc/bindings.cpp is to its kernels (bindings.cpp:22-26, 538-572): every wrapper checks that its
// tensors are CUDA, contiguous and of the right dtype and shape with TORCH_CHECK (a Python RuntimeError), allocates
// outputs with torch (so that, inside CUDA-graph capture, only torch's caching allocator allocates), and launches on
// at::cuda::getCurrentCUDAStream().  No arithmetic lives here.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "../../include/colinfer_b200.h"

namespace {

using Opt = c10::optional<at::Tensor>;

void check(const at::Tensor& t, at::ScalarType dt, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (this path has no CPU implementation)");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(t.scalar_type() == dt, name, " must be ", dt, ", got ", t.scalar_type());
}
void cuda_ok(int code, const char* what) {
    TORCH_CHECK(code == 0, what, " failed: CUDA error ", code, code == 1 ? " (invalid value / shape)" : "");
}
void* stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int dtype_code(const at::Tensor& logits) {
    if (logits.scalar_type() == at::kFloat) return COLINFER_F32;
    if (logits.scalar_type() == at::kBFloat16) return COLINFER_BF16;
    TORCH_CHECK(false, "logits must be float32 or bfloat16, got ", logits.scalar_type());
}

// The slot parameters of SamplerParams as the C struct.
colinfer_sampler_params params_of(int64_t B, const at::Tensor& temperature, const at::Tensor& top_k, const at::Tensor& top_p,
                                  const at::Tensor& log_min_p, const Opt& seed, const Opt& rep, const Opt& pres, const Opt& freq,
                                  const Opt& history, const Opt& hist_len) {
    colinfer_sampler_params p{};
    check(temperature, at::kFloat, "temperature"); check(top_k, at::kInt, "top_k");
    check(top_p, at::kFloat, "top_p"); check(log_min_p, at::kFloat, "log_min_p");
    TORCH_CHECK(temperature.numel() == B && top_k.numel() == B && top_p.numel() == B && log_min_p.numel() == B,
                "temperature, top_k, top_p, log_min_p must have one entry per slot (", B, ")");
    p.temperature = temperature.data_ptr<float>(); p.top_k = top_k.data_ptr<int32_t>();
    p.top_p = top_p.data_ptr<float>(); p.log_min_p = log_min_p.data_ptr<float>();
    if (seed) { check(*seed, at::kLong, "seed"); TORCH_CHECK(seed->numel() == B, "seed must have one entry per slot"); p.seed = seed->data_ptr<int64_t>(); }
    if (rep) { check(*rep, at::kFloat, "repetition_penalty"); TORCH_CHECK(rep->numel() == B, "repetition_penalty [B]"); p.repetition_penalty = rep->data_ptr<float>(); }
    if (pres) { check(*pres, at::kFloat, "presence_penalty"); TORCH_CHECK(pres->numel() == B, "presence_penalty [B]"); p.presence_penalty = pres->data_ptr<float>(); }
    if (freq) { check(*freq, at::kFloat, "frequency_penalty"); TORCH_CHECK(freq->numel() == B, "frequency_penalty [B]"); p.frequency_penalty = freq->data_ptr<float>(); }
    if (history) {
        check(*history, at::kInt, "history");
        TORCH_CHECK(history->dim() == 2 && history->size(0) == B, "history must be int32 [B, H]");
        p.history = history->data_ptr<int32_t>();
        p.hist_stride = (int32_t)history->size(1);
        if (hist_len) { check(*hist_len, at::kInt, "hist_len"); TORCH_CHECK(hist_len->numel() == B, "hist_len must be int32 [B]"); p.hist_len = hist_len->data_ptr<int32_t>(); }
    }
    return p;
}

// ops().philox_uniform(seed, offset, out): writes in place (csrc/bindings.cpp:538-544 of the reference)
void philox_uniform(const at::Tensor& seed, const at::Tensor& offset, at::Tensor out) {
    check(seed, at::kLong, "seed"); check(offset, at::kLong, "offset"); check(out, at::kFloat, "out");
    TORCH_CHECK(out.dim() == 2 && seed.numel() == out.size(0) && offset.numel() == out.size(0), "out [B, n], seed / offset [B]");
    c10::cuda::CUDAGuard guard(out.device());
    cuda_ok(colinfer_philox_uniform(seed.data_ptr<int64_t>(), offset.data_ptr<int64_t>(), out.data_ptr<float>(), (int)out.size(0),
                                    (int)out.size(1), stream()), "philox_uniform");
}

// apply_mask(logits [B, R, V], mask [B, R, W]) -> masked copy (engine/runtime/sampler.py:50-56)
at::Tensor apply_mask(const at::Tensor& logits, const at::Tensor& mask) {
    check(logits, at::kFloat, "logits"); check(mask, at::kInt, "mask");
    const int64_t V = logits.size(-1), rows = logits.numel() / std::max<int64_t>(V, 1);
    TORCH_CHECK(mask.dim() >= 1 && mask.numel() == rows * mask.size(-1) && mask.size(-1) >= (V + 31) / 32, "mask [..., W] with W >= ceil(V / 32)");
    c10::cuda::CUDAGuard guard(logits.device());
    at::Tensor out = at::empty_like(logits);
    cuda_ok(colinfer_apply_mask(logits.data_ptr<float>(), mask.data_ptr<int32_t>(), out.data_ptr<float>(), rows, (int)V, (int)mask.size(-1), stream()),
            "apply_mask");
    return out;
}

// draw(logits [B, R, V], the slot parameters, pos [B]) -> ids [B, R] (+ status [B, R] int32, + row statistics [B, R, 32] uint8)
std::vector<at::Tensor> draw(const at::Tensor& logits, const at::Tensor& temperature, const at::Tensor& top_k, const at::Tensor& top_p,
                             const at::Tensor& log_min_p, const Opt& seed, const Opt& rep, const Opt& pres, const Opt& freq,
                             const Opt& history, const Opt& hist_len, const Opt& pos, const Opt& mask, const Opt& u, bool want_status,
                             bool want_stats, int64_t flags) {
    TORCH_CHECK(logits.dim() == 3, "logits [B, R, V]");
    TORCH_CHECK(logits.is_cuda() && logits.is_contiguous(), "logits must be a contiguous CUDA tensor");
    const int dt = dtype_code(logits);
    const int64_t B = logits.size(0), R = logits.size(1), V = logits.size(2);
    colinfer_sampler_params p = params_of(B, temperature, top_k, top_p, log_min_p, seed, rep, pres, freq, history, hist_len);
    const int32_t* mask_ptr = nullptr; int mask_rows = 0, W = 0;
    if (mask) {
        if (mask->is_cuda() || !mask->is_pinned()) check(*mask, at::kInt, "mask");   // pinned host rows are read in place (mapped memory)
        else TORCH_CHECK(mask->is_contiguous() && mask->scalar_type() == at::kInt, "mask must be contiguous int32");
        TORCH_CHECK(mask->dim() == 3 && mask->size(0) == B && mask->size(1) >= R && mask->size(2) >= (V + 31) / 32,
                    "mask [B, R, W] int32 with W >= ceil(V / 32)");
        mask_ptr = mask->data_ptr<int32_t>(); mask_rows = (int)mask->size(1); W = (int)mask->size(2);
    }
    const void* pos_ptr = nullptr; int pos_i64 = 0; const float* u_ptr = nullptr;
    if (u) {
        check(*u, at::kFloat, "u");
        TORCH_CHECK(u->numel() == B * R, "u [B, R]");
        u_ptr = u->data_ptr<float>();
    } else {
        TORCH_CHECK(pos.has_value(), "pos is required when no uniforms are passed");
        TORCH_CHECK(pos->is_cuda() && pos->is_contiguous() && (pos->scalar_type() == at::kInt || pos->scalar_type() == at::kLong),
                    "pos must be a contiguous int32 or int64 CUDA tensor");
        TORCH_CHECK(pos->numel() == B, "pos [B]");
        TORCH_CHECK(seed.has_value(), "SamplerParams.seed is required when no uniforms are passed");
        pos_ptr = pos->data_ptr(); pos_i64 = pos->scalar_type() == at::kLong;
    }
    c10::cuda::CUDAGuard guard(logits.device());
    at::Tensor out = at::empty({B, R}, logits.options().dtype(at::kLong));
    std::vector<at::Tensor> res{out};
    at::Tensor st, rs;
    if (want_status) { st = at::empty({B, R}, logits.options().dtype(at::kInt)); res.push_back(st); }
    if (want_stats) { rs = at::empty({B, R, (int64_t)sizeof(colinfer_row_stats)}, logits.options().dtype(at::kByte)); res.push_back(rs); }
    if (B * R == 0) return res;
    cuda_ok(colinfer_sample(logits.data_ptr(), dt, mask_ptr, mask_rows, W, &p, pos_ptr, pos_i64, u_ptr, out.data_ptr<int64_t>(),
                            want_stats ? reinterpret_cast<colinfer_row_stats*>(rs.data_ptr()) : nullptr,
                            want_status ? st.data_ptr<int32_t>() : nullptr, (int)B, (int)R, (int)V, (int)flags, stream()), "draw");
    return res;
}

// spec_accept(pred, tok, stop_ids, active) -> (out_tok, n) (engine/spec/mtp.py:406-415, 422-423)
std::vector<at::Tensor> spec_accept(const at::Tensor& pred, const at::Tensor& tok, const Opt& stop_ids, const Opt& active) {
    check(pred, at::kLong, "pred"); check(tok, at::kLong, "tok");
    TORCH_CHECK(pred.dim() == 2 && pred.sizes() == tok.sizes(), "pred, tok [B, k+1]");
    const int64_t B = pred.size(0), k1 = pred.size(1);
    int S = 0;
    if (stop_ids) { check(*stop_ids, at::kLong, "stop_ids"); TORCH_CHECK(stop_ids->dim() == 2 && stop_ids->size(0) == B, "stop_ids [B, S]"); S = (int)stop_ids->size(1); }
    if (active) { check(*active, at::kInt, "active"); TORCH_CHECK(active->numel() == B, "active [B]"); }
    c10::cuda::CUDAGuard guard(pred.device());
    at::Tensor out_tok = at::empty({B, k1}, pred.options()), n = at::empty({B}, pred.options().dtype(at::kInt));
    cuda_ok(colinfer_spec_accept(pred.data_ptr<int64_t>(), tok.data_ptr<int64_t>(), S ? stop_ids->data_ptr<int64_t>() : nullptr,
                                 active ? active->data_ptr<int32_t>() : nullptr, out_tok.data_ptr<int64_t>(), n.data_ptr<int32_t>(),
                                 (int)B, (int)k1, S, stream()), "spec_accept");
    return {out_tok, n};
}

// spec_advance(out_tok, n, y, history?, hist_len?, pos?): the scheduler's bookkeeping after a cycle, in place on the device
// (engine/runtime/scheduler.py:635-641)
void spec_advance(const at::Tensor& out_tok, const at::Tensor& n, at::Tensor y, const Opt& history, const Opt& hist_len, const Opt& pos) {
    check(out_tok, at::kLong, "out_tok"); check(n, at::kInt, "n"); check(y, at::kLong, "y");
    TORCH_CHECK(out_tok.dim() == 2 && n.numel() == out_tok.size(0) && y.numel() == out_tok.size(0), "out_tok [B, k+1], n [B], y [B]");
    const int64_t B = out_tok.size(0), k1 = out_tok.size(1);
    int64_t H = 0;
    if (history) {
        check(*history, at::kInt, "history");
        TORCH_CHECK(hist_len.has_value(), "hist_len is required with history");
        check(*hist_len, at::kInt, "hist_len");
        TORCH_CHECK(history->dim() == 2 && history->size(0) == B && hist_len->numel() == B, "history [B, H], hist_len [B]");
        H = history->size(1);
    }
    if (pos) { check(*pos, at::kLong, "pos"); TORCH_CHECK(pos->numel() == B, "pos [B]"); }
    c10::cuda::CUDAGuard guard(out_tok.device());
    cuda_ok(colinfer_spec_advance(out_tok.data_ptr<int64_t>(), n.data_ptr<int32_t>(), y.data_ptr<int64_t>(),
                                  H ? history->data_ptr<int32_t>() : nullptr, H ? hist_len->data_ptr<int32_t>() : nullptr,
                                  pos ? pos->data_ptr<int64_t>() : nullptr, (int)B, (int)k1, (int)H, stream()), "spec_advance");
}

// lowrank_draft(ap, g2, w, vocab_ids?, sf?, gs, n_cands, ctas_per_slot, scratch, want_index) -> ids, p (+ idx, ex): the greedy
// draft of the low-rank heads in one launch (engine/spec/mtp.py:301-309, engine/spec/mtp4.py:416-423).  scratch: a uint8
// tensor of colinfer_draft_pick_scratch_bytes(N) bytes that is zero-filled before its first use (the mirror keeps it).
std::vector<at::Tensor> lowrank_draft(const at::Tensor& ap, const at::Tensor& g2, const at::Tensor& w, const Opt& vocab_ids, const Opt& sf,
                                      double gs, int64_t n_cands, int64_t ctas_per_slot, at::Tensor scratch, bool want_index) {
    check(ap, at::kFloat, "ap"); check(g2, at::kBFloat16, "g2");
    TORCH_CHECK(ap.dim() == 2 && g2.dim() == 2 && g2.size(0) == ap.size(0), "ap [N, Vd], g2 [N, K]");
    const int64_t N = ap.size(0), Vd = ap.size(1), K = g2.size(1);
    const bool fp4 = sf.has_value();
    if (fp4) {
        check(w, at::kByte, "w");
        TORCH_CHECK(sf->is_cuda() && sf->is_contiguous() && (sf->scalar_type() == at::kByte || sf->scalar_type() == at::kFloat8_e4m3fn),
                    "sf must be a contiguous CUDA tensor of uint8 or float8_e4m3fn");
        TORCH_CHECK(w.dim() == 2 && w.size(1) * 2 == K && K % 16 == 0 && sf->numel() == w.size(0) * (K / 16),
                    "w [rows, K / 2], sf [rows, K / 16] with K % 16 == 0");
    } else {
        check(w, at::kBFloat16, "w");
        TORCH_CHECK(w.dim() == 2 && w.size(1) == K && K % 8 == 0, "w [rows, K] with K % 8 == 0");
    }
    if (vocab_ids) { check(*vocab_ids, at::kLong, "vocab_ids"); TORCH_CHECK(vocab_ids->numel() == Vd, "vocab_ids [Vd]"); }
    TORCH_CHECK(n_cands >= 1 && n_cands <= std::min<int64_t>(Vd, 1024), "n_cands must lie in 1 .. min(Vd, 1024)");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(g2.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(w.data_ptr()) % 16 == 0,
                "g2 and w must be 16-byte aligned");
    check(scratch, at::kByte, "scratch");
    TORCH_CHECK(scratch.numel() >= colinfer_draft_pick_scratch_bytes((int)N), "scratch is too small");
    c10::cuda::CUDAGuard guard(ap.device());
    at::Tensor ids = at::empty({N}, ap.options().dtype(at::kLong)), p = at::empty({N}, ap.options());
    std::vector<at::Tensor> res{ids, p};
    at::Tensor idx, ex;
    if (want_index) { idx = at::empty({N}, ap.options().dtype(at::kInt)); ex = at::empty({N}, ap.options()); res.push_back(idx); res.push_back(ex); }
    if (N == 0) return res;
    cuda_ok(colinfer_draft_pick(ap.data_ptr<float>(), g2.data_ptr(), w.data_ptr(), fp4 ? sf->data_ptr() : nullptr, fp4 ? (float)gs : 1.0f,
                                fp4 ? COLINFER_W_NVFP4 : COLINFER_W_BF16, vocab_ids ? vocab_ids->data_ptr<int64_t>() : nullptr,
                                ids.data_ptr<int64_t>(), p.data_ptr<float>(), want_index ? idx.data_ptr<int32_t>() : nullptr,
                                want_index ? ex.data_ptr<float>() : nullptr, (int)N, (int)Vd, (int)K, (int)n_cands, w.size(0),
                                (int)ctas_per_slot, scratch.data_ptr(), scratch.numel(), stream()), "draft_pick");
    return res;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "Thin PyTorch extension over libcolinfer_b200.so (the B200 logits -> token path)";
    m.def("philox_uniform", &philox_uniform, "out[b, i] = U(0, 1] of Philox4x32-10 keyed by seed[b] at counter offset[b] + i (in place)");
    m.def("apply_mask", &apply_mask, "logits with every token whose mask bit is clear set to -inf (a new tensor)");
    m.def("draw", &draw, "fused penalties + mask + temperature + min-p / top-k / top-p + argmax or seeded draw: one launch");
    m.def("spec_accept", &spec_accept, "exact-match accept, bonus token and stop cut of the speculative cycle");
    m.def("spec_advance", &spec_advance, "the bookkeeping after a cycle, in place on the device");
    m.def("lowrank_draft", &lowrank_draft, "the greedy draft of the low-rank heads: top candidates, exact rescoring, argmax, probability: one launch");
}
