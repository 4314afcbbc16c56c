"""Mirror of the reference's engine/spec/accept.py: processed_probs, inverse_cdf, draw -- same names, argument
meaning and return values, computed by the fused sm_100a kernels.

draw() is the hot call: where the reference loops over slots in Python and issues ~25 torch / FlashInfer launches per
slot (accept.py:43-52), this issues ONE launch for all B x R rows, reads every logit from HBM once, and takes the
position from device memory (graph-capturable, no host sync).  Keyword-only extensions (absent in the reference, all
optional): mask= fuses apply_mask, u= supplies explicit uniforms, status= returns per-row status words.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from ..kernels import _stream, check_tensor


def _params_struct(p, B: int) -> _lib.SamplerParamsC:
    s = _lib.SamplerParamsC()
    for name, dt in (("temperature", torch.float32), ("top_k", torch.int32), ("top_p", torch.float32),
                     ("log_min_p", torch.float32)):
        t = getattr(p, name)
        check_tensor(t, dt, name)
        if t.numel() != B:
            raise RuntimeError(f"{name} must have one entry per slot ({B}), got {t.numel()}")
        setattr(s, name, t.data_ptr())
    seed = getattr(p, "seed", None)
    if seed is not None:
        check_tensor(seed, torch.int64, "seed")
        if seed.numel() != B:
            raise RuntimeError(f"seed must have one entry per slot ({B})")
        s.seed = seed.data_ptr()
    for name in ("repetition_penalty", "presence_penalty", "frequency_penalty"):
        t = getattr(p, name, None)
        if t is not None:
            check_tensor(t, torch.float32, name)
            if t.numel() != B:
                raise RuntimeError(f"{name} must have one entry per slot ({B})")
            setattr(s, name, t.data_ptr())
    hist = getattr(p, "history", None)
    if hist is not None:
        check_tensor(hist, torch.int32, "history")
        if hist.dim() != 2 or hist.size(0) != B:
            raise RuntimeError("history must be int32 [B, H]")
        s.history = hist.data_ptr()
        s.hist_stride = hist.size(1)
        hl = getattr(p, "hist_len", None)
        if hl is not None:
            check_tensor(hl, torch.int32, "hist_len")
            if hl.numel() != B:
                raise RuntimeError("hist_len must be int32 [B]")
            s.hist_len = hl.data_ptr()
    return s


def _dtype_code(logits: torch.Tensor) -> int:
    if logits.dtype == torch.float32:
        return _lib.F32
    if logits.dtype == torch.bfloat16:
        return _lib.BF16
    raise RuntimeError(f"logits must be float32 or bfloat16, got {logits.dtype}")


def processed_probs(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                    log_min_p: torch.Tensor) -> torch.Tensor:
    """logits [R, V] fp32 (rows of one request) -> renormalised probabilities [R, V] after the filters.
    temperature / top_k / top_p / log_min_p: 1-element device tensors (the slot's parameters).
    (engine/spec/accept.py:23-33)"""
    check_tensor(logits, torch.float32, "logits")
    if logits.dim() != 2:
        raise RuntimeError("logits [R, V]")
    for t, dt, name in ((temperature, torch.float32, "temperature"), (top_k, torch.int32, "top_k"),
                        (top_p, torch.float32, "top_p"), (log_min_p, torch.float32, "log_min_p")):
        check_tensor(t, dt, name)
        if t.numel() != 1:
            raise RuntimeError(f"{name} must have 1 element")
    R, V = logits.shape
    out = torch.empty_like(logits)
    scratch = torch.empty(max(R, 1) * _lib.ROW_STATS_BYTES, dtype=torch.uint8, device=logits.device)
    _lib.check(_lib.lib().colinfer_processed_probs(logits.data_ptr(), temperature.data_ptr(), top_k.data_ptr(),
                                                   top_p.data_ptr(), log_min_p.data_ptr(), out.data_ptr(),
                                                   scratch.data_ptr(), R, V, _stream()), "processed_probs")
    return out


def inverse_cdf(P: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """P [R, V] probabilities, u [R] uniforms in (0, 1] -> [R] int64: the first index whose CDF reaches u
    (never a zero-probability token).  (engine/spec/accept.py:36-40)"""
    check_tensor(P, torch.float32, "P")
    if P.dim() != 2:
        raise RuntimeError("P [R, V]")
    u = u.contiguous()
    check_tensor(u, torch.float32, "u")
    if u.numel() != P.size(0):
        raise RuntimeError("u [R]")
    out = torch.empty(P.size(0), dtype=torch.int64, device=P.device)
    _lib.check(_lib.lib().colinfer_inverse_cdf(P.data_ptr(), u.data_ptr(), out.data_ptr(), P.size(0), P.size(1),
                                               _stream()), "inverse_cdf")
    return out


def draw(logits: torch.Tensor, p, pos: torch.Tensor, *, mask: torch.Tensor | None = None,
         u: torch.Tensor | None = None, status: bool = False, stats: bool = False, flags: int = 0):
    """logits [B, R, V] fp32 (or bf16): row r of slot b predicts the token at position pos[b] + r.
    p: SamplerParams for the B slots.  Returns the sampled tokens [B, R] int64 (argmax for slots with temperature 0).
    (engine/spec/accept.py:43-52)

    mask [B, R, W] int32: grammar bitmask applied inside the same pass (what apply_mask would do first).  Besides a CUDA
    tensor, a pinned host tensor is taken as it is (RowMasks(zero_copy=True)): the kernel reads it over PCIe.
    u [B, R] fp32: explicit uniforms in (0, 1] instead of Philox(seed, pos).
    status / stats: also return the per-row status words int32 [B, R] / the raw row statistics uint8 [B, R, 32].
    flags: COLINFER_* flag bits of colinfer_sample (kernel choice, test flags)."""
    ext = _lib.ext()
    if ext is not None:
        # the thin C++ extension: the same checks (TORCH_CHECK), outputs from torch's allocator, torch's current stream
        flags = int(flags)
        if not flags & _lib.KERNEL_MASK:
            flags |= _lib.default_kernel_flags
        g = lambda name: getattr(p, name, None)  # noqa: E731
        res = ext.draw(logits, p.temperature, p.top_k, p.top_p, p.log_min_p, g("seed"), g("repetition_penalty"),
                       g("presence_penalty"), g("frequency_penalty"), g("history"), g("hist_len"), pos if u is None else None,
                       mask, u, bool(status), bool(stats), flags)
        return res[0] if len(res) == 1 else tuple(res)
    if logits.dim() != 3:
        raise RuntimeError("logits [B, R, V]")
    check_tensor(logits, None, "logits")
    dt = _dtype_code(logits)
    B, R, V = logits.shape
    ps = _params_struct(p, B)
    mask_ptr, mask_rows, W = None, 0, 0
    if mask is not None:
        if not (isinstance(mask, torch.Tensor) and not mask.is_cuda and mask.is_pinned() and mask.is_contiguous()
                and mask.dtype == torch.int32):
            check_tensor(mask, torch.int32, "mask")
        if mask.dim() != 3 or mask.size(0) != B or mask.size(1) < R or mask.size(2) < (V + 31) // 32:
            raise RuntimeError("mask [B, R, W] int32 with W >= ceil(V / 32)")
        mask_ptr, mask_rows, W = mask.data_ptr(), mask.size(1), mask.size(2)
    pos_ptr, pos_i64, u_ptr = None, 0, None
    if u is not None:
        check_tensor(u, torch.float32, "u")
        if u.numel() != B * R:
            raise RuntimeError("u [B, R]")
        u_ptr = u.data_ptr()
    else:
        if pos.dtype not in (torch.int32, torch.int64):
            raise RuntimeError("pos must be int32 or int64")
        check_tensor(pos, None, "pos")
        if pos.numel() != B:
            raise RuntimeError("pos [B]")
        if getattr(p, "seed", None) is None:
            raise RuntimeError("SamplerParams.seed is required when no uniforms are passed")
        pos_ptr, pos_i64 = pos.data_ptr(), int(pos.dtype == torch.int64)
    out = torch.empty(B, R, dtype=torch.int64, device=logits.device)
    if B * R == 0 and not (status or stats):
        return out
    st = torch.empty(B, R, dtype=torch.int32, device=logits.device) if status else None
    rs = torch.empty(B, R, _lib.ROW_STATS_BYTES, dtype=torch.uint8, device=logits.device) if stats else None
    flags = int(flags)
    if not flags & _lib.KERNEL_MASK:
        flags |= _lib.default_kernel_flags
    _lib.check(_lib.lib().colinfer_sample(logits.data_ptr(), dt, mask_ptr, mask_rows, W, C.byref(ps), pos_ptr, pos_i64,
                                          u_ptr, out.data_ptr(), rs.data_ptr() if stats else None,
                                          st.data_ptr() if status else None, B, R, V, flags, _stream()), "draw")
    if status or stats:
        return (out,) + ((st,) if status else ()) + ((rs,) if stats else ())
    return out


def processed_probs_noalloc(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                            log_min_p: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """processed_probs into a caller-provided `out` [R, V] without any allocation: the per-row scratch is a fixed array
    inside the CUDA library (at most 4096 rows; calls that overlap on the GPU race on it).  For hosts that may not
    allocate at call time; not part of the reference's interface."""
    check_tensor(logits, torch.float32, "logits")
    check_tensor(out, torch.float32, "out")
    if logits.dim() != 2 or out.shape != logits.shape:
        raise RuntimeError("logits, out [R, V]")
    for t, dt, name in ((temperature, torch.float32, "temperature"), (top_k, torch.int32, "top_k"),
                        (top_p, torch.float32, "top_p"), (log_min_p, torch.float32, "log_min_p")):
        check_tensor(t, dt, name)
        if t.numel() != 1:
            raise RuntimeError(f"{name} must have 1 element")
    R, V = logits.shape
    _lib.check(_lib.lib().colinfer_processed_probs_noalloc(logits.data_ptr(), temperature.data_ptr(), top_k.data_ptr(),
                                                           top_p.data_ptr(), log_min_p.data_ptr(), out.data_ptr(), R, V,
                                                           _stream()), "processed_probs_noalloc")
    return out
