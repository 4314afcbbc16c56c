"""The speculative-verify step: exact-match accept with the stop cut (what the reference's cycle bodies do inline,
engine/spec/mtp.py:406-415, 422-423 and engine/spec/mtp4.py:538-547) and the rejection verify with the (p - q)+
residual resample (not in the reference)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from ..kernels import _stream, check_tensor
from .accept import _dtype_code, _params_struct


def spec_accept(pred: torch.Tensor, tok: torch.Tensor, stop_ids: torch.Tensor | None = None,
                active: torch.Tensor | None = None):
    """pred [B, k+1] int64: the target's own token at every verified row (argmax or draw()); tok [B, k+1] int64: the
    verified inputs (tok[:, 1:] are the drafts); stop_ids [B, S] int64 (-1 unused); active [B] int32.
    Returns (out_tok [B, k+1] int64, n [B] int32): n counts the emitted tokens (accepted drafts + 1; 0 for inactive
    slots), out_tok[:, :n-1] are the accepted drafts and out_tok[:, n-1] is the bonus token."""
    ext = _lib.ext()
    if ext is not None:
        out_tok, n = ext.spec_accept(pred, tok, stop_ids, active)
        return out_tok, n
    check_tensor(pred, torch.int64, "pred")
    check_tensor(tok, torch.int64, "tok")
    if pred.dim() != 2 or pred.shape != tok.shape:
        raise RuntimeError("pred, tok [B, k+1]")
    B, k1 = pred.shape
    S = 0
    if stop_ids is not None:
        check_tensor(stop_ids, torch.int64, "stop_ids")
        if stop_ids.dim() != 2 or stop_ids.size(0) != B:
            raise RuntimeError("stop_ids [B, S]")
        S = stop_ids.size(1)
    if active is not None:
        check_tensor(active, torch.int32, "active")
        if active.numel() != B:
            raise RuntimeError("active [B]")
    out_tok = torch.empty(B, k1, dtype=torch.int64, device=pred.device)
    n = torch.empty(B, dtype=torch.int32, device=pred.device)
    _lib.check(_lib.lib().colinfer_spec_accept(pred.data_ptr(), tok.data_ptr(),
                                               stop_ids.data_ptr() if S else None,
                                               active.data_ptr() if active is not None else None,
                                               out_tok.data_ptr(), n.data_ptr(), B, k1, S, _stream()), "spec_accept")
    return out_tok, n


def spec_advance(out_tok: torch.Tensor, n: torch.Tensor, y: torch.Tensor, history: torch.Tensor | None = None,
                 hist_len: torch.Tensor | None = None, pos: torch.Tensor | None = None) -> None:
    """The scheduler's bookkeeping after a cycle (engine/runtime/scheduler.py:635-641: `tokens.append(y); tokens += o[:-1];
    y = o[-1]`) without reading n back: in place, for every slot with n > 0, y int64 [B] and the accepted drafts are
    appended to history int32 [B, H] / hist_len int32 [B] (the most recent H ids are kept), y becomes the bonus token,
    pos int64 [B] moves on by n."""
    ext = _lib.ext()
    if ext is not None and hasattr(ext, "spec_advance"):
        ext.spec_advance(out_tok, n, y, history, hist_len, pos)
        return
    check_tensor(out_tok, torch.int64, "out_tok")
    check_tensor(n, torch.int32, "n")
    check_tensor(y, torch.int64, "y")
    if out_tok.dim() != 2 or n.numel() != out_tok.size(0) or y.numel() != out_tok.size(0):
        raise RuntimeError("out_tok [B, k+1], n [B], y [B]")
    B, k1 = out_tok.shape
    H = 0
    if history is not None:
        check_tensor(history, torch.int32, "history")
        if hist_len is None:
            raise RuntimeError("hist_len is required with history")
        check_tensor(hist_len, torch.int32, "hist_len")
        if history.dim() != 2 or history.size(0) != B or hist_len.numel() != B:
            raise RuntimeError("history [B, H], hist_len [B]")
        H = history.size(1)
    if pos is not None:
        check_tensor(pos, torch.int64, "pos")
        if pos.numel() != B:
            raise RuntimeError("pos [B]")
    _lib.check(_lib.lib().colinfer_spec_advance(out_tok.data_ptr(), n.data_ptr(), y.data_ptr(),
                                                history.data_ptr() if H else None, hist_len.data_ptr() if H else None,
                                                pos.data_ptr() if pos is not None else None, B, k1, H, _stream()), "spec_advance")


def spec_verify(target_logits: torch.Tensor, draft_logits: torch.Tensor, draft_ids: torch.Tensor, p,
                ua: torch.Tensor, us: torch.Tensor, mask: torch.Tensor | None = None):
    """Rejection verify.  target_logits [B, k+1, V], draft_logits [B, k, V] (fp32 or bf16), draft_ids [B, k] int64,
    p: SamplerParams (its penalties, if any, apply to every row of both models with the slot's history), ua [B, k] accept
    uniforms, us [B, k+1] sampling uniforms, mask [B, k+1, W] int32 applied to both models' rows.  Accept draft i iff ua_i * q_i(d_i) <= p_i(d_i); at the first
    rejection emit a draw from normalize(max(p - q, 0)); with no rejection emit a draw from p_k.  temperature <= 0:
    accept while the draft equals the target's argmax.  Returns (out_tok [B, k+1] int64 padded with -1, n [B] int32)."""
    check_tensor(target_logits, None, "target_logits")
    check_tensor(draft_logits, target_logits.dtype, "draft_logits")
    dt = _dtype_code(target_logits)
    if target_logits.dim() != 3 or draft_logits.dim() != 3:
        raise RuntimeError("target_logits [B, k+1, V], draft_logits [B, k, V]")
    B, k1, V = target_logits.shape
    k = k1 - 1
    if k < 1 or tuple(draft_logits.shape) != (B, k, V):
        raise RuntimeError("draft_logits must be [B, k, V] with k >= 1")
    check_tensor(draft_ids, torch.int64, "draft_ids")
    check_tensor(ua, torch.float32, "ua")
    check_tensor(us, torch.float32, "us")
    if draft_ids.numel() != B * k or ua.numel() != B * k or us.numel() != B * k1:
        raise RuntimeError("draft_ids, ua [B, k]; us [B, k+1]")
    ps = _params_struct(p, B)
    mask_ptr, W = None, 0
    if mask is not None:
        check_tensor(mask, torch.int32, "mask")
        if mask.dim() != 3 or mask.size(0) != B or mask.size(1) != k1 or mask.size(2) < (V + 31) // 32:
            raise RuntimeError("mask [B, k+1, W]")
        mask_ptr, W = mask.data_ptr(), mask.size(2)
    L = _lib.lib()
    dev = target_logits.device
    stats = torch.empty(L.colinfer_spec_verify_stats_bytes(B, k), dtype=torch.uint8, device=dev)
    ids = torch.empty(B, k1, dtype=torch.int64, device=dev)
    out_tok = torch.empty(B, k1, dtype=torch.int64, device=dev)
    n = torch.empty(B, dtype=torch.int32, device=dev)
    _lib.check(L.colinfer_spec_verify(target_logits.data_ptr(), draft_logits.data_ptr(), dt, mask_ptr, W, C.byref(ps),
                                      draft_ids.data_ptr(), ua.data_ptr(), us.data_ptr(), out_tok.data_ptr(),
                                      n.data_ptr(), stats.data_ptr(), ids.data_ptr(), B, k, V, _stream()), "spec_verify")
    return out_tok, n
