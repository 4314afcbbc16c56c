"""Logprobs of emitted tokens, the mirror of Scheduler._logprobs (engine/runtime/scheduler.py:714-722).

The reference runs log_softmax over the raw rows, gathers the emitted tokens and takes topk: three full-vocabulary
passes and an [r, V] temporary per call.  Here one CUDA kernel reads each row once (colinfer_logprobs)."""
from __future__ import annotations

import torch

from .. import _lib
from ..kernels import _stream, check_tensor

MAX_TOP = 32


def logprobs_tensors(rows: torch.Tensor, toks: torch.Tensor, n_top: int):
    """rows [r, V] fp32 / bf16 raw logits (CUDA, contiguous), toks [r] int64 -> (chosen fp32 [r], top_ids int64
    [r, n_top], top_lp fp32 [r, n_top]) on the device; nothing is synchronised."""
    if rows.dim() != 2:
        raise RuntimeError("rows [r, V]")
    check_tensor(rows, None, "rows")
    check_tensor(toks, torch.int64, "toks")
    r, V = rows.shape
    if toks.numel() != r:
        raise RuntimeError("one token per row")
    if not 0 <= n_top <= min(MAX_TOP, V):
        raise RuntimeError(f"n_top in [0, {min(MAX_TOP, V)}]")
    dt = _lib.F32 if rows.dtype == torch.float32 else _lib.BF16
    if rows.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("rows must be float32 or bfloat16")
    chosen = torch.empty(r, dtype=torch.float32, device=rows.device)
    top_ids = torch.empty(r, n_top, dtype=torch.int64, device=rows.device)
    top_lp = torch.empty(r, n_top, dtype=torch.float32, device=rows.device)
    if r:
        _lib.check(_lib.lib().colinfer_logprobs(rows.data_ptr(), dt, toks.data_ptr(), n_top, chosen.data_ptr(),
                                                top_ids.data_ptr() if n_top else None,
                                                top_lp.data_ptr() if n_top else None, r, V, _stream()), "logprobs")
    return chosen, top_ids, top_lp


def logprobs(rows: torch.Tensor, toks: list[int], n_top: int):
    """rows [r, V] raw logits of the positions that produced toks -> [(logprob, [(id, logprob) x n_top])], the
    reference's return value (engine/runtime/scheduler.py:714-722)."""
    t = torch.tensor(toks, dtype=torch.int64, device=rows.device)
    chosen, ids, lps = logprobs_tensors(rows.contiguous(), t, n_top)
    chosen, ids, lps = chosen.tolist(), ids.tolist(), lps.tolist()
    return [(chosen[i], list(zip(ids[i], lps[i]))) for i in range(len(toks))]
