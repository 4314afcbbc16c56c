"""The greedy draft of the low-rank draft heads (the step that feeds verify): the `if self.lr_B is not None` block of
MtpHead.draft (engine/spec/mtp.py:301-309) and Mtp4Head.draft (engine/spec/mtp4.py:416-423) as one launch."""
from __future__ import annotations

import torch

from .. import _lib
from ..kernels import _stream, check_tensor

LOWRANK_CANDS = 256     # engine/spec/mtp.py:70


_scratch_cache: dict = {}


def _scratch(dev: torch.device, nbytes: int) -> torch.Tensor:
    """The kernel's scratch (each slot's posted results and a counter that every call leaves at zero): zero-filled once
    and kept per device and stream; a call inside CUDA-graph capture takes a fresh zero-filled one from the graph's pool."""
    if torch.cuda.is_current_stream_capturing():
        return torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), torch.cuda.current_stream(dev).cuda_stream)
    buf = _scratch_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = _scratch_cache[key] = torch.zeros(max(nbytes, 1 << 16), dtype=torch.uint8, device=dev)
    return buf


def lowrank_draft(ap: torch.Tensor, g2: torch.Tensor, w: torch.Tensor, vocab_ids: torch.Tensor | None = None,
                  sf: torch.Tensor | None = None, gs: float | None = None, n_cands: int = LOWRANK_CANDS,
                  ctas_per_slot: int = 0, want_index: bool = False):
    """ap fp32 [N, Vd]: the low-rank head's approximate logits over the draft vocabulary (lr_B(lr_A(g2)) in the reference);
    g2 bf16 [N, K]: the drafter's outputs; w: the lm_head itself, bf16 [rows, K], or NVFP4 (uint8 [rows, K / 2] with sf
    [rows, K / 16] E4M3 scales and the global scale gs); vocab_ids int64 [Vd]: draft-vocabulary index -> token id = lm_head
    row.  Returns (ids int64 [N], p fp32 [N]) as the reference's block does: of the n_cands largest approximations the
    token with the largest exact logit, and exp(that logit - logsumexp(ap)) clamped to 1.  want_index: also the winning
    draft-vocabulary index (int32 [N]) and its exact logit (fp32 [N])."""
    ext = _lib.ext()
    if ext is not None and hasattr(ext, "lowrank_draft") and isinstance(ap, torch.Tensor) and ap.is_cuda and ap.dim() == 2:
        nbytes = _lib.lib().colinfer_draft_pick_scratch_bytes(ap.size(0))
        res = ext.lowrank_draft(ap, g2, w, vocab_ids, sf, float(gs) if gs is not None else 1.0, int(n_cands), int(ctas_per_slot),
                                _scratch(ap.device, max(int(nbytes), 1)), bool(want_index))
        return tuple(res)
    check_tensor(ap, torch.float32, "ap")
    check_tensor(g2, torch.bfloat16, "g2")
    if ap.dim() != 2 or g2.dim() != 2 or g2.size(0) != ap.size(0):
        raise RuntimeError("ap [N, Vd], g2 [N, K]")
    N, Vd = ap.shape
    K = g2.size(1)
    fp4 = sf is not None
    if fp4:
        check_tensor(w, torch.uint8, "w")
        if sf.dtype not in (torch.uint8, torch.float8_e4m3fn):
            raise RuntimeError("sf must be uint8 or float8_e4m3fn")
        check_tensor(sf, None, "sf")
        if gs is None or w.dim() != 2 or w.size(1) * 2 != K or K % 16 or sf.numel() != w.size(0) * (K // 16):
            raise RuntimeError("w [rows, K / 2], sf [rows, K / 16] with K % 16 == 0, and gs")
    else:
        check_tensor(w, torch.bfloat16, "w")
        if w.dim() != 2 or w.size(1) != K or K % 8:
            raise RuntimeError("w [rows, K] with K % 8 == 0")
    if vocab_ids is not None:
        check_tensor(vocab_ids, torch.int64, "vocab_ids")
        if vocab_ids.numel() != Vd:
            raise RuntimeError("vocab_ids [Vd]")
    if not 1 <= n_cands <= min(Vd, 1024):
        raise RuntimeError("n_cands must lie in 1 .. min(Vd, 1024)")
    if g2.data_ptr() % 16 or w.data_ptr() % 16:
        raise RuntimeError("g2 and w must be 16-byte aligned")
    dev = ap.device
    ids = torch.empty(N, dtype=torch.int64, device=dev)
    p = torch.empty(N, dtype=torch.float32, device=dev)
    idx = torch.empty(N, dtype=torch.int32, device=dev) if want_index else None
    ex = torch.empty(N, dtype=torch.float32, device=dev) if want_index else None
    if N:
        lib = _lib.lib()
        nbytes = lib.colinfer_draft_pick_scratch_bytes(N)
        scratch = _scratch(dev, nbytes)
        _lib.check(lib.colinfer_draft_pick(ap.data_ptr(), g2.data_ptr(), w.data_ptr(), sf.data_ptr() if fp4 else None,
                                           float(gs) if fp4 else 1.0, 1 if fp4 else 0,
                                           vocab_ids.data_ptr() if vocab_ids is not None else None, ids.data_ptr(), p.data_ptr(),
                                           idx.data_ptr() if want_index else None, ex.data_ptr() if want_index else None,
                                           N, Vd, K, n_cands, w.size(0), ctas_per_slot, scratch.data_ptr(), nbytes, _stream()),
                   "draft_pick")
    return (ids, p, idx, ex) if want_index else (ids, p)
