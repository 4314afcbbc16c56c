"""Mirror of the reference's engine/runtime/sampler.py: SamplerParams, apply_mask, sample.

Order (as in the reference): [penalties ->] [mask ->] temperature -> min-p (relative to the top token) -> top-k ->
top-p -> sample.  temperature == 0 selects the argmax for that slot, whatever the other parameters are.  The position
keys the randomness: the token at absolute position t is drawn by inverse CDF with u = Philox(seed, counter t).
"""
from __future__ import annotations

import math

import torch

from .. import _lib
from ..kernels import _stream, check_tensor
from ..spec.accept import draw


class SamplerParams:
    """Per-slot device buffers (engine/runtime/sampler.py:23-47).  The tensor attributes are part of the interface
    (callers fill them directly).  Added by this project, neutral by default: repetition_penalty, presence_penalty,
    frequency_penalty (fp32 [B]) and history (int32 [B, H]) / hist_len (int32 [B]), set with set_penalties() /
    set_history()."""

    _NAMES = ("temperature", "top_k", "top_p", "log_min_p", "seed")
    _PEN = ("repetition_penalty", "presence_penalty", "frequency_penalty")

    def __init__(self, batch: int, vocab: int, device):
        self.vocab = vocab
        self.temperature = torch.zeros(batch, dtype=torch.float32, device=device)
        self.top_k = torch.full((batch,), vocab, dtype=torch.int32, device=device)
        self.top_p = torch.ones(batch, dtype=torch.float32, device=device)
        self.log_min_p = torch.full((batch,), -math.inf, dtype=torch.float32, device=device)
        self.seed = torch.zeros(batch, dtype=torch.int64, device=device)
        self.repetition_penalty = None
        self.presence_penalty = None
        self.frequency_penalty = None
        self.history = None
        self.hist_len = None

    def view(self, lo: int, hi: int) -> "SamplerParams":
        """Parameters of slots [lo, hi), sharing this object's device buffers."""
        v = SamplerParams.__new__(SamplerParams)
        v.vocab = self.vocab
        for name in self._NAMES + self._PEN + ("history", "hist_len"):
            t = getattr(self, name)
            setattr(v, name, None if t is None else t[lo:hi])
        return v

    def set(self, slot: int, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, seed: int = 0):
        """top_k <= 0 disables top-k, and so does a top_k of at least the vocabulary (the buffer is int32); min_p <= 0
        disables min-p."""
        self.temperature[slot] = float(temperature)
        self.top_k[slot] = min(int(top_k), self.vocab) if top_k > 0 else self.vocab
        self.top_p[slot] = float(top_p)
        self.log_min_p[slot] = math.log(min_p) if min_p > 0 else -math.inf
        self.seed[slot] = int(seed)

    def _ensure_penalties(self):
        if self.repetition_penalty is None:
            dev, n = self.temperature.device, self.temperature.numel()
            self.repetition_penalty = torch.ones(n, dtype=torch.float32, device=dev)
            self.presence_penalty = torch.zeros(n, dtype=torch.float32, device=dev)
            self.frequency_penalty = torch.zeros(n, dtype=torch.float32, device=dev)

    def set_penalties(self, slot: int, repetition: float = 1.0, presence: float = 0.0, frequency: float = 0.0):
        """(1, 0, 0) is neutral: the row is left bit for bit as it was."""
        self._ensure_penalties()
        self.repetition_penalty[slot] = float(repetition)
        self.presence_penalty[slot] = float(presence)
        self.frequency_penalty[slot] = float(frequency)

    def set_history(self, history: torch.Tensor, hist_len: torch.Tensor | None = None):
        """history int32 [B, H]: the token ids each slot's penalties count; hist_len int32 [B] valid entries."""
        self.history, self.hist_len = history, hist_len


def apply_mask(logits: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """logits [B, R, V] fp32, mask [B, R, W] int32 token bitmask (token t: bit t % 32 of word t // 32) -> the logits
    with the tokens outside the mask at -inf, as a new tensor.  An all-ones mask leaves every value as it was.
    Graph-capturable.  (engine/runtime/sampler.py:50-56.)  draw(..., mask=mask) fuses this step instead."""
    check_tensor(logits, torch.float32, "logits")
    check_tensor(mask, torch.int32, "mask")
    if logits.dim() != 3 or mask.dim() != 3 or mask.shape[:2] != logits.shape[:2]:
        raise RuntimeError("logits [B, R, V], mask [B, R, W]")
    B, R, V = logits.shape
    if mask.size(2) < (V + 31) // 32:
        raise RuntimeError("mask has fewer than ceil(V / 32) words")
    out = torch.empty_like(logits)
    _lib.check(_lib.lib().colinfer_apply_mask(logits.data_ptr(), mask.data_ptr(), out.data_ptr(), B * R, V,
                                              mask.size(2), _stream()), "apply_mask")
    return out


def sample(logits: torch.Tensor, p: SamplerParams, pos: torch.Tensor, **kw) -> torch.Tensor:
    """logits [B, V] fp32 -> token ids [B] int64.  pos [B]: the position of the token being sampled (device).
    Graph-capturable (no host syncs).  (engine/runtime/sampler.py:59-62)"""
    if "mask" in kw and kw["mask"] is not None and kw["mask"].dim() == 2:
        kw["mask"] = kw["mask"][:, None]
    if "u" in kw and kw["u"] is not None and kw["u"].dim() == 1:
        kw["u"] = kw["u"][:, None]
    res = draw(logits[:, None], p, pos, **kw)
    if isinstance(res, tuple):
        return (res[0][:, 0],) + tuple(t[:, 0] for t in res[1:])
    return res[:, 0]
