"""The reference's torch path for logits -> token, restated so that it runs on host cores.  TEST / BASELINE
INFRASTRUCTURE ONLY: the benchmark times it as the CPU baseline; the product never imports it.

It follows the reference's order of torch operations (engine/runtime/sampler.py:50-56 for the mask;
engine/spec/accept.py:23-52 for temperature, min-p, softmax, top-k, top-p, cumsum and the inverse-CDF count), in fp32,
multi-threaded by torch's intra-op pool, vectorised over rows where the reference loops over slots in Python.  The two
FlashInfer calls (GPU only) are replaced by sort-based thresholds with the same kept sets (every probability >= the
k-th largest; every probability >= the value at which the descending cumulative mass reaches top_p).  Penalties (absent
in the reference) use the bincount formulation of this project's definition.  Uniforms come from the numpy Philox of
oracle.py (negligible cost).
"""
from __future__ import annotations

import numpy as np
import torch

from . import oracle as O


def apply_mask(logits: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """[N, V] fp32, [N, W] int32 -> masked copy (bit t % 32 of word t // 32)."""
    N, V = logits.shape
    shifts = torch.arange(32, dtype=torch.int32)
    bits = ((mask[:, :, None] >> shifts) & 1).reshape(N, -1)[:, :V]
    return logits.masked_fill(bits == 0, float("-inf"))


def penalties(logits: torch.Tensor, history: torch.Tensor, hist_len: torch.Tensor, rep, pres, freq) -> torch.Tensor:
    N, V = logits.shape
    H = history.shape[1]
    valid = (torch.arange(H)[None, :] < hist_len[:, None]) & (history >= 0) & (history < V)
    counts = torch.zeros(N, V + 1, dtype=torch.float32)
    counts.scatter_add_(1, torch.where(valid, history.long(), torch.full_like(history, V).long()), valid.float())
    counts = counts[:, :V]
    seen = counts > 0
    rep, pres, freq = rep[:, None], pres[:, None], freq[:, None]
    scaled = torch.where(logits > 0, logits / rep, logits * rep)
    out = torch.where(seen, scaled, logits)
    out = out - freq * counts
    return out - pres * seen.float()


def processed_probs(logits, temperature, top_k, top_p, log_min_p):
    """[N, V] rows with per-row parameters [N] -> renormalised probabilities [N, V]."""
    N, V = logits.shape
    z = logits / temperature.clamp_min(1e-6)[:, None]
    z = z.masked_fill(z < z.amax(-1, keepdim=True) + log_min_p[:, None], float("-inf"))
    p = torch.softmax(z, -1)
    srt, _ = torch.sort(p, -1, descending=True)
    kth = srt.gather(1, (top_k.long().clamp(1, V) - 1)[:, None])
    p = torch.where(p >= kth, p, torch.zeros_like(p))
    p = p / p.sum(-1, keepdim=True)
    srt, _ = torch.sort(p, -1, descending=True)
    cum = srt.cumsum(-1)
    reach = (cum >= (top_p[:, None] * cum[:, -1:])).int().argmax(-1)
    piv = srt.gather(1, reach[:, None])
    piv = torch.where(top_p[:, None] >= 1.0, torch.zeros_like(piv), piv)
    p = torch.where(p >= piv, p, torch.zeros_like(p))
    return p / p.sum(-1, keepdim=True)


def inverse_cdf(P, u):
    c = P.cumsum(-1)
    return (c < (u * c[:, -1])[:, None]).sum(-1).clamp_max(P.shape[-1] - 1)


def draw(logits, params, pos=None, mask=None, u=None, chunk: int = 32):
    """logits [B, R, V] (fp32 or bf16) CPU tensor; params: dict of CPU tensors [B]; returns int64 [B, R]."""
    B, R, V = logits.shape
    if u is None:
        u = torch.from_numpy(O.philox_uniform(params["seed"].numpy(), pos.numpy().astype(np.int64), R))
    out = torch.empty(B, R, dtype=torch.int64)
    rep = lambda t: t.repeat_interleave(R)  # noqa: E731
    flat = logits.reshape(B * R, V)
    uf = u.reshape(-1)
    for lo in range(0, B * R, chunk):
        hi = min(lo + chunk, B * R)
        slot = torch.arange(lo, hi) // R
        x = flat[lo:hi].float()
        if "history" in params:
            x = penalties(x, params["history"][slot], params["hist_len"][slot], params["repetition_penalty"][slot],
                          params["presence_penalty"][slot], params["frequency_penalty"][slot])
        if mask is not None:
            x = apply_mask(x, mask.reshape(B * R, -1)[lo:hi])
        greedy = x.argmax(-1)
        T = params["temperature"][slot]
        P = processed_probs(x, T, params["top_k"][slot], params["top_p"][slot], params["log_min_p"][slot])
        tok = inverse_cdf(P, uf[lo:hi])
        out.view(-1)[lo:hi] = torch.where(T > 0, tok, greedy)
    return out
