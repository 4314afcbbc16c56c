"""Seeded synthetic inputs of the five benchmark configurations of the logits -> token path.

They stand in for real model logits and llguidance grammar masks (no checkpoint, tokenizer or dataset is needed or
used).  One generator per configuration, shared by the parity tests, the smoke check and the benchmark, so that every
implementation sees the same tensors.  Everything is produced on the CPU with torch.Generator seeds and returned as a
dict of CPU tensors; to_device() moves a dict to the GPU.
"""
from __future__ import annotations

import math

import numpy as np
import torch

V_QWEN = 151_936
V_LARGE = 262_144


def pack_mask(allowed: torch.Tensor) -> torch.Tensor:
    """bool [..., V] -> int32 [..., ceil(V / 32)]: token t is bit t % 32 of word t // 32 (the reference's convention,
    engine/runtime/grammar.py:28-30)."""
    a = allowed.numpy().astype(np.uint8)
    V = a.shape[-1]
    W = (V + 31) // 32
    pad = W * 32 - V
    if pad:
        a = np.concatenate([a, np.zeros(a.shape[:-1] + (pad,), np.uint8)], -1)
    words = np.packbits(a, axis=-1, bitorder="little").view(np.uint32).view(np.int32)
    return torch.from_numpy(words.reshape(a.shape[:-1] + (W,)).copy())


def open_unit(g: torch.Generator, *shape) -> torch.Tensor:
    """Uniforms in (0, 1] (the range of the engine's Philox uniforms)."""
    return (1.0 - torch.rand(*shape, generator=g, dtype=torch.float32)).clamp_min(1e-7)


def _params(B, V, temperature, top_k, top_p, min_p, seed=None):
    """Device-value arrays as SamplerParams.set stores them."""
    def arr(x, dt):
        t = torch.as_tensor(x, dtype=dt)
        return t.expand(B).clone() if t.dim() == 0 else t.clone()
    tk = arr(top_k, torch.int64)
    tk = torch.where((tk <= 0) | (tk >= V), torch.full_like(tk, V), tk).to(torch.int32)
    mp = arr(min_p, torch.float64)
    lmp = torch.where(mp > 0, mp.clamp_min(1e-300).log(), torch.full_like(mp, -math.inf)).to(torch.float32)
    return dict(temperature=arr(temperature, torch.float32), top_k=tk, top_p=arr(top_p, torch.float32), log_min_p=lmp,
                seed=arr(seed if seed is not None else torch.arange(B), torch.int64))


def config0(V: int = V_QWEN, H: int = 512):
    """Single-row sampling with penalties, temperature, top-k, top-p, min-p, one explicit uniform; plus greedy."""
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(1, 1, V, generator=g) * 2.0
    history = torch.randint(0, V, (1, H), generator=g, dtype=torch.int32)
    u = open_unit(torch.Generator().manual_seed(1), 1, 1)
    p = _params(1, V, 0.7, 50, 0.9, 0.05)
    p.update(repetition_penalty=torch.tensor([1.1]), presence_penalty=torch.tensor([0.5]),
             frequency_penalty=torch.tensor([0.2]), history=history, hist_len=torch.tensor([H], dtype=torch.int32))
    return dict(name="config0", logits=logits, params=p, u=u, pos=torch.tensor([17], dtype=torch.int32))


def config1(V: int = V_QWEN, allow: float = 0.02):
    """Grammar-constrained step: masked argmax and masked temperature-1.0 draw."""
    logits = torch.randn(1, 1, V, generator=torch.Generator().manual_seed(2)) * 2.0
    g = torch.Generator().manual_seed(3)
    allowed = torch.rand(1, 1, V, generator=g) < allow
    if not allowed.any():
        allowed[0, 0, int(torch.randint(0, V, (1,), generator=g))] = True
    u = open_unit(g, 1, 1)
    return dict(name="config1", logits=logits, mask=pack_mask(allowed), params=_params(1, V, 1.0, 0, 1.0, 0.0), u=u,
                pos=torch.tensor([5], dtype=torch.int32))


def config2(V: int = V_QWEN, k: int = 8, B: int = 1):
    """Speculative verify: target [B, k+1, V], draft = target[:, :k] + N(0, 0.5^2); uniforms for the draft's own
    sampling (ud), the accept tests (ua) and the target's sampling (us); temperature 0.8, top-p 0.95."""
    target = torch.randn(B, k + 1, V, generator=torch.Generator().manual_seed(4)) * 2.0
    draft = target[:, :k] + torch.randn(B, k, V, generator=torch.Generator().manual_seed(5)) * 0.5
    g = torch.Generator().manual_seed(6)
    return dict(name="config2", target=target, draft=draft.contiguous(), ud=open_unit(g, B, k), ua=open_unit(g, B, k),
                us=open_unit(g, B, k + 1), params=_params(B, V, 0.8, 0, 0.95, 0.0), k=k)


def config3(B: int, V: int = V_QWEN, H: int = 2048):
    """Batched sampling sweep: per-row histories, temperature U[0.5, 1.2], top_k in {0, 20, 100}, top_p U[0.8, 1.0],
    penalties (1.1, 0.5, 0.2), per-row seeds and positions."""
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(B, 1, V, generator=g) * 2.0
    history = torch.randint(0, V, (B, H), generator=g, dtype=torch.int32)
    temperature = 0.5 + 0.7 * torch.rand(B, generator=g)
    top_k = torch.tensor([0, 20, 100])[torch.randint(0, 3, (B,), generator=g)]
    top_p = 0.8 + 0.2 * torch.rand(B, generator=g)
    p = _params(B, V, temperature, top_k, top_p, 0.0, seed=torch.arange(B) * 7919 + 13)
    p.update(repetition_penalty=torch.full((B,), 1.1), presence_penalty=torch.full((B,), 0.5),
             frequency_penalty=torch.full((B,), 0.2), history=history,
             hist_len=torch.full((B,), H, dtype=torch.int32))
    pos = torch.randint(0, 4096, (B,), generator=g, dtype=torch.int32)
    return dict(name=f"config3_B{B}", logits=logits, params=p, pos=pos)


def config4(B: int = 512, V: int = V_LARGE, allow: float = 0.3, head: int = 100):
    """Large-vocabulary bf16 stress: heavy head (+8 on `head` tokens per row), 30 % grammar mask, top_k 1000,
    top_p 0.98, min_p 0.01, seeded draw."""
    g = torch.Generator().manual_seed(8)
    logits = torch.randn(B, 1, V, generator=g) * 2.0
    idx = torch.stack([torch.randperm(V, generator=g)[:head] for _ in range(B)])
    logits[:, 0].scatter_add_(1, idx, torch.full((B, head), 8.0))
    allowed = torch.rand(B, 1, V, generator=g) < allow
    p = _params(B, V, 1.0, 1000, 0.98, 0.01, seed=torch.arange(B) + 1000)
    pos = torch.randint(0, 4096, (B,), generator=g, dtype=torch.int32)
    return dict(name=f"config4_B{B}", logits=logits.to(torch.bfloat16), mask=pack_mask(allowed), params=p, pos=pos)


def to_device(x, device="cuda"):
    if isinstance(x, torch.Tensor):
        return x.to(device)
    if isinstance(x, dict):
        return {k: to_device(v, device) for k, v in x.items()}
    return x


def sampler_params(p: dict, V: int, device="cuda"):
    """A SamplerParams object holding the arrays of a workload's `params` dict."""
    from .runtime.sampler import SamplerParams
    B = p["temperature"].numel()
    sp = SamplerParams(B, V, device)
    for name in ("temperature", "top_k", "top_p", "log_min_p", "seed"):
        getattr(sp, name).copy_(p[name])
    for name in ("repetition_penalty", "presence_penalty", "frequency_penalty", "history", "hist_len"):
        if name in p:
            setattr(sp, name, p[name].to(device).contiguous())
    return sp


def bytes_per_row(V: int, elt: int, masked: bool, hist: int) -> int:
    """Algorithmic bytes of one sampled row: one read of every input plus the outputs."""
    return V * elt + (4 * ((V + 31) // 32) if masked else 0) + 4 * hist + 32 + 8
