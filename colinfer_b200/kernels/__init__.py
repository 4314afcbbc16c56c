"""Mirror of the reference's engine/kernels: ops() returns an object with the native operators of this path.

Only philox_uniform is a native operator of this path in the reference (csrc/sampling.cu:25-35, bound at
csrc/bindings.cpp:538-544, 637); the same name, argument order and error behaviour are kept.
"""
from __future__ import annotations

import torch

from .. import _lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check_tensor(t: torch.Tensor, dtype, name: str) -> None:
    """The reference's CHECK_CUDA_TENSOR: a contiguous CUDA tensor of the given dtype, else RuntimeError."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (this path has no CPU implementation)")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")


class _Ops:
    @staticmethod
    def philox_uniform(seed: torch.Tensor, offset: torch.Tensor, out: torch.Tensor) -> None:
        """out fp32 [B, n] = per-slot seeded uniforms in (0, 1] at counters offset[b] + i (seed, offset: int64 [B]).
        Writes in place; the caller allocates out."""
        ext = _lib.ext()
        if ext is not None:
            return ext.philox_uniform(seed, offset, out)
        check_tensor(seed, torch.int64, "seed")
        check_tensor(offset, torch.int64, "offset")
        check_tensor(out, torch.float32, "out")
        if out.dim() != 2 or seed.numel() != out.size(0) or offset.numel() != out.size(0):
            raise RuntimeError("out [B, n], seed / offset [B]")
        _lib.check(_lib.lib().colinfer_philox_uniform(seed.data_ptr(), offset.data_ptr(), out.data_ptr(),
                                                      out.size(0), out.size(1), _stream()), "philox_uniform")

    @staticmethod
    def rescore_bf16(x: torch.Tensor, w: torch.Tensor, cand: torch.Tensor) -> torch.Tensor:
        """Exact logits of candidate rows of a BF16 matrix: x bf16 [B, K], w bf16 [V, K], cand int64 [B, NC] -> fp32
        [B, NC] (csrc/bindings.cpp:561-572 of the reference: same checks, same result bit for bit)."""
        check_tensor(x, torch.bfloat16, "x")
        check_tensor(w, torch.bfloat16, "w")
        check_tensor(cand, torch.int64, "cand")
        K = x.size(-1)
        B, NC = x.numel() // K, cand.size(-1)
        if w.dim() != 2 or w.size(1) != K or K % 8 or cand.numel() != B * NC:
            raise RuntimeError("x [B, K], w [V, K] with K % 8 == 0, cand [B, NC]")
        if x.data_ptr() % 16 or w.data_ptr() % 16:
            raise RuntimeError("x and w must be 16-byte aligned")
        out = torch.empty(B, NC, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().colinfer_rescore_bf16(x.data_ptr(), w.data_ptr(), cand.data_ptr(), out.data_ptr(), B, K, NC,
                                                    w.size(0), _stream()), "rescore_bf16")
        return out

    @staticmethod
    def rescore_nvfp4(x: torch.Tensor, w: torch.Tensor, sf: torch.Tensor, gs: float, cand: torch.Tensor) -> torch.Tensor:
        """Exact logits of candidate rows of an NVFP4 matrix: x bf16 [B, K], w uint8 [V, K / 2] (E2M1 pairs), sf [V, K / 16]
        E4M3 scales (uint8 or float8_e4m3fn), global scale gs, cand int64 [B, NC] -> fp32 [B, NC]
        (csrc/bindings.cpp:547-558)."""
        check_tensor(x, torch.bfloat16, "x")
        check_tensor(w, torch.uint8, "w")
        check_tensor(cand, torch.int64, "cand")
        if sf.dtype not in (torch.uint8, torch.float8_e4m3fn):
            raise RuntimeError("sf must be uint8 or float8_e4m3fn")
        check_tensor(sf, None, "sf")
        K = x.size(-1)
        B, NC = x.numel() // K, cand.size(-1)
        if w.dim() != 2 or w.size(1) * 2 != K or K % 16 or cand.numel() != B * NC or sf.numel() != w.size(0) * (K // 16):
            raise RuntimeError("x [B, K], w [V, K / 2], sf [V, K / 16] with K % 16 == 0, cand [B, NC]")
        if x.data_ptr() % 16 or w.data_ptr() % 16:
            raise RuntimeError("x and w must be 16-byte aligned")
        out = torch.empty(B, NC, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().colinfer_rescore_nvfp4(x.data_ptr(), w.data_ptr(), sf.data_ptr(), float(gs), cand.data_ptr(),
                                                     out.data_ptr(), B, K, NC, w.size(0), _stream()), "rescore_nvfp4")
        return out


_ops = None


def ops() -> _Ops:
    global _ops
    if _ops is None:
        _lib.lib()  # fail loudly here if the library has not been built
        _ops = _Ops()
    return _ops
