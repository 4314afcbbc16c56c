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
        check_tensor(seed, torch.int64, "seed")
        check_tensor(offset, torch.int64, "offset")
        check_tensor(out, torch.float32, "out")
        if out.dim() != 2 or seed.numel() != out.size(0) or offset.numel() != out.size(0):
            raise RuntimeError("out [B, n], seed / offset [B]")
        _lib.check(_lib.lib().colinfer_philox_uniform(seed.data_ptr(), offset.data_ptr(), out.data_ptr(),
                                                      out.size(0), out.size(1), _stream()), "philox_uniform")


_ops = None


def ops() -> _Ops:
    global _ops
    if _ops is None:
        _lib.lib()  # fail loudly here if the library has not been built
        _ops = _Ops()
    return _ops
