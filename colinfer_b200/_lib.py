"""ctypes binding of libcolinfer_b200.so (the C ABI declared in include/colinfer_b200.h).

There is no CPU path: if the library is missing this module raises, and every op needs CUDA tensors.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcolinfer_b200.so")

F32, BF16 = 0, 1
ROW_DEGENERATE, ROW_TIMEOUT, ROW_HIST_SLOW, ROW_SELECT_SLOW = 1, 2, 4, 8
FORCE_DISTRIBUTION, TEST_MISS_BAND, TEST_DROP_COPY = 1, 0x4000, 0x2000
KERNEL_AUTO, KERNEL_STREAM = 0, 0x100
KERNEL_CLUSTER = {1: 0x200, 2: 0x300, 4: 0x400, 8: 0x500}
KERNEL_MASK = 0x700

# Kernel-choice bits that draw() adds to calls which do not choose themselves: a knob of this Python module for tests and
# benchmarks (the C library keeps no settings between calls).
default_kernel_flags = KERNEL_AUTO


def kernel_flags(cluster: int) -> int:
    """0: automatic, -1: the streaming kernel, 1 / 2 / 4 / 8: the cluster-resident kernel with that cluster size."""
    if cluster == 0:
        return KERNEL_AUTO
    if cluster == -1:
        return KERNEL_STREAM
    return KERNEL_CLUSTER[cluster]



class SamplerParamsC(C.Structure):
    _fields_ = [("temperature", C.c_void_p), ("top_k", C.c_void_p), ("top_p", C.c_void_p), ("log_min_p", C.c_void_p),
                ("seed", C.c_void_p), ("repetition_penalty", C.c_void_p), ("presence_penalty", C.c_void_p),
                ("frequency_penalty", C.c_void_p), ("history", C.c_void_p), ("hist_len", C.c_void_p),
                ("hist_stride", C.c_int32)]


class Geometry(C.Structure):
    _fields_ = [("cluster", C.c_int32), ("slice_elems", C.c_int32), ("smem_bytes", C.c_int32), ("bulk_copy", C.c_int32)]


ROW_STATS_BYTES = 32  # sizeof(colinfer_row_stats): 3 x f32, i32, i64, u64

# name -> (restype, argtypes); every symbol include/colinfer_b200.h declares
SIGNATURES = {
    "colinfer_philox_uniform": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "colinfer_apply_mask": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "colinfer_sample": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.POINTER(SamplerParamsC),
                                  C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "colinfer_processed_probs": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                           C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "colinfer_processed_probs_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                   C.c_int, C.c_int, C.c_void_p]),
    "colinfer_noalloc_max_rows": (C.c_int, []),
    "colinfer_inverse_cdf": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "colinfer_spec_accept": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "colinfer_spec_advance": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                        C.c_int, C.c_void_p]),
    "colinfer_spec_verify": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.POINTER(SamplerParamsC),
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "colinfer_logprobs": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_int, C.c_int, C.c_void_p]),
    "colinfer_rescore_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                        C.c_int64, C.c_void_p]),
    "colinfer_rescore_nvfp4": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_int,
                                         C.c_int, C.c_int, C.c_int64, C.c_void_p]),
    "colinfer_draft_pick_scratch_bytes": (C.c_int64, [C.c_int]),
    "colinfer_draft_pick": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int,
                                      C.c_void_p, C.c_int64, C.c_void_p]),
    "colinfer_spec_verify_stats_bytes": (C.c_int64, [C.c_int, C.c_int]),
    "colinfer_spec_verify_ids_bytes": (C.c_int64, [C.c_int, C.c_int]),
    "colinfer_sample_geometry": (C.c_int, [C.c_int, C.c_int, C.c_void_p, C.c_int, C.POINTER(Geometry)]),
    "colinfer_max_active_clusters": (C.c_int, [C.c_int, C.c_int]),
    "colinfer_gather_ids": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                      C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "colinfer_version": (C.c_int, []),
}

_lib = None
_ext = False            # False: not looked for yet; None: not built


def ext():
    """The thin PyTorch C++ extension over the C ABI (colinfer_b200/_colinfer_torch.so, built by build.build_torch_ext), or
    None when it has not been built: the Python mirrors then call the library through ctypes (same results)."""
    global _ext
    if _ext is False:
        _ext = None
        if os.path.exists(os.path.join(_HERE, "_colinfer_torch.so")) and os.environ.get("COLINFER_NO_TORCH_EXT") != "1":
            try:
                import importlib

                import torch  # noqa: F401  (its libraries must be loaded first)
                lib()
                _ext = importlib.import_module("colinfer_b200._colinfer_torch")
            except Exception:                              # noqa: BLE001  (an extension built for another torch: fall back to ctypes)
                _ext = None
    return _ext


def lib():
    """The loaded library.  Raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m colinfer_b200.build` "
                               "(there is no CPU or eager fallback for this path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(code: int, what: str) -> None:
    """cudaError_t -> RuntimeError, the exception type the reference's bindings raise (TORCH_CHECK)."""
    if code != 0:
        raise RuntimeError(f"{what} failed: CUDA error {code}" + (" (invalid value / shape)" if code == 1 else ""))
