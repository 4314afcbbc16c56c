"""Builds the CUDA library of this package, in-tree, for sm_100a: colinfer_b200/libcolinfer_b200.so.

`python -m colinfer_b200.build` (or build() from the graft entry) runs nvcc on the sources in csrc/.  nvcc cross-compiles,
so no GPU is needed to build.  The library has a plain C ABI (include/colinfer_b200.h) and does not link against torch.

The streaming kernel is compiled once per instantiation (csrc/stream_part.cu with -DCOLINFER_STREAM_PART=0..8), side by
side, which keeps a full build to about a minute.  Objects are kept under colinfer_b200/build/obj and reused while they
are newer than every source and header.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build", "obj")
LIB = os.path.join(HERE, "libcolinfer_b200.so")
STREAM_PARTS = 9
# (source, object name, extra flags)
UNITS = [("sample.cu", "sample.o", []), ("ops.cu", "ops.o", []), ("logprobs.cu", "logprobs.o", []),
         ("rescore.cu", "rescore.o", []), ("gather.cu", "gather.o", []), ("draft_pick.cu", "draft_pick.o", []), ("stream_host.cu", "stream_host.o", [])] + \
        [("stream_part.cu", f"stream_part_{i}.o", [f"-DCOLINFER_STREAM_PART={i}"]) for i in range(STREAM_PARTS)]
# --fmad=false: fp32 expressions on a decision path are never contracted behind the source's back (the reference builds its
# kernels the same way); the fused multiply-adds the kernels want are written as fmaf().
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--fmad=false", "-Xcompiler", "-fPIC"]


def _deps():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))] + \
           [os.path.join(ROOT, "include", "colinfer_b200.h")]


def needs_build() -> bool:
    return not os.path.exists(LIB) or os.path.getmtime(LIB) < max(os.path.getmtime(p) for p in _deps())


def build(force: bool = False, verbose: bool = False, only: set[str] | None = None) -> str:
    """Compile csrc/*.cu into libcolinfer_b200.so (skipped when it is newer than every source).

    only: object names to recompile even though the others are stale too (a development shortcut: the stale objects
    are linked as they are)."""
    if not force and not needs_build() and only is None:
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    extra = os.environ.get("COLINFER_NVCC_EXTRA", "").split()
    flags = NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else [])
    os.makedirs(OBJ, exist_ok=True)
    newest = max(os.path.getmtime(p) for p in _deps())

    def compile_one(unit):
        src, name, defs = unit
        obj = os.path.join(OBJ, name)
        fresh = os.path.exists(obj) and os.path.getmtime(obj) >= newest
        if only is not None:
            if name not in only and os.path.exists(obj):
                return obj, ""
        elif fresh and not force:
            return obj, ""
        cmd = [nvcc, *flags, *defs, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return obj, r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(len(UNITS), os.cpu_count() or 4))) as pool:
        done = list(pool.map(compile_one, UNITS))
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *[o for o, _ in done]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write("".join(e for _, e in done) + res.stderr)
    return LIB


EXT = os.path.join(HERE, "_colinfer_torch.so")


def build_torch_ext(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/torch_ext.cpp -- the thin PyTorch C++ extension over the C ABI -- into colinfer_b200/_colinfer_torch.so.
    It links against libcolinfer_b200.so next to it (rpath $ORIGIN) and needs torch's headers; no GPU is needed."""
    src = os.path.join(CSRC, "torch_ext.cpp")
    deps = [src, os.path.join(ROOT, "include", "colinfer_b200.h")]
    if not force and os.path.exists(EXT) and os.path.getmtime(EXT) >= max(os.path.getmtime(p) for p in deps):
        return EXT
    if not os.path.exists(LIB):
        build()
    import shutil

    from torch.utils import cpp_extension
    bdir = os.path.join(HERE, "build", "torch_ext")
    os.makedirs(bdir, exist_ok=True)
    cpp_extension.load(name="_colinfer_torch", sources=[src], extra_cflags=["-O2"], with_cuda=True,
                       # -l:libstdc++.so.6 first: a compiler driver whose own libstdc++.so link dangles would otherwise link
                       # the static libstdc++ into the extension, whose streams are then not the process's (and crash)
                       extra_ldflags=["-l:libstdc++.so.6", f"-L{HERE}", "-lcolinfer_b200", "-Wl,-rpath,'$$ORIGIN'", "-Wl,-rpath,'$$ORIGIN/../..'"],
                       build_directory=bdir,
                       is_python_module=False, verbose=verbose)
    shutil.copyfile(os.path.join(bdir, "_colinfer_torch.so"), EXT)
    return EXT


if __name__ == "__main__":
    names = {a.split("=", 1)[1] for a in sys.argv if a.startswith("--only=")}
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, only=names or None))
    if "--ext" in sys.argv:
        print(build_torch_ext(force="--force" in sys.argv, verbose="-v" in sys.argv))
