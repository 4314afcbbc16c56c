"""Builds the CUDA library of this package, in-tree, for sm_100a: colinfer_b200/libcolinfer_b200.so.

`python -m colinfer_b200.build` (or build() from the graft entry) runs nvcc on the sources in csrc/.  nvcc cross-compiles,
so no GPU is needed to build.  The library has a plain C ABI (include/colinfer_b200.h) and does not link against torch.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcolinfer_b200.so")
SOURCES = ("sample.cu", "stream.cu", "ops.cu", "logprobs.cu", "rescore.cu")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC"]


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def needs_build() -> bool:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "colinfer_b200.h")]
    return not os.path.exists(LIB) or os.path.getmtime(LIB) < _newest(deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/*.cu into libcolinfer_b200.so (skipped when it is newer than every source)."""
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    flags = [f for f in NVCC_FLAGS if f != "-shared"] + (["-Xptxas", "-v"] if verbose else [])
    # one nvcc per source, side by side (stream.cu holds eight kernel instantiations and dominates), then the link
    with tempfile.TemporaryDirectory(prefix="colinfer_b200_obj_") as tmp:
        def compile_one(src):
            obj = os.path.join(tmp, src.replace(".cu", ".o"))
            cmd = [nvcc, *flags, "-c", os.path.join(CSRC, src), "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
            return obj, r.stderr
        with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
            done = list(pool.map(compile_one, SOURCES))
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *[o for o, _ in done]]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
        res.stderr = "".join(e for _, e in done) + res.stderr
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
