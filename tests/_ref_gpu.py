"""Shared by the CPU and GPU tests: the cases of tests/golden/ref_gpu_vectors.npz (what the reference's expressions gave
on a GPU with FlashInfer, tests/golden/make_gpu_golden.py) and the rows they were computed from."""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))


def cases():
    """[(name, workload, u [B, 1], effective logits [B, 1, V])]: penalties and mask already applied to the logits."""
    import make_gpu_golden as G
    from colinfer_b200 import workloads as wl
    from oracle import oracle as O
    out = []
    w = wl.config0()
    out.append(("config0", w, w["u"].numpy()))
    w = wl.config1()
    out.append(("config1", w, w["u"].numpy()))
    w = wl.config3(64)
    out.append(("config3_b64", w, O.philox_uniform(w["params"]["seed"].numpy(), w["pos"].numpy().astype(np.int64), 1)))
    w, u = G.tie_case()
    out.append(("ties", w, u))
    return [(n, w, u, G.effective_logits(w)) for n, w, u in out]


def load():
    return np.load(os.path.join(HERE, "golden", "ref_gpu_vectors.npz"))
