"""The C-ABI library and the host-side mirror of the reference's interface, without a GPU: the library builds and
loads, exports every symbol the header declares, and the host logic (SamplerParams, shape / device checks, geometry)
behaves like the reference's."""
import ctypes as C
import math
import os
import re

import pytest
import torch

from colinfer_b200 import _lib
from colinfer_b200.runtime.sampler import SamplerParams, apply_mask, sample
from colinfer_b200.spec.accept import draw, inverse_cdf, processed_probs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_lib):
    header = open(os.path.join(ROOT, "include", "colinfer_b200.h")).read()
    declared = set(re.findall(r"^(?:int|int64_t)\s+(colinfer_[a-z_0-9]+)\s*\(", header, re.M))
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    handle = C.CDLL(built_lib)
    for name in declared:
        assert hasattr(handle, name), name
    assert _lib.lib().colinfer_version() >= 100


def test_struct_layouts_match_header(built_lib):
    assert C.sizeof(_lib.SamplerParamsC) == 11 * 8          # ten pointers + int32 (padded)
    assert C.sizeof(_lib.Geometry) == 16
    assert _lib.ROW_STATS_BYTES == 32


def test_geometry_of_the_benchmark_vocabularies(built_lib):
    g = _lib.Geometry()
    L = _lib.lib()
    assert L.colinfer_sample_geometry(151936, _lib.F32, None, 0, C.byref(g)) == 0
    assert g.cluster * g.slice_elems >= 151936 and g.slice_elems % 128 == 0 and g.bulk_copy == 1
    assert g.smem_bytes <= 113 * 1024                          # two CTAs per SM
    assert L.colinfer_sample_geometry(262144, _lib.BF16, None, 0, C.byref(g)) == 0
    assert g.cluster * g.slice_elems >= 262144 and g.smem_bytes <= 227 * 1024
    assert L.colinfer_sample_geometry(50, _lib.F32, None, 0, C.byref(g)) == 0 and g.cluster == 1 and g.bulk_copy == 0
    assert L.colinfer_sample_geometry(10_000_000, _lib.F32, None, 0, C.byref(g)) == 1   # beyond the resident-row limit
    assert L.colinfer_sample_geometry(151936, _lib.F32, None, 3, C.byref(g)) == 1 and L.colinfer_sample_geometry(151936, _lib.F32, None, 8, C.byref(g)) == 0


def test_sampler_params_host_logic(golden):
    """engine/runtime/sampler.py:23-47 on CPU tensors, against the values the reference's class stores."""
    cases = golden["set_cases"]
    sp = SamplerParams(len(cases), 151936, "cpu")
    assert sp.top_k.tolist() == [151936] * len(cases) and sp.top_p.tolist() == [1.0] * len(cases)
    assert all(math.isinf(x) and x < 0 for x in sp.log_min_p.tolist())
    for i, ((t, k, p, mp), seed) in enumerate(zip(cases, golden["set_case_seeds"])):
        sp.set(i, temperature=t, top_k=int(k), top_p=p, min_p=mp, seed=int(seed))
    assert torch.equal(sp.temperature, torch.from_numpy(golden["set_temperature"]))
    assert torch.equal(sp.top_k, torch.from_numpy(golden["set_top_k"]))
    assert torch.equal(sp.top_p, torch.from_numpy(golden["set_top_p"]))
    assert torch.equal(sp.log_min_p, torch.from_numpy(golden["set_log_min_p"]))
    assert torch.equal(sp.seed, torch.from_numpy(golden["set_seed"]))
    v = sp.view(1, 3)
    assert torch.equal(v.top_k, torch.from_numpy(golden["view_top_k"]))
    v.temperature[0] = 9.0                                     # a view shares storage
    assert sp.temperature[1] == 9.0
    sp.set_penalties(2, 1.1, 0.5, 0.2)
    assert sp.repetition_penalty.tolist()[:3] == [1.0, 1.0, pytest.approx(1.1)] and sp.view(2, 3).presence_penalty[0] == 0.5


def test_top_k_beyond_int32_means_no_top_k():
    """Reference tests/test_sampler.py:104-107."""
    p = SamplerParams(1, 1000, "cpu")
    p.set(0, temperature=1.0, top_k=3_000_000_000)
    assert int(p.top_k[0]) == 1000


def test_no_cpu_fallback(built_lib):
    """Every op refuses CPU tensors with RuntimeError (the reference's CHECK_CUDA_TENSOR behaviour); nothing computes
    on the host."""
    from colinfer_b200.kernels import ops
    from colinfer_b200.spec.verify import spec_accept
    p = SamplerParams(2, 64, "cpu")
    logits = torch.zeros(2, 1, 64)
    with pytest.raises(RuntimeError):
        draw(logits, p, torch.zeros(2, dtype=torch.int32))
    with pytest.raises(RuntimeError):
        sample(logits[:, 0], p, torch.zeros(2, dtype=torch.int32))
    with pytest.raises(RuntimeError):
        apply_mask(logits, torch.zeros(2, 1, 2, dtype=torch.int32))
    with pytest.raises(RuntimeError):
        processed_probs(logits[0], p.temperature[:1], p.top_k[:1], p.top_p[:1], p.log_min_p[:1])
    with pytest.raises(RuntimeError):
        inverse_cdf(torch.ones(2, 64), torch.ones(2))
    with pytest.raises(RuntimeError):
        ops().philox_uniform(p.seed, p.seed, torch.empty(2, 4))
    with pytest.raises(RuntimeError):
        spec_accept(torch.zeros(2, 4, dtype=torch.int64), torch.zeros(2, 4, dtype=torch.int64))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or eager fallback"):
        _lib.lib()


def test_workload_generators_are_deterministic():
    from colinfer_b200 import workloads as wl
    a, b = wl.config3(4, V=4096, H=64), wl.config3(4, V=4096, H=64)
    assert torch.equal(a["logits"], b["logits"]) and torch.equal(a["params"]["history"], b["params"]["history"])
    assert set(a["params"]["top_k"].tolist()) <= {20, 100, 4096}
    m = wl.pack_mask(torch.tensor([[True] + [False] * 31 + [False, True]]))
    assert m.tolist() == [[1, 2]]
    c1 = wl.config1(V=4099)
    assert c1["mask"].shape == (1, 1, 129)
    assert wl.bytes_per_row(151936, 4, False, 2048) == 615976
