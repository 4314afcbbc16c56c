"""The allocation-free variant of processed_probs (colinfer_processed_probs_noalloc) against the ordinary entry point.

It exists for hosts that bind the C ABI without an allocator to draw scratch from (graph replay, fixed memory budgets):
its per-row scratch is a fixed array inside the library.  Collected last on purpose (the file name sorts after every
other test file): should it fail, everything else has already run.  Called through the C ABI, twice in a row with
different inputs, because the fixed array keeps whatever the previous call wrote.
"""
import math

import pytest
import torch

from colinfer_b200 import _lib

pytestmark = pytest.mark.gpu


def _both(logits, t, k, p, lmp):
    L = _lib.lib()
    dev = logits.device
    one = lambda v, dt: torch.tensor([v], dtype=dt, device=dev)  # noqa: E731
    T, K, P, M = one(t, torch.float32), one(k, torch.int32), one(p, torch.float32), one(lmp, torch.float32)
    R, V = logits.shape
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.empty_like(logits)
    scratch = torch.empty(R * _lib.ROW_STATS_BYTES, dtype=torch.uint8, device=dev)
    assert L.colinfer_processed_probs(logits.data_ptr(), T.data_ptr(), K.data_ptr(), P.data_ptr(), M.data_ptr(),
                                      want.data_ptr(), scratch.data_ptr(), R, V, stream) == 0
    got = torch.full_like(logits, float("nan"))
    assert L.colinfer_processed_probs_noalloc(logits.data_ptr(), T.data_ptr(), K.data_ptr(), P.data_ptr(), M.data_ptr(),
                                              got.data_ptr(), R, V, stream) == 0
    torch.cuda.synchronize()
    return got, want


def test_noalloc_matches_the_ordinary_entry_point_twice_in_a_row():
    assert torch.cuda.is_available()
    g = torch.Generator().manual_seed(77)
    # first call: many rows, wide distribution; second call: fewer rows, other vocabulary and filters -- entries left in
    # the fixed array by the first call must not leak into the second
    a = (torch.randn(37, 4099, generator=g) * 2).cuda()
    got, want = _both(a, 0.9, 4099, 0.9, float("-inf"))
    torch.testing.assert_close(got, want, rtol=1e-6, atol=0)
    assert torch.equal(got > 0, want > 0)
    b = (torch.randn(5, 151936, generator=g) * 3).cuda()
    got, want = _both(b, 0.7, 50, 0.95, math.log(0.02))
    torch.testing.assert_close(got, want, rtol=1e-6, atol=0)
    assert torch.equal(got > 0, want > 0)
    assert abs(float(got[0].double().sum()) - 1.0) < 1e-5


def test_noalloc_rejects_more_rows_than_the_fixed_array_holds():
    L = _lib.lib()
    cap = L.colinfer_noalloc_max_rows()
    assert cap == 4096
    x = torch.zeros(1, 8, device="cuda")
    one = torch.ones(1, device="cuda")
    k = torch.full((1,), 8, dtype=torch.int32, device="cuda")
    rc = L.colinfer_processed_probs_noalloc(x.data_ptr(), one.data_ptr(), k.data_ptr(), one.data_ptr(), one.data_ptr(),
                                            x.data_ptr(), cap + 1, 8, torch.cuda.current_stream().cuda_stream)
    assert rc == 1                                                 # cudaErrorInvalidValue, nothing launched
