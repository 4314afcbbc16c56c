"""Generates tests/golden/ref_cpu_vectors.npz by running the parts of the reference that execute on a CPU:
engine.runtime.sampler.SamplerParams / apply_mask and engine.spec.accept.inverse_cdf, imported unmodified from a
colinfer checkout (its path is the first argument; nothing is written there and engine.kernels.ops() is never called).

    python tests/golden/make_golden.py [path-to-colinfer]

The .npz holds the inputs and the reference's outputs; the tests compare the oracle and the CUDA kernels with them.
processed_probs / draw cannot run without a GPU (FlashInfer) and are pinned by the reference's known-answer vectors
instead (tests/test_spec_accept.py:39-48 of the reference, restated in tests/test_oracle.py).
Also writes tests/golden/ref_logprobs.npz from engine.runtime.scheduler.Scheduler._logprobs.
"""
import math
import os
import sys

import numpy as np
import torch

ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("COLINFER_REF", "")
if not os.path.isdir(os.path.join(ref, "engine")):
    sys.exit("usage: make_golden.py <reference checkout>   (or set COLINFER_REF)")
sys.path.insert(0, ref)
sys.dont_write_bytecode = True
from engine.runtime.sampler import SamplerParams, apply_mask  # noqa: E402
from engine.spec.accept import inverse_cdf  # noqa: E402

out = {}
g = torch.Generator().manual_seed(1234)

# apply_mask: [B, R, V] with V not a multiple of 32, random masks, one all-ones row and one single-token row
B, R, V = 2, 3, 70
W = (V + 31) // 32
logits = torch.randn(B, R, V, generator=g) * 3
mask = torch.randint(-2**31, 2**31 - 1, (B, R, W), generator=g, dtype=torch.int64).to(torch.int32)
mask[0, 0] = -1
mask[1, 2] = 0
mask[1, 2, 1] = 1 << 5
out["mask_logits"], out["mask_words"] = logits.numpy(), mask.numpy()
out["mask_out"] = apply_mask(logits, mask).numpy()

# a larger vocabulary (the reference models' 248,320) on one row
V2 = 248320
out["mask_big_seed"] = np.array([4321])
gg = torch.Generator().manual_seed(4321)
l2b = torch.randn(1, 1, V2, generator=gg)
m2b = torch.randint(-2**31, 2**31 - 1, (1, 1, (V2 + 31) // 32), generator=gg, dtype=torch.int64).to(torch.int32)
o2b = apply_mask(l2b, m2b)[0, 0]
out["mask_big_kept_count"] = np.array([int(torch.isfinite(o2b).sum())])
out["mask_big_kept_sum"] = np.array([float(o2b[torch.isfinite(o2b)].double().sum())])
out["mask_big_first_kept"] = torch.nonzero(torch.isfinite(o2b))[:64, 0].numpy()

# inverse_cdf: rows with zero-probability tokens, boundary uniforms
Vc, Rc = 50, 64
P = torch.softmax(torch.randn(Rc, Vc, generator=g) * 1.5, -1)
P[:, 7] = 0
P[3, :5] = 0
P[4, -6:] = 0
P = P / P.sum(-1, keepdim=True)
u = torch.rand(Rc, generator=g).clamp_min(1e-7)
u[0], u[1], u[2] = 1.0, 1e-7, 0.5
out["icdf_P"], out["icdf_u"] = P.numpy(), u.numpy()
out["icdf_out"] = inverse_cdf(P, u).numpy()
# unnormalised weights (inverse_cdf scales u by the row sum)
Wt = torch.rand(8, 1000, generator=g) * (torch.rand(8, 1000, generator=g) < 0.3)
Wt[:, 17] = 0.5
uw = torch.rand(8, generator=g).clamp_min(1e-7)
out["icdf_W"], out["icdf_uw"] = Wt.numpy(), uw.numpy()
out["icdf_wout"] = inverse_cdf(Wt, uw).numpy()

# SamplerParams.set: the stored device values
cases = [(0.0, 0, 1.0, 0.0, 0), (0.7, 50, 0.9, 0.05, 123), (1.3, 3_000_000_000, 0.5, 1e-3, 2**62 - 1),
         (100.0, -4, 1e-3, 1.0, 7), (1e-9, 151936, 1.0, 0.4, 1), (0.8, 151935, 0.95, 0.02, 42)]
sp = SamplerParams(len(cases), 151936, "cpu")
for i, c in enumerate(cases):
    sp.set(i, temperature=c[0], top_k=c[1], top_p=c[2], min_p=c[3], seed=c[4])
out["set_cases"] = np.array([c[:4] for c in cases], dtype=np.float64)
out["set_case_seeds"] = np.array([c[4] for c in cases], dtype=np.int64)
out["set_temperature"], out["set_top_k"] = sp.temperature.numpy(), sp.top_k.numpy()
out["set_top_p"], out["set_log_min_p"], out["set_seed"] = sp.top_p.numpy(), sp.log_min_p.numpy(), sp.seed.numpy()
v = sp.view(1, 3)
out["view_top_k"] = v.top_k.numpy()

dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_cpu_vectors.npz")
np.savez_compressed(dst, **out)
print("wrote", dst, {k: v.shape for k, v in out.items()})

# Logprobs of emitted tokens: Scheduler._logprobs (engine/runtime/scheduler.py:714-722) is a pure torch function of
# its arguments and runs on a CPU.  Small rows are stored; the full-vocabulary rows are regenerated from their seed.
from engine.runtime.scheduler import Scheduler  # noqa: E402
lp = {}
g2 = torch.Generator().manual_seed(99)
rows = torch.randn(5, 1000, generator=g2) * 4
rows[1, 10:14] = rows[1].max() + 1.0            # a four-way tie at the top
rows[2, ::3] = -math.inf                        # masked-out logits
toks = [3, 11, 4, 999, 0]
res = Scheduler._logprobs(None, rows, toks, 5)
lp["small_rows"], lp["small_toks"] = rows.numpy(), np.array(toks)
lp["small_chosen"] = np.array([r[0] for r in res], dtype=np.float64)
lp["small_top_ids"] = np.array([[t[0] for t in r[1]] for r in res], dtype=np.int64)
lp["small_top_lp"] = np.array([[t[1] for t in r[1]] for r in res], dtype=np.float64)
g3 = torch.Generator().manual_seed(2024)
big = torch.randn(3, 151936, generator=g3) * 2.5
btoks = [151935, 0, 77777]
res = Scheduler._logprobs(None, big, btoks, 20)
lp["big_seed"], lp["big_toks"] = np.array([2024]), np.array(btoks)
lp["big_chosen"] = np.array([r[0] for r in res], dtype=np.float64)
lp["big_top_ids"] = np.array([[t[0] for t in r[1]] for r in res], dtype=np.int64)
lp["big_top_lp"] = np.array([[t[1] for t in r[1]] for r in res], dtype=np.float64)
res0 = Scheduler._logprobs(None, rows, toks, 0)
lp["small_chosen_n0"] = np.array([r[0] for r in res0], dtype=np.float64)
assert all(r[1] == [] for r in res0)
dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_logprobs.npz")
np.savez_compressed(dst, **lp)
print("wrote", dst, {k: v.shape for k, v in lp.items()})
