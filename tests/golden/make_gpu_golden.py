"""Golden vectors from the reference's GPU arithmetic: tests/golden/ref_gpu_vectors.npz.  TEST INFRASTRUCTURE.

The reference's processed_probs (engine/spec/accept.py:23-33) is four torch expressions around two FlashInfer calls
(top_k_renorm_probs, top_p_renorm_probs), and its inverse_cdf (accept.py:36-40) is a cumsum and a count.  FlashInfer
needs a GPU and the reference checkout does not travel to a GPU box, so this script states those few expressions
itself, in the reference's order, and runs them with the FlashInfer installed on the box (its version is recorded in
the output; the reference pins flashinfer-python 0.7.0.post1).  The vectors pin what the oracle and the kernels are
compared with: kept sets (ties at a pivot all kept), renormalised probabilities and drawn tokens.

    python tests/golden/make_gpu_golden.py [out.npz]      (on a box with a GPU and FlashInfer; default: next to this script)

Inputs are the seeded workloads of colinfer_b200/workloads.py (the tests regenerate them); penalties and the grammar
mask -- which the reference applies before this step or not at all -- are applied with the numpy oracle first.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from colinfer_b200 import workloads as wl  # noqa: E402
from oracle import oracle as O  # noqa: E402

TOPN = 16


def ref_processed(logits, temperature, top_k, top_p, log_min_p):
    """accept.py:23-33: logits [R, V] fp32 on the GPU; the four parameters are 1-element device tensors."""
    import flashinfer.sampling as fs
    z = logits / temperature.clamp_min(1e-6)
    z = z.masked_fill(z < z.amax(-1, keepdim=True) + log_min_p, float("-inf"))
    p = torch.softmax(z, -1)
    R = p.shape[0]
    p = fs.top_k_renorm_probs(p, top_k.expand(R).contiguous())
    return fs.top_p_renorm_probs(p, top_p.expand(R).contiguous())


def ref_inverse_cdf(P, u):
    """accept.py:36-40."""
    c = P.cumsum(-1)
    return (c < (u * c[:, -1])[:, None]).sum(-1).clamp_max(P.shape[-1] - 1)


def effective_logits(w):
    """The rows as the filters see them: penalties, then the grammar mask (numpy oracle, exact fp32 steps)."""
    lg = w["logits"].float().numpy().copy()
    p = w["params"]
    B, R, _ = lg.shape
    for b in range(B):
        for r in range(R):
            row = lg[b, r]
            if "history" in p:
                row = O.penalties(row, p["history"][b, :int(p["hist_len"][b])].numpy(), float(p["repetition_penalty"][b]),
                                  float(p["presence_penalty"][b]), float(p["frequency_penalty"][b]))
            if "mask" in w:
                row = O.apply_mask(row, w["mask"][b, r].numpy())
            lg[b, r] = row
    return lg


def run_case(name, w, u, out):
    """Every row of a workload through the reference's expressions; per row: token, greedy token, kept count, smallest
    kept and largest dropped logit, the TOPN largest probabilities and their tokens."""
    lg = effective_logits(w)
    B, R, V = lg.shape
    p = {k: v.cuda() for k, v in w["params"].items() if k in ("temperature", "top_k", "top_p", "log_min_p")}
    d = torch.from_numpy(lg).cuda()
    tok = np.zeros((B, R), np.int64)
    greedy = d.argmax(-1).cpu().numpy()
    nkept = np.zeros((B, R), np.int64)
    kmin = np.zeros((B, R), np.float32)
    dmax = np.zeros((B, R), np.float32)
    top_i = np.zeros((B, R, TOPN), np.int64)
    top_p = np.zeros((B, R, TOPN), np.float32)
    for b in range(B):
        if not float(p["temperature"][b]) > 0:
            tok[b] = greedy[b]
            continue
        P = ref_processed(d[b], p["temperature"][b:b + 1], p["top_k"][b:b + 1], p["top_p"][b:b + 1], p["log_min_p"][b:b + 1])
        tok[b] = ref_inverse_cdf(P, torch.from_numpy(u[b]).cuda()).cpu().numpy()
        kept = P > 0
        nkept[b] = kept.sum(-1).cpu().numpy()
        kmin[b] = torch.where(kept, d[b], torch.full_like(d[b], float("inf"))).amin(-1).cpu().numpy()
        dmax[b] = torch.where(kept, torch.full_like(d[b], float("-inf")), d[b]).amax(-1).cpu().numpy()
        tv, ti = P.topk(TOPN, -1)
        top_i[b], top_p[b] = ti.cpu().numpy(), tv.cpu().numpy()
    for key, val in (("tok", tok), ("greedy", greedy), ("nkept", nkept), ("kept_min_logit", kmin), ("dropped_max_logit", dmax),
                     ("top_idx", top_i), ("top_prob", top_p), ("u", u)):
        out[f"{name}_{key}"] = val


def tie_case(V=wl.V_QWEN):
    """Rows rounded to bf16 (a hundred tokens share every value) under the filters whose pivots then fall on ties."""
    g = torch.Generator().manual_seed(31)
    combos = [(1.0, 0, 0.9, 0.0), (0.8, 100, 1.0, 0.0), (1.0, 1000, 0.98, 0.01), (0.7, 50, 0.9, 0.0), (1.2, 0, 0.5, 0.0),
              (0.9, 5000, 0.95, 0.0), (1.0, 20, 0.6, 0.05), (0.6, 0, 0.999, 0.0)]
    B = len(combos)
    logits = (torch.randn(B, 1, V, generator=g) * 2.0).bfloat16().float()
    params = wl._params(B, V, [c[0] for c in combos], [c[1] for c in combos], [c[2] for c in combos], [c[3] for c in combos],
                        list(range(500, 500 + B)))
    return dict(name="ties", logits=logits, params=params, pos=torch.arange(B, dtype=torch.int32)), wl.open_unit(g, B, 1).numpy()


def main():
    import flashinfer
    dst = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "ref_gpu_vectors.npz")
    out = {"flashinfer_version": np.array(flashinfer.__version__), "torch_version": np.array(torch.__version__),
           "topn": np.array(TOPN)}
    w = wl.config0()
    run_case("config0", w, w["u"].numpy(), out)
    w = wl.config1()
    run_case("config1", w, w["u"].numpy(), out)
    w = wl.config3(64)
    u = O.philox_uniform(w["params"]["seed"].numpy(), w["pos"].numpy().astype(np.int64), 1)
    run_case("config3_b64", w, u, out)
    w, u = tie_case()
    run_case("ties", w, u, out)
    os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
    np.savez_compressed(dst, **out)
    print("wrote", dst, "flashinfer", flashinfer.__version__, {k: v.shape for k, v in out.items() if k.endswith("_tok")})


if __name__ == "__main__":
    main()
