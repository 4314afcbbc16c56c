"""The torch restatement of the reference path that the benchmark times on host cores agrees with the oracle."""
import numpy as np
import torch

from colinfer_b200 import workloads as wl
from oracle import oracle as O
from oracle import torch_cpu_path as T


def test_torch_cpu_path_agrees_with_oracle():
    V = 4096
    w = wl.config3(12, V=V, H=128)
    got = T.draw(w["logits"], w["params"], w["pos"]).numpy()
    pr = {k: v.numpy() for k, v in w["params"].items() if k not in ("history", "hist_len")}
    want, info = O.draw(w["logits"].numpy(), pr, w["pos"].numpy(), history=w["params"]["history"].numpy(),
                        hist_len=w["params"]["hist_len"].numpy())
    bad = np.flatnonzero(got.reshape(-1) != want.reshape(-1))
    assert all(min(info[i]["margin"], info[i]["margin_top_p"]) < 1e-4 for i in bad) and len(bad) <= 1


def test_torch_cpu_path_mask_and_greedy():
    w = wl.config1(V=5000, allow=0.05)
    got = T.draw(w["logits"], w["params"], mask=w["mask"], u=w["u"])
    pr = {k: v.numpy() for k, v in w["params"].items()}
    want, _ = O.draw(w["logits"].numpy(), pr, None, mask=w["mask"].numpy(), u=w["u"].numpy())
    assert got.numpy().tolist() == want.tolist()
    assert torch.equal(T.apply_mask(w["logits"][0], w["mask"][0]),
                       torch.from_numpy(O.apply_mask(w["logits"][0].numpy(), w["mask"][0].numpy())))
