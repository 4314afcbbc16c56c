"""Randomised parity sweeps: draw() and the rejection verify against the oracle over random shapes, dtypes, masks,
penalties and filter settings, through every kernel the host can pick.  Tokens must equal the oracle's unless the oracle's
decision margin is below 1e-6 (1e-5 for the accept test); for the verify, a draft below the mass horizon (no mass in the
kernels, p ~ 1e-11 in float64) is rejected by design and is counted apart."""
import numpy as np
import pytest
import torch

from colinfer_b200 import _lib
from colinfer_b200 import workloads as wl
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _penalty_params(rng, params, B, V, H_choices):
    H = int(rng.choice(H_choices))
    hist = torch.tensor(rng.integers(-2, V + 2, size=(B, H)), dtype=torch.int32)
    if rng.random() < 0.5:
        hist[:, : H // 2] = hist[:, :1]                            # heavy repeats
    hl = torch.tensor(rng.integers(0, H + 1, size=B), dtype=torch.int32)
    params["repetition_penalty"] = torch.tensor(rng.choice([1.0, 1.2, 2.0, 0.8], size=B), dtype=torch.float32)
    params["presence_penalty"] = torch.tensor(rng.choice([0.0, 0.5, -0.5, 3.0], size=B), dtype=torch.float32)
    params["frequency_penalty"] = torch.tensor(rng.choice([0.0, 0.1, -0.1, 1.0], size=B), dtype=torch.float32)
    params["history"], params["hist_len"] = hist, hl
    return hist, hl


@pytest.mark.parametrize("seed", [11, 12])
def test_draw_random_sweep(seed):
    from colinfer_b200.spec.accept import draw
    _lib.lib()
    checked = boundary = 0
    for case in range(120):
        rng = np.random.default_rng(seed * 100000 + case)
        g = torch.Generator().manual_seed(seed * 100000 + case)
        V = int(rng.choice([1, 2, 3, 31, 32, 33, 100, 127, 128, 129, 1000, 4099, 8192, 20000]))
        B, R = int(rng.choice([1, 2, 3, 5, 9, 40])), int(rng.choice([1, 1, 2, 4]))
        dtype = torch.bfloat16 if rng.random() < 0.3 else torch.float32
        kind = rng.choice(["normal", "peaked", "flat", "ties", "neg_inf", "wide_scale"])
        x = torch.randn(B, R, V, generator=g)
        if kind == "normal":
            x = x * float(rng.choice([0.5, 2.0, 5.0]))
        elif kind == "peaked":
            x = x * 2.0
            x[..., int(rng.integers(0, V))] += float(rng.choice([5.0, 15.0, 40.0]))
        elif kind == "flat":
            x = x * 1e-3
        elif kind == "ties":
            x = (x * 3).round() * 0.5
        elif kind == "neg_inf":
            x = x * 2.0
            x[torch.rand(B, R, V, generator=g) < 0.5] = -float("inf")
        else:
            x = x * 30.0
        logits = x.to(dtype)
        params = wl._params(B, V, torch.tensor(rng.choice([0.0, 0.3, 0.7, 1.0, 1.5], size=B), dtype=torch.float32),
                            torch.tensor(rng.choice([0, 1, 2, 5, 20, 100, 1000, V, V + 5], size=B)),
                            torch.tensor(rng.choice([1.0, 0.99, 0.9, 0.5, 0.1, 1e-4], size=B), dtype=torch.float32),
                            torch.tensor(rng.choice([0.0, 0.0, 0.01, 0.2, 0.9], size=B)), seed=torch.tensor(rng.integers(0, 2 ** 40, size=B)))
        mask = None
        if rng.random() < 0.4:
            allowed = torch.rand(B, R, V, generator=g) < float(rng.choice([0.05, 0.5, 0.95]))
            if rng.random() < 0.8:
                allowed[..., int(rng.integers(0, V))] = True
            mask = wl.pack_mask(allowed)
        hist = hl = None
        if rng.random() < 0.5:
            hist, hl = _penalty_params(rng, params, B, V, [1, 7, 64, 512, 3000])
        pos = torch.tensor(rng.integers(0, 10 ** 6, size=B), dtype=torch.int64)
        sp = wl.sampler_params(params, V, "cuda")
        pr = {k: v.numpy() for k, v in params.items() if k not in ("history", "hist_len")}
        want, info = O.draw(logits.float().numpy(), pr, pos.numpy(), mask=None if mask is None else mask.numpy(),
                            history=None if hist is None else hist.numpy(), hist_len=None if hl is None else hl.numpy())
        for cluster in (0, -1, 1, 8):                               # automatic, streaming kernel, clusters of 1 and of 8 CTAs
            try:
                got = draw(logits.cuda(), sp, pos.cuda(), mask=None if mask is None else mask.cuda(), flags=_lib.kernel_flags(cluster))
            except RuntimeError:
                assert cluster in (1, 8)                            # a forced geometry may not hold the row
                continue
            got, w = got.cpu().numpy().reshape(-1), want.reshape(-1)
            checked += len(w)
            for i in np.flatnonzero(got != w):
                assert min(info[i]["margin"], info[i]["margin_top_p"]) < 1e-6, (case, cluster, i, got[i], w[i], V, B, R, dtype, kind)
                boundary += 1
    print(f"[parity] random sweep of draw, seed {seed}: {checked} row checks, {boundary} inside the margin")
    assert boundary <= max(2, checked // 2000)


@pytest.mark.parametrize("seed", [21, 22])
def test_spec_verify_random_sweep(seed):
    from colinfer_b200.spec.accept import draw
    from colinfer_b200.spec.verify import spec_verify
    _lib.lib()
    slots = boundary = horizon = 0
    for case in range(120):
        rng = np.random.default_rng(seed * 100000 + case)
        g = torch.Generator().manual_seed(seed * 100000 + case)
        V, B, k = int(rng.choice([2, 33, 128, 1000, 4099, 20000])), int(rng.choice([1, 2, 5, 20])), int(rng.choice([1, 2, 4, 8]))
        dtype = torch.bfloat16 if rng.random() < 0.25 else torch.float32
        target = (torch.randn(B, k + 1, V, generator=g) * float(rng.choice([1.0, 3.0]))).to(dtype)
        draft = (target[:, :k].float() + torch.randn(B, k, V, generator=g) * float(rng.choice([0.1, 1.0, 3.0]))).to(dtype).contiguous()
        params = wl._params(B, V, torch.tensor(rng.choice([0.0, 0.5, 1.0], size=B), dtype=torch.float32), torch.tensor(rng.choice([0, 3, 50], size=B)),
                            torch.tensor(rng.choice([1.0, 0.9, 0.3], size=B), dtype=torch.float32), torch.tensor(rng.choice([0.0, 0.05], size=B)))
        mask = None
        if rng.random() < 0.4:
            allowed = torch.rand(B, k + 1, V, generator=g) < 0.6
            allowed[..., 0] = True
            mask = wl.pack_mask(allowed)
        hist = hl = None
        if rng.random() < 0.5:
            hist, hl = _penalty_params(rng, params, B, V, [4, 64, 700])
        sp = wl.sampler_params(params, V, "cuda")
        ud, ua, us = wl.open_unit(g, B, k), wl.open_unit(g, B, k), wl.open_unit(g, B, k + 1)
        if rng.random() < 0.5:                                      # drafts drawn from q, or drafts that ignore q
            d_ids = draw(draft.cuda(), sp, None, u=ud.cuda(), mask=None if mask is None else mask[:, :k].contiguous().cuda())
        else:
            d_ids = torch.tensor(rng.integers(0, V, size=(B, k))).cuda()
        out, n = spec_verify(target.cuda(), draft.cuda(), d_ids, sp, ua.cuda(), us.cuda(), mask=None if mask is None else mask.cuda())
        out, n, d_np = out.cpu().numpy(), n.cpu().numpy(), d_ids.cpu().numpy()
        pr = {kk: v.numpy() for kk, v in params.items() if kk not in ("history", "hist_len")}
        for b in range(B):
            kw = {}
            if hist is not None:
                kw = dict(history=hist[b, :int(hl[b])].numpy(), rep=float(pr["repetition_penalty"][b]), pres=float(pr["presence_penalty"][b]),
                          freq=float(pr["frequency_penalty"][b]))
            r = O.spec_verify_reject(target[b].float().numpy(), draft[b].float().numpy(), d_np[b], pr["temperature"][b], pr["top_k"][b],
                                     pr["top_p"][b], pr["log_min_p"][b], ua[b].numpy(), us[b].numpy(),
                                     target_mask=None if mask is None else mask[b].numpy(), **kw)
            slots += 1
            if n[b] == r["n_accept"] + 1 and out[b, r["n_accept"]] == r["token"] and list(out[b, :r["n_accept"]]) == list(d_np[b, :r["n_accept"]]):
                continue
            j = int(n[b]) - 1                                       # the position the kernel stopped at
            below = False
            if j < k and pr["temperature"][b] > 0:
                row = target[b, j].float().numpy()
                if hist is not None:
                    row = O.penalties(row, kw["history"], kw["rep"], kw["pres"], kw["freq"])
                if mask is not None:
                    row = O.apply_mask(row, mask[b, j].numpy())
                p = O.processed(row, pr["temperature"][b], pr["top_k"][b], pr["top_p"][b], pr["log_min_p"][b])["probs"]
                below = p[int(d_np[b, j])] < p.max() * 2.0 ** -29
            if below:
                horizon += 1
            else:
                assert min(r["margin"], r["accept_margin"]) < 1e-5, (case, b, n[b], out[b], r, V, k, dtype)
                boundary += 1
    print(f"[parity] random sweep of the verify, seed {seed}: {slots} slots, {boundary} inside the margin, {horizon} drafts below the mass horizon")
    assert boundary <= max(2, slots // 500)


def test_draft_pick_and_logprobs_random_sweep():
    from colinfer_b200.runtime.logprobs import logprobs_tensors
    from colinfer_b200.spec.draft import lowrank_draft
    _lib.lib()
    bits = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    for case in range(40):
        rng = np.random.default_rng(3100000 + case)
        g = torch.Generator().manual_seed(3100000 + case)
        # ---- the one-launch draft of the low-rank heads
        Vd = int(rng.choice([256, 300, 1000, 4096, 8190, 20000]))
        K, N = int(rng.choice([8, 64, 264])), int(rng.choice([1, 2, 9, 12, 40, 80]))
        NC, rows_w = int(min(Vd, rng.choice([1, 16, 256, 1000]))), Vd + int(rng.integers(0, 50))
        w = (torch.randn(rows_w, K, generator=g) * 0.05).bfloat16().cuda()
        x = torch.randn(N, K, generator=g).bfloat16().cuda()
        vid = torch.randperm(rows_w, generator=g)[:Vd].cuda() if rng.random() < 0.8 else None
        kind = rng.choice(["track", "normal", "ties", "crowded", "neg_inf"])
        if kind == "track":
            ap = x.float() @ w[vid if vid is not None else slice(0, Vd)].float().T + 0.3 * torch.randn(N, Vd, generator=g).cuda()
        elif kind == "normal":
            ap = torch.randn(N, Vd, generator=g).cuda() * 3
        elif kind == "ties":
            ap = (torch.randn(N, Vd, generator=g) * 2).round().cuda()
        elif kind == "crowded":
            ap = (5.0 + 1e-4 * torch.randn(N, Vd, generator=g)).cuda()
        else:
            ap = torch.randn(N, Vd, generator=g)
            ap[torch.rand(N, Vd, generator=g) < 0.9] = -float("inf")
            ap = ap.cuda()
        ap = ap.contiguous()
        ctas = int(rng.choice([0, 0, 1, 2, 4, 8, 16]))
        ids, p, idx, ex = lowrank_draft(ap, x, w, vid, n_cands=NC, ctas_per_slot=ctas, want_index=True)
        want = O.draft_pick(ap.cpu().numpy(), bits(x), None if vid is None else vid.cpu().numpy(), NC, w_bits=bits(w))
        what = (case, N, Vd, K, NC, ctas, kind)
        assert np.array_equal(idx.cpu().numpy(), want[2]) and np.array_equal(ids.cpu().numpy(), want[0]), what
        assert np.array_equal(ex.cpu().numpy().view(np.uint32), want[3].view(np.uint32)), what
        fin = np.isfinite(want[1])
        np.testing.assert_allclose(p.cpu().numpy()[fin], want[1][fin], rtol=2e-5, atol=1e-30)
        # ---- logprobs of emitted tokens
        V, r = int(rng.choice([1, 5, 33, 128, 1000, 4099, 20000])), int(rng.choice([1, 3, 17, 200]))
        n_top = int(min(V, rng.choice([0, 1, 5, 20, 32])))
        dtype = torch.bfloat16 if rng.random() < 0.3 else torch.float32
        rows = torch.randn(r, V, generator=g) * float(rng.choice([1.0, 4.0]))
        kind = rng.choice(["normal", "ties", "peaked", "neg_inf"])
        if kind == "ties":
            rows = (rows * 2).round() * 0.5
        elif kind == "peaked":
            rows[:, int(rng.integers(0, V))] += 30.0
        elif kind == "neg_inf":
            rows[torch.rand(r, V, generator=g) < 0.7] = -float("inf")
            rows[:, 0] = 0.0
        rows = rows.to(dtype)
        toks = torch.tensor(rng.integers(0, V, size=r))
        c, ti, tl = (t.cpu().numpy() for t in logprobs_tensors(rows.cuda(), toks.cuda(), n_top))
        wc, wi, wl_ = O.logprobs(rows.float().numpy(), toks.numpy(), n_top)
        fin = np.isfinite(wc)
        np.testing.assert_allclose(c[fin], wc[fin], atol=3e-5, rtol=0)
        if n_top:
            fin = np.isfinite(wl_)
            np.testing.assert_allclose(tl[fin], wl_[fin], atol=3e-5, rtol=0)
            xv = rows.float().numpy()
            for i in range(r):                                      # equal logits may swap places: the values must agree
                assert np.array_equal(xv[i][ti[i]], xv[i][wi[i]]), (case, i)
