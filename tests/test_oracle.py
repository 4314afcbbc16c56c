"""The CPU oracle against the pins the reference offers for this path: its CPU-runnable functions (golden vectors made
by tests/golden/make_golden.py), the known-answer vectors and properties of its own tests, the published Philox4x32-10
known answers, and an independent sort-based restatement of the filters (the method of the reference's
tests/test_sampler.py:13-27)."""
import math

import numpy as np
import pytest

from oracle import oracle as O


# ------------------------------------------------------------------------------------------------ Philox
def test_philox_known_answers():
    """Known-answer vectors of Philox4x32-10 (Salmon et al. 2011, Random123 kat_vectors)."""
    kats = [([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
            ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
            ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
             [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1])]
    for ctr, key, want in kats:
        assert [int(x) for x in O.philox4x32_10(ctr, key)] == want


def test_philox_uniform_properties():
    """Reference tests/test_spec_accept.py:51-62: reproducible, in (0, 1], a slot's stream depends only on its own
    seed / offset."""
    u = O.philox_uniform([7, 7, 123], [0, 0, 5 << 20], 4096)
    assert np.array_equal(u[0], u[1]) and not np.array_equal(u[0], u[2])
    assert u.min() > 0.0 and u.max() <= 1.0 and abs(u.mean() - 0.5) < 0.02
    v = O.philox_uniform([123], [5 << 20], 4096)
    assert np.array_equal(v[0], u[2])
    # consecutive counters: the stream at offset o + 3 is the stream at offset o shifted by 3
    assert np.array_equal(O.philox_uniform([9], [3], 100)[0], O.philox_uniform([9], [0], 103)[0, 3:])
    # extremes of the 32-bit word map into (0, 1]
    assert O.u32_to_uniform(np.uint32(0)) > 0 and O.u32_to_uniform(np.uint32(0xFFFFFFFF)) <= 1.0


# ------------------------------------------------------------------------------------------------ golden vectors
def test_apply_mask_matches_reference(golden):
    got = O.apply_mask(golden["mask_logits"], golden["mask_words"])
    assert np.array_equal(got, golden["mask_out"])


def test_apply_mask_large_vocab_summary(golden):
    import torch
    V = 248320
    g = torch.Generator().manual_seed(int(golden["mask_big_seed"][0]))
    l = torch.randn(1, 1, V, generator=g)
    m = torch.randint(-2**31, 2**31 - 1, (1, 1, (V + 31) // 32), generator=g, dtype=torch.int64).to(torch.int32)
    out = O.apply_mask(l.numpy(), m.numpy())[0, 0]
    fin = np.isfinite(out)
    assert int(fin.sum()) == int(golden["mask_big_kept_count"][0])
    assert np.array_equal(np.flatnonzero(fin)[:64], golden["mask_big_first_kept"])
    assert float(out[fin].astype(np.float64).sum()) == float(golden["mask_big_kept_sum"][0])


def test_inverse_cdf_matches_reference(golden):
    assert np.array_equal(O.inverse_cdf(golden["icdf_P"], golden["icdf_u"]), golden["icdf_out"])
    assert np.array_equal(O.inverse_cdf(golden["icdf_W"], golden["icdf_uw"]), golden["icdf_wout"])


def test_sampler_params_set_matches_reference(golden):
    for i, ((t, k, p, mp), seed) in enumerate(zip(golden["set_cases"], golden["set_case_seeds"])):
        s = O.sampler_params_set(151936, t, int(k), p, mp, int(seed))
        assert s["temperature"] == golden["set_temperature"][i]
        assert s["top_k"] == golden["set_top_k"][i]
        assert s["top_p"] == golden["set_top_p"][i]
        assert s["log_min_p"] == golden["set_log_min_p"][i]
    assert O.mask_words(151936) == 4748 and O.mask_words(33) == 2


# ------------------------------------------------------------------------------------------------ known answers
def test_processed_probs_known_answers():
    """Reference tests/test_spec_accept.py:39-48 (atol 1e-5)."""
    logits = np.log(np.array([[0.5, 0.3, 0.15, 0.05]], dtype=np.float32))
    want = np.array([0.625, 0.375, 0, 0])
    for k, p, lmp in ((2, 1.0, -np.inf), (4, 0.7, -np.inf), (4, 1.0, math.log(0.4))):
        got = O.processed_probs(logits, 1.0, k, p, np.float32(lmp))[0]
        assert np.allclose(got, want, atol=1e-5, rtol=0)


def sort_based(logits, t, k, p, min_p):
    """Independent restatement by sorting, the method of the reference's tests/test_sampler.py:13-27 (float64)."""
    z = logits.astype(np.float64) / t
    probs = np.exp(z - z.max())
    probs /= probs.sum()
    keep = probs >= min_p * probs.max()
    order = np.argsort(-z, kind="stable")
    keep_k = np.zeros_like(keep)
    keep_k[order[:k]] = True
    keep &= keep_k
    pr = np.where(keep, probs, 0.0)
    pr /= pr.sum()
    idx = np.argsort(-pr, kind="stable")
    srt = pr[idx]
    cut = (np.cumsum(srt) - srt) < p
    final = np.zeros_like(pr)
    final[idx[cut]] = srt[cut]
    return final / final.sum()


@pytest.mark.parametrize("t,k,p,min_p", [(1.0, 0, 1.0, 0.0), (0.7, 20, 1.0, 0.0), (1.0, 0, 0.8, 0.0), (1.3, 50, 0.9, 0.05)])
def test_filters_agree_with_sort_based_restatement(t, k, p, min_p):
    """The four parameter sets of the reference's test_distribution (tests/test_sampler.py:30), V = 1000."""
    V = 1000
    rng = np.random.default_rng(0)
    for trial in range(5):
        base = (rng.standard_normal(V) * 2).astype(np.float32)
        prm = O.sampler_params_set(V, t, k, p, min_p)
        got = O.processed(base, prm["temperature"], prm["top_k"], prm["top_p"], prm["log_min_p"])
        want = sort_based(base, t, k if k > 0 else V, p, min_p)
        assert np.array_equal(got["probs"] > 0, want > 0)
        assert np.allclose(got["probs"], want, rtol=1e-5, atol=1e-12)


def test_ties_are_all_kept():
    l = np.array([2.0, 1.0, 1.0, 1.0, 0.0, -1.0], dtype=np.float32)
    pr = O.processed(l, 1.0, 2, 1.0, -np.inf)["probs"]
    assert (pr[:4] > 0).all() and (pr[4:] == 0).all()          # the k-th largest value ties three ways
    pr = O.processed(l, 1.0, 6, 0.6, -np.inf)["probs"]         # mass 0.49 for the top token: the cut falls in the tie
    assert (pr[:4] > 0).all() and (pr[4:] == 0).all()


def test_inverse_cdf_never_picks_zero_probability():
    """Reference tests/test_spec_accept.py:12-21."""
    rng = np.random.default_rng(1)
    P = np.exp(rng.standard_normal(50) * 1.5)
    P[7] = 0
    P /= P.sum()
    u = np.maximum(rng.random(20000).astype(np.float32), 1e-7)
    x = np.array([O.inverse_cdf_row(P, ui)[0] for ui in u])
    emp = np.bincount(x, minlength=50) / len(x)
    assert emp[7] == 0 and 0.5 * np.abs(emp - P).sum() < 0.02
    assert O.inverse_cdf_row(P, 1.0)[0] == 49 and O.inverse_cdf_row(P, 1e-7)[0] == 0


def test_argmax_lowest_index_on_ties():
    """Reference tests/test_grammar.py:131-133: outside the mask everything is -inf, the argmax is the lowest allowed."""
    l = np.zeros(64, dtype=np.float32)
    l[40] = 10
    mask = np.array([[-1, 0]], dtype=np.int32)                   # LowHalf: tokens 0..31
    res = O.draw_row(l, 0.0, 64, 1.0, -np.inf, 0.5, mask=mask[0])
    assert res["token"] == 0
    l[5] = 3
    assert O.draw_row(l, 0.0, 64, 1.0, -np.inf, 0.5, mask=mask[0])["token"] == 5


# ------------------------------------------------------------------------------------------------ penalties
def test_neutral_penalties_leave_every_bit():
    rng = np.random.default_rng(2)
    l = (rng.standard_normal(500) * 3).astype(np.float32)
    h = rng.integers(0, 500, 200)
    assert np.array_equal(O.penalties(l, h, 1.0, 0.0, 0.0).view(np.uint32), l.view(np.uint32))


def test_penalties_definition():
    l = np.array([2.0, -2.0, 1.0, 0.5, -1.0], dtype=np.float32)
    out = O.penalties(l, [0, 1, 1, 3, 3, 3, 9, -1], 2.0, 0.25, 0.5)
    want = np.array([2.0 / 2 - 0.5 * 1 - 0.25, -2.0 * 2 - 0.5 * 2 - 0.25, 1.0, 0.5 / 2 - 0.5 * 3 - 0.25, -1.0], dtype=np.float32)
    assert np.array_equal(out, want)


# ------------------------------------------------------------------------------------------------ accept
def test_spec_accept_lengths():
    """Reference tests/test_mtp4.py:285-312: n == j + 1 for j correct drafts, every n in 1..k+1 occurs."""
    k = 7
    pred = np.arange(100, 100 + k + 1)[None, :]
    for j in range(k + 1):
        drafts = pred[0, :k].copy()
        if j < k:
            drafts[j] = 5
        tok = np.concatenate([[1], drafts])[None, :]
        out, n = O.spec_accept(pred, tok, np.full((1, 8), -1), [1])
        assert n[0] == j + 1
        assert list(out[0, :j]) == list(pred[0, :j]) and out[0, j] == pred[0, j]


def test_spec_accept_stop_cut_and_inactive():
    pred = np.array([[10, 11, 12, 13]])
    tok = np.array([[1, 10, 11, 12]])
    out, n = O.spec_accept(pred, tok, np.array([[11, -1]]), [1])
    assert n[0] == 2 and out[0, 1] == 11                        # cut at the accepted stop token, which is emitted
    out, n = O.spec_accept(pred, tok, np.array([[12, -1]]), [1])
    assert n[0] == 3 and out[0, 2] == 12
    out, n = O.spec_accept(pred, tok, np.array([[13, -1]]), [1])
    assert n[0] == 4 and out[0, 3] == 13                        # the bonus token is not a draft: no cut
    out, n = O.spec_accept(pred, tok, np.array([[-1, -1]]), [0])
    assert n[0] == 0


def test_verify_reject_keeps_target_distribution():
    """Rejection sampling emits exactly p whatever q is: first emitted token over many uniform draws."""
    rng = np.random.default_rng(3)
    V, trials = 12, 6000
    tl = (rng.standard_normal((2, V)) * 1.5).astype(np.float32)
    dl = (tl[:1] + rng.standard_normal((1, V))).astype(np.float32)
    p = O.processed(tl[0], 1.0, V, 1.0, -np.inf)["probs"]
    q = O.processed(dl[0], 1.0, V, 1.0, -np.inf)["probs"]
    counts = np.zeros(V)
    for _ in range(trials):
        d, _m = O.inverse_cdf_row(q, max(rng.random(), 1e-7))
        r = O.spec_verify_reject(tl, dl, [d], 1.0, V, 1.0, -np.inf, [max(rng.random(), 1e-7)],
                                 np.maximum(rng.random(2), 1e-7).astype(np.float32))
        counts[d if r["n_accept"] == 1 else r["token"]] += 1
    assert 0.5 * np.abs(counts / trials - p).sum() < 0.03


# ------------------------------------------------------------------------------------------------ logprobs (reference vectors)
def _tie_groups_equal(ids_a, lp_a, ids_b, lp_b, tol):
    """Same values position by position; ids equal as sets inside every run of equal values (topk leaves ties open),
    except a run cut off by the end of the list, where either choice of tied tokens is a valid top-n."""
    ids_a, ids_b = np.asarray(ids_a), np.asarray(ids_b)
    lp_a, lp_b = np.asarray(lp_a, dtype=np.float64), np.asarray(lp_b, dtype=np.float64)
    both_inf = np.isinf(lp_a) & np.isinf(lp_b)
    with np.errstate(invalid="ignore"):
        assert np.all(both_inf | (np.abs(lp_a - lp_b) <= tol)), (lp_a, lp_b)
    i, n = 0, len(ids_a)
    while i < n:
        j = i
        while j + 1 < n and lp_b[j + 1] == lp_b[i]:
            j += 1
        if j + 1 < n:
            assert set(ids_a[i:j + 1].tolist()) == set(ids_b[i:j + 1].tolist()), (ids_a, ids_b)
        i = j + 1


def test_logprobs_match_reference_vectors():
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_logprobs.npz"))
    chosen, ids, lp = O.logprobs(g["small_rows"], g["small_toks"], 5)
    assert np.allclose(chosen, g["small_chosen"], atol=2e-6)
    for r in range(len(chosen)):
        _tie_groups_equal(ids[r], lp[r], g["small_top_ids"][r], g["small_top_lp"][r], 2e-6)
    c0, i0, l0 = O.logprobs(g["small_rows"], g["small_toks"], 0)
    assert np.allclose(c0, g["small_chosen_n0"], atol=2e-6) and i0.shape == (5, 0)
    import torch
    big = (torch.randn(3, 151936, generator=torch.Generator().manual_seed(int(g["big_seed"][0]))) * 2.5).numpy()
    chosen, ids, lp = O.logprobs(big, g["big_toks"], 20)
    assert np.allclose(chosen, g["big_chosen"], atol=5e-6)
    for r in range(3):
        _tie_groups_equal(ids[r], lp[r], g["big_top_ids"][r], g["big_top_lp"][r], 5e-6)


# ------------------------------------------------------------------------------------------------ draft-head rescoring
def _bf16_bits(t):
    import torch
    return t.bfloat16().view(torch.int16).numpy().view(np.uint16)


def test_rescore_oracles_equal_the_dense_products():
    """The reference's own tests (tests/test_draft_head.py:8-40) compare its kernels with the dense fp32 products of
    the candidate rows (rtol = atol = 1e-5 for BF16, 1e-4 for NVFP4): the oracle's ordered fp32 sums must as well."""
    import torch
    g = torch.Generator().manual_seed(1)
    V, K, B, C = 500, 2560, 3, 40
    w = (torch.randn(V, K, generator=g) * 0.02).bfloat16()
    x = torch.randn(B, K, generator=g).bfloat16()
    cand = torch.randint(0, V, (B, C), generator=g)
    out = O.rescore_bf16(_bf16_bits(x), _bf16_bits(w), cand.numpy())
    ref = torch.stack([w[cand[b]].double() @ x[b].double() for b in range(B)]).numpy()
    assert np.allclose(out, ref, rtol=1e-5, atol=1e-5)
    # row invariance: a slot alone, a prefix of the candidates
    assert np.array_equal(O.rescore_bf16(_bf16_bits(x[2:3]), _bf16_bits(w), cand[2:3].numpy()), out[2:3])
    assert np.array_equal(O.rescore_bf16(_bf16_bits(x), _bf16_bits(w), cand[:, :7].numpy()), out[:, :7])
    # NVFP4: random packed rows and scales
    K2 = 1024
    wq = torch.randint(0, 256, (V, K2 // 2), generator=g, dtype=torch.int64).to(torch.uint8)
    sf = torch.randint(0x20, 0x60, (V, K2 // 16), generator=g, dtype=torch.int64).to(torch.uint8)   # finite, moderate scales
    x2 = torch.randn(B, K2, generator=g).bfloat16()
    gs = 0.0123
    out = O.rescore_nvfp4(_bf16_bits(x2), wq.numpy(), sf.numpy(), gs, cand.numpy())
    lo, hi = wq & 0xF, wq >> 4
    tab = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float64)
    W = torch.empty(V, K2, dtype=torch.float64)
    W[:, 0::2], W[:, 1::2] = tab[lo.long()], tab[hi.long()]
    W = W * torch.from_numpy(O.e4m3_to_f64(sf.numpy())).repeat_interleave(16, 1) * gs
    ref = torch.stack([W[cand[b]] @ x2[b].double() for b in range(B)]).numpy()
    assert np.allclose(out, ref, rtol=1e-4, atol=1e-4)
    # E4M3 decode against torch's own cast
    codes = torch.arange(256, dtype=torch.int64).to(torch.uint8)
    want = codes.view(torch.float8_e4m3fn).double().numpy()
    got = O.e4m3_to_f64(codes.numpy())
    assert np.array_equal(np.isnan(got), np.isnan(want)) and np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])


def test_oracle_agrees_with_the_reference_expressions_run_on_a_gpu():
    """tests/golden/ref_gpu_vectors.npz: the reference's processed_probs / inverse_cdf expressions with the FlashInfer
    ops it calls, run on a B200 (make_gpu_golden.py).  The oracle must give the same tokens, the same kept sets (ties at
    a pivot all kept) and the same probabilities to 1e-5 relative."""
    import _ref_gpu
    g = _ref_gpu.load()
    n_rows = 0
    for name, w, u, lg in _ref_gpu.cases():
        p = w["params"]
        V = lg.shape[-1]
        for b in range(lg.shape[0]):
            T, k, tp, lmp = float(p["temperature"][b]), int(p["top_k"][b]), float(p["top_p"][b]), float(p["log_min_p"][b])
            r = O.draw_row(lg[b, 0], T, k, tp, lmp, u[b, 0])
            assert int(g[name + "_greedy"][b, 0]) == r["greedy"]
            tok = int(g[name + "_tok"][b, 0])
            assert tok == r["token"] or min(r["margin"], r["margin_top_p"]) < 1e-6, (name, b, tok, r)
            if not T > 0:
                continue
            pr = O.processed(lg[b, 0], T, k, tp, lmp)
            kept = pr["w"] > 0
            if k < V or tp < 1.0:                                  # (without a filter fp32 underflow alone decides the support)
                assert float(g[name + "_dropped_max_logit"][b, 0]) < float(g[name + "_kept_min_logit"][b, 0])
                if int(kept.sum()) != int(g[name + "_nkept"][b, 0]):
                    # the top-p target fell within 1e-6 of a cumulative-mass step: fp32 and float64 sums may cut one token apart
                    assert pr["margin_top_p"] < 1e-6 and abs(int(kept.sum()) - int(g[name + "_nkept"][b, 0])) <= 2, (name, b)
                    continue
                assert float(lg[b, 0][kept].min()) == float(g[name + "_kept_min_logit"][b, 0])
            ti, tv = g[name + "_top_idx"][b, 0], g[name + "_top_prob"][b, 0].astype(np.float64)
            assert np.allclose(pr["probs"][ti], tv, rtol=1e-5, atol=1e-30), (name, b)
            n_rows += 1
    assert n_rows >= 70
