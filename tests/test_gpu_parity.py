"""Parity of the CUDA path (called through the C ABI) with the CPU oracle and with the reference's own pins.

Integer work (Philox words, masks, argmax, accept decisions, token ids) is compared bit for bit.  Sampled tokens must be
identical to the oracle's whenever the oracle's decision margins (distance of u * mass from the nearest CDF step, of
the top-p target from the nearest cumulative-mass step) exceed MARGIN; probabilities are compared at 1e-5 relative.
"""
import ctypes as C
import math
import os

import numpy as np
import pytest
import torch

from colinfer_b200 import _lib
from colinfer_b200 import workloads as wl
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MARGIN = 1e-6          # fp32 exponentials differ from float64 ones by ~1e-7 relative


@pytest.fixture(autouse=True, params=["auto", "stream"])
def _kernel_choice(request):
    """Every test runs twice: with the automatic kernel choice (few rows: cluster-resident kernel, else the streaming
    kernel) and with the streaming kernel forced, so that small cases cover both kernels."""
    assert torch.cuda.is_available(), "the gpu tests need a CUDA device"
    _lib.lib()
    _lib.default_kernel_flags = _lib.kernel_flags(0 if request.param == "auto" else -1)
    yield request.param
    _lib.default_kernel_flags = _lib.KERNEL_AUTO


def mods():
    from colinfer_b200.kernels import ops
    from colinfer_b200.runtime.sampler import SamplerParams, apply_mask, sample
    from colinfer_b200.spec.accept import draw, inverse_cdf, processed_probs
    from colinfer_b200.spec.verify import spec_accept, spec_verify
    return dict(ops=ops, SamplerParams=SamplerParams, apply_mask=apply_mask, sample=sample, draw=draw,
                inverse_cdf=inverse_cdf, processed_probs=processed_probs, spec_accept=spec_accept, spec_verify=spec_verify)


def np_params(p):
    d = {k: v.cpu().numpy() for k, v in p.items() if k not in ("history", "hist_len")}
    return d


def check_tokens(got, want, info, what=""):
    """Token identity, except where the oracle says the decision was closer than MARGIN to flipping."""
    got, want = np.asarray(got).reshape(-1), np.asarray(want).reshape(-1)
    bad = np.flatnonzero(got != want)
    for i in bad:
        m = min(info[i]["margin"], info[i]["margin_top_p"])
        assert m < MARGIN, f"{what}: row {i}: got {got[i]}, oracle {want[i]}, margin {m:.3e}"
    assert len(bad) <= max(1, len(got) // 200), f"{what}: {len(bad)} boundary rows of {len(got)}"
    print(f"[parity] {what}: {len(got)} rows, {len(bad)} differ from the oracle (all within the {MARGIN:g} margin)")
    return len(bad)


def run_workload(w, V, cluster=None, use_philox=False):
    """draw() on a workload dict vs the oracle.  Returns (#boundary mismatches, tokens)."""
    m = mods()
    if cluster is not None:
        _lib.default_kernel_flags = _lib.kernel_flags(cluster)
    dev = "cuda"
    logits = w["logits"].to(dev)
    sp = wl.sampler_params(w["params"], V, dev)
    mask = w.get("mask")
    u = w.get("u")
    pos = w["pos"].to(dev)
    kw = dict(mask=None if mask is None else mask.to(dev))
    if u is not None and not use_philox:
        kw["u"] = u.to(dev)
    out, st = m["draw"](logits, sp, pos, status=True, **kw)
    torch.cuda.synchronize()
    pr = np_params(w["params"])
    hist = w["params"].get("history")
    want, info = O.draw(logits.float().cpu().numpy(), pr, w["pos"].numpy(),
                        mask=None if mask is None else mask.numpy(),
                        history=None if hist is None else hist.numpy(),
                        hist_len=None if hist is None else w["params"]["hist_len"].numpy(),
                        u=None if (u is None or use_philox) else u.numpy())
    assert (st.cpu().numpy() & ~(_lib.ROW_HIST_SLOW | _lib.ROW_SELECT_SLOW) == 0).all(), st.unique()
    nb = check_tokens(out.cpu().numpy(), want, info, w.get("name", ""))
    return nb, out


# ------------------------------------------------------------------------------------------------ Philox
def test_philox_uniform_bit_exact_vs_oracle():
    m = mods()
    seed = torch.tensor([7, 7, 123, -5, 2**62 - 1], device="cuda")
    off = torch.tensor([0, 0, 5 << 20, (1 << 40) + 3, 2**33 + 1], device="cuda")
    for n in (1, 3, 16, 4096):
        u = torch.empty(5, n, device="cuda")
        m["ops"]().philox_uniform(seed, off, u)
        assert np.array_equal(u.cpu().numpy(), O.philox_uniform(seed.cpu().numpy(), off.cpu().numpy(), n))
    assert float(u.min()) > 0.0 and float(u.max()) <= 1.0
    with pytest.raises(RuntimeError):
        m["ops"]().philox_uniform(seed[:2], off, u)             # shape check, as the reference's binding raises


def test_philox_uniform_bit_exact_vs_reference_kernel():
    """The reference's own csrc/sampling.cu, built unmodified into oracle/_ref by oracle/Makefile."""
    path = os.path.join(ROOT, "oracle", "_ref", "libref_sampling.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libref_sampling.so was not built (needs the reference checkout at build time)")
    ref = C.CDLL(path)
    fn = getattr(ref, "_Z21launch_philox_uniformPKlS0_PfiiP11CUstream_st")
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    m = mods()
    g = torch.Generator().manual_seed(0)
    B = 64
    seed = torch.randint(-2**62, 2**62, (B,), generator=g).cuda()
    off = torch.randint(0, 2**40, (B,), generator=g).cuda()
    for n in (1, 9, 16, 700):
        a, b = torch.empty(B, n, device="cuda"), torch.zeros(B, n, device="cuda")
        m["ops"]().philox_uniform(seed, off, a)
        assert fn(seed.data_ptr(), off.data_ptr(), b.data_ptr(), B, n, torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(a, b)


# ------------------------------------------------------------------------------------------------ mask
def test_apply_mask_matches_reference_vectors(golden):
    m = mods()
    out = m["apply_mask"](torch.from_numpy(golden["mask_logits"]).cuda(), torch.from_numpy(golden["mask_words"]).cuda())
    assert np.array_equal(out.cpu().numpy(), golden["mask_out"])


@pytest.mark.parametrize("V", [1, 31, 33, 1000, 4099, 151936])
def test_apply_mask_sizes_and_identity(V):
    m = mods()
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(2, 2, V, generator=g)
    allowed = torch.rand(2, 2, V, generator=g) < 0.4
    mask = wl.pack_mask(allowed)
    out = m["apply_mask"](logits.cuda(), mask.cuda()).cpu()
    assert np.array_equal(out.numpy(), O.apply_mask(logits.numpy(), mask.numpy()))
    ones = torch.full_like(mask, -1)
    assert torch.equal(m["apply_mask"](logits.cuda(), ones.cuda()).cpu(), logits)       # all-ones: identity, new tensor


# ------------------------------------------------------------------------------------------------ draw: small grids
GRID = [(0.0, 0, 1.0, 0.0), (1.0, 0, 1.0, 0.0), (0.7, 20, 1.0, 0.0), (1.0, 0, 0.8, 0.0), (1.3, 50, 0.9, 0.05),
        (0.5, 1, 1.0, 0.0), (1.0, 0, 1e-4, 0.0), (1e-9, 0, 0.9, 0.0), (2.0, 5000, 0.999, 0.3)]


@pytest.mark.parametrize("cluster", [-1, 1, 2, 4, 8])
@pytest.mark.parametrize("V", [1, 31, 33, 1000, 4099])
def test_draw_vs_oracle_grid(V, cluster):
    m = mods()
    _lib.default_kernel_flags = _lib.kernel_flags(cluster)
    g = torch.Generator().manual_seed(100 + V)
    B, R = len(GRID), 2
    logits = torch.randn(B, R, V, generator=g) * 2
    sp = m["SamplerParams"](B, V, "cuda")
    for b, (T, k, tp, mp) in enumerate(GRID):
        sp.set(b, temperature=T, top_k=k, top_p=tp, min_p=mp, seed=b)
    u = wl.open_unit(g, B, R)
    allowed = torch.rand(B, R, V, generator=g) < 0.5
    allowed[..., V // 2] = True
    mask = wl.pack_mask(allowed)
    H = 48
    hist = torch.randint(0, V, (B, H), generator=g, dtype=torch.int32)
    hist[:, :8] = hist[:, 8:16]                                   # duplicates
    hist[:, 20] = V + 5                                            # out of range: skipped
    hist[:, 21] = -3
    sp.set_history(hist.cuda(), torch.full((B,), H - 4, dtype=torch.int32, device="cuda"))
    for b in range(B):
        sp.set_penalties(b, 1.3, 0.4, 0.25)
    out, st = m["draw"](logits.cuda(), sp, torch.zeros(B, dtype=torch.int32, device="cuda"), u=u.cuda(), mask=mask.cuda(),
                        status=True)
    pr = dict(temperature=sp.temperature.cpu().numpy(), top_k=sp.top_k.cpu().numpy(), top_p=sp.top_p.cpu().numpy(),
              log_min_p=sp.log_min_p.cpu().numpy(), repetition_penalty=sp.repetition_penalty.cpu().numpy(),
              presence_penalty=sp.presence_penalty.cpu().numpy(), frequency_penalty=sp.frequency_penalty.cpu().numpy())
    want, info = O.draw(logits.numpy(), pr, None, mask=mask.numpy(), history=hist.numpy(),
                        hist_len=np.full(B, H - 4), u=u.numpy())
    assert ((st & ~(_lib.ROW_HIST_SLOW | _lib.ROW_SELECT_SLOW)) == 0).all()   # slower exact paths are fine at toy sizes
    check_tokens(out.cpu().numpy(), want, info, f"V={V} cluster={cluster}")


def test_masked_argmax_picks_lowest_allowed_index():
    """Reference tests/test_grammar.py:116-160 (the LowHalf stub): next token has logit 10, all others 0; outside the
    mask the argmax is the lowest allowed token."""
    m = mods()
    V = 64
    logits = torch.zeros(3, 1, V)
    logits[0, 0, 40] = 10
    logits[1, 0, 5] = 10
    logits[2, 0, 31] = 10
    mask = torch.zeros(3, 1, 2, dtype=torch.int32)
    mask[:, :, 0] = -1
    sp = m["SamplerParams"](3, V, "cuda")
    out = m["draw"](logits.cuda(), sp, torch.zeros(3, dtype=torch.int32, device="cuda"), mask=mask.cuda())
    assert out[:, 0].tolist() == [0, 5, 31]
    masked = m["apply_mask"](logits.cuda(), mask.cuda())
    assert masked.argmax(-1)[:, 0].tolist() == [0, 5, 31]


def test_degenerate_rows_report_status_and_never_trap():
    m = mods()
    V = 200
    logits = torch.randn(3, 1, V)
    mask = torch.full((3, 1, 7), -1, dtype=torch.int32)
    mask[0] = 0                                                    # nothing allowed
    mask[1] = 0
    mask[1, 0, 3] = 1 << 9                                         # exactly one token allowed: 105
    sp = m["SamplerParams"](3, V, "cuda")
    for b in range(3):
        sp.set(b, temperature=1.0, top_k=10, top_p=0.9, seed=b)
    out, st = m["draw"](logits.cuda(), sp, torch.zeros(3, dtype=torch.int32, device="cuda"), mask=mask.cuda(), status=True)
    assert st[:, 0].tolist() == [_lib.ROW_DEGENERATE, 0, 0]
    assert out[0, 0] == 0 and out[1, 0] == 105 and 0 <= out[2, 0] < V
    assert m["draw"](torch.empty(0, 1, V, device="cuda"), m["SamplerParams"](0, V, "cuda"),
                     torch.zeros(0, dtype=torch.int32, device="cuda")).shape == (0, 1)


def test_bounded_wait_of_the_cluster_kernel_reports_a_timeout():
    """The cluster-resident kernel waits for its bulk copies with a limit.  With the test flag the copies are never
    issued (nothing is armed, nothing is in flight): every wait runs out, the rows report COLINFER_ROW_TIMEOUT, the
    kernel returns, and the next launch on the same context is clean."""
    m = mods()
    V, B = 151936, 4
    w = wl.config3(B, V=V, H=64)
    for k in ("history", "hist_len", "repetition_penalty", "presence_penalty", "frequency_penalty"):
        w["params"].pop(k)
    sp = wl.sampler_params(w["params"], V, "cuda")
    logits, pos = w["logits"].cuda(), w["pos"].cuda()
    good = m["draw"](logits, sp, pos, flags=_lib.KERNEL_CLUSTER[8])
    out, st = m["draw"](logits, sp, pos, status=True, flags=_lib.KERNEL_CLUSTER[8] | _lib.TEST_DROP_COPY)
    torch.cuda.synchronize()
    assert ((st & _lib.ROW_TIMEOUT) != 0).all()
    again, st2 = m["draw"](logits, sp, pos, status=True, flags=_lib.KERNEL_CLUSTER[8])
    assert torch.equal(again, good) and int(st2.abs().sum()) == 0


def test_neutral_penalties_are_a_bit_exact_no_op():
    m = mods()
    V, B = 4099, 6
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(B, 1, V, generator=g) * 2).cuda()
    hist = torch.randint(0, V, (B, 300), generator=g, dtype=torch.int32).cuda()
    pos = torch.arange(B, dtype=torch.int32, device="cuda")
    outs = []
    for with_hist in (False, True):
        sp = m["SamplerParams"](B, V, "cuda")
        for b in range(B):
            sp.set(b, temperature=0.9 if b else 0.0, top_k=0, top_p=0.95, seed=b + 3)
        if with_hist:
            sp.set_history(hist)
            sp.set_penalties(0, 1.0, 0.0, 0.0)
        o, rs = m["draw"](logits, sp, pos, stats=True)
        outs.append((o, rs))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("rp", [1.2, 0.8])
@pytest.mark.parametrize("cluster", [-1, 1])
def test_many_distinct_history_ids_use_the_slow_count_path(cluster, rp):
    """More than 2048 distinct history ids in one table: counts come from scanning the history.  The streaming kernel
    builds no table for a greedy row whose penalties can only lower a logit (rp >= 1) as long as its lists decide it."""
    m = mods()
    V, H = 8192, 6000
    _lib.default_kernel_flags = _lib.kernel_flags(cluster)
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(1, 1, V, generator=g) * 2
    hist = torch.randint(0, V, (1, H), generator=g, dtype=torch.int32)
    sp = m["SamplerParams"](1, V, "cuda")
    sp.set(0, temperature=0.0)
    sp.set_history(hist.cuda())
    sp.set_penalties(0, rp, 0.3, 0.7)
    out, st = m["draw"](logits.cuda(), sp, torch.zeros(1, dtype=torch.int32, device="cuda"), status=True)
    want = O.argmax(O.penalties(logits[0, 0].numpy(), hist[0].numpy(), rp, 0.3, 0.7))
    assert int(out) == want
    if cluster == -1 and rp >= 1.0:
        assert int(st) in (0, _lib.ROW_HIST_SLOW)      # (the tables are built after all when the lists do not decide the row)
    else:
        assert int(st) == _lib.ROW_HIST_SLOW


@pytest.mark.parametrize("V", [20000, 151936])
@pytest.mark.parametrize("k,tp", [(0, 0.6), (3000, 1.0), (5000, 0.7), (0, 0.999), (40, 0.9)])
@pytest.mark.parametrize("pen", [False, True])
def test_heavy_ties_take_the_exact_select(V, k, tp, pen):
    """Thousands of equal logits around the pivot overflow every candidate list: the radix select must give the same
    kept set (all ties kept) and the same draw as the oracle -- also for penalised slots, whose rows start on the
    patch-afterwards path and have to leave it."""
    g = torch.Generator().manual_seed(V + k)
    B = 6
    logits = torch.randn(B, 1, V, generator=g)
    tie = torch.randperm(V, generator=g)[:8000]
    logits[:, 0, tie] = 3.25                                       # 8000 tokens share the maximum
    logits[1::2, 0, tie[:10]] = 5.0                                # odd rows: a small head above the plateau
    params = wl._params(B, V, 0.9, k, tp, 0.0, list(range(11, 11 + B)))
    if pen:
        H = 300
        hist = torch.randint(0, V, (B, H), generator=g, dtype=torch.int32)
        hist[:, :40] = tie[:40].to(torch.int32)                    # penalties hit the plateau and the head
        params.update(history=hist, hist_len=torch.full((B,), H, dtype=torch.int32),
                      repetition_penalty=torch.full((B,), 1.3), presence_penalty=torch.full((B,), 0.25),
                      frequency_penalty=torch.full((B,), 0.1))
    w = dict(logits=logits, params=params, pos=torch.arange(B, dtype=torch.int32), u=wl.open_unit(g, B, 1), name="ties")
    nb, out = run_workload(w, V)
    assert nb == 0


# ------------------------------------------------------------------------------------------------ processed_probs / inverse_cdf
def test_processed_probs_known_answers():
    """Reference tests/test_spec_accept.py:39-48."""
    m = mods()
    logits = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]], device="cuda"))
    one = lambda v, dt=torch.float32: torch.tensor([v], dtype=dt, device="cuda")  # noqa: E731
    want = torch.tensor([0.625, 0.375, 0, 0], device="cuda")
    p = m["processed_probs"](logits, one(1.0), one(2, torch.int32), one(1.0), one(float("-inf")))
    torch.testing.assert_close(p[0], want, atol=1e-5, rtol=0)
    p = m["processed_probs"](logits, one(1.0), one(4, torch.int32), one(0.7), one(float("-inf")))
    torch.testing.assert_close(p[0], want, atol=1e-5, rtol=0)
    p = m["processed_probs"](logits, one(1.0), one(4, torch.int32), one(1.0), one(math.log(0.4)))
    torch.testing.assert_close(p[0], want, atol=1e-5, rtol=0)


@pytest.mark.parametrize("V", [1000, 151936])
@pytest.mark.parametrize("T,k,tp,mp", [(1.0, 0, 1.0, 0.0), (0.7, 20, 1.0, 0.0), (1.0, 0, 0.8, 0.0), (1.3, 50, 0.9, 0.05), (0.0, 0, 0.9, 0.0)])
def test_processed_probs_vs_oracle(V, T, k, tp, mp):
    m = mods()
    g = torch.Generator().manual_seed(V + k)
    logits = torch.randn(3, V, generator=g) * 2
    prm = O.sampler_params_set(V, T, k, tp, mp)
    one = lambda v, dt: torch.tensor([v], dtype=dt, device="cuda")  # noqa: E731
    got = m["processed_probs"](logits.cuda(), one(float(prm["temperature"]), torch.float32), one(int(prm["top_k"]), torch.int32),
                               one(float(prm["top_p"]), torch.float32), one(float(prm["log_min_p"]), torch.float32)).cpu().numpy()
    for r in range(3):
        pr = O.processed(logits[r].numpy(), prm["temperature"], prm["top_k"], prm["top_p"], prm["log_min_p"])
        if pr["margin_top_p"] < MARGIN:
            continue
        want = pr["probs"]
        assert np.array_equal(got[r] > 0, want > 1e-44), "support set"
        nz = want > 1e-30
        assert np.allclose(got[r][nz], want[nz], rtol=1e-5, atol=0)
        assert abs(got[r].astype(np.float64).sum() - 1.0) < 1e-5


def test_inverse_cdf_matches_reference_vectors(golden):
    m = mods()
    out = m["inverse_cdf"](torch.from_numpy(golden["icdf_P"]).cuda(), torch.from_numpy(golden["icdf_u"]).cuda())
    assert np.array_equal(out.cpu().numpy(), golden["icdf_out"])
    out = m["inverse_cdf"](torch.from_numpy(golden["icdf_W"]).cuda(), torch.from_numpy(golden["icdf_uw"]).cuda())
    assert np.array_equal(out.cpu().numpy(), golden["icdf_wout"])


def test_inverse_cdf_row_without_mass_gives_index_zero():
    """engine/spec/accept.py:36-40 counts the prefixes below u * total: none when the row has no mass at all."""
    m = mods()
    P = torch.zeros(3, 77, device="cuda")
    P[1, 40] = 0.25
    out = m["inverse_cdf"](P, torch.tensor([0.3, 0.3, 1.0], device="cuda"))
    assert out.tolist() == [0, 40, 0]


def test_inverse_cdf_marginal_is_exact():
    """Reference tests/test_spec_accept.py:12-21."""
    m = mods()
    torch.manual_seed(0)
    V, trials = 50, 200000
    P = torch.softmax(torch.randn(1, V, device="cuda") * 1.5, -1)
    P[0, 7] = 0
    P /= P.sum()
    x = m["inverse_cdf"](P.expand(trials, V).contiguous(), torch.rand(trials, device="cuda").clamp_min(1e-7))
    emp = torch.bincount(x, minlength=V).float() / trials
    assert emp[7] == 0
    assert 0.5 * (emp - P[0]).abs().sum().item() < 0.01


# ------------------------------------------------------------------------------------------------ the reference's sampler tests
def expected(logits, t, k, p, min_p):
    """The reference's exact truncated softmax (tests/test_sampler.py:13-27), on the CPU in float64."""
    z = logits.double() / t
    probs = torch.softmax(z, -1)
    keep = probs >= min_p * probs.max()
    order = torch.argsort(z, descending=True)
    keep_k = torch.zeros_like(keep)
    keep_k[order[:k]] = True
    keep &= keep_k
    pr = torch.softmax(z.masked_fill(~keep, float("-inf")), -1)
    srt, idx = torch.sort(pr, descending=True)
    cut = (srt.cumsum(0) - srt) < p
    final = torch.zeros_like(pr)
    final[idx[cut]] = srt[cut]
    return final / final.sum()


@pytest.mark.parametrize("t,k,p,min_p", [(1.0, 0, 1.0, 0.0), (0.7, 20, 1.0, 0.0), (1.0, 0, 0.8, 0.0), (1.3, 50, 0.9, 0.05)])
def test_distribution(t, k, p, min_p):
    """Reference tests/test_sampler.py:30-49: 100k draws, nothing outside the allowed set, total variation < 0.03."""
    m = mods()
    V = 1000
    torch.manual_seed(0)
    base = torch.randn(V) * 2
    B, rounds = 4000, 25
    params = m["SamplerParams"](B, V, "cuda")
    params.temperature.fill_(t)
    params.top_k.fill_(k if k > 0 else V)
    params.top_p.fill_(p)
    params.log_min_p.fill_(math.log(min_p) if min_p > 0 else float("-inf"))
    params.seed.copy_(torch.arange(B, device="cuda") * 7919)
    counts = torch.zeros(V, device="cuda")
    logits = base.cuda().expand(B, V).contiguous()
    for r in range(rounds):
        counts += torch.bincount(m["sample"](logits, params, torch.full((B,), r, device="cuda")), minlength=V).float()
    emp = (counts / counts.sum()).cpu().double()
    want = expected(base, t, k if k > 0 else V, p, min_p)
    assert emp[want == 0].sum() == 0, "sampled a token outside the allowed set"
    assert 0.5 * (emp - want).abs().sum().item() < 0.03


def test_slot_independence():
    """Reference tests/test_sampler.py:52-62."""
    m = mods()
    V = 1000
    torch.manual_seed(3)
    logits = torch.randn(2, V, device="cuda")
    outs = []
    for other_seed in (0, 12345):
        p = m["SamplerParams"](2, V, "cuda")
        p.set(0, temperature=1.0, seed=other_seed)
        p.set(1, temperature=1.0, seed=9)
        outs.append([int(m["sample"](logits, p, torch.full((2,), i, device="cuda"))[1]) for i in range(10)])
    assert outs[0] == outs[1]


def test_greedy_slots_and_seed_determinism():
    """Reference tests/test_sampler.py:65-78."""
    m = mods()
    V = 1000
    torch.manual_seed(1)
    logits = torch.randn(3, V, device="cuda")
    p = m["SamplerParams"](3, V, "cuda")
    p.set(0, temperature=0.0)
    p.set(1, temperature=1.0, seed=7)
    p.set(2, temperature=1.0, seed=7)
    pos = lambda i: torch.full((3,), i, device="cuda")  # noqa: E731
    out = m["sample"](logits, p, pos(0))
    assert out[0] == logits[0].argmax()
    a = [int(m["sample"](logits, p, pos(i))[1]) for i in range(20)]
    b = [int(m["sample"](logits, p, pos(i))[1]) for i in range(20)]
    assert a == b and len(set(a)) > 1
    assert [int(m["sample"](logits[[1, 1, 1]], p, pos(i))[2]) for i in range(20)] == a


def test_captured_in_cuda_graph_follows_position():
    """Reference tests/test_sampler.py:81-101: capturable, the position is read from device memory at replay."""
    m = mods()
    V = 1000
    torch.manual_seed(2)
    logits = torch.zeros(2, V, device="cuda")
    p = m["SamplerParams"](2, V, "cuda")
    p.set(0, temperature=1.0, seed=3)
    p.set(1, temperature=1.0, seed=4)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    pos = torch.zeros(2, dtype=torch.int32, device="cuda")
    with torch.cuda.stream(s):
        m["sample"](logits, p, pos)
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = m["sample"](logits, p, pos)
        pos += 1
    draws = []
    for _ in range(30):
        g.replay()
        draws.append(tuple(out.tolist()))
    assert len(set(draws)) > 20


def test_draw_rows_match_single_row_draws():
    """Reference tests/test_spec_accept.py:24-36 (V = 248,320, R = 4): verifying k+1 rows at once draws what k+1
    single-row steps draw at those positions."""
    m = mods()
    torch.manual_seed(1)
    V, R = 248320, 4
    logits = torch.randn(2, R, V, device="cuda") * 3
    p = m["SamplerParams"](2, V, "cuda")
    p.set(0, temperature=0.8, top_k=20, top_p=0.95, seed=11)
    p.set(1, temperature=1.0, top_p=0.9, min_p=0.02, seed=12)
    pos = torch.tensor([100, 7], device="cuda", dtype=torch.int32)
    many = m["draw"](logits, p, pos)
    one = torch.stack([m["draw"](logits[:, r:r + 1].contiguous(), p, pos + r)[:, 0] for r in range(R)], 1)
    assert torch.equal(many, one)
    # and the oracle agrees, Philox uniforms included
    pr = dict(temperature=p.temperature.cpu().numpy(), top_k=p.top_k.cpu().numpy(), top_p=p.top_p.cpu().numpy(),
              log_min_p=p.log_min_p.cpu().numpy(), seed=p.seed.cpu().numpy())
    want, info = O.draw(logits.cpu().numpy(), pr, pos.cpu().numpy())
    check_tokens(many.cpu().numpy(), want, info, "V=248320")


# ------------------------------------------------------------------------------------------------ benchmark configurations
def test_config0_single_row():
    w = wl.config0()
    nb, out = run_workload(w, wl.V_QWEN)
    assert nb == 0
    # greedy on the same logits (temperature 0): the argmax of the penalised row
    w["params"]["temperature"] = torch.zeros(1)
    nb, out = run_workload(w, wl.V_QWEN)
    assert nb == 0
    # and with the Philox uniform at (seed, pos) instead of the explicit one
    w = wl.config0()
    assert run_workload(w, wl.V_QWEN, use_philox=True)[0] == 0


def test_config1_grammar_mask():
    w = wl.config1()
    assert run_workload(w, wl.V_QWEN)[0] == 0
    w["params"]["temperature"] = torch.zeros(1)
    nb, out = run_workload(w, wl.V_QWEN)
    allowed = O.mask_bits(w["mask"][0, 0].numpy(), wl.V_QWEN)
    assert nb == 0 and allowed[int(out)]


@pytest.mark.parametrize("B", [8, 64])
def test_config3_batched_sweep_vs_oracle(B):
    w = wl.config3(B)
    nb, _ = run_workload(w, wl.V_QWEN, use_philox=True)
    assert nb == 0                                                 # on these seeds no row differs at all


def test_config3_all_1024_rows_vs_oracle():
    """The benchmarked batch itself, every row against the oracle (the oracle runs on the host cores in parallel)."""
    from _oracle_pool import oracle_draw_rows
    m = mods()
    B, V = 1024, wl.V_QWEN
    w = wl.config3(B)
    sp = wl.sampler_params(w["params"], V, "cuda")
    out, st = m["draw"](w["logits"].cuda(), sp, w["pos"].cuda(), status=True)
    torch.cuda.synchronize()
    want, info = oracle_draw_rows(w["logits"].numpy(), np_params(w["params"]), w["pos"].numpy(),
                                  history=w["params"]["history"].numpy(), hist_len=w["params"]["hist_len"].numpy())
    assert (st.cpu().numpy() & ~(_lib.ROW_HIST_SLOW | _lib.ROW_SELECT_SLOW) == 0).all()
    assert check_tokens(out.cpu().numpy(), want, info, "config3 B=1024, all rows") == 0


def test_config4_all_512_rows_vs_oracle():
    """The bf16 large-vocabulary stress at full size (512 x 262,144, 30 % grammar mask), every row against the oracle."""
    from _oracle_pool import oracle_draw_rows
    m = mods()
    V = wl.V_LARGE
    w = wl.config4()
    sp = wl.sampler_params(w["params"], V, "cuda")
    out, st = m["draw"](w["logits"].cuda(), sp, w["pos"].cuda(), mask=w["mask"].cuda(), status=True)
    torch.cuda.synchronize()
    want, info = oracle_draw_rows(w["logits"].float().numpy(), np_params(w["params"]), w["pos"].numpy(), mask=w["mask"].numpy())
    assert (st.cpu().numpy() & ~_lib.ROW_SELECT_SLOW == 0).all()
    got = out.cpu().numpy()
    assert check_tokens(got, want, info, "config4 B=512, all rows") == 0
    for b in range(0, 512, 37):
        assert O.mask_bits(w["mask"][b, 0].numpy(), V)[int(got[b, 0])]


def test_config3_full_batch_properties():
    """B = 1024 at full size: deterministic across launches, independent of the batch a row rides in (row invariance),
    and equal to the oracle on a sample of rows."""
    m = mods()
    B, V = 1024, wl.V_QWEN
    w = wl.config3(B)
    dev = "cuda"
    logits = w["logits"].to(dev)
    sp = wl.sampler_params(w["params"], V, dev)
    pos = w["pos"].to(dev)
    a = m["draw"](logits, sp, pos)
    b = m["draw"](logits, sp, pos)
    assert torch.equal(a, b)
    a, st = m["draw"](logits, sp, pos, status=True)
    assert torch.equal(a, b)
    # the oracle sample: fixed rows plus every row that took a slower exact path (a missed band estimate, a full list)
    slow = torch.nonzero(st.reshape(-1) != 0).reshape(-1).tolist()
    rows = sorted(set([0, 1, 17, 333, 512, 1023] + slow[:10]))
    for r in rows:
        one = m["draw"](logits[r:r + 1].contiguous(), sp.view(r, r + 1), pos[r:r + 1].contiguous())
        assert torch.equal(one[0], a[r])
    perm = torch.randperm(B, generator=torch.Generator().manual_seed(0))
    sp2 = wl.sampler_params({k: v[perm] for k, v in w["params"].items()}, V, dev)
    c = m["draw"](logits[perm.to(dev)].contiguous(), sp2, pos[perm.to(dev)].contiguous())
    assert torch.equal(c, a[perm.to(dev)])
    sub = {k: (v[rows] if isinstance(v, torch.Tensor) and v.size(0) == B else v) for k, v in w.items() if k != "params"}
    sub["params"] = {k: v[rows] for k, v in w["params"].items()}
    want, info = O.draw(sub["logits"].numpy(), np_params(sub["params"]), sub["pos"].numpy(),
                        history=sub["params"]["history"].numpy(), hist_len=sub["params"]["hist_len"].numpy())
    check_tokens(a[rows].cpu().numpy(), want, info, "config3 B=1024 sample")
    # every sampled token lies in [0, V) and greedy rows would be the penalised argmax
    assert int(a.min()) >= 0 and int(a.max()) < V


def test_missed_band_estimate_retries_exactly(_kernel_choice):
    """The top-p band is an estimate; with the test hook it is misplaced (above the pivot on odd rows, below on even
    ones): the exact window pass must find the pivot's bucket and the tokens must not change."""
    if _kernel_choice != "stream":
        pytest.skip("the hook belongs to the streaming kernel")
    m = mods()
    V = wl.V_QWEN
    w = wl.config3(32)
    w["params"]["top_k"][:] = V                                     # top-p rows only
    dev = "cuda"
    logits, pos = w["logits"].to(dev), w["pos"].to(dev)
    for strip in (False, True):
        pr = dict(w["params"])
        if strip:
            for k in ("history", "hist_len", "repetition_penalty", "presence_penalty", "frequency_penalty"):
                pr.pop(k)
        sp = wl.sampler_params(pr, V, dev)
        a, sa = m["draw"](logits, sp, pos, status=True)
        b, sb = m["draw"](logits, sp, pos, status=True, flags=_lib.TEST_MISS_BAND)
        assert torch.equal(a, b)
        assert int((sb & _lib.ROW_SELECT_SLOW).ne(0).sum()) >= 24   # the hook took effect
        assert int((sa & _lib.ROW_SELECT_SLOW).ne(0).sum()) <= 2
    want, info = O.draw(w["logits"].numpy(), np_params(w["params"]), w["pos"].numpy(),
                        history=w["params"]["history"].numpy(), hist_len=w["params"]["hist_len"].numpy())
    sp = wl.sampler_params(w["params"], V, dev)
    got = m["draw"](logits, sp, pos, flags=_lib.TEST_MISS_BAND)
    check_tokens(got.cpu().numpy(), want, info, "missed band")


def test_config4_bf16_large_vocab():
    w = wl.config4(B=6)
    nb, out = run_workload(w, wl.V_LARGE, use_philox=True)
    allowed = np.stack([O.mask_bits(w["mask"][b, 0].numpy(), wl.V_LARGE) for b in range(6)])
    assert all(allowed[b, int(out[b, 0])] for b in range(6))


# ------------------------------------------------------------------------------------------------ speculative verify
def test_spec_accept_vs_oracle():
    m = mods()
    g = torch.Generator().manual_seed(11)
    for k in (1, 3, 7, 15):
        B = 257
        pred = torch.randint(0, 6, (B, k + 1), generator=g)
        tok = torch.randint(0, 6, (B, k + 1), generator=g)
        agree = torch.rand(B, k, generator=g) < 0.7
        tok[:, 1:] = torch.where(agree, pred[:, :k], tok[:, 1:])
        stop = torch.randint(-1, 8, (B, 8), generator=g)
        stop[stop > 5] = -1
        active = (torch.rand(B, generator=g) < 0.9).int()
        out, n = m["spec_accept"](pred.cuda(), tok.cuda(), stop.cuda(), active.cuda())
        want_out, want_n = O.spec_accept(pred.numpy(), tok.numpy(), stop.numpy(), active.numpy())
        assert np.array_equal(n.cpu().numpy(), want_n) and np.array_equal(out.cpu().numpy(), want_out)
        out2, n2 = m["spec_accept"](pred.cuda(), tok.cuda())
        w2o, w2n = O.spec_accept(pred.numpy(), tok.numpy(), np.full((B, 1), -1), np.ones(B))
        assert np.array_equal(n2.cpu().numpy(), w2n) and np.array_equal(out2.cpu().numpy(), w2o)


def test_spec_accept_lengths_cover_every_n():
    """Reference tests/test_mtp4.py:285-312: n == j + 1 for j correct drafts."""
    m = mods()
    k = 7
    pred = torch.arange(100, 100 + k + 1)[None].repeat(k + 1, 1)
    tok = torch.ones(k + 1, k + 1, dtype=torch.int64)
    tok[:, 1:] = pred[:, :k]
    for j in range(k):
        tok[j, 1 + j] = 5
    out, n = m["spec_accept"](pred.cuda(), tok.cuda())
    assert n.tolist() == list(range(1, k + 2))
    for j in range(k + 1):
        assert out[j, j] == pred[j, j]


def _stub_logits(ctx, V):
    """A deterministic stand-in for a model: the logits of the next token are a fixed function of the last three tokens."""
    seed = 0
    for t in ctx[-3:]:
        seed = (seed * 1000003 + int(t) + 17) % (2**31 - 1)
    return torch.randn(V, generator=torch.Generator().manual_seed(seed)) * 2.0


@pytest.mark.parametrize("sampled", [False, True])
def test_speculative_cycles_reproduce_plain_decoding(sampled):
    """The reference's end-to-end property (tests/test_mtp4.py:284-328): cycles of verify -- draw() over the k + 1 rows
    at positions pos + r, then the exact-match accept -- emit the same stream as decoding one token at a time with
    sample(), whatever the drafts are; every accept length 1 .. k + 1 occurs."""
    m = mods()
    V, k, N = 4096, 2, 48
    sp = m["SamplerParams"](1, V, "cuda")
    if sampled:
        sp.set(0, temperature=0.8, top_k=50, top_p=0.95, seed=1234)
    prompt = [3, 1, 4, 1, 5]
    # plain decoding: the token at sequence index p is drawn with the uniform at counter p
    want = list(prompt)
    for _ in range(N + 8):
        row = _stub_logits(want, V)[None].cuda()
        want.append(int(m["sample"](row, sp, torch.tensor([len(want)], dtype=torch.int32, device="cuda"))))
    g = torch.Generator().manual_seed(5)
    seq, seen = list(prompt), set()
    while len(seq) < len(prompt) + N:
        n0 = len(seq)
        j = int(torch.randint(0, k + 1, (1,), generator=g))        # j right drafts, then a wrong one
        drafts = [want[n0 + i] for i in range(k)]
        if j < k:
            drafts[j] = (drafts[j] + 1) % V
        rows = torch.stack([_stub_logits(seq + drafts[:r], V) for r in range(k + 1)])[None].cuda()   # [1, k + 1, V]
        pred = m["draw"](rows, sp, torch.tensor([n0], dtype=torch.int32, device="cuda"))
        tok = torch.tensor([[seq[-1]] + drafts], dtype=torch.int64, device="cuda")
        out_tok, n = m["spec_accept"](pred, tok)
        n = int(n[0])
        assert n == j + 1
        seen.add(n)
        seq += out_tok[0, :n].tolist()
    assert seq[:len(prompt) + N] == want[:len(prompt) + N]
    assert seen == set(range(1, k + 2))


def verify_case(target, draft, ud, ua, us, params, V, k, mask=None):
    """Draft tokens are drawn from the draft's processed distribution with ud; then the verify is compared."""
    m = mods()
    B = target.shape[0]
    sp = wl.sampler_params(params, V, "cuda")
    kw = {} if mask is None else dict(mask=mask[:, :k].contiguous().cuda())
    d_ids = m["draw"](draft.cuda(), sp, None, u=ud.cuda(), **kw)
    out, n = m["spec_verify"](target.cuda(), draft.cuda(), d_ids, sp, ua.cuda(), us.cuda(),
                              mask=None if mask is None else mask.cuda())
    torch.cuda.synchronize()
    out, n, d_np = out.cpu().numpy(), n.cpu().numpy(), d_ids.cpu().numpy()
    pr = np_params(params)
    boundary = 0
    for b in range(B):
        r = O.spec_verify_reject(target[b].float().numpy(), draft[b].float().numpy(), d_np[b], pr["temperature"][b], pr["top_k"][b],
                                 pr["top_p"][b], pr["log_min_p"][b], ua[b].numpy(), us[b].numpy(),
                                 target_mask=None if mask is None else mask[b].numpy())
        ok = (n[b] == r["n_accept"] + 1 and out[b, r["n_accept"]] == r["token"]
              and list(out[b, :r["n_accept"]]) == list(d_np[b, :r["n_accept"]]) and (out[b, n[b]:] == -1).all())
        if not ok:
            assert min(r["margin"], r["accept_margin"]) < 1e-5, (b, n[b], out[b], r)
            boundary += 1
    assert boundary <= max(1, B // 100)
    return n


def test_config2_speculative_verify_greedy_and_sampled():
    w = wl.config2()
    V, k = wl.V_QWEN, w["k"]
    n = verify_case(w["target"], w["draft"], w["ud"], w["ua"], w["us"], w["params"], V, k)
    assert 1 <= int(n[0]) <= k + 1
    greedy = dict(w["params"])
    greedy["temperature"] = torch.zeros(1)
    verify_case(w["target"], w["draft"], w["ud"], w["ua"], w["us"], greedy, V, k)


def test_spec_verify_small_vocab_many_slots():
    g = torch.Generator().manual_seed(21)
    B, k, V = 96, 4, 1000
    target = torch.randn(B, k + 1, V, generator=g) * 2
    draft = (target[:, :k] + torch.randn(B, k, V, generator=g) * 0.7).contiguous()
    allowed = torch.rand(B, k + 1, V, generator=g) < 0.6
    allowed[..., 3] = True
    params = wl._params(B, V, torch.where(torch.arange(B) % 5 == 0, 0.0, 0.9), 40, 0.9, 0.02)
    n = verify_case(target, draft, wl.open_unit(g, B, k), wl.open_unit(g, B, k), wl.open_unit(g, B, k + 1), params, V, k,
                    mask=wl.pack_mask(allowed))
    assert len(set(n.tolist())) >= 3                               # several accept lengths occur


def test_spec_verify_never_accepts_a_token_the_target_excludes():
    """Drafts that are not drawn from q (a suffix or argmax drafter): a draft id the grammar mask forbids, or one outside
    the target's top-k, has p = 0 (and possibly q = 0 too) -- it must be rejected and never emitted."""
    m = mods()
    g = torch.Generator().manual_seed(77)
    B, k, V = 64, 3, 512
    target = torch.randn(B, k + 1, V, generator=g) * 2
    draft = (target[:, :k] + torch.randn(B, k, V, generator=g) * 0.3).contiguous()
    allowed = torch.rand(B, k + 1, V, generator=g) < 0.7
    allowed[..., 5] = True
    mask = wl.pack_mask(allowed)
    params = wl._params(B, V, 0.8, 10, 1.0, 0.0)
    sp = wl.sampler_params(params, V, "cuda")
    # even slots: the first draft is a masked token; odd slots: the target's 30th largest allowed logit (outside top-10)
    d_ids = torch.zeros(B, k, dtype=torch.int64)
    for b in range(B):
        row = target[b, 0].clone()
        if b % 2 == 0:
            d_ids[b, 0] = int(torch.nonzero(~allowed[b, 0])[0])
        else:
            row[~allowed[b, 0]] = -float("inf")
            d_ids[b, 0] = int(torch.argsort(row, descending=True)[29])
        d_ids[b, 1:] = 5
    ua = torch.full((B, k), 1e-7)                                  # the most permissive accept uniforms
    us = wl.open_unit(g, B, k + 1)
    out, n = m["spec_verify"](target.cuda(), draft.cuda(), d_ids.cuda(), sp, ua.cuda(), us.cuda(), mask=mask.cuda())
    out, n = out.cpu(), n.cpu()
    assert (n == 1).all()                                          # rejected at the first position
    for b in range(B):
        tok = int(out[b, 0])
        assert tok != int(d_ids[b, 0]) and bool(allowed[b, 0, tok])
        r = O.spec_verify_reject(target[b].numpy(), draft[b].numpy(), d_ids[b].numpy(), 0.8, 10, 1.0, -np.inf, ua[b].numpy(),
                                 us[b].numpy(), target_mask=mask[b].numpy())
        assert r["n_accept"] == 0
        assert tok == r["token"] or r["margin"] < 1e-5


def test_error_paths_raise_and_do_not_crash():
    """Errors found behind the tensor checks -- a vocabulary beyond the kernels' limit, a slot count that does not match --
    come back as RuntimeError with the numbers in the message (formatting them once crashed an extension that had been
    linked against a second copy of the C++ runtime)."""
    m = mods()
    V = 600000                                                     # beyond the streaming kernel's penalty bitmap and the clusters' slices
    logits = torch.zeros(1, 1, V, device="cuda")
    sp = m["SamplerParams"](1, V, "cuda")
    sp.set(0, temperature=1.0, top_k=5, top_p=0.9, seed=1)
    pos = torch.zeros(1, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError):
        m["draw"](logits, sp, pos, flags=_lib.kernel_flags(8))
    sp2 = m["SamplerParams"](2, 1000, "cuda")
    with pytest.raises(RuntimeError, match="slot"):
        m["draw"](torch.zeros(1, 1, 1000, device="cuda"), sp2, pos)


def test_spec_verify_and_the_mass_horizon():
    """A draft token the kernels give no mass (more than ~21.5 temperatures below the target row's maximum; p ~ 1e-11 in
    float64) counts as excluded by the target and is rejected, whatever the draft thought of it; one well above the
    horizon follows the oracle's accept test.  Found by a randomised sweep with drafts that were not drawn from q."""
    m = mods()
    V, k, T = 2000, 1, 0.5
    g = torch.Generator().manual_seed(4)
    target = torch.randn(2, k + 1, V, generator=g)
    target[:, 0, 7] = 20.0                                         # the maximum of the first row
    target[0, 0, 11] = 20.0 - 25.0 * T                             # slot 0's draft: 25 temperatures below it
    target[1, 0, 11] = 20.0 - 10.0 * T                             # slot 1's draft: 10 temperatures below it
    draft = target[:, :k].clone()
    draft[:, 0, 11] -= 5.0                                         # the drafter likes it even less: q < p, the test would accept
    d_ids = torch.full((2, k), 11, dtype=torch.int64)
    params = wl._params(2, V, T, 0, 1.0, 0.0)
    sp = wl.sampler_params(params, V, "cuda")
    ua, us = torch.full((2, k), 0.5), torch.full((2, k + 1), 0.4)
    out, n = m["spec_verify"](target.cuda(), draft.cuda(), d_ids.cuda(), sp, ua.cuda(), us.cuda())
    r0 = O.spec_verify_reject(target[0].numpy(), draft[0].numpy(), d_ids[0].numpy(), T, V, 1.0, -np.inf, ua[0].numpy(), us[0].numpy())
    r1 = O.spec_verify_reject(target[1].numpy(), draft[1].numpy(), d_ids[1].numpy(), T, V, 1.0, -np.inf, ua[1].numpy(), us[1].numpy())
    assert r0["n_accept"] == 1 and r1["n_accept"] == 1             # in float64 both drafts pass p > 0 and ua * q <= p
    assert int(n[0]) == 1 and int(out[0, 0]) != 11                 # below the horizon: rejected, another token emitted
    assert int(n[1]) == 2 and int(out[1, 0]) == 11 and int(out[1, 1]) == r1["token"]


def test_spec_verify_with_penalties_vs_oracle():
    """The slot's penalties apply to every target and draft row of the verify (this project's definition).  Histories hold
    the targets' most likely tokens and the drafts themselves, so that acceptance and the residual both depend on them;
    neutral factors leave the result of the penalty-free call."""
    m = mods()
    for (B, k, V, H) in [(24, 3, 5000, 64), (3, 4, wl.V_QWEN, 2048)]:
        g = torch.Generator().manual_seed(B + V)
        target = torch.randn(B, k + 1, V, generator=g) * 2.5
        draft = (target[:, :k] + torch.randn(B, k, V, generator=g) * 0.6).contiguous()
        params = wl._params(B, V, torch.where(torch.arange(B) % 6 == 0, 0.0, 0.8), 50, 0.95, 0.0)
        hist = torch.randint(0, V, (B, H), generator=g, dtype=torch.int64)
        top = target[:, :k].topk(8, -1).indices.reshape(B, -1)          # the most likely tokens of every target row
        hist[:, :top.size(1)] = top
        hist[:, top.size(1):2 * top.size(1)] = top                      # twice: counts of 2
        hist[:, -3:] = torch.tensor([-1, V, V + 7])                     # ids outside the vocabulary are skipped
        hl = torch.randint(2 * top.size(1), H + 1, (B,), generator=g, dtype=torch.int64)
        rep = torch.where(torch.arange(B) % 4 == 3, 1.0, 1.3)
        pres = torch.where(torch.arange(B) % 4 == 3, 0.0, 0.5)
        freq = torch.where(torch.arange(B) % 4 == 3, 0.0, 0.25)
        sp = wl.sampler_params(params, V, "cuda")
        for b in range(B):
            sp.set_penalties(b, float(rep[b]), float(pres[b]), float(freq[b]))
        sp.set_history(hist.int().cuda(), hl.int().cuda())
        ud, ua, us = wl.open_unit(g, B, k), wl.open_unit(g, B, k), wl.open_unit(g, B, k + 1)
        d_ids = m["draw"](draft.cuda(), sp, None, u=ud.cuda())           # drafts drawn from the penalised q
        out, n = m["spec_verify"](target.cuda(), draft.cuda(), d_ids, sp, ua.cuda(), us.cuda())
        out, n, d_np = out.cpu().numpy(), n.cpu().numpy(), d_ids.cpu().numpy()
        pr = np_params(params)
        boundary, lens = 0, set()
        for b in range(B):
            r = O.spec_verify_reject(target[b].numpy(), draft[b].numpy(), d_np[b], pr["temperature"][b], pr["top_k"][b], pr["top_p"][b],
                                     pr["log_min_p"][b], ua[b].numpy(), us[b].numpy(), history=hist[b, :int(hl[b])].numpy(),
                                     rep=float(rep[b]), pres=float(pres[b]), freq=float(freq[b]))
            ok = (n[b] == r["n_accept"] + 1 and out[b, r["n_accept"]] == r["token"]
                  and list(out[b, :r["n_accept"]]) == list(d_np[b, :r["n_accept"]]))
            lens.add(int(n[b]))
            if not ok:
                assert min(r["margin"], r["accept_margin"]) < 1e-5, (b, n[b], out[b], r)
                boundary += 1
        assert boundary <= 1 and len(lens) >= 2
        # neutral factors: the penalty-free call, bit for bit
        sp0 = wl.sampler_params(params, V, "cuda")
        base = m["spec_verify"](target.cuda(), draft.cuda(), d_ids, sp0, ua.cuda(), us.cuda())
        for b in range(B):
            sp0.set_penalties(b, 1.0, 0.0, 0.0)
        sp0.set_history(hist.int().cuda(), hl.int().cuda())
        neutral = m["spec_verify"](target.cuda(), draft.cuda(), d_ids, sp0, ua.cuda(), us.cuda())
        assert torch.equal(base[0], neutral[0]) and torch.equal(base[1], neutral[1])
        # and the penalties do change decisions on these inputs
        assert not (torch.equal(base[0].cpu(), torch.from_numpy(out)) and torch.equal(base[1].cpu(), torch.from_numpy(n)))


def test_spec_verify_preserves_the_target_distribution():
    """The first emitted token of a rejection verify follows p_0 whatever the draft distribution is."""
    m = mods()
    V, B = 64, 60000
    g = torch.Generator().manual_seed(4)
    tl = torch.randn(1, 2, V, generator=g) * 1.5
    dl = tl[:, :1] + torch.randn(1, 1, V, generator=g)
    sp = m["SamplerParams"](B, V, "cuda")
    sp.temperature.fill_(1.0)
    target = tl.expand(B, 2, V).contiguous().cuda()
    draft = dl.expand(B, 1, V).contiguous().cuda()
    d_ids = m["draw"](draft, sp, None, u=wl.open_unit(g, B, 1).cuda())
    out, n = m["spec_verify"](target, draft, d_ids, sp, wl.open_unit(g, B, 1).cuda(), wl.open_unit(g, B, 2).cuda())
    emp = torch.bincount(out[:, 0], minlength=V).double().cpu() / B
    p = torch.softmax(tl[0, 0].double(), -1)
    assert 0.5 * (emp - p).abs().sum().item() < 0.02


# ------------------------------------------------------------------------------------------------ the reference's GPU arithmetic
def test_kernels_agree_with_the_reference_expressions_run_on_a_gpu():
    """tests/golden/ref_gpu_vectors.npz (the reference's processed_probs / inverse_cdf expressions with FlashInfer, run on
    a B200): same tokens from draw() -- penalties, mask and filters fused -- and, from processed_probs, the same kept
    sets and probabilities to 1e-5 relative."""
    import _ref_gpu
    m = mods()
    g = _ref_gpu.load()
    one = lambda v, dt=torch.float32: torch.tensor([v], dtype=dt, device="cuda")  # noqa: E731
    for name, w, u, lg in _ref_gpu.cases():
        V = lg.shape[-1]
        sp = wl.sampler_params(w["params"], V, "cuda")
        mask = w.get("mask")
        out = m["draw"](w["logits"].cuda(), sp, None, u=torch.from_numpy(u).cuda(), mask=None if mask is None else mask.cuda())
        got, want = out.cpu().numpy().reshape(-1), g[name + "_tok"].reshape(-1)
        p = w["params"]
        for b in np.flatnonzero(got != want):
            r = O.draw_row(lg[b, 0], float(p["temperature"][b]), int(p["top_k"][b]), float(p["top_p"][b]), float(p["log_min_p"][b]), u[b, 0])
            assert min(r["margin"], r["margin_top_p"]) < MARGIN, (name, b, got[b], want[b])
        print(f"[parity] {name}: {len(got)} rows, {int((got != want).sum())} differ from the FlashInfer vectors")
        for b in range(0, lg.shape[0], 7):                          # processed_probs on the effective logits of some rows
            T, k, tp, lmp = float(p["temperature"][b]), int(p["top_k"][b]), float(p["top_p"][b]), float(p["log_min_p"][b])
            if not T > 0:
                continue
            P = m["processed_probs"](torch.from_numpy(lg[b]).cuda(), one(T), one(k, torch.int32), one(tp), one(lmp))[0].cpu().numpy()
            if (k < V or tp < 1.0) and int((P > 0).sum()) != int(g[name + "_nkept"][b, 0]):
                assert O.processed(lg[b, 0], T, k, tp, lmp)["margin_top_p"] < MARGIN, (name, b)   # a cut within the margin of a step
            ti, tv = g[name + "_top_idx"][b, 0], g[name + "_top_prob"][b, 0]
            assert np.allclose(P[ti], tv, rtol=1e-5, atol=1e-30), (name, b)


# ------------------------------------------------------------------------------------------------ the mass horizon
# Masses are integers in units of 2^-30 of the largest token's: a logit more than ~21.5 temperatures below the maximum
# has mass 0 and can never be drawn, one a little above that is rounded coarsely.  Against the reference's fp32 softmax
# this moves at most V * 2^-31 of the mass (7.1e-5 at 151,936 tokens) -- the bound the next tests pin.
HORIZON_BOUND = 151936 * 2.0 ** -31


def _bulk_row(gap_t, T, V=151936, seed=3):
    """One dominant token; every other logit `gap_t` temperatures below it (with a little jitter)."""
    g = torch.Generator().manual_seed(seed)
    row = 3.0 - gap_t * T + 0.05 * torch.randn(V, generator=g)
    row[1000] = 3.0
    return row


@pytest.mark.parametrize("gap_t", [18.0, 20.0, 21.0, 23.0, 24.0])
def test_mass_horizon_moves_at_most_its_bound(gap_t):
    m = mods()
    V, T = 151936, 0.7
    row = _bulk_row(gap_t, T)
    one = lambda v, dt=torch.float32: torch.tensor([v], dtype=dt, device="cuda")  # noqa: E731
    got = m["processed_probs"](row[None].cuda(), one(T), one(V, torch.int32), one(1.0), one(float("-inf")))[0].cpu().numpy().astype(np.float64)
    pr = O.processed(row.numpy(), T, V, 1.0, -np.inf)
    want = pr["probs"]
    assert np.abs(got - want).sum() <= 2.0 * HORIZON_BOUND + 1e-6      # total variation <= the bound
    assert not np.any((got > 0) & ~(want > 0))                          # nothing outside the reference's support
    assert np.all(want[(want > 0) & ~(got > 0)] <= 2.0 ** -30)          # what is dropped is below one mass unit each
    # draws: the token's interval of the reference CDF lies within the bound of u
    us = [0.5, 0.99999, 1.0 - 2.0 ** -24, 1.0]
    sp = m["SamplerParams"](len(us), V, "cuda")
    for b in range(len(us)):
        sp.set(b, temperature=T, seed=b)
    toks = m["draw"](row[None, None].expand(len(us), 1, V).contiguous().cuda(), sp, None, u=torch.tensor(us, device="cuda")[:, None])
    cdf = np.cumsum(want)
    for u, t in zip(us, toks[:, 0].tolist()):
        assert want[t] > 0
        lo, hi = (cdf[t - 1] if t else 0.0), cdf[t]
        assert lo - 2.0 * HORIZON_BOUND <= np.float32(u) <= hi + 2.0 * HORIZON_BOUND, (u, t, lo, hi)


def test_top_k_reaching_below_the_horizon_keeps_the_reference_support_above_it():
    """A peaked row whose k-th largest logit lies below the horizon: the reference keeps k tokens, 49 of them with
    probability ~1e-13; here they carry no mass.  The probabilities agree to far better than 1e-5."""
    m = mods()
    V, T = 151936, 1.0
    row = _bulk_row(30.0, T, seed=5)
    one = lambda v, dt=torch.float32: torch.tensor([v], dtype=dt, device="cuda")  # noqa: E731
    got = m["processed_probs"](row[None].cuda(), one(T), one(50, torch.int32), one(1.0), one(float("-inf")))[0].cpu().numpy().astype(np.float64)
    want = O.processed(row.numpy(), T, 50, 1.0, -np.inf)["probs"]
    assert int((want > 0).sum()) == 50 and got[1000] > 0
    assert not np.any((got > 0) & ~(want > 0))
    assert np.abs(got - want).sum() < 1e-9


# ------------------------------------------------------------------------------------------------ logprobs of emitted tokens
def _check_logprobs(rows, toks, n_top, tol=2e-5):
    from colinfer_b200.runtime.logprobs import logprobs_tensors
    from test_oracle import _tie_groups_equal
    chosen, ids, lps = logprobs_tensors(rows.cuda().contiguous(), torch.tensor(toks, dtype=torch.int64, device="cuda"), n_top)
    wc, wi, wl_ = O.logprobs(rows.float().numpy(), np.asarray(toks), n_top)
    got_c = chosen.cpu().numpy().astype(np.float64)
    both_inf = np.isinf(got_c) & np.isinf(wc)
    with np.errstate(invalid="ignore"):
        assert np.all(both_inf | (np.abs(got_c - wc) <= tol)), (got_c, wc)
    for r in range(rows.size(0)):
        _tie_groups_equal(ids[r].cpu().numpy(), lps[r].cpu().numpy(), wi[r], wl_[r], tol)
    return chosen, ids, lps


def test_logprobs_match_reference_vectors_on_gpu():
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_logprobs.npz"))
    from colinfer_b200.runtime.logprobs import logprobs
    from test_oracle import _tie_groups_equal
    res = logprobs(torch.from_numpy(g["small_rows"]).cuda(), g["small_toks"].tolist(), 5)
    for r, (lp, alts) in enumerate(res):
        assert abs(lp - g["small_chosen"][r]) <= 2e-5
        _tie_groups_equal([a[0] for a in alts], [a[1] for a in alts], g["small_top_ids"][r], g["small_top_lp"][r], 2e-5)
    assert [x[1] for x in logprobs(torch.from_numpy(g["small_rows"]).cuda(), g["small_toks"].tolist(), 0)] == [[]] * 5
    big = torch.randn(3, 151936, generator=torch.Generator().manual_seed(int(g["big_seed"][0]))) * 2.5
    res = logprobs(big.cuda(), g["big_toks"].tolist(), 20)
    for r, (lp, alts) in enumerate(res):
        assert abs(lp - g["big_chosen"][r]) <= 2e-5
        _tie_groups_equal([a[0] for a in alts], [a[1] for a in alts], g["big_top_ids"][r], g["big_top_lp"][r], 2e-5)


@pytest.mark.parametrize("V", [1, 31, 33, 1000, 4099, 151936])
@pytest.mark.parametrize("n_top", [0, 1, 5, 20])
def test_logprobs_vs_oracle(V, n_top):
    if n_top > V:
        pytest.skip("n_top <= V")
    g = torch.Generator().manual_seed(V * 31 + n_top)
    rows = torch.randn(5, V, generator=g) * 3
    if V > 40:
        rows[1, 5:9] = rows[1].max() + 2.0                          # ties at the top
        rows[2, ::2] = -math.inf                                    # half masked
        rows[3] = rows[3].sort().values                             # ascending: every batch raises the bound
    toks = [int(t) for t in torch.randint(0, V, (5,), generator=g)]
    _check_logprobs(rows, toks, n_top)


def test_logprobs_long_ties_take_the_slow_path_and_bf16():
    V = 151936
    g = torch.Generator().manual_seed(5)
    rows = torch.randn(3, V, generator=g)
    rows[0, torch.randperm(V, generator=g)[:9000]] = 4.5            # 9000 equal maxima: every list overflows
    rows[1] = 0.0                                                   # a constant row
    toks = [7, 0, V - 1]
    _, ids, _ = _check_logprobs(rows, toks, 20)
    assert ids[1].tolist() == list(range(20))                       # equal logits: lower token first
    _check_logprobs(rows.bfloat16().float(), toks, 20)              # same values through the bf16 loader
    from colinfer_b200.runtime.logprobs import logprobs_tensors
    c16, i16, l16 = logprobs_tensors(rows.bfloat16().cuda(), torch.tensor(toks, device="cuda"), 20)
    c32, i32, l32 = logprobs_tensors(rows.bfloat16().float().cuda(), torch.tensor(toks, device="cuda"), 20)
    assert torch.equal(i16, i32) and torch.allclose(l16, l32, atol=1e-6) and torch.allclose(c16, c32, atol=1e-6)


# ------------------------------------------------------------------------------------------------ draft-head rescoring
def _bf16_bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def _ref_sampling_lib():
    path = os.path.join(ROOT, "oracle", "_ref", "libref_sampling.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libref_sampling.so was not built (needs the reference checkout at build time)")
    return C.CDLL(path)


@pytest.mark.parametrize("K", [8, 264, 2560, 5120])
def test_rescore_bf16_bit_exact(K):
    """Bit-identical to the oracle's ordered fp32 sums and to the reference's own kernel; close to the dense product
    (tests/test_draft_head.py:25-40 of the reference); row invariant; wrong shapes raise."""
    ops = mods()["ops"]()
    g = torch.Generator().manual_seed(K)
    V, B, NC = 5000, 4, 256
    w = (torch.randn(V, K, generator=g) * 0.02).bfloat16().cuda()
    x = torch.randn(B, K, generator=g).bfloat16().cuda()
    cand = torch.randint(0, V, (B, NC), generator=g).cuda()
    out = ops.rescore_bf16(x, w, cand)
    ref = torch.stack([w[cand[b]].float() @ x[b].float() for b in range(B)])
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    want = O.rescore_bf16(_bf16_bits(x), _bf16_bits(w), cand.cpu().numpy())
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert torch.equal(ops.rescore_bf16(x[2:3].contiguous(), w, cand[2:3].contiguous()), out[2:3])
    assert torch.equal(ops.rescore_bf16(x, w, cand[:, :7].contiguous()), out[:, :7])
    if K > 8:
        with pytest.raises(RuntimeError):
            ops.rescore_bf16(x, w[:, :K - 4].contiguous(), cand)    # K must match x
    lib = _ref_sampling_lib()
    fn = getattr(lib, "_Z19launch_rescore_bf16PKvS0_PKlPfiiiP11CUstream_st")
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    theirs = torch.zeros(B, NC, device="cuda")
    assert fn(x.data_ptr(), w.data_ptr(), cand.data_ptr(), theirs.data_ptr(), B, K, NC, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, theirs)


@pytest.mark.parametrize("K", [16, 1040, 5120])
def test_rescore_nvfp4_bit_exact(K):
    ops = mods()["ops"]()
    g = torch.Generator().manual_seed(K + 1)
    V, B, NC = 3000, 3, 64
    wq = torch.randint(0, 256, (V, K // 2), generator=g, dtype=torch.int64).to(torch.uint8).cuda()
    sf = torch.randint(0x20, 0x60, (V, K // 16), generator=g, dtype=torch.int64).to(torch.uint8).cuda()
    x = torch.randn(B, K, generator=g).bfloat16().cuda()
    cand = torch.randint(0, V, (B, NC), generator=g).cuda()
    gs = 0.00731
    out = ops.rescore_nvfp4(x, wq, sf, gs, cand)
    want = O.rescore_nvfp4(_bf16_bits(x), wq.cpu().numpy(), sf.cpu().numpy(), gs, cand.cpu().numpy())
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert torch.equal(ops.rescore_nvfp4(x[1:2].contiguous(), wq, sf, gs, cand[1:2].contiguous()), out[1:2])
    lib = _ref_sampling_lib()
    fn = getattr(lib, "_Z20launch_rescore_nvfp4PKvS0_S0_fPKlPfiiiP11CUstream_st")
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    theirs = torch.zeros(B, NC, device="cuda")
    assert fn(x.data_ptr(), wq.data_ptr(), sf.data_ptr(), gs, cand.data_ptr(), theirs.data_ptr(), B, K, NC,
              torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, theirs)


def test_rescore_bad_candidate_ids_give_nan_not_a_fault():
    ops = mods()["ops"]()
    V, K = 100, 64
    w = torch.randn(V, K).bfloat16().cuda()
    x = torch.randn(1, K).bfloat16().cuda()
    cand = torch.tensor([[0, V, -1, 5]], device="cuda")
    out = ops.rescore_bf16(x, w, cand)
    assert torch.isnan(out[0, 1]) and torch.isnan(out[0, 2]) and torch.isfinite(out[0, [0, 3]]).all()


# ------------------------------------------------------------------------------------------------ peaked rows
@pytest.mark.parametrize("gap", [3.0, 12.0, 40.0])
@pytest.mark.parametrize("pen", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_peaked_rows_vs_oracle(gap, pen, dtype):
    """Rows as a language model produces them: a handful of tokens far above a broad bulk.  The sample that places the
    fine histogram usually misses them (the row maximum lies `gap` above everything else, up to beyond the histogram's
    range), nuclei are a few tokens wide, and penalties hit exactly the leading tokens."""
    V, B = wl.V_QWEN, 24
    g = torch.Generator().manual_seed(int(gap * 10) + pen)
    logits = torch.randn(B, 1, V, generator=g) * 1.5
    for b in range(B):
        lead = torch.randperm(V, generator=g)[:1 + b % 5]
        logits[b, 0, lead] = logits[b, 0].max() + gap - 0.7 * torch.arange(len(lead), dtype=torch.float32)
    T = [0.6, 1.0, 1.4][0:3] * (B // 3)
    top_k = ([0] * 6 + [40] * 3 + [2000] * 3) * 2
    top_p = ([0.5, 0.9, 0.99, 0.999, 1.0, 0.95] * 4)
    min_p = [0.0] * 20 + [0.02] * 4
    params = wl._params(B, V, T, top_k, top_p, min_p, list(range(100, 100 + B)))
    if pen:
        H = 64
        hist = torch.randint(0, V, (B, H), generator=g, dtype=torch.int32)
        hist[:, 0] = logits[:, 0].argmax(-1).to(torch.int32)       # the leading token was just emitted
        hist[:, 1] = hist[:, 0]
        params.update(history=hist, hist_len=torch.full((B,), H, dtype=torch.int32),
                      repetition_penalty=torch.full((B,), 1.2), presence_penalty=torch.full((B,), 0.4),
                      frequency_penalty=torch.full((B,), 0.3))
    logits = logits.to(dtype)                                       # bf16: a hundred tokens share every value of the bulk
    w = dict(logits=logits, params=params, pos=torch.arange(B, dtype=torch.int32), u=wl.open_unit(g, B, 1), name="peaked")
    nb, out = run_workload(w, V)
    assert nb <= 1
