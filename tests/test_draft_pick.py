"""The one-launch greedy draft of the low-rank draft heads (colinfer_draft_pick) against the oracle and against the
reference's own expressions (engine/spec/mtp.py:301-309, engine/spec/mtp4.py:416-423) run with torch on the same GPU.

The winning index, the token id and the exact logit are compared bit for bit (the candidate set, the accumulation
order of the exact logits and the tie rules are all defined); the probability at 1e-5 relative (the log-sum-exp is an
fp32 sum whose order differs from torch's)."""
import numpy as np
import pytest
import torch

from colinfer_b200 import _lib
from oracle import oracle as O

pytestmark = pytest.mark.gpu
P_RTOL = 1e-5


def _bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def _draft():
    from colinfer_b200.spec.draft import lowrank_draft
    assert torch.cuda.is_available(), "the gpu tests need a CUDA device"
    _lib.lib()
    return lowrank_draft


def _head(V, K, Vd, N, seed, perm=True):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(V, K, generator=g) * 0.05).bfloat16().cuda()
    x = torch.randn(N, K, generator=g).bfloat16().cuda()
    vid = (torch.randperm(V, generator=g)[:Vd] if perm else torch.arange(Vd)).cuda()
    # approximations that track the exact logits loosely, as a low-rank head does
    ap = (x.float() @ w[vid].float().T + 0.3 * torch.randn(N, Vd, generator=g).cuda()).contiguous()
    return w, x, vid, ap


def _check(out, ap, x, vid, n_cands, w=None, wq=None, sf=None, gs=None):
    ids, p, idx, ex = out
    want = O.draft_pick(ap.cpu().numpy(), _bits(x), None if vid is None else vid.cpu().numpy(), n_cands,
                        w_bits=None if w is None else _bits(w), w_u8=None if wq is None else wq.cpu().numpy(),
                        sf_u8=None if sf is None else sf.cpu().numpy(), gs=gs)
    assert np.array_equal(idx.cpu().numpy(), want[2]), (idx.cpu().numpy(), want[2])
    assert np.array_equal(ids.cpu().numpy(), want[0])
    assert np.array_equal(ex.cpu().numpy().view(np.uint32), want[3].view(np.uint32))
    np.testing.assert_allclose(p.cpu().numpy(), want[1], rtol=P_RTOL, atol=1e-30)
    return want


@pytest.mark.parametrize("ctas", [0, 1, 2, 4, 8, 16])
@pytest.mark.parametrize("N,Vd,K", [(1, 69632, 2560), (5, 20000, 264), (3, 4099, 64), (20, 147456, 64), (2, 160000, 64)])
def test_draft_pick_vs_oracle_bf16(ctas, N, Vd, K):
    draft = _draft()
    w, x, vid, ap = _head(Vd + 500, K, Vd, N, seed=Vd + K)
    out = draft(ap, x, w, vid, n_cands=256, ctas_per_slot=ctas, want_index=True)
    _check(out, ap, x, vid, 256, w=w)
    ids2, p2 = draft(ap, x, w, vid, n_cands=256, ctas_per_slot=ctas)
    assert torch.equal(ids2, out[0]) and torch.equal(p2, out[1])


def test_draft_pick_equals_the_references_expressions():
    """topk -> rescore -> argmax -> gathers -> exp(ex - logsumexp).clamp_max(1), with torch and this library's rescoring op
    (bit-identical to the reference's), on rows without equal approximations."""
    from colinfer_b200.kernels import ops
    draft = _draft()
    for N in (1, 16, 50, 200):
        w, x, vid, ap = _head(30000, 256, 24000, N, seed=N)
        ids, p = draft(ap, x, w, vid)
        cand = ap.topk(256, -1).indices
        ex = ops().rescore_bf16(x, w, vid[cand])
        best = ex.argmax(-1, keepdim=True)
        want_ids = vid[cand.gather(-1, best)].view(-1)
        want_p = torch.exp(ex.gather(-1, best) - torch.logsumexp(ap, -1, keepdim=True)).clamp_max(1.0).view(-1)
        assert torch.equal(ids, want_ids)
        torch.testing.assert_close(p, want_p, rtol=P_RTOL, atol=1e-30)


@pytest.mark.parametrize("K", [16, 1040])
def test_draft_pick_nvfp4(K):
    draft = _draft()
    g = torch.Generator().manual_seed(K)
    V, Vd, N = 6000, 5000, 4
    wq = torch.randint(0, 256, (V, K // 2), generator=g, dtype=torch.int64).to(torch.uint8).cuda()
    sf = torch.randint(0x20, 0x60, (V, K // 16), generator=g, dtype=torch.int64).to(torch.uint8).cuda()
    x = torch.randn(N, K, generator=g).bfloat16().cuda()
    vid = torch.randperm(V, generator=g)[:Vd].cuda()
    ap = torch.randn(N, Vd, generator=g).cuda()
    gs = 0.0131
    for ctas in (0, 1, 4):
        out = draft(ap, x, wq, vid, sf=sf, gs=gs, n_cands=64, ctas_per_slot=ctas, want_index=True)
        _check(out, ap, x, vid, 64, wq=wq, sf=sf, gs=gs)


@pytest.mark.parametrize("kind", ["crowded", "crowded_fine", "quantised", "all_equal", "mostly_minus_inf", "few_finite", "two_values"])
@pytest.mark.parametrize("ctas,Vd", [(0, 30011), (2, 30011), (16, 30012), (0, 30012), (4, 30012)])
def test_draft_pick_hard_rows(kind, ctas, Vd):
    """Rows whose values crowd into one histogram bin (the second and third level run), rows with many equal values at the
    NC-th place (index order decides; more of them than the collection holds: the ordered count runs), and rows that are
    mostly -inf."""
    draft = _draft()
    N, K, NC = 3, 128, 256                                      # Vd divisible by 4: the CTAs of a slot may share the row as a cluster
    w, x, vid, ap = _head(Vd + 100, K, Vd, N, seed=len(kind))
    g = torch.Generator().manual_seed(7)
    if kind == "crowded":
        ap = (10.0 + 1e-3 * torch.randn(N, Vd, generator=g)).cuda()
    elif kind == "crowded_fine":
        ap = (10.0 + 2e-6 * torch.randint(0, 40, (N, Vd), generator=g).float()).cuda()   # a few dozen adjacent floats
    elif kind == "quantised":
        ap = (torch.randn(N, Vd, generator=g) * 4).round().mul(0.5).cuda()
    elif kind == "all_equal":
        ap = torch.zeros(N, Vd).cuda()
    elif kind == "mostly_minus_inf":
        ap = torch.full((N, Vd), float("-inf"))
        pos = torch.randperm(Vd, generator=g)[:1000]
        ap[:, pos] = torch.randn(N, 1000, generator=g)
        ap = ap.cuda()
    elif kind == "few_finite":                                   # fewer finite values than candidates
        ap = torch.full((N, Vd), float("-inf"))
        ap[:, 5:105] = torch.randn(N, 100, generator=g)
        ap = ap.cuda()
    elif kind == "two_values":
        ap = (torch.rand(N, Vd, generator=g) < 0.5).float().cuda()
    out = draft(ap.contiguous(), x, w, vid, n_cands=NC, ctas_per_slot=ctas, want_index=True)
    _check(out, ap, x, vid, NC, w=w)


def test_draft_pick_small_and_identity_vocabulary():
    draft = _draft()
    w, x, _, ap = _head(300, 64, 300, 2, seed=3, perm=False)
    for nc in (1, 7, 300):
        out = draft(ap, x, w, None, n_cands=nc, want_index=True)
        want = _check(out, ap, x, None, nc, w=w)
        if nc == 1:
            assert np.array_equal(want[2], ap.argmax(-1).cpu().numpy())
        if nc == 300:                                            # every row is a candidate: the exact argmax
            exact = (w.float() @ x.float().T).T.argmax(-1)
            assert (out[2].long() == exact).float().mean() >= 0.5


def test_draft_pick_rows_outside_the_matrix_are_never_chosen():
    draft = _draft()
    w, x, vid, ap = _head(5000, 64, 4000, 2, seed=11)
    top = ap.topk(3, -1).indices
    vid2 = vid.clone()
    vid2[top[0, 0]] = 10 ** 9                                    # the best approximations of slot 0 point outside the matrix
    vid2[top[0, 1]] = -4
    ids, p, idx, ex = draft(ap, x, w, vid2, want_index=True)
    assert int(idx[0]) not in (int(top[0, 0]), int(top[0, 1])) and 0 <= int(ids[0]) < 5000
    assert torch.isfinite(ex).all()


def test_draft_pick_wrong_shapes_raise():
    draft = _draft()
    w, x, vid, ap = _head(600, 64, 500, 2, seed=5)
    with pytest.raises(RuntimeError):
        draft(ap, x[:, :60].contiguous(), w, vid)                # K must match w
    with pytest.raises(RuntimeError):
        draft(ap, x, w, vid[:-1])
    with pytest.raises(RuntimeError):
        draft(ap, x, w, vid, n_cands=501)
    with pytest.raises(RuntimeError):
        draft(ap.cpu(), x, w, vid)
    with pytest.raises(RuntimeError):
        draft(ap, x, w, vid, ctas_per_slot=3)


def test_draft_pick_inside_a_cuda_graph():
    draft = _draft()
    w, x, vid, ap = _head(9000, 128, 8000, 4, seed=9)
    eager = draft(ap, x, w, vid)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        draft(ap, x, w, vid)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            ids, p = draft(ap, x, w, vid)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(ids, eager[0]) and torch.equal(p, eager[1])
