"""The callers either side of the sampler: the mask rows' staging (engine/runtime/scheduler.py:222-223, 672-681) and the
bookkeeping after a cycle (scheduler.py:635-641), the latter kept on the device."""
import numpy as np
import pytest
import torch

from colinfer_b200 import _lib
from colinfer_b200.runtime.masks import RowMasks, mask_words
from oracle import oracle as O


class FakeConstraint:
    """Stands in for grammar.Constraint (llguidance is not part of this path): row i allows the tokens congruent to
    i + salt modulo 3, and rows after `refuse_at` are left as they are, as the real one leaves them."""

    def __init__(self, vocab, salt=0, refuse_at=None):
        self.vocab, self.salt, self.refuse_at = vocab, salt, refuse_at

    def masks(self, drafts, out):
        assert out.dtype == np.int32 and out.shape[0] == len(drafts) + 1
        for i in range(out.shape[0]):
            if self.refuse_at is not None and i > self.refuse_at:
                break
            allow = (np.arange(self.vocab) % 3) == ((i + self.salt) % 3)
            bits = np.zeros(out.shape[1] * 32, dtype=np.uint8)
            bits[:self.vocab] = allow
            out[i] = np.packbits(bits.reshape(-1, 32), axis=1, bitorder="little").view("<u4").reshape(-1).view(np.int32)


def test_row_masks_on_cpu_follow_the_reference_method():
    V = 1000
    rm = RowMasks(n_slots=3, margin=5, vocab=V, device="cpu", depth=2)
    assert rm.masks.shape == (3, 5, mask_words(V)) and int(rm.masks.min()) == -1
    for step in range(5):                                        # the ring comes round: nothing to wait for on CPU
        rows = rm.rows(FakeConstraint(V, salt=step), 1, [7, 8])
        assert rows.shape == (1, 3, mask_words(V))
        want = np.full((3, mask_words(V)), -1, dtype=np.int32)
        FakeConstraint(V, salt=step).masks([7, 8], want)
        assert np.array_equal(rows[0].numpy(), want)
    rows = rm.rows(FakeConstraint(V, refuse_at=0), 2, [1, 2, 3])   # rows after the refused draft stay all-ones
    assert int(rows[0, 1:].min()) == -1 and int(rows[0, 0].min()) != -1
    with pytest.raises(RuntimeError):
        rm.rows(FakeConstraint(V), 0, [0] * 5)
    rm.reset(1)
    assert int(rm.masks[1].min()) == -1 and rm.waits == 0


def test_spec_advance_oracle_matches_the_schedulers_lines():
    """tokens.append(y); tokens += o[:-1]; y = o[-1] (engine/runtime/scheduler.py:637-639) on Python lists."""
    rng = np.random.default_rng(0)
    B, k1, H = 6, 4, 8
    out_tok = rng.integers(0, 100, (B, k1))
    n = np.array([1, 4, 0, 2, 3, 4], dtype=np.int32)
    y = rng.integers(0, 100, B)
    hist = rng.integers(0, 100, (B, H)).astype(np.int32)
    hl = np.array([0, 2, 5, 7, 8, 6], dtype=np.int32)
    pos = np.arange(B) * 10
    y2, h2, hl2, pos2 = O.spec_advance(out_tok, n, y, hist, hl, pos)
    for b in range(B):
        tokens = list(hist[b, :hl[b]])
        if n[b] > 0:
            o = list(out_tok[b, :n[b]])
            tokens.append(y[b]); tokens += o[:-1]
            assert y2[b] == o[-1] and pos2[b] == pos[b] + n[b]
        else:
            assert y2[b] == y[b] and pos2[b] == pos[b]
        assert list(h2[b, :hl2[b]]) == tokens[-H:]


@pytest.mark.gpu
@pytest.mark.parametrize("B,k1,H", [(1, 1, 4), (7, 8, 16), (64, 9, 2048), (5, 4, 5000), (3, 4, 0)])
def test_spec_advance_vs_oracle(B, k1, H):
    from colinfer_b200.spec.verify import spec_advance
    _lib.lib()
    g = torch.Generator().manual_seed(B + H)
    out_tok = torch.randint(0, 150000, (B, k1), generator=g)
    n = torch.randint(0, k1 + 1, (B,), generator=g).int()
    y = torch.randint(0, 150000, (B,), generator=g)
    hist = torch.randint(0, 150000, (B, max(H, 1)), generator=g).int()[:, :H].contiguous()
    hl = torch.randint(0, H + 1, (B,), generator=g).int()
    if B > 2 and H:
        hl[0], hl[1] = H, max(H - 1, 0)                           # full and nearly full histories
    pos = torch.randint(0, 1000, (B,), generator=g)
    want = O.spec_advance(out_tok.numpy(), n.numpy(), y.numpy(), hist.numpy() if H else np.zeros((B, 0), np.int32), hl.numpy(), pos.numpy())
    d = [t.cuda() for t in (out_tok, n, y, hist, hl, pos)]
    if H:
        spec_advance(d[0], d[1], d[2], d[3], d[4], d[5])
    else:
        spec_advance(d[0], d[1], d[2], None, None, d[5])
    torch.cuda.synchronize()
    assert np.array_equal(d[2].cpu().numpy(), want[0]) and np.array_equal(d[5].cpu().numpy(), want[3])
    if H:
        assert np.array_equal(d[4].cpu().numpy(), want[2])
        for b in range(B):
            assert np.array_equal(d[3][b, :want[2][b]].cpu().numpy(), want[1][b, :want[2][b]])
    with pytest.raises(RuntimeError):
        spec_advance(d[0], d[1], d[2][:-1] if B > 1 else d[2].cpu(), None, None, None)


@pytest.mark.gpu
def test_a_penalised_cycle_keeps_its_history_on_the_device():
    """draw -> spec_accept -> spec_advance, three cycles: the history the penalties count in grows on the device exactly as
    the scheduler's token list does on the host."""
    from colinfer_b200.runtime.sampler import SamplerParams
    from colinfer_b200.spec.accept import draw
    from colinfer_b200.spec.verify import spec_accept, spec_advance
    B, k, V, H = 4, 3, 5000, 64
    g = torch.Generator().manual_seed(1)
    sp = SamplerParams(B, V, "cuda")
    for b in range(B):
        sp.set(b, temperature=0.0)
        sp.set_penalties(b, 1.3, 0.4, 0.2)
    hist = torch.zeros(B, H, dtype=torch.int32, device="cuda")
    hl = torch.zeros(B, dtype=torch.int32, device="cuda")
    sp.set_history(hist, hl)
    y = torch.randint(0, V, (B,), generator=g).cuda()
    pos = torch.zeros(B, dtype=torch.int64, device="cuda")
    tokens = [[] for _ in range(B)]
    y_host = y.cpu().tolist()
    for cycle in range(3):
        logits = (torch.randn(B, k + 1, V, generator=g) * 3).cuda()
        drafts = torch.randint(0, V, (B, k), generator=g).cuda()
        pred = draw(logits, sp, pos)
        drafts[:, 0] = pred[:, 0]                                 # the first draft is always accepted
        tok = torch.cat([y[:, None], drafts], 1)
        out_tok, n = spec_accept(pred, tok)
        # the host's version of the bookkeeping, from values read back (scheduler.py:635-639)
        nb, o = n.cpu().tolist(), out_tok.cpu().tolist()
        for b in range(B):
            tokens[b].append(y_host[b]); tokens[b] += o[b][:nb[b] - 1]; y_host[b] = o[b][nb[b] - 1]
        spec_advance(out_tok, n, y, hist, hl, pos)
        assert y.cpu().tolist() == y_host
        for b in range(B):
            assert hist[b, :int(hl[b])].cpu().tolist() == tokens[b]
        assert pos.cpu().tolist() == [len(t) for t in tokens]      # pos moved on by the emitted tokens
        # the next greedy draw is penalised with exactly these ids (the oracle gets the host's list)
        nxt = (torch.randn(B, 1, V, generator=g) * 3).cuda()
        got = draw(nxt, sp, pos)
        for b in range(B):
            want = O.draw_row(nxt[b, 0].cpu().numpy(), 0.0, V, 1.0, -np.inf, 1.0, history=np.array(tokens[b], dtype=np.int64),
                              rep=1.3, pres=0.4, freq=0.2)["token"]
            assert int(got[b, 0]) == int(want)


@pytest.mark.gpu
def test_row_masks_ring_and_zero_copy_feed_the_sampler():
    """The staged rows (copied, or read in place from pinned memory) give the tokens of the same rows on the device."""
    from colinfer_b200.runtime.sampler import SamplerParams
    from colinfer_b200.spec.accept import draw
    V, R = 4099, 3
    g = torch.Generator().manual_seed(2)
    logits = (torch.randn(1, R, V, generator=g) * 3).cuda()
    sp = SamplerParams(1, V, "cuda")
    sp.set(0, temperature=0.8, top_k=50, top_p=0.9, seed=5)
    pos = torch.tensor([3], device="cuda")
    ref_rows = np.full((R, mask_words(V)), -1, dtype=np.int32)
    FakeConstraint(V, salt=1).masks([1, 2], ref_rows)
    want = draw(logits, sp, pos, mask=torch.from_numpy(ref_rows)[None].cuda())
    assert all(int(t) % 3 == (i + 1) % 3 for i, t in enumerate(want[0].tolist()))
    for zero_copy in (False, True):
        rm = RowMasks(n_slots=2, margin=4, vocab=V, device="cuda", depth=2, zero_copy=zero_copy)
        for step in range(5):                                    # more steps than buffers: the ring comes round
            rows = rm.rows(FakeConstraint(V, salt=1), 0, [1, 2])
            got = draw(logits, sp, pos, mask=rows)
            rm.release()
            assert torch.equal(got, want)
        assert rows.is_cuda != zero_copy
