"""CPU oracle of colinfer's logits -> token path.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import this module; the product
package never does (it has no CPU path at all and raises when its CUDA library is missing).

It restates, in numpy, what the reference computes on this path.  fp32 steps that the reference performs as single
IEEE operations (the division by the temperature, the row maximum, the min-p threshold add and compare, the penalty
multiply / subtract) are done in numpy float32 and are therefore bit-identical to any correct implementation.  Steps
whose rounding the reference itself does not fix (the softmax exponentials and every sum: torch sums in a device
dependent order and FlashInfer's renormalisation uses float atomics) are evaluated in float64, i.e. the oracle returns
the mathematically exact answer for the fp32 inputs, together with *margins* that say how far each discrete decision
(top-p cut, inverse-CDF crossing) was from flipping.  A fp32 implementation must agree with the oracle on every decision
whose margin is not vanishing.

Reference lines followed (paths inside the colinfer tree):
  philox_uniform      csrc/sampling.cu:11-30
  apply_mask          engine/runtime/sampler.py:50-56 (bit t%32 of word t//32), engine/runtime/grammar.py:28-30
  sampler_params_set  engine/runtime/sampler.py:40-47
  processed           engine/spec/accept.py:23-33 (temperature -> min-p -> softmax -> top-k renorm -> top-p renorm);
                      the two FlashInfer calls (flashinfer-python 0.7.0.post1, not part of the tree) are restated from
                      their published behaviour: top-k keeps every probability >= the k-th largest; top-p keeps every
                      probability >= the value at which the descending cumulative mass first reaches top_p; both divide
                      by the kept sum.  tests/test_sampler.py:13-27 is the reference's own CPU restatement of the same
                      filters and is cross-checked in the tests.
  inverse_cdf         engine/spec/accept.py:36-40
  draw                engine/spec/accept.py:43-52
  spec_accept         engine/spec/mtp.py:406-415, 422-423
Not in the reference (defined by this project, parity unpinned): penalties(), spec_verify_reject().
"""
from __future__ import annotations

import math

import numpy as np

F32 = np.float32
NEG_INF = F32(-np.inf)

# ---------------------------------------------------------------------------------------------------- Philox
_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(counter, key):
    """Philox4x32-10 (Salmon et al. 2011).  counter: 4 uint32 arrays (or ints), key: 2.  Returns 4 uint32 arrays."""
    c = [np.asarray(x, dtype=np.uint64) & _MASK32 for x in counter]
    k0 = np.asarray(key[0], dtype=np.uint64) & _MASK32
    k1 = np.asarray(key[1], dtype=np.uint64) & _MASK32
    for r in range(10):
        if r:
            k0 = (k0 + np.uint64(_W0)) & _MASK32
            k1 = (k1 + np.uint64(_W1)) & _MASK32
        p0 = _M0 * c[0]
        p1 = _M1 * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK32
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK32
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
    return [x.astype(np.uint32) for x in c]


def philox_u32(seed, n):
    """The 32-bit word that csrc/sampling.cu:11-24 returns for (key = mix(seed), counter index n).  seed, n: int
    arrays (broadcastable).  key = seed * 6364136223846793005 + 1442695040888963407 mod 2^64 (sampling.cu:27)."""
    with np.errstate(over="ignore"):
        key = np.asarray(seed).astype(np.uint64) * np.uint64(6364136223846793005) + np.uint64(1442695040888963407)
    n = np.asarray(n).astype(np.uint64)
    key, n = np.broadcast_arrays(key, n)
    ctr = [(n >> np.uint64(2)) & _MASK32, (n >> np.uint64(34)) & _MASK32, np.zeros_like(n), np.zeros_like(n)]
    w = philox4x32_10(ctr, [key & _MASK32, key >> np.uint64(32)])
    sel = (n & np.uint64(3)).astype(np.int64)
    return np.choose(sel, w)


def u32_to_uniform(x):
    """sampling.cu:29: x * 2^-32 + 2^-33 as two separate fp32 operations -> (0, 1]."""
    xf = np.asarray(x, dtype=np.uint32).astype(F32)         # round to nearest even, as the device conversion does
    return (xf * F32(2.3283064e-10) + F32(2.3283064e-10) / F32(2.0)).astype(F32)


def philox_uniform(seed, offset, n):
    """out[b, i] = U(0, 1] at counter offset[b] + i of the stream keyed by seed[b] (sampling.cu:25-30)."""
    seed = np.asarray(seed, dtype=np.int64).reshape(-1, 1)
    offset = np.asarray(offset, dtype=np.int64).reshape(-1, 1)
    idx = offset.astype(np.uint64) + np.arange(n, dtype=np.uint64)[None, :]
    return u32_to_uniform(philox_u32(seed.astype(np.uint64), idx))


# ---------------------------------------------------------------------------------------------------- parameters
def sampler_params_set(vocab, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, seed=0):
    """engine/runtime/sampler.py:40-47: the device values that SamplerParams.set stores for one slot."""
    return dict(temperature=F32(temperature),
                top_k=np.int32(min(int(top_k), vocab) if top_k > 0 else vocab),
                top_p=F32(top_p),
                log_min_p=F32(math.log(min_p)) if min_p > 0 else NEG_INF,
                seed=np.int64(seed))


# ---------------------------------------------------------------------------------------------------- mask / penalties
def mask_words(vocab):
    """engine/runtime/grammar.py:28-30."""
    return (vocab + 31) // 32


def mask_bits(mask_row, vocab):
    """bool[V]: token t allowed iff bit t % 32 of word t // 32 is set (tests/test_grammar.py:47-48)."""
    w = np.asarray(mask_row).astype(np.int64) & 0xFFFFFFFF
    bits = (w[:, None] >> np.arange(32)[None, :]) & 1
    return bits.reshape(-1)[:vocab].astype(bool)


def apply_mask(logits, mask):
    """engine/runtime/sampler.py:50-56.  logits [..., V] fp32, mask [..., W] int32 -> masked copy."""
    logits = np.asarray(logits, dtype=F32)
    V = logits.shape[-1]
    out = logits.copy().reshape(-1, V)
    m = np.asarray(mask).reshape(-1, np.asarray(mask).shape[-1])
    for r in range(out.shape[0]):
        out[r, ~mask_bits(m[r], V)] = NEG_INF
    return out.reshape(logits.shape)


def penalties(logits, history, rep, pres, freq):
    """Repetition / presence / frequency penalties of one row (not in the reference; this project's definition).
    cnt[v] = occurrences of v in history (ids outside [0, V) are skipped).  For cnt[v] > 0, in fp32 and as separate
    operations:  l = l / rep if l > 0 else l * rep;  l = l - freq * cnt[v];  l = l - pres.
    (rep, pres, freq) = (1, 0, 0) leaves every bit unchanged."""
    l = np.asarray(logits, dtype=F32).copy()
    V = l.shape[-1]
    h = np.asarray(history, dtype=np.int64).reshape(-1)
    h = h[(h >= 0) & (h < V)]
    if h.size == 0 or (F32(rep) == F32(1) and F32(pres) == F32(0) and F32(freq) == F32(0)):
        return l
    ids, cnt = np.unique(h, return_counts=True)
    x = l[ids]
    with np.errstate(invalid="ignore", over="ignore"):
        x = np.where(x > 0, x / F32(rep), x * F32(rep)).astype(F32)
        x = (x - (F32(freq) * cnt.astype(F32)).astype(F32)).astype(F32)
        x = (x - F32(pres)).astype(F32)
    l[ids] = x
    return l


# ---------------------------------------------------------------------------------------------------- distribution
def processed(logits, temperature, top_k, top_p, log_min_p):
    """One row of engine/spec/accept.py:23-33.  Returns a dict:
      w        float64[V]  unnormalised kept weights exp(z - m) (0 outside the kept set)
      probs    float64[V]  w / sum(w): the renormalised probabilities that processed_probs returns
      z, m     the fp32 scaled logits and their maximum
      z_cut    the smallest kept z (fp32); the kept set is exactly {z >= z_cut}
      margin_top_p   distance of the top-p target from the nearest cumulative-mass step, as a fraction of the mass
      degenerate     True if the row has no finite maximum (all -inf / NaN): the caller falls back to index 0."""
    l = np.asarray(logits, dtype=F32)
    V = l.shape[0]
    Tc = max(F32(temperature), F32(1e-6))
    with np.errstate(over="ignore", invalid="ignore", divide="ignore"):
        z = (l / Tc).astype(F32)
        m = z.max()
        if not np.isfinite(m):
            w = np.zeros(V)
            return dict(w=w, probs=w, z=z, m=m, z_cut=m, margin_top_p=np.inf, degenerate=True)
        thr = F32(m + F32(log_min_p))
        z = np.where(z < thr, NEG_INF, z).astype(F32)
        d = (z - m).astype(F32)
    e = np.exp(d.astype(np.float64))
    z_cut = NEG_INF
    k = int(top_k)
    if 0 < k < V:
        zk = np.partition(z, V - k)[V - k]                      # k-th largest
        z_cut = max(z_cut, zk)
    keep = z >= z_cut
    margin = np.inf
    tp = float(F32(top_p))
    if tp < 1.0:
        idx = np.flatnonzero(keep & (e > 0))
        order = idx[np.argsort(-z[idx], kind="stable")]
        ev = e[order]
        cum = np.cumsum(ev)
        target = tp * cum[-1]
        j = int(np.searchsorted(cum, target, side="left"))      # first position with cum >= target
        j = min(j, len(order) - 1)
        zp = z[order[j]]
        # ties at the pivot are all kept: extend to the last position holding the pivot value
        jj = j
        while jj + 1 < len(order) and z[order[jj + 1]] == zp:
            jj += 1
        j0 = j
        while j0 > 0 and z[order[j0 - 1]] == zp:
            j0 -= 1
        incl = cum[jj]
        excl = cum[j0 - 1] if j0 > 0 else 0.0
        margin = min(incl - target, target - excl) / cum[-1]
        z_cut = max(z_cut, zp)
        keep = z >= z_cut
    w = np.where(keep, e, 0.0)
    return dict(w=w, probs=w / w.sum(), z=z, m=m, z_cut=F32(z_cut), margin_top_p=margin, degenerate=False)


def processed_probs(logits, temperature, top_k, top_p, log_min_p):
    """logits [R, V] -> float64 [R, V] renormalised probabilities (accept.py:23-33)."""
    logits = np.asarray(logits, dtype=F32)
    return np.stack([processed(r, temperature, top_k, top_p, log_min_p)["probs"] for r in logits])


def inverse_cdf_row(w, u):
    """accept.py:36-40 for one row of (possibly unnormalised) weights: #{j : c_j < u * c_last}, clamped to V - 1.
    Returns (index, margin): margin = distance of u * c_last from the nearest CDF step, as a fraction of c_last."""
    c = np.cumsum(np.asarray(w, dtype=np.float64))
    t = float(F32(u)) * c[-1]
    i = int(np.searchsorted(c, t, side="left"))
    V = c.shape[0]
    i = min(i, V - 1)
    below = c[i - 1] if i > 0 else 0.0
    margin = min(c[i] - t, t - below) / c[-1] if c[-1] > 0 else 0.0
    return i, margin


def inverse_cdf(P, u):
    P = np.asarray(P)
    return np.array([inverse_cdf_row(P[r], np.asarray(u).reshape(-1)[r])[0] for r in range(P.shape[0])], dtype=np.int64)


def argmax(logits):
    """Lowest index among equal maxima (tests/test_grammar.py:131-133; torch and numpy agree on this)."""
    return int(np.argmax(np.asarray(logits, dtype=F32)))


def draw_row(logits, temperature, top_k, top_p, log_min_p, u, mask=None, history=None, rep=1.0, pres=0.0, freq=0.0):
    """Penalties -> mask -> (temperature > 0 ? inverse-CDF draw from the processed distribution : argmax).
    Returns dict(token, greedy, margin, margin_top_p, degenerate)."""
    l = np.asarray(logits, dtype=F32)
    if history is not None:
        l = penalties(l, history, rep, pres, freq)
    if mask is not None:
        l = apply_mask(l, mask)
    g = argmax(l)
    if not (F32(temperature) > 0):
        return dict(token=g, greedy=g, margin=np.inf, margin_top_p=np.inf, degenerate=False)
    pr = processed(l, temperature, top_k, top_p, log_min_p)
    if pr["degenerate"]:
        return dict(token=g, greedy=g, margin=np.inf, margin_top_p=np.inf, degenerate=True)
    i, margin = inverse_cdf_row(pr["w"], u)
    return dict(token=i, greedy=g, margin=margin, margin_top_p=pr["margin_top_p"], degenerate=False)


def draw(logits, params, pos, mask=None, history=None, hist_len=None, u=None):
    """accept.py:43-52.  logits [B, R, V]; params: dict of arrays [B] (temperature, top_k, top_p, log_min_p, seed and
    optionally repetition_penalty, presence_penalty, frequency_penalty); pos [B].  Row r of slot b uses the uniform at
    counter pos[b] + r unless u [B, R] is given.  Returns (tokens int64 [B, R], info: list of per-row dicts)."""
    logits = np.asarray(logits, dtype=F32)
    B, R, V = logits.shape
    if u is None:
        u = philox_uniform(params["seed"], np.asarray(pos, dtype=np.int64), R)
    out = np.zeros((B, R), dtype=np.int64)
    info = []
    for b in range(B):
        h = None
        if history is not None:
            n = int(hist_len[b]) if hist_len is not None else history.shape[1]
            h = history[b, :n]
        for r in range(R):
            res = draw_row(logits[b, r], params["temperature"][b], params["top_k"][b], params["top_p"][b],
                           params["log_min_p"][b], u[b, r],
                           mask=None if mask is None else mask[b, r], history=h,
                           rep=params.get("repetition_penalty", np.ones(B, F32))[b],
                           pres=params.get("presence_penalty", np.zeros(B, F32))[b],
                           freq=params.get("frequency_penalty", np.zeros(B, F32))[b])
            out[b, r] = res["token"]
            info.append(res)
    return out, info


# ---------------------------------------------------------------------------------------------------- speculative verify
def spec_accept(pred, tok, stop_ids, active):
    """engine/spec/mtp.py:406-415, 422-423.  pred [B, k+1] the target's own tokens at the verified rows, tok [B, k+1]
    the verified inputs (tok[:, 1:] are the drafts), stop_ids [B, S] (-1 = unused), active [B].
    Returns (out_tok int64 [B, k+1], n int32 [B])."""
    pred = np.asarray(pred, dtype=np.int64)
    tok = np.asarray(tok, dtype=np.int64)
    stop_ids = np.asarray(stop_ids, dtype=np.int64)
    B, K1 = pred.shape
    k = K1 - 1
    out_tok = np.zeros((B, K1), dtype=np.int64)
    n_out = np.zeros(B, dtype=np.int32)
    for b in range(B):
        d = tok[b, 1:]
        n = 1
        while n - 1 < k and pred[b, n - 1] == d[n - 1]:
            n += 1
        bonus = pred[b, n - 1]
        for i in range(min(k, n - 1)):
            if (d[i] == stop_ids[b]).any():
                n, bonus = i + 1, d[i]
                break
        n *= int(active[b])
        row = np.concatenate([d, [bonus]])
        if n >= 1:
            row[n - 1] = bonus
        out_tok[b], n_out[b] = row, n
    return out_tok, n_out


def spec_verify_reject(target_logits, draft_logits, draft_ids, temperature, top_k, top_p, log_min_p, ua, us,
                       target_mask=None, history=None, rep=1.0, pres=0.0, freq=0.0):
    """Rejection verify with the (p - q)+ residual (not in the reference; this project's definition) for one slot.
    target_logits [k+1, V], draft_logits [k, V], draft_ids [k], ua [k] accept uniforms, us [k+1] sampling uniforms.
    p_i, q_i = processed() of target / draft row i (the same parameters; the slot's penalties, then the mask, if any,
    apply to every row of both).
    temperature <= 0: accept while draft == argmax(target row), emit the argmax of the first mismatching row.
    Else accept draft i iff p_i(d_i) > 0 and ua_i * q_i(d_i) <= p_i(d_i); at the first rejection j emit inverse_cdf(max(p_j - q_j, 0),
    us_j) (from p_j if that residual has no mass); if none is rejected emit inverse_cdf(p_k, us_k).
    Returns dict(n_accept, token, margins)."""
    tl = np.asarray(target_logits, dtype=F32)
    dl = np.asarray(draft_logits, dtype=F32)
    k = dl.shape[0]
    if history is not None:
        tl = np.stack([penalties(tl[i], history, rep, pres, freq) for i in range(k + 1)])
        dl = np.stack([penalties(dl[i], history, rep, pres, freq) for i in range(k)])
    if target_mask is not None:
        tl = np.stack([apply_mask(tl[i], target_mask[i]) for i in range(k + 1)])
        dl = np.stack([apply_mask(dl[i], target_mask[i]) for i in range(k)])
    if not (F32(temperature) > 0):
        j = 0
        while j < k and argmax(tl[j]) == int(draft_ids[j]):
            j += 1
        return dict(n_accept=j, token=argmax(tl[j]), margin=np.inf, accept_margin=np.inf)
    accept_margin = np.inf
    for j in range(k + 1):
        p = processed(tl[j], temperature, top_k, top_p, log_min_p)["probs"]
        if j == k:
            tok, margin = inverse_cdf_row(p, us[j])
            return dict(n_accept=k, token=tok, margin=margin, accept_margin=accept_margin)
        q = processed(dl[j], temperature, top_k, top_p, log_min_p)["probs"]
        d = int(draft_ids[j])
        lhs, rhs = float(F32(ua[j])) * q[d], p[d]
        accept_margin = min(accept_margin, abs(lhs - rhs) / max(rhs, lhs, 1e-300))
        if rhs > 0 and lhs <= rhs:                     # a token the target gives no probability is never accepted
            continue
        res = np.maximum(p - q, 0.0)
        if res.sum() <= 0:
            res = p
        tok, margin = inverse_cdf_row(res, us[j])
        return dict(n_accept=j, token=tok, margin=margin, accept_margin=accept_margin)


# ------------------------------------------------------------------------------------------------ logprobs
def logprobs(rows, toks, n_top):
    """Logprob of each emitted token and the n_top most likely alternatives, from the RAW logits of the positions that
    produced them (engine/runtime/scheduler.py:714-722: log_softmax, gather, topk).

    rows [r, V], toks [r], n_top >= 0.  Returns (chosen float64 [r], top_ids int64 [r, n_top], top_lp float64
    [r, n_top]); alternatives in descending order, equal values in ascending token order (torch.topk leaves the order
    of ties open; the tests compare tie groups as sets).  log-sum-exp in float64."""
    x = np.asarray(rows, dtype=np.float64)
    r, V = x.shape
    m = np.max(x, axis=1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    lse = m[:, 0] + np.log(np.sum(np.exp(x - m), axis=1))
    lsm = x - lse[:, None]
    chosen = lsm[np.arange(r), np.asarray(toks, dtype=np.int64)]
    top_ids = np.zeros((r, n_top), dtype=np.int64)
    top_lp = np.zeros((r, n_top), dtype=np.float64)
    for i in range(r):
        order = np.lexsort((np.arange(V), -x[i]))[:n_top]           # value descending, then index ascending
        top_ids[i], top_lp[i] = order, lsm[i, order]
    return chosen, top_ids, top_lp


# ------------------------------------------------------------------------------------------------ draft-head rescoring
_E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float64)


def bf16_to_f64(u16):
    """bfloat16 bit patterns (uint16) -> float64."""
    return (np.asarray(u16, dtype=np.uint32) << 16).view(np.float32).astype(np.float64)


def e4m3_to_f64(u8):
    """FP8 E4M3 (finite-only variant: no infinities, 0x7f / 0xff are NaN) bit patterns -> float64."""
    u8 = np.asarray(u8, dtype=np.int64)
    sign = np.where(u8 & 0x80, -1.0, 1.0)
    e, m = (u8 >> 3) & 0xF, u8 & 7
    val = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * 2.0 ** (e.astype(np.float64) - 7))
    val = np.where((e == 15) & (m == 7), np.nan, val)
    return sign * val


def _fma32(a, b, c):
    """fp32 fused multiply-add of values whose product is exact in float64 (bf16 / fp4 / fp8 operands against fp32)."""
    return (a * b + c.astype(np.float64)).astype(np.float32)


def _warp_xor_sum(acc):
    """acc [..., 32] fp32 per lane -> every lane's value after the xor-shuffle sums 16, 8, 4, 2, 1 (lane 0 is the result)."""
    acc = acc.copy()
    lanes = np.arange(32)
    for o in (16, 8, 4, 2, 1):
        acc = (acc + acc[..., lanes ^ o]).astype(np.float32)
    return acc[..., 0]


def rescore_bf16(x_bits, w_bits, cand):
    """Exact logits of candidate rows of a BF16 matrix in the reference kernel's accumulation order
    (csrc/sampling.cu:88-109): one warp per candidate, lane l takes the 8-element chunks l, l + 32, ... in order, one
    fp32 fma per element, then the xor-shuffle sum.  x_bits uint16 [B, K], w_bits uint16 [V, K], cand [B, NC]."""
    x, w = bf16_to_f64(x_bits), bf16_to_f64(w_bits)
    B, K = x.shape
    NC = cand.shape[1]
    chunks = K // 8
    out = np.zeros((B, NC), dtype=np.float32)
    for b in range(B):
        rows = w[cand[b]]                                          # [NC, K]
        acc = np.zeros((NC, 32), dtype=np.float32)
        for c0 in range(0, chunks, 32):
            lanes = np.arange(32)
            cc = c0 + lanes
            ok = cc < chunks
            for i in range(8):
                k = np.where(ok, cc * 8 + i, 0)
                upd = _fma32(rows[:, k], x[b, k][None, :], acc)
                acc = np.where(ok[None, :], upd, acc)
        out[b] = _warp_xor_sum(acc)
    return out


def rescore_nvfp4(x_bits, w_u8, sf_u8, gs, cand):
    """The NVFP4 variant (csrc/sampling.cu:45-75): per 16-element block s = sum of fma(w, x) in element order (byte i of
    the block: element 2i in the low nibble, 2i + 1 in the high one), acc = fma(s, scale, acc) over the lane's blocks
    l, l + 32, ...; xor-shuffle sum; times gs in fp32."""
    x = bf16_to_f64(x_bits)
    B, K = x.shape
    NC = cand.shape[1]
    blocks = K // 16
    w_u8 = np.asarray(w_u8, dtype=np.uint8)
    lo, hi = w_u8 & 0xF, w_u8 >> 4
    dec = lambda n: np.where(n & 8, -1.0, 1.0) * _E2M1[n & 7]
    wv = np.empty((w_u8.shape[0], K), dtype=np.float64)
    wv[:, 0::2], wv[:, 1::2] = dec(lo), dec(hi)
    sc = e4m3_to_f64(np.asarray(sf_u8, dtype=np.uint8).reshape(w_u8.shape[0], blocks))
    out = np.zeros((B, NC), dtype=np.float32)
    for b in range(B):
        rows, scs = wv[cand[b]], sc[cand[b]]
        acc = np.zeros((NC, 32), dtype=np.float32)
        for b0 in range(0, blocks, 32):
            bb = b0 + np.arange(32)
            ok = bb < blocks
            s = np.zeros((NC, 32), dtype=np.float32)
            for i in range(16):
                k = np.where(ok, bb * 16 + i, 0)
                s = _fma32(rows[:, k], x[b, k][None, :], s)
            upd = _fma32(s.astype(np.float64), scs[:, np.where(ok, bb, 0)], acc)
            acc = np.where(ok[None, :], upd, acc)
        out[b] = (_warp_xor_sum(acc) * np.float32(gs)).astype(np.float32)
    return out


def draft_pick(ap, x_bits, vocab_ids, n_cands, w_bits=None, w_u8=None, sf_u8=None, gs=None):
    """The greedy draft of the low-rank heads (engine/spec/mtp.py:301-309, engine/spec/mtp4.py:416-423): the n_cands largest
    entries of each row of ap (equal values: lower index first -- the order torch.topk's sorted list has apart from ties),
    their exact logits in the rescoring kernels' accumulation order, the first maximum of those in that list, and
    p = min(1, exp(ex - logsumexp(ap))).  ap fp32 [N, Vd]; vocab_ids [Vd] or None.  Returns (token ids [N], p float64 [N],
    winning draft-vocabulary index [N], its exact logit fp32 [N], margin [N] = gap between the two largest exact logits of
    different candidates, 0 where they tie)."""
    ap = np.asarray(ap, dtype=np.float32)
    N, Vd = ap.shape
    vid = np.arange(Vd, dtype=np.int64) if vocab_ids is None else np.asarray(vocab_ids, dtype=np.int64)
    ids, ps, idxs, exs, margins = [], [], [], [], []
    for n in range(N):
        order = np.lexsort((np.arange(Vd), -ap[n].astype(np.float64)))[:n_cands]     # value descending, index ascending
        rows = vid[order][None, :]
        if w_bits is not None:
            ex = rescore_bf16(x_bits[n:n + 1], w_bits, rows)[0]
        else:
            ex = rescore_nvfp4(x_bits[n:n + 1], w_u8, sf_u8, gs, rows)[0]
        best = int(np.argmax(ex))                                                   # first maximum in list order
        m = ap[n].astype(np.float64).max()
        lse = m + np.log(np.exp(ap[n].astype(np.float64) - m).sum())
        srt = np.sort(ex.astype(np.float64))
        ids.append(int(vid[order[best]])); idxs.append(int(order[best])); exs.append(ex[best])
        ps.append(min(1.0, float(np.exp(np.float64(ex[best]) - lse))))
        margins.append(float(srt[-1] - srt[-2]) if len(srt) > 1 else np.inf)
    return (np.array(ids, dtype=np.int64), np.array(ps), np.array(idxs, dtype=np.int64), np.array(exs, dtype=np.float32),
            np.array(margins))


def spec_advance(out_tok, n, y, history, hist_len, pos):
    """The scheduler's bookkeeping after a cycle (engine/runtime/scheduler.py:635-641) on arrays: for each slot with n > 0,
    tokens += [y] + out_tok[:n-1], y = out_tok[n-1], pos += n; the history keeps its most recent H ids.  Returns new
    (y, history, hist_len, pos); the inputs are not modified."""
    y, history, hist_len, pos = np.array(y), np.array(history), np.array(hist_len), np.array(pos)
    B, H = history.shape
    for b in range(B):
        nb = int(n[b])
        if nb <= 0:
            continue
        o = [int(t) for t in out_tok[b][:nb]]
        toks = [int(t) for t in history[b, :hist_len[b]]] + [int(y[b])] + o[:-1]
        toks = toks[-H:] if H else []
        history[b, :len(toks)] = toks
        hist_len[b] = len(toks)
        y[b] = o[-1]
        pos[b] += nb
    return y, history, hist_len, pos
