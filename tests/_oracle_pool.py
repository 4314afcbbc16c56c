"""The CPU oracle over every row of a large workload, spread over the host cores (test helper).

O.draw is pure numpy and takes tens of milliseconds per 151,936-token row; full-size parity cases (1024 or 512 rows)
run it in worker processes.  Workers are spawned (never forked from a process that holds a CUDA context) and import
nothing but numpy and the oracle."""
from __future__ import annotations

import multiprocessing as mp
import os

import numpy as np


def _chunk(args):
    from oracle import oracle as O
    logits, params, pos, mask, history, hist_len, u = args
    tokens, info = O.draw(logits, params, pos, mask=mask, history=history, hist_len=hist_len, u=u)
    keep = ("token", "greedy", "margin", "margin_top_p", "degenerate")
    return tokens, [{k: d[k] for k in keep} for d in info]


def oracle_draw_rows(logits, params, pos, mask=None, history=None, hist_len=None, u=None, workers=None):
    """O.draw(logits [B, R, V], ...) -> (tokens [B, R], info list), computed in `workers` processes over blocks of slots."""
    B = logits.shape[0]
    workers = workers or max(1, min(len(os.sched_getaffinity(0)), 16, B))
    bounds = np.linspace(0, B, workers * 2 + 1).astype(int)
    jobs = []
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        if hi > lo:
            jobs.append((logits[lo:hi], {k: v[lo:hi] for k, v in params.items()}, None if pos is None else pos[lo:hi],
                         None if mask is None else mask[lo:hi], None if history is None else history[lo:hi],
                         None if hist_len is None else hist_len[lo:hi], None if u is None else u[lo:hi]))
    if workers == 1:
        parts = [_chunk(j) for j in jobs]
    else:
        with mp.get_context("spawn").Pool(workers) as pool:
            parts = pool.map(_chunk, jobs)
    tokens = np.concatenate([p[0] for p in parts], 0)
    info = [d for p in parts for d in p[1]]
    return tokens, info
