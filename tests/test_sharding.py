"""Row sharding and the id gather of the multi-GPU path, as two gloo ranks on the CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from colinfer_b200.sharding import gather_ids, shard_range, shard_rows


def test_shard_ranges_partition_the_rows():
    for n in (0, 1, 7, 8, 1024, 1025):
        for world in (1, 2, 3, 8):
            parts = [shard_range(n, world, r) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_shard_rows_of_a_workload_dict():
    from colinfer_b200 import workloads as wl
    w = wl.config3(5, V=256, H=16)
    s = shard_rows(w, 5, 2, 1)
    assert s["logits"].shape[0] == 2 and s["params"]["history"].shape == (2, 16) and s["name"] == w["name"]
    assert torch.equal(s["params"]["seed"], w["params"]["seed"][3:])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_rows, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lo, hi = shard_range(n_rows, world, rank)
        # stand-in for the rank's sampled ids: a function of the global row index
        local = (torch.arange(lo, hi) * 3 + 1)[:, None].repeat(1, 2)
        full = gather_ids(local, n_rows)
        q.put((rank, full.tolist()))
        ok = False
        try:
            gather_ids(local[:-1], n_rows)                   # a rank that lost a row is an error, not a hang
        except ValueError:
            ok = True
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows", [8, 7])
def test_gather_ids_two_ranks(n_rows):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n_rows, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(4)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = [[3 * i + 1, 3 * i + 1] for i in range(n_rows)]
    fulls = [g[1] for g in got if isinstance(g[1], list)]
    flags = [g[1] for g in got if isinstance(g[1], bool)]
    assert len(fulls) == 2 and all(f == want for f in fulls) and flags == [True, True]
