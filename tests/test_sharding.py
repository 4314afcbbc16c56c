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


class _FakeIpc:
    """Stands in for the CUDA IPC calls: a handle names (owner rank, address); opening it yields a tagged address."""
    def __init__(self, rank):
        self.rank, self.opened = rank, []

    def export(self, ptr):
        return f"{self.rank}:{ptr}".encode().ljust(64, b"\0")

    def open(self, handle):
        owner, ptr = handle.rstrip(b"\0").decode().split(":")
        self.opened.append(int(owner))
        return 10_000_000 * (int(owner) + 1) + int(ptr)            # "where rank `owner`'s memory appears in this process"


def _exchange_worker(rank, world, port, q):
    from colinfer_b200.sharding import exchange_tables
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ipc = _FakeIpc(rank)
        bufs, flags = exchange_tables(ipc, 1000 + rank, 2000 + rank, world, rank,
                                      lambda out, obj: dist.all_gather_object(out, obj))
        q.put((rank, bufs, flags, sorted(ipc.opened)))
    finally:
        dist.destroy_process_group()


def test_peer_gather_pointer_exchange_two_ranks():
    """The bookkeeping of the peer gather's set-up on two gloo ranks: every rank ends with one buffer and one flag
    pointer per rank, in rank order, its own memory never re-opened, every other rank's mapped exactly twice."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_exchange_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, bufs, flags, opened in got:
        other = 1 - rank
        assert bufs[rank] == 1000 + rank and flags[rank] == 2000 + rank
        assert bufs[other] == 10_000_000 * (other + 1) + 1000 + other
        assert flags[other] == 10_000_000 * (other + 1) + 2000 + other
        assert opened == [other, other]


@pytest.mark.gpu
def test_gather_kernel_single_rank_and_bounded_wait():
    """colinfer_gather_ids on one GPU.  (a) A world of one rank: its ids come back, step after step, from alternating
    halves.  (b) The bounded wait: a second rank that never raises its flag (nothing sets it) makes the wait run out
    after its limit; the kernel returns with COLINFER_GATHER_TIMEOUT, nothing hangs and the next launch is clean."""
    from colinfer_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda")
    n = 10
    st = torch.cuda.current_stream().cuda_stream
    # (a)
    buf = torch.zeros(2 * n, dtype=torch.int64, device=dev)
    flags = torch.zeros(1, dtype=torch.int64, device=dev)
    tables = torch.tensor([[buf.data_ptr()], [flags.data_ptr()]], dtype=torch.int64, device=dev)
    step = torch.zeros(1, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.empty(n, dtype=torch.int64, device=dev)
    for s in range(1, 4):
        ids = torch.arange(n, device=dev) * s
        assert lib.colinfer_gather_ids(ids.data_ptr(), n, 0, tables[0].data_ptr(), tables[1].data_ptr(), 1, 0, step.data_ptr(), n,
                                       out.data_ptr(), 0, status.data_ptr(), st) == 0
        torch.cuda.synchronize()
        assert torch.equal(out, ids) and int(step) == s and int(flags) == s and int(status) == 0
        assert torch.equal(buf[(s & 1) * n:(s & 1) * n + n], ids)
    # (b) rank 0 of two; "rank 1" is a second buffer on the same GPU whose flag stays 0
    buf1 = torch.zeros(2 * n, dtype=torch.int64, device=dev)
    flags0, flags1 = torch.zeros(2, dtype=torch.int64, device=dev), torch.zeros(2, dtype=torch.int64, device=dev)
    tables = torch.tensor([[buf.data_ptr(), buf1.data_ptr()], [flags0.data_ptr(), flags1.data_ptr()]], dtype=torch.int64, device=dev)
    step.zero_()
    ids = torch.arange(5, device=dev) + 100
    rc = lib.colinfer_gather_ids(ids.data_ptr(), 5, 0, tables[0].data_ptr(), tables[1].data_ptr(), 2, 0, step.data_ptr(), n,
                                 out.data_ptr(), 200_000, status.data_ptr(), st)          # limit: 200,000 cycles (~0.1 ms)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status) == 1                                        # COLINFER_GATHER_TIMEOUT
    assert int(flags1[0]) == 1 and torch.equal(buf1[n:n + 5], ids)  # its own ids and flag did reach "rank 1"
    status.zero_()
    assert lib.colinfer_gather_ids(ids.data_ptr(), 5, 0, tables[0].data_ptr(), tables[1].data_ptr(), 2, 0, step.data_ptr(), n,
                                   out.data_ptr(), 200_000, status.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(step) == 2 and int(status) == 1                     # still alone, still bounded; the context is fine
    assert lib.colinfer_gather_ids(ids.data_ptr(), 11, 0, tables[0].data_ptr(), tables[1].data_ptr(), 2, 0, step.data_ptr(), n,
                                   out.data_ptr(), 0, status.data_ptr(), st) == 1         # more rows than the buffer holds
