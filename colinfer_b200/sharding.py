"""Row sharding of a batched sampling step across the GPUs of one node.

Rows are independent (a row's result never depends on another row), so the batch is split into contiguous blocks of
rows, one block per rank; every rank runs the single-GPU kernels on its block and the only communication is the final
gather of the sampled ids (8 bytes per row) -- torch.distributed all_gather, NCCL over NVLink on GPUs, gloo in the CPU
tests.  The reference is single-GPU (one request stream, at most 3 slots); this is the scale-out this project adds.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n_rows: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [lo, hi) of `rank`: contiguous blocks, the first n_rows % world ranks hold one row more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad world / rank")
    base, extra = divmod(n_rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_rows(x, n_rows: int, world: int, rank: int):
    """The rank's block of a tensor whose first dimension is the row (slot) dimension; dicts are sharded per value,
    anything that is not a tensor of n_rows rows is passed through."""
    lo, hi = shard_range(n_rows, world, rank)
    if isinstance(x, dict):
        return {k: shard_rows(v, n_rows, world, rank) for k, v in x.items()}
    if isinstance(x, torch.Tensor) and x.dim() >= 1 and x.size(0) == n_rows:
        return x[lo:hi].contiguous()
    return x


def gather_ids(local: torch.Tensor, n_rows: int, group=None) -> torch.Tensor:
    """All ranks' sampled ids in row order.  local: this rank's ids [rows_of_rank, ...]; returns [n_rows, ...] on every
    rank.  Blocks may differ by one row, so each rank pads to the largest block before the all_gather."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    lo, hi = shard_range(n_rows, world, rank)
    if local.size(0) != hi - lo:
        raise ValueError(f"rank {rank} holds {local.size(0)} rows, expected {hi - lo}")
    if n_rows % world == 0 and local.is_contiguous():
        # equal blocks: one collective straight into the result, no padding, no concatenation
        out = torch.empty((n_rows,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local, group=group)
        return out
    biggest = shard_range(n_rows, world, 0)[1]
    pad = torch.zeros((biggest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: hi - lo] = local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    out = []
    for r, part in enumerate(parts):
        a, b = shard_range(n_rows, world, r)
        out.append(part[: b - a])
    return torch.cat(out, 0)


def sharded_draw(logits_local: torch.Tensor, params_local, pos_local: torch.Tensor, n_rows: int, group=None, **kw):
    """draw() on this rank's rows followed by the id gather: every rank returns the ids of all n_rows slots."""
    from .spec.accept import draw
    ids = draw(logits_local, params_local, pos_local, **kw)
    return gather_ids(ids, n_rows, group)
