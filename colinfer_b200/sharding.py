"""Row sharding of a batched sampling step across the GPUs of one node.

Rows are independent (a row's result never depends on another row), so the batch is split into contiguous blocks of
rows, one block per rank; every rank runs the single-GPU kernels on its block and the only communication is the final
gather of the sampled ids (8 bytes per row) -- torch.distributed all_gather, NCCL over NVLink on GPUs, gloo in the CPU
tests.  The reference is single-GPU (one request stream, at most 3 slots); this is the scale-out this project adds.
"""
from __future__ import annotations

import ctypes as C

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


# ---------------------------------------------------------------------------------------------------- peer gather
class CudaIpc:
    """The handful of CUDA runtime calls the peer gather needs (device memory that other processes can map), through the
    runtime library torch has already loaded.  A test double with the same four methods stands in on the CPU."""
    HANDLE_BYTES = 64

    def __init__(self):
        self.rt = None
        for name in ("libcudart.so.12", "libcudart.so"):
            try:
                self.rt = C.CDLL(name)
                break
            except OSError:
                continue
        if self.rt is None:
            raise RuntimeError("the CUDA runtime library is not loadable")

    def _check(self, code, what):
        if code != 0:
            raise RuntimeError(f"{what} failed: CUDA error {code}")

    def alloc_zeroed(self, nbytes: int) -> int:
        ptr = C.c_void_p()
        self._check(self.rt.cudaMalloc(C.byref(ptr), C.c_size_t(nbytes)), "cudaMalloc")
        self._check(self.rt.cudaMemset(ptr, 0, C.c_size_t(nbytes)), "cudaMemset")
        self._check(self.rt.cudaDeviceSynchronize(), "cudaDeviceSynchronize")
        return ptr.value

    def export(self, ptr: int) -> bytes:
        h = (C.c_ubyte * self.HANDLE_BYTES)()
        self._check(self.rt.cudaIpcGetMemHandle(C.byref(h), C.c_void_p(ptr)), "cudaIpcGetMemHandle")
        return bytes(h)

    def open(self, handle: bytes) -> int:
        class Handle(C.Structure):
            _fields_ = [("reserved", C.c_ubyte * self.HANDLE_BYTES)]
        h = Handle()
        C.memmove(C.byref(h), handle, self.HANDLE_BYTES)
        ptr = C.c_void_p()
        self.rt.cudaIpcOpenMemHandle.argtypes = [C.POINTER(C.c_void_p), Handle, C.c_uint]
        self._check(self.rt.cudaIpcOpenMemHandle(C.byref(ptr), h, 1), "cudaIpcOpenMemHandle")   # 1: enable peer access lazily
        return ptr.value

    def free(self, ptr: int) -> None:
        self.rt.cudaFree(C.c_void_p(ptr))


def exchange_tables(ipc, own_buf: int, own_flags: int, world: int, rank: int, all_gather_object):
    """The pointer exchange of the peer gather: every rank exports its gather buffer and its flag array, collects all
    ranks' handles, and maps the others' into its own address space.  Returns ([buffer pointer per rank], [flag pointer
    per rank]) with this rank's own pointers at index `rank` (its own memory is never re-opened)."""
    mine = (ipc.export(own_buf), ipc.export(own_flags))
    handles = [None] * world
    all_gather_object(handles, mine)
    bufs, flags = [], []
    for r, (hb, hf) in enumerate(handles):
        bufs.append(own_buf if r == rank else ipc.open(hb))
        flags.append(own_flags if r == rank else ipc.open(hf))
    return bufs, flags


class PeerGather:
    """The id gather as one small kernel over NVLink (colinfer_gather_ids): every rank's GPU stores its ids into every
    rank's buffer and waits for the others' flags -- no collective call behind the sampler.  Built once per (n_rows,
    group); gather(local) returns all ranks' ids in row order (a buffer that the next call overwrites).  Every rank must own a GPU of the node (peer access over NVLink or PCIe)."""

    def __init__(self, n_rows: int, group=None, ipc=None):
        from . import _lib
        self.lib = _lib.lib()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.n_rows = n_rows
        self.lo, self.hi = shard_range(n_rows, self.world, self.rank)
        self.ipc = ipc or CudaIpc()
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.buf_ptr = self.ipc.alloc_zeroed(2 * n_rows * 8)
        self.flag_ptr = self.ipc.alloc_zeroed(max(self.world, 1) * 8)
        bufs, flags = exchange_tables(self.ipc, self.buf_ptr, self.flag_ptr, self.world, self.rank,
                                      lambda out, obj: dist.all_gather_object(out, obj, group=group))
        self.tables = torch.tensor([bufs, flags], dtype=torch.int64, device=self.dev)      # [2, world] device pointers
        self.step = torch.zeros(1, dtype=torch.int64, device=self.dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.out = torch.empty(n_rows, dtype=torch.int64, device=self.dev)
        dist.barrier(group=group)                          # every rank has mapped every buffer before the first store

    def gather(self, local: torch.Tensor) -> torch.Tensor:
        from . import _lib
        if local.dtype != torch.int64 or not local.is_cuda or not local.is_contiguous() or local.numel() != self.hi - self.lo:
            raise RuntimeError(f"rank {self.rank} gathers {self.hi - self.lo} contiguous int64 ids on the GPU")
        _lib.check(self.lib.colinfer_gather_ids(local.data_ptr(), self.hi - self.lo, self.lo, self.tables[0].data_ptr(),
                                                self.tables[1].data_ptr(), self.world, self.rank, self.step.data_ptr(),
                                                self.n_rows, self.out.data_ptr(), 0, self.status.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream), "gather_ids")
        return self.out

    def close(self) -> None:
        """Frees this rank's buffers (after every rank has stopped gathering)."""
        if self.buf_ptr:
            self.ipc.free(self.buf_ptr)
            self.ipc.free(self.flag_ptr)
            self.buf_ptr = self.flag_ptr = 0

    def timed_out(self) -> bool:
        """True if a wait of some earlier call gave up (a rank was missing); synchronises the stream."""
        return bool(int(self.status.item()) & 1)


def sharded_draw(logits_local: torch.Tensor, params_local, pos_local: torch.Tensor, n_rows: int, group=None, **kw):
    """draw() on this rank's rows followed by the id gather: every rank returns the ids of all n_rows slots."""
    from .spec.accept import draw
    ids = draw(logits_local, params_local, pos_local, **kw)
    return gather_ids(ids, n_rows, group)
