"""The grammar-mask rows of a step on their way to the sampler: the buffers of the reference's scheduler
(engine/runtime/scheduler.py:222-223: `masks` int32 [n_slots, margin, W] on the device, `mask_host` pinned) and its
`_row_masks` (scheduler.py:672-681), without the stream synchronisation that method ends with.

The reference fills ONE pinned buffer, copies it and then waits for the whole stream, because the next cycle refills
that buffer.  Here the pinned side is a ring: a buffer is only waited for when the ring comes round to it while its
copy (or the kernel reading it) is still in flight, so the host returns to the grammar engine at once.  With
`zero_copy` the rows are not copied at all: pinned memory is mapped into the device's address space, and the sampling
kernel reads the ~19 KB of a row over PCIe while it runs (`draw(..., mask=rows)` with the returned tensor).
"""
from __future__ import annotations

import torch


def mask_words(vocab: int) -> int:
    """int32 words of a token bitmask: token t is bit t % 32 of word t // 32 (engine/runtime/grammar.py:28-30)."""
    return (vocab + 31) // 32


class RowMasks:
    """n_slots x margin mask rows on `device` and a ring of `depth` pinned staging buffers.

    rows(constraint, b, drafts) is the reference's `_row_masks(req, b, drafts)` with `req.constraint` passed directly:
    `constraint.masks(drafts, out)` fills out[i] (numpy int32 [len(drafts) + 1, W]) with the mask after drafts[:i]
    (engine/runtime/grammar.py:42-48); rows it leaves alone stay all-ones."""

    def __init__(self, n_slots: int, margin: int, vocab: int, device, depth: int = 4, zero_copy: bool = False):
        self.dev = torch.device(device)
        self.W = mask_words(vocab)
        self.margin, self.depth, self.zero_copy = margin, max(1, depth), zero_copy
        cuda = self.dev.type == "cuda"
        self.masks = torch.full((n_slots, margin, self.W), -1, dtype=torch.int32, device=self.dev)
        self.host = torch.full((self.depth, margin, self.W), -1, dtype=torch.int32, pin_memory=cuda)
        self._events = [torch.cuda.Event() if cuda else None for _ in range(self.depth)]
        self._busy = [False] * self.depth
        self._next = 0
        self.waits = 0          # how often the ring had to wait for a buffer (0 in steady state with enough depth)

    def reset(self, b: int) -> None:
        """A slot without a grammar: every token allowed (scheduler.py:523)."""
        self.masks[b].fill_(-1)

    def _take(self) -> int:
        i = self._next
        self._next = (i + 1) % self.depth
        if self._busy[i] and self._events[i] is not None:
            if not self._events[i].query():
                self.waits += 1
                self._events[i].synchronize()
        self._busy[i] = False
        return i

    def rows(self, constraint, b: int, drafts: list[int]) -> torch.Tensor:
        """Fills the masks of slot b's verify rows [y, drafts...] from the grammar and returns them as [1, r, W] for the
        sampler (device rows; with zero_copy the pinned rows themselves).  No stream synchronisation; call `release()`
        after the launch that reads the rows when zero_copy is on."""
        r = len(drafts) + 1
        if r > self.margin:
            raise RuntimeError(f"{r} rows do not fit the margin of {self.margin}")
        i = self._take()
        host = self.host[i, :r]
        host.fill_(-1)
        constraint.masks(list(drafts), host.numpy())
        self._last = i
        if self.zero_copy and self.dev.type == "cuda":
            self._busy[i] = True                                    # until release() records the event behind the reader
            return host.unsqueeze(0)
        self.masks[b, :r].copy_(host, non_blocking=True)
        if self._events[i] is not None:
            self._events[i].record()
            self._busy[i] = True
        return self.masks[b:b + 1, :r]

    def release(self) -> None:
        """zero_copy only: marks the point in the current stream after which the rows returned last may be refilled."""
        if self.zero_copy and self._events[self._last] is not None:
            self._events[self._last].record()
