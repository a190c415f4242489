"""Mapped-tile layer sharded over the ranks of a ``torch.distributed`` group.

The reference runs the tiles of a mapped layer one after the other on one device
(``TileModuleArray.forward``, src/aihwkit/simulator/tiles/array.py:155-182); the only coupling
between tiles is the sum over in-splits after each tile's ADC (``result.add_``, :173-176).  Here
every rank owns a contiguous block of in-splits (all out-splits of them), computes the partial
``[m, out_size]`` sum of its tiles on its GPU, and the partials are summed with one collective
(NCCL over NVLink on GPUs; gloo in the CPU tests of the host logic).

Noise keys depend on the global tile coordinates only, so the result does not depend on the
number of ranks.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def split_sizes(size: int, split_max: int) -> List[int]:
    """``TileModuleArray.get_split_sizes`` (array.py:82-97)."""
    if split_max <= 0:
        return [size]
    n = (size + split_max - 1) // split_max
    base, extra = divmod(size, n)
    return [base + (1 if i < extra else 0) for i in range(n)]


def in_split_range(n_in_splits: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block of in-splits owned by ``rank`` (balanced; may be empty)."""
    base, extra = divmod(n_in_splits, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def column_range(in_size: int, split_max: int, rank: int, world: int) -> Tuple[int, int]:
    """Input columns ``[c0, c1)`` a rank reads: the union of its in-splits."""
    sizes = split_sizes(in_size, split_max)
    b, e = in_split_range(len(sizes), rank, world)
    return sum(sizes[:b]), sum(sizes[:e])


class ShardedTileArray:
    """One rank's share of a mapped analog layer plus the partial-sum collective.

    ``local_factory(begin, end)`` builds the object that computes the local partial sum
    (``aihwkit_b200.rpu_base.tiles.TileArray`` on a GPU; any callable stand-in in CPU tests)."""

    def __init__(self, out_size: int, in_size: int, max_output_size: int, max_input_size: int,
                 local_factory, group: Optional[dist.ProcessGroup] = None):
        self.out_size, self.in_size = out_size, in_size
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.in_sizes = split_sizes(in_size, max_input_size)
        self.out_sizes = split_sizes(out_size, max_output_size)
        self.begin, self.end = in_split_range(len(self.in_sizes), self.rank, self.world)
        self.local = local_factory(self.begin, self.end)

    @property
    def n_local_tiles(self) -> int:
        return (self.end - self.begin) * len(self.out_sizes)

    def forward_partial(self, x: torch.Tensor, **kw) -> torch.Tensor:
        return self.local.forward(x, **kw)

    def reduce(self, partial: torch.Tensor, dst: Optional[int] = 0) -> torch.Tensor:
        """Sum the partial outputs: to ``dst`` (``dist.reduce``) or to every rank (``dst=None``)."""
        if not self.distributed or self.world == 1:
            return partial
        if dst is None:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
        else:
            dist.reduce(partial, dst=dst, op=dist.ReduceOp.SUM, group=self.group)
        return partial

    def forward(self, x: torch.Tensor, dst: Optional[int] = 0, **kw) -> torch.Tensor:
        return self.reduce(self.forward_partial(x, **kw), dst)

    def forward_overlapped(self, x: torch.Tensor, dst: Optional[int] = 0, n_chunks: int = 4,
                           **kw) -> torch.Tensor:
        """Forward with the partial-sum collective overlapped with the kernels: the batch is cut
        into ``n_chunks`` row blocks; the collective of block ``k`` runs (on the process group's
        own stream) while the tiles compute block ``k + 1``.  Same result as :meth:`forward`."""
        if not self.distributed or self.world == 1 or n_chunks <= 1:
            return self.forward(x, dst, **kw)
        m = x.size(0)
        if getattr(self, "_ov_partial", None) is None or self._ov_partial.size(0) != m:
            self._ov_partial = torch.empty(m, self.out_size, dtype=torch.float32, device=x.device)
        rows = (m + n_chunks - 1) // n_chunks
        works = []
        for r0 in range(0, m, rows):
            part = self._ov_partial[r0 : r0 + rows]
            self.local.forward(x[r0 : r0 + rows], out=part, non_blocking=True, **kw)
            if dst is None:
                works.append(dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            else:
                works.append(dist.reduce(part, dst=dst, op=dist.ReduceOp.SUM, group=self.group,
                                         async_op=True))
        for w in works:
            w.wait()
        return self._ov_partial

    def forward_host(self, x_local_host: torch.Tensor, out_host: Optional[torch.Tensor] = None,
                     dst: int = 0, chunk_rows: int = 1024) -> Optional[torch.Tensor]:
        """End-to-end forward from host memory on every rank.

        ``x_local_host`` is this rank's own input columns ``[m, local_in_size]`` in page-locked
        host memory (inputs are scattered over the ranks, not broadcast).  Row chunks are copied
        to the device on a side stream while earlier chunks are in the kernels; the partial
        outputs are summed to ``dst`` with one collective and copied to ``out_host`` there.
        With a single rank the library's own pipelined host entry point does all of it."""
        if self.world == 1:
            return self.local.forward(x_local_host, out=out_host)
        dev = self.local.device
        m = x_local_host.size(0)
        if not hasattr(self, "_copy_stream"):
            self._copy_stream = torch.cuda.Stream(device=dev)
            self._stage = None
        if self._stage is None or self._stage[0].size(0) < chunk_rows or self._partial.size(0) != m:
            self._stage = [torch.empty(chunk_rows, max(self.local.local_in_size, 1), device=dev)
                           for _ in range(2)]
            self._partial = torch.empty(m, self.out_size, device=dev)
            self._events = [[torch.cuda.Event(), torch.cuda.Event()] for _ in range(2)]
        main = torch.cuda.current_stream(dev)
        if self.local.local_in_size == 0:
            self._partial.zero_()
        else:
            for c, r0 in enumerate(range(0, m, chunk_rows)):
                b = c & 1
                rows = min(chunk_rows, m - r0)
                h2d_done, comp_done = self._events[b]
                with torch.cuda.stream(self._copy_stream):
                    if c >= 2:
                        self._copy_stream.wait_event(comp_done)  # staging buffer b is free again
                    self._stage[b][:rows].copy_(x_local_host[r0 : r0 + rows], non_blocking=True)
                    h2d_done.record(self._copy_stream)
                main.wait_event(h2d_done)
                self.local.forward_local(self._stage[b][:rows], out=self._partial[r0 : r0 + rows])
                comp_done.record(main)
        self.reduce(self._partial, dst)
        if self.rank == dst and out_host is not None:
            out_host.copy_(self._partial, non_blocking=True)
            return out_host
        return None
