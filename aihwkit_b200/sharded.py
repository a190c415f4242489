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
