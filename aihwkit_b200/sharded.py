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

    # ---- reduce-scatter by direct stores --------------------------------------------------------
    def enable_scatter(self, m: int, codes: Optional[bool] = None) -> None:
        """Prepare :meth:`forward_reduce_scatter` for batches of ``m`` rows: every rank allocates
        two sets of ``world`` slots of ``rows x out_size`` floats (double buffering over steps),
        shares them with the other ranks of the node through CUDA IPC handles, and builds the
        pointer tables the kernel scatters through.

        ``codes``: send the signed-byte ADC code of every in-split (plus one factor per row and
        in-split) instead of the fp32 sum over the rank's in-splits - a quarter of the bytes on
        the wire per in-split, so it pays while a rank holds fewer than four in-splits.  Default:
        used when every rank's tiles are eligible (``TileArray.scatter_codes_supported``) and no
        rank holds more than three in-splits."""
        import ctypes as C

        from . import _cabi

        lib = _cabi.lib()
        item = 256  # work-item height of the kernel: ownership changes on item boundaries
        per_rank = (m + self.world - 1) // self.world
        self._sc_rows = (per_rank + item - 1) // item * item
        self._sc_m = m
        dev_index = self.local.device.index
        slot_floats = self._sc_rows * self.out_size
        # codes variant: agreed on by all ranks
        mine = (self.end - self.begin, bool(self.local.scatter_codes_supported()) if self.end > self.begin else False)
        infos = [None] * self.world
        dist.all_gather_object(infos, mine, group=self.group)
        self._sc_planes = [int(i[0]) for i in infos]
        if min(self._sc_planes) == 0:
            # every rank sees the same list, so every rank raises: a rank without tiles would
            # launch no kernel and never signal its peers, which would wait for it on the GPU
            empty = [q for q, n in enumerate(self._sc_planes) if n == 0]
            raise RuntimeError(
                f"the fused reduce-scatter needs at least one in-split per rank; ranks {empty} of "
                f"{self.world} own none ({len(self.in_sizes)} in-splits)")
        eligible = all(i[1] for i in infos) and (self._sc_rows % 32 == 0) and self.world <= 16
        if codes is None:
            codes = eligible and max(self._sc_planes) <= 3
        elif codes and not eligible:
            raise RuntimeError("the scatter of ADC codes is not available for this layer")
        self._sc_codes = bool(codes)
        max_planes = max(self._sc_planes)
        self._sc_code_stride = max_planes * self._sc_rows * self.out_size  # bytes per sender slot
        self._sc_fac_stride = max_planes * self._sc_rows                   # floats per sender slot
        if self._sc_codes:
            alloc_bytes = self.world * (self._sc_code_stride + 4 * self._sc_fac_stride)
        else:
            alloc_bytes = 4 * slot_floats * self.world
        # a rank whose allocation or mapping fails tells the others through the same exchange, so
        # that every rank raises (and none waits in a collective the failed one never joins)
        handles, self._sc_mine, self._sc_peers, failure = [], [], [], None
        try:
            for _ in range(2):
                ptr, h = C.c_void_p(), C.create_string_buffer(64)
                _cabi.check(lib.ab200_peer_alloc(alloc_bytes, dev_index, C.byref(ptr), h))
                self._sc_mine.append(ptr.value)
                handles.append(h.raw)
        except RuntimeError as exc:
            failure = f"rank {self.rank}: {exc}"
        gathered = [None] * self.world
        dist.all_gather_object(gathered, failure or handles, group=self.group)
        failure = next((g for g in gathered if isinstance(g, str)), None)
        self._sc_tables, self._sc_fac_tables = [], []
        if failure is None:
            try:
                for b in range(2):
                    ptrs, fptrs = [], []
                    for q in range(self.world):
                        if q == self.rank:
                            base = self._sc_mine[b]
                        else:
                            p = C.c_void_p()
                            _cabi.check(lib.ab200_peer_open(gathered[q][b], dev_index, C.byref(p)))
                            self._sc_peers.append(p.value)
                            base = p.value
                        if self._sc_codes:
                            # this rank's code planes and factors at owner q
                            ptrs.append(base + self._sc_code_stride * self.rank)
                            fptrs.append(base + self._sc_code_stride * self.world
                                         + 4 * self._sc_fac_stride * self.rank)
                        else:
                            ptrs.append(base + 4 * slot_floats * self.rank)  # this rank's slot at owner q
                    self._sc_tables.append(torch.tensor(ptrs, dtype=torch.int64, device=self.local.device))
                    if self._sc_codes:
                        self._sc_fac_tables.append(
                            torch.tensor(fptrs, dtype=torch.int64, device=self.local.device))
            except RuntimeError as exc:
                failure = f"rank {self.rank}: {exc}"
        opened = [None] * self.world
        dist.all_gather_object(opened, failure, group=self.group)
        failure = next((g for g in opened if g is not None), None)
        if failure is not None:
            self.disable_scatter()
            raise RuntimeError(f"peer memory for the fused reduce-scatter is not available ({failure})")
        self._sc_flag = torch.zeros(1, device=self.local.device)
        self._sc_step = 0
        dist.barrier(group=self.group)

    def forward_reduce_scatter(self, x_local: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Forward of the sharded layer with the sum over the ranks' in-splits done by direct
        stores: every rank's kernel writes its partial sums into its slot at the owner of each
        row block (peer memory over NVLink, tile by tile while it computes; the ranks sweep the
        owners in staggered order), a barrier follows, and every owner adds its ``world`` slots.
        Returns this rank's rows ``[rows, out_size]`` of the summed output: rank ``q`` owns rows
        ``[q * rows, (q + 1) * rows)`` with ``rows = self.scatter_rows``; all on the GPU, no host
        synchronisation."""
        from . import _cabi

        import ctypes as C

        b = self._sc_step & 1
        self._sc_step += 1
        rotate = ((self.rank + 1) % self.world) * self._sc_rows
        if out is None:
            out = torch.empty(self._sc_rows, self.out_size, device=self.local.device)
        stream = int(torch.cuda.current_stream(self.local.device).cuda_stream)
        if self._sc_codes:
            self.local.forward_scatter_codes(x_local, self._sc_tables[b], self._sc_fac_tables[b],
                                             self._sc_rows, rotate)
            dist.all_reduce(self._sc_flag, group=self.group)  # every rank's stores have landed
            valid = max(0, min(self._sc_rows, x_local.size(0) - self.rank * self._sc_rows))
            planes = (C.c_int * self.world)(*self._sc_planes)
            base = self._sc_mine[b]
            _cabi.check(_cabi.lib().ab200_sum_code_slots(
                base, self._sc_code_stride, base + self._sc_code_stride * self.world,
                self._sc_fac_stride, self.world, planes, self._sc_rows, valid, self.out_size,
                out.data_ptr(), stream))
            return out
        self.local.forward_scatter(x_local, self._sc_tables[b], self._sc_rows, rotate)
        dist.all_reduce(self._sc_flag, group=self.group)  # every rank's stores have landed
        _cabi.check(_cabi.lib().ab200_sum_slots(self._sc_mine[b], self.world,
                                                self._sc_rows * self.out_size, out.data_ptr(), stream))
        return out

    @property
    def scatter_rows(self) -> int:
        return self._sc_rows

    def disable_scatter(self) -> None:
        """Close the peers' buffers and free this rank's (after a barrier: nobody writes any more)."""
        from . import _cabi

        if getattr(self, "_sc_mine", None) is None:
            return
        self._sc_tables = []
        torch.cuda.synchronize(self.local.device)
        dist.barrier(group=self.group)
        lib = _cabi.lib()
        for p in self._sc_peers:
            _cabi.check(lib.ab200_peer_close(p))
        dist.barrier(group=self.group)
        for p in self._sc_mine:
            _cabi.check(lib.ab200_peer_free(p))
        self._sc_mine = None

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
