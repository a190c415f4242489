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


def tile_grid(n_in_splits: int, n_out_splits: int, world: int) -> Tuple[int, int]:
    """Ranks along the in-splits and along the out-splits, ``(g_in, g_out)`` with ``g_in * g_out
    == world``: as many ranks as possible share the in-splits (their partial sums are the only
    thing that has to be added up), the rest divide the out-splits."""
    g_in = 1
    for g in range(1, world + 1):
        if world % g == 0 and g <= max(1, n_in_splits):
            g_in = g
    return g_in, world // g_in


def block_of_rank(n_in_splits: int, n_out_splits: int, rank: int, world: int):
    """The block of tiles of ``rank`` in the 2-D map: ``((in_begin, in_end), (out_begin, out_end))``;
    ranks sit in-split-major (``rank = r_in * g_out + r_out``). A block may be empty."""
    g_in, g_out = tile_grid(n_in_splits, n_out_splits, world)
    r_in, r_out = divmod(rank, g_out)
    return in_split_range(n_in_splits, r_in, g_in), in_split_range(n_out_splits, r_out, g_out)


class ShardedTileArray:
    """One rank's share of a mapped analog layer plus the partial-sum collective.

    ``local_factory(begin, end)`` builds the object that computes the local partial sum
    (``aihwkit_b200.rpu_base.tiles.TileArray`` on a GPU; any callable stand-in in CPU tests)."""

    def __init__(self, out_size: int, in_size: int, max_output_size: int, max_input_size: int,
                 local_factory, group: Optional[dist.ProcessGroup] = None, two_d: bool = False):
        """``two_d``: map the tiles onto a grid of ranks over in-splits AND out-splits
        (:func:`tile_grid`) - for layers with fewer in-splits than ranks; ``local_factory`` is
        then called as ``local_factory(in_begin, in_end, out_begin, out_end)``."""
        self.out_size, self.in_size = out_size, in_size
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.in_sizes = split_sizes(in_size, max_input_size)
        self.out_sizes = split_sizes(out_size, max_output_size)
        if two_d:
            (self.begin, self.end), (self.out_begin, self.out_end) = block_of_rank(
                len(self.in_sizes), len(self.out_sizes), self.rank, self.world)
            self.local = local_factory(self.begin, self.end, self.out_begin, self.out_end)
        else:
            self.begin, self.end = in_split_range(len(self.in_sizes), self.rank, self.world)
            self.out_begin, self.out_end = 0, len(self.out_sizes)
            self.local = local_factory(self.begin, self.end)

    @property
    def n_local_tiles(self) -> int:
        return (self.end - self.begin) * (self.out_end - self.out_begin)

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
    ITEM_ROWS = 256  # work-item height of the kernel: ownership changes on item boundaries
    FLAG_BYTES = 256

    def enable_scatter(self, m: int, codes: Optional[bool] = None, cyclic: bool = False,
                       buffers: int = 2) -> None:
        """Prepare :meth:`forward_reduce_scatter` for batches of ``m`` rows: every rank allocates
        ``buffers`` sets of ``world`` slots of ``rows x out_size`` floats (two: double buffering
        over steps; four: steps pipelined two deep, see ``forward_reduce_scatter(pipelined=True)``)
        plus one arrival flag per sender, shares them with the other ranks of the node through
        CUDA IPC handles, and builds the pointer tables the kernel scatters through.

        ``cyclic``: deal the 256-row blocks of the batch to the ranks in turn (block ``b`` is
        block ``b // world`` of rank ``b % world``) instead of giving rank ``q`` the rows
        ``[q * rows, (q + 1) * rows)``; every part of a batch then feeds all owners alike, which
        is what :meth:`forward_reduce_scatter_host` pipelines over.

        ``codes``: send the signed-byte ADC code of every in-split (plus one factor per row and
        in-split) instead of the fp32 sum over the rank's in-splits - a quarter of the bytes on
        the wire per in-split, so it pays while a rank holds fewer than four in-splits.  Default:
        used when every rank's tiles are eligible (``TileArray.scatter_codes_supported``) and no
        rank holds more than three in-splits."""
        import ctypes as C

        from . import _cabi

        lib = _cabi.lib()
        item = self.ITEM_ROWS
        if cyclic:
            n_blocks = (m + item - 1) // item
            self._sc_rows = (n_blocks + self.world - 1) // self.world * item
        else:
            per_rank = (m + self.world - 1) // self.world
            self._sc_rows = (per_rank + item - 1) // item * item
        self._sc_blk = item if cyclic else 0
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
            data_bytes = self.world * (self._sc_code_stride + 4 * self._sc_fac_stride)
        else:
            data_bytes = 4 * slot_floats * self.world
        # arrival flags (one int per sender) behind the slots of the first buffer
        self._sc_flag_off = (data_bytes + 255) // 256 * 256
        alloc_bytes = self._sc_flag_off + max(self.FLAG_BYTES, 4 * self.world)
        # a rank whose allocation or mapping fails tells the others through the same exchange, so
        # that every rank raises (and none waits for a rank that gave up)
        handles, self._sc_mine, self._sc_peers, failure = [], [], [], None
        try:
            for _ in range(buffers):
                ptr, h = C.c_void_p(), C.create_string_buffer(64)
                _cabi.check(lib.ab200_peer_alloc(alloc_bytes, dev_index, C.byref(ptr), h))
                self._sc_mine.append(ptr.value)
                handles.append(h.raw)
        except RuntimeError as exc:
            failure = f"rank {self.rank}: {exc}"
        gathered = [None] * self.world
        dist.all_gather_object(gathered, failure or handles, group=self.group)
        failure = next((g for g in gathered if isinstance(g, str)), None)
        self._sc_tables, self._sc_fac_tables, self._sc_flag_table = [], [], None
        if failure is None:
            try:
                for b in range(buffers):
                    ptrs, fptrs, flags = [], [], []
                    for q in range(self.world):
                        if q == self.rank:
                            base = self._sc_mine[b]
                        else:
                            p = C.c_void_p()
                            _cabi.check(lib.ab200_peer_open(gathered[q][b], dev_index, C.byref(p)))
                            self._sc_peers.append(p.value)
                            base = p.value
                        flags.append(base + self._sc_flag_off + 4 * self.rank)
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
                    if b == 0:
                        # this rank's arrival flag at every owner (the first buffer holds them)
                        self._sc_flag_table = torch.tensor(flags, dtype=torch.int64,
                                                           device=self.local.device)
            except RuntimeError as exc:
                failure = f"rank {self.rank}: {exc}"
        opened = [None] * self.world
        dist.all_gather_object(opened, failure, group=self.group)
        failure = next((g for g in opened if g is not None), None)
        if failure is not None:
            self.disable_scatter()
            raise RuntimeError(f"peer memory for the fused reduce-scatter is not available ({failure})")
        self._sc_flags_local = self._sc_mine[0] + self._sc_flag_off
        self._sc_step = 0
        self._sc_epoch = 0
        self._sc_wait_ms = 2000.0
        self._sc_nbuf = buffers
        self._sc_side = None      # stream of the owner's sums when steps are pipelined
        self._sc_sum_done = None  # events: sum of step j recorded in slot j % 4
        self._sc_sum_seen = [-1] * 4  # step whose sum the event in each slot belongs to
        dist.barrier(group=self.group)

    def _owned_rows(self, r0: int, rows: int) -> Tuple[int, int]:
        """Rows of this rank's buffer that the rows ``[r0, r0 + rows)`` of the batch fill:
        ``(first local row, count)``.  ``r0`` must start a round of the deal when blocks are
        dealt in turn."""
        if self._sc_blk == 0:
            lo = max(r0, self.rank * self._sc_rows)
            hi = min(r0 + rows, (self.rank + 1) * self._sc_rows)
            return (max(lo - self.rank * self._sc_rows, 0), max(hi - lo, 0))
        blk = self._sc_blk
        if r0 % (blk * self.world) != 0:
            raise RuntimeError("a part of the batch must start on a multiple of 256 * world rows")
        count = 0
        for b in range(r0 // blk, (r0 + rows + blk - 1) // blk):
            if b % self.world == self.rank:
                count += min(blk, r0 + rows - b * blk)
        return (r0 // self.world, count)

    def _check_wait_status(self) -> None:
        import ctypes as C

        from . import _cabi

        n = C.c_int(0)
        _cabi.check(_cabi.lib().ab200_wait_status(self.local.device.index, C.byref(n)))
        if n.value:
            raise RuntimeError(
                f"reduce-scatter: {n.value} wait(s) for the other ranks' partial sums ran out "
                f"(rank {self.rank}); a rank is missing or far behind")

    def _scatter_part(self, x_part: torch.Tensor, r0: int, b: int, out: torch.Tensor,
                      events=None, sum_stream=None) -> Tuple[int, int]:
        """One launch of the scatter kernel on the rows ``[r0, r0 + rows)`` of the batch followed
        by this owner's sum of what all ranks sent for them (which first waits, on the GPU and
        bounded, for the senders' arrival flags).  Returns the owner's local row range.
        ``events``: three CUDA events recorded before the scatter, between the two and after the
        sum (a phase breakdown for benchmarks)."""
        import ctypes as C

        from . import _cabi

        lib = _cabi.lib()
        self._sc_epoch += 1
        plan = _cabi.ScatterPlan()
        if self._sc_codes:
            plan.code_table_dev = self._sc_tables[b].data_ptr()
            plan.fac_table_dev = self._sc_fac_tables[b].data_ptr()
        else:
            plan.out_table_dev = self._sc_tables[b].data_ptr()
        plan.flag_table_dev = self._sc_flag_table.data_ptr()
        plan.n_owners = self.world
        plan.rows_per_owner = self._sc_rows
        # the ranks sweep the owners in staggered order, so that no owner receives from all
        # ranks at once
        plan.rotate_rows = (self.rank * self._sc_blk if self._sc_blk
                            else ((self.rank + 1) % self.world) * self._sc_rows)
        plan.row_base = r0
        plan.owner_block_rows = self._sc_blk
        plan.epoch = self._sc_epoch
        if events is not None:
            events[0].record()
        self.local.forward_scatter_plan(x_part, plan)
        if events is not None:
            events[1].record()
        lr0, n = self._owned_rows(r0, x_part.size(0))
        if sum_stream is not None:
            # the owner's sum runs on its own stream, behind this step's scatter kernel
            sum_stream.wait_stream(torch.cuda.current_stream(self.local.device))
            stream = int(sum_stream.cuda_stream)
        else:
            stream = int(torch.cuda.current_stream(self.local.device).cuda_stream)
        base = self._sc_mine[b]
        if self._sc_codes:
            planes = (C.c_int * self.world)(*self._sc_planes)
            _cabi.check(lib.ab200_sum_code_slots_wait(
                base, self._sc_code_stride, base + self._sc_code_stride * self.world,
                self._sc_fac_stride, self.world, planes, self._sc_rows, lr0, n, self.out_size,
                out.data_ptr(), self._sc_flags_local, self.world, self._sc_epoch,
                self._sc_wait_ms, stream))
        else:
            _cabi.check(lib.ab200_sum_slots_wait(
                base, self.world, self._sc_rows * self.out_size, lr0, n, self.out_size,
                out.data_ptr(), self._sc_flags_local, self.world, self._sc_epoch,
                self._sc_wait_ms, stream))
        if events is not None:
            events[2].record()
        return lr0, n

    def forward_reduce_scatter(self, x_local: torch.Tensor, out: Optional[torch.Tensor] = None,
                               events=None, pipelined: bool = False) -> torch.Tensor:
        """Forward of the sharded layer with the sum over the ranks' in-splits done by direct
        stores: every rank's kernel writes its partial sums into its slot at the owner of each
        row block (peer memory over NVLink, tile by tile while it computes) and, once all its
        stores are out, raises its arrival flag at every owner; every owner's sum kernel waits
        for the flags of all senders (bounded: a missing rank makes the next call raise) and adds
        its ``world`` slots.  No collective, no host synchronisation.  Returns this rank's rows
        ``[rows, out_size]`` of the summed output: rank ``q`` owns rows ``[q * rows, (q + 1) *
        rows)`` with ``rows = self.scatter_rows`` (or, with ``cyclic`` ownership, the 256-row
        blocks ``q, q + world, ...`` of the batch, packed).

        ``pipelined`` (needs ``enable_scatter(..., buffers=4)``): consecutive calls overlap - the
        owner's sum of step ``j`` runs on a side stream while the kernels of step ``j + 1`` run
        on the caller's.  Step ``j`` writes slot set ``j % 4``; its kernel is held back (by an
        event, on the host's stream order, no device-side wait) until this rank's sum of step
        ``j - 2`` is done.  That sum has seen every rank's arrival flag of step ``j - 2``, and
        every rank launched that step after its own sum of step ``j - 4``: so all owners have
        finished reading slot set ``j % 4`` before anyone writes it again.  The result is
        complete when :meth:`scatter_flush` (or a device synchronisation) returns."""
        self._check_wait_status()
        dev = self.local.device
        j = self._sc_step
        b = j % self._sc_nbuf
        self._sc_step += 1
        if out is None:
            out = torch.empty(self._sc_rows, self.out_size, device=dev)
        main = torch.cuda.current_stream(dev)
        if not pipelined:
            if self._sc_side is not None:
                main.wait_stream(self._sc_side)  # sums of earlier pipelined steps
            _, n = self._scatter_part(x_local, 0, b, out, events)
            if n < self._sc_rows:
                out[n:].zero_()  # rows of the buffer beyond the batch
            return out
        if self._sc_nbuf < 4:
            raise RuntimeError("pipelined steps need enable_scatter(..., buffers=4)")
        if self._sc_side is None:
            self._sc_side = torch.cuda.Stream(device=dev)
            self._sc_sum_done = [torch.cuda.Event() for _ in range(4)]
        if j >= 2 and self._sc_sum_seen[(j - 2) % 4] == j - 2:
            main.wait_event(self._sc_sum_done[(j - 2) % 4])
        else:
            # step j - 2 was not a pipelined one (its sum ran on the caller's stream): wait for
            # whatever the side stream still holds, which orders this step behind all earlier sums
            main.wait_stream(self._sc_side)
        out.record_stream(self._sc_side)
        _, n = self._scatter_part(x_local, 0, b, out, events, sum_stream=self._sc_side)
        if n < self._sc_rows:
            with torch.cuda.stream(self._sc_side):
                out[n:].zero_()
        self._sc_sum_done[j % 4].record(self._sc_side)
        self._sc_sum_seen[j % 4] = j
        return out

    def scatter_flush(self) -> None:
        """Make the caller's stream wait for the sums of all pipelined steps issued so far."""
        if getattr(self, "_sc_side", None) is not None:
            torch.cuda.current_stream(self.local.device).wait_stream(self._sc_side)

    def forward_reduce_scatter_host(self, x_local_host: torch.Tensor, out_rows_host: torch.Tensor,
                                    chunk_rows: int = 2048) -> torch.Tensor:
        """The same end to end from and to page-locked host memory, pipelined over parts of the
        batch (needs ``enable_scatter(..., cyclic=True)``): while part ``c`` is in the kernels,
        part ``c + 1`` of this rank's input columns is on its way to the device and this rank's
        rows of part ``c - 1`` are on their way back.  ``x_local_host``: ``[m, local_in_size]``;
        ``out_rows_host``: ``[scatter_rows, out_size]``, filled with this rank's blocks.  Returns
        when the result is in host memory."""
        if not self._sc_blk:
            raise RuntimeError("forward_reduce_scatter_host needs enable_scatter(m, cyclic=True)")
        self._check_wait_status()
        dev = self.local.device
        m = x_local_host.size(0)
        round_rows = self._sc_blk * self.world
        chunk_rows = max(round_rows, chunk_rows // round_rows * round_rows)
        if getattr(self, "_sh_streams", None) is None:
            self._sh_streams = (torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev))
            self._sh_x = None
        if self._sh_x is None or self._sh_x[0].size(0) < chunk_rows:
            self._sh_x = [torch.empty(chunk_rows, self.local.local_in_size, device=dev) for _ in range(2)]
            self._sh_out = torch.empty(self._sc_rows, self.out_size, device=dev)
            self._sh_ev = [[torch.cuda.Event(), torch.cuda.Event()] for _ in range(2)]
        s_h2d, s_d2h = self._sh_streams
        main = torch.cuda.current_stream(dev)
        b = self._sc_step % self._sc_nbuf
        self._sc_step += 1
        self.scatter_flush()
        s_h2d.wait_stream(main)
        for c, r0 in enumerate(range(0, m, chunk_rows)):
            rows = min(chunk_rows, m - r0)
            xb = c & 1
            h2d_done, comp_done = self._sh_ev[xb]
            with torch.cuda.stream(s_h2d):
                if c >= 2:
                    s_h2d.wait_event(comp_done)  # staging buffer xb has been read
                self._sh_x[xb][:rows].copy_(x_local_host[r0:r0 + rows], non_blocking=True)
                h2d_done.record(s_h2d)
            main.wait_event(h2d_done)
            lr0, n = self._scatter_part(self._sh_x[xb][:rows], r0, b, self._sh_out)
            comp_done.record(main)
            if n:
                s_d2h.wait_event(comp_done)
                with torch.cuda.stream(s_d2h):
                    out_rows_host[lr0:lr0 + n].copy_(self._sh_out[lr0:lr0 + n], non_blocking=True)
        s_d2h.synchronize()
        main.synchronize()
        self._check_wait_status()
        return out_rows_host

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
