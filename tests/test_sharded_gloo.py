"""Host logic of the sharded mapped layer on CPU: two gloo ranks each own a block of in-splits,
compute their partial sum (with the numpy oracle standing in for the GPU tiles) and the
collective adds them up to what one rank computes for the whole layer."""

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _OracleArray:
    """Partial sum over in-splits [begin, end) with the single-tile oracle."""

    def __init__(self, W, cfg, max_tile, begin, end):
        from aihwkit_b200.sharded import split_sizes

        self.W, self.cfg, self.max_tile = W, cfg, max_tile
        self.begin, self.end = begin, end
        self.in_sizes = split_sizes(W.shape[1], max_tile)
        self.out_sizes = split_sizes(W.shape[0], max_tile)

    def forward(self, x, out=None, **_):
        y = self._forward(x)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def _forward(self, x):
        from oracle import analog_tile_oracle as O

        io = O.IO.from_c(self.cfg.forward_io)
        X = x.numpy()
        y = np.zeros((X.shape[0], self.W.shape[0]), np.float32)
        offs = np.concatenate([[0], np.cumsum(self.in_sizes)])
        for ii in range(self.begin, self.end):
            c0, c1 = offs[ii], offs[ii + 1]
            r0 = 0
            for osz in self.out_sizes:
                y[:, r0 : r0 + osz] += O.forward(self.W[r0 : r0 + osz, c0:c1], X[:, c0:c1], io)
                r0 += osz
        return torch.from_numpy(y)


def _worker(rank, world, port, out_path):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.sharded import ShardedTileArray
    from tests import helpers as H

    rng = np.random.default_rng(0)
    out_size, in_size, max_tile, m = 96, 200, 64, 10
    W = rng.normal(0, 0.1, (out_size, in_size)).astype(np.float32)
    X = torch.from_numpy(rng.normal(0, 1, (m, in_size)).astype(np.float32))
    cfg = H.inference_params(noise=False)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=1)
    arr = ShardedTileArray(out_size, in_size, max_tile, max_tile,
                           lambda b, e: _OracleArray(W, cfg, max_tile, b, e))
    assert arr.world == world and len(arr.in_sizes) == 4
    y = arr.forward(X, dst=0)
    y_all = arr.reduce(arr.forward_partial(X), dst=None)
    # row blocks whose collectives are issued asynchronously, ragged last block
    y_ov = arr.forward_overlapped(X, dst=None, n_chunks=3).clone()
    y_ov0 = arr.forward_overlapped(X, dst=0, n_chunks=4)
    if rank == 0:
        full = _OracleArray(W, cfg, max_tile, 0, 4).forward(X)
        ok = torch.allclose(y, full, atol=1e-5) and torch.allclose(y_all, full, atol=1e-5)
        ok = ok and torch.allclose(y_ov, full, atol=1e-5) and torch.allclose(y_ov0, full, atol=1e-5)
        with open(out_path, "w") as f:
            f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_partial_sums_reduce_to_full_layer(tmp_path, world):
    out = tmp_path / "result.txt"
    port = 29500 + (os.getpid() % 400) + world
    mp.spawn(_worker, args=(world, port, str(out)), nprocs=world, join=True)
    assert out.read_text() == "ok"


def _empty_rank_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aihwkit_b200.sharded import ShardedTileArray

    class _Local:
        device = torch.device("cpu")

        def scatter_codes_supported(self):
            return False

    # two in-splits on three ranks: the last rank owns none
    arr = ShardedTileArray(64, 100, 64, 64, lambda b, e: _Local())
    msg = "no error"
    try:
        arr.enable_scatter(256)
    except RuntimeError as exc:
        msg = str(exc)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(msg)
    dist.barrier()
    dist.destroy_process_group()


def test_scatter_setup_raises_on_every_rank_when_one_owns_no_in_split(tmp_path):
    """A rank without tiles would never signal its peers; the set-up refuses on all ranks alike
    instead of letting the others wait for it."""
    world = 3
    port = 29950 + (os.getpid() % 40)
    mp.spawn(_empty_rank_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    msgs = [(tmp_path / f"rank{r}.txt").read_text() for r in range(world)]
    assert all("at least one in-split per rank" in m for m in msgs), msgs
    assert len(set(msgs)) == 1


def test_two_d_tile_map_covers_every_tile_once():
    """Blocks over in-splits and out-splits: every tile of the layer belongs to exactly one rank,
    for the layer shapes of the transformer benchmark on 1 to 8 ranks."""
    sys.path.insert(0, ROOT)
    from aihwkit_b200.sharded import block_of_rank, split_sizes, tile_grid

    for in_size, out_size in ((768, 2304), (768, 768), (768, 3072), (3072, 768), (4096, 4096)):
        n_in, n_out = len(split_sizes(in_size, 512)), len(split_sizes(out_size, 512))
        for world in (1, 2, 3, 4, 8):
            g_in, g_out = tile_grid(n_in, n_out, world)
            assert g_in * g_out == world and g_in <= max(1, n_in)
            owner = {}
            for rank in range(world):
                (ib, ie), (ob, oe) = block_of_rank(n_in, n_out, rank, world)
                for i in range(ib, ie):
                    for o in range(ob, oe):
                        assert (i, o) not in owner
                        owner[(i, o)] = rank
            assert len(owner) == n_in * n_out
