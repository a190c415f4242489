"""Sharded layer on two GPUs: the reduce-scatter by direct peer stores (fp32 partial sums, and the
signed-byte ADC codes of every in-split; rows owned in contiguous ranges or dealt in blocks; on the
device and pipelined from / to host memory) against the NCCL reduce of the same partial sums.
Needs two CUDA devices (skipped otherwise).  The owners' sum kernels wait for the senders' arrival
flags with a bound; the kernels that raise them run on the other GPU."""

import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_path):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from aihwkit_b200.rpu_base import devices as D, tiles as T
    from aihwkit_b200.sharded import ShardedTileArray, column_range
    from tests import helpers as H

    rng = np.random.default_rng(0)
    out_size, in_size, max_tile, m = 1024, 2048, 512, 1000
    W = rng.normal(0, 1 / np.sqrt(in_size), (out_size, in_size)).astype(np.float32)
    X = rng.normal(0, 1, (m, in_size)).astype(np.float32)
    cfg = H.inference_params(noise=True)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=8)
    ok = True
    for trial in range(3):  # NCCL reference, fp32 partial sums, signed-byte ADC codes
        arr = ShardedTileArray(out_size, in_size, max_tile, max_tile,
                               lambda b, e: T.TileArray(cfg, out_size, in_size, max_tile, max_tile,
                                                        cuda_device=rank, in_split_range=(b, e)))
        arr.local.set_weights(torch.from_numpy(W))
        c0, c1 = column_range(in_size, max_tile, rank, world)
        x_local = torch.from_numpy(np.ascontiguousarray(X[:, c0:c1])).cuda()
        if trial == 0:
            full = arr.reduce(arr.local.forward_local(x_local), dst=None)  # NCCL all-reduce
            ref = full.cpu().numpy()
        else:
            arr.enable_scatter(m, codes=(trial == 2))
            rows = arr.scatter_rows
            for step in range(3):  # several steps: double-buffered slots
                mine = arr.forward_reduce_scatter(x_local)
            torch.cuda.synchronize()
            lo, hi = rank * rows, min(m, (rank + 1) * rows)
            # the call counter advanced: compare with a fresh NCCL result of the same call number
            arr2 = ShardedTileArray(out_size, in_size, max_tile, max_tile,
                                    lambda b, e: T.TileArray(cfg, out_size, in_size, max_tile, max_tile,
                                                             cuda_device=rank, in_split_range=(b, e)))
            arr2.local.set_weights(torch.from_numpy(W))
            for step in range(3):
                full2 = arr2.reduce(arr2.local.forward_local(x_local), dst=None)
            want = full2[lo:hi].cpu().numpy()
            got = mine[: hi - lo].cpu().numpy()
            tol = 1e-6 if trial == 1 else 1e-5  # codes: the clip bound sits a hair below the top code
            ok = ok and np.allclose(got, want, rtol=tol, atol=tol) and not np.array_equal(want, ref[lo:hi])
            arr.disable_scatter()
            # blocks dealt in turn, end to end from and to page-locked host memory, in parts
            arr.enable_scatter(m, codes=(trial == 2), cyclic=True)
            arr.local.set_seed(77)
            x_host = torch.from_numpy(np.ascontiguousarray(X[:, c0:c1])).pin_memory()
            y_host = torch.empty(arr.scatter_rows, out_size).pin_memory()
            arr.forward_reduce_scatter_host(x_host, y_host, chunk_rows=512)
            arr2.local.set_seed(77)
            fulls = [arr2.reduce(arr2.local.forward_local(x_local), dst=None) for _ in range(2)]
            blk = 256
            for bi in range(rank, (m + blk - 1) // blk, world):
                part = bi * blk // 512  # the part (and call counter) the block went through with
                n = min(blk, m - bi * blk)
                lrow = (bi // world) * blk
                ok = ok and np.allclose(y_host[lrow:lrow + n].numpy(),
                                        fulls[part][bi * blk:bi * blk + n].cpu().numpy(), rtol=tol, atol=tol)
            arr.disable_scatter()
            # consecutive steps pipelined two deep over four slot sets: the sum of a step runs on
            # a side stream beside the kernels of the next; every step has its own input and
            # must give what NCCL gives for the same call number
            arr.enable_scatter(m, codes=(trial == 2), cyclic=True, buffers=4)
            arr.local.set_seed(99)
            arr2.local.set_seed(99)
            xs = [x_local * (0.5 + 0.25 * k) for k in range(7)]
            outs = [arr.forward_reduce_scatter(xk, pipelined=True) for xk in xs]
            outs.append(arr.forward_reduce_scatter(xs[0]))  # a plain step behind pipelined ones
            outs.append(arr.forward_reduce_scatter(xs[1], pipelined=True))  # and a pipelined one again
            arr.scatter_flush()
            torch.cuda.synchronize()
            for k, xk in enumerate(xs + [xs[0], xs[1]]):
                fullk = arr2.reduce(arr2.local.forward_local(xk), dst=None)
                for bi in range(rank, (m + blk - 1) // blk, world):
                    n = min(blk, m - bi * blk)
                    lrow = (bi // world) * blk
                    ok = ok and np.allclose(outs[k][lrow:lrow + n].cpu().numpy(),
                                            fullk[bi * blk:bi * blk + n].cpu().numpy(), rtol=tol, atol=tol)
            arr.disable_scatter()
    with open(f"{out_path}.{rank}", "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_reduce_scatter_by_peer_stores_matches_nccl(tmp_path):
    import torch.multiprocessing as mp

    out = str(tmp_path / "result")
    mp.spawn(_worker, args=(2, 29650 + os.getpid() % 200, out), nprocs=2, join=True)
    assert open(out + ".0").read() == "ok" and open(out + ".1").read() == "ok"
