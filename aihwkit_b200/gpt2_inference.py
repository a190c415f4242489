"""Analog inference of a transformer with the layer shapes of GPT-2 small: every linear layer of
the blocks runs on mapped analog tiles, everything else stays digital fp32.

    python -m aihwkit_b200.gpt2_inference [--layers 12] [--batch 16] [--seq 1024] [--steps 5]
    python -m torch.distributed.run --nproc-per-node N ... -m aihwkit_b200.gpt2_inference ...

Shapes only: the weights are random (N(0, 0.02), seeded), the token ids uniform over the
vocabulary; no checkpoint and no text is involved.  Per block: QKV 768 -> 2304, attention output
768 -> 768, MLP 768 -> 3072 -> 768.  Each of them is a mapped-tile layer
(``TileModuleArray``, src/aihwkit/simulator/tiles/array.py:30-198) with tiles of at most 512 x 512
(768 -> [384, 384], 2304 -> 4 x 461 + 460, 3072 -> 6 x 512) and the inference IO settings
(8-bit DAC / ADC, out_noise 0.04, additive weight noise 0.0175, ABS_MAX noise management).
Embeddings, LayerNorm, attention, GELU, residuals and the vocabulary projection are fp32 torch ops,
as they are digital in the reference too (``AnalogLinear`` only replaces ``nn.Linear``,
src/aihwkit/nn/conversion.py).

Two ways to use N ranks (``--shard``):
  ``sequences`` (default): sequences are independent, so every rank takes ``batch / N`` sequences
      and holds all tiles; no collective on the data path.
  ``tiles``: the tiles of every analog layer are dealt to the ranks - over the in-splits first,
      over the out-splits where a layer has fewer in-splits than ranks (768 -> 2 in-splits) - every
      rank computes the partial output of its block of tiles for ALL tokens, and one NCCL
      all-reduce per layer adds the partial outputs up (``TileModuleArray``'s ``result.add_`` over
      in-splits, tiles/array.py:173-176, across GPUs).  The digital parts run replicated.
Prints one JSON line (rank 0): tokens/s of the whole forward, the share of the analog layers, and
their logical TFLOP/s.
"""

from __future__ import annotations

import argparse
import json
import os
from typing import List

import torch
import torch.nn.functional as F

VOCAB, N_POS = 50257, 1024


def inference_config(seed: int, max_tile: int = 512):
    from .rpu_base import devices as D

    p = D.AnalogTileParameter()
    io = p.forward_io
    io.inp_res = io.out_res = 1.0 / 254.0
    io.out_noise = 0.04
    io.w_noise = 0.0175
    io.w_noise_type = D.WeightNoiseType.AdditiveConstant
    io.out_bound, io.inp_bound = 10.0, 1.0
    io.noise_management = D.NoiseManagementType.AbsMax
    io.bound_management = D.BoundManagementType.None_
    p.update.pulse_type = D.PulseType.None_
    return p._config(max_tile, max_tile, D.IdealResistiveDeviceParameter(), seed=seed)


class AnalogLinear:
    """``y = sum over tiles of alpha_tile * tile(x) + bias``: every tile stores its block of the
    weight matrix divided by ``alpha_tile = max|w_tile|`` so that it fills the conductance range
    [-1, 1] (the reference's weight-scaling omega = 1, layer-wise per tile,
    src/aihwkit/simulator/tiles/periphery.py:437-500); the scales and the digital bias are applied
    inside the mapped layer's kernels, so a layer is two launches (DAC, MVM)."""

    def __init__(self, in_features: int, out_features: int, device: int, seed: int,
                 gen: torch.Generator, max_tile: int = 512, shard_tiles: bool = False):
        from .rpu_base import tiles as T
        from .sharded import ShardedTileArray

        w = torch.randn(out_features, in_features, generator=gen) * 0.02
        cfg = inference_config(seed, max_tile)
        self.sharded = None
        if shard_tiles:
            # this rank's block of the layer's tiles; the ranks' partial outputs are all-reduced
            self.sharded = ShardedTileArray(
                out_features, in_features, max_tile, max_tile,
                lambda b, e, ob, oe: T.TileArray(cfg, out_features, in_features, max_tile, max_tile,
                                                 cuda_device=device, in_split_range=(b, e),
                                                 out_split_range=(ob, oe)),
                two_d=True)
            self.array = self.sharded.local
        else:
            self.array = T.TileArray(cfg, out_features, in_features, max_tile, max_tile,
                                     cuda_device=device)
        self.array.set_seed(seed)
        self.array.set_weights(w, weight_scaling_omega=1.0)
        self.array.set_bias(torch.zeros(out_features))
        self.in_features, self.out_features = in_features, out_features

    @property
    def n_tiles(self) -> int:
        return self.array.num_in_splits * self.array.num_out_splits

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        y = self.array.forward(x.reshape(-1, self.in_features), is_test=True, non_blocking=True)
        if self.sharded is not None:
            y = self.sharded.reduce(y, dst=None)  # all-reduce of the shards' partial outputs
        return y.reshape(*x.shape[:-1], self.out_features)


class Block:
    def __init__(self, d_model: int, n_head: int, device: int, seed: int, gen: torch.Generator,
                 shard_tiles: bool = False):
        dev = f"cuda:{device}"
        self.n_head = n_head
        self.ln1_w, self.ln1_b = torch.ones(d_model, device=dev), torch.zeros(d_model, device=dev)
        self.ln2_w, self.ln2_b = torch.ones(d_model, device=dev), torch.zeros(d_model, device=dev)
        self.qkv = AnalogLinear(d_model, 3 * d_model, device, seed + 1, gen, shard_tiles=shard_tiles)
        self.proj = AnalogLinear(d_model, d_model, device, seed + 2, gen, shard_tiles=shard_tiles)
        self.fc = AnalogLinear(d_model, 4 * d_model, device, seed + 3, gen, shard_tiles=shard_tiles)
        self.fc_out = AnalogLinear(4 * d_model, d_model, device, seed + 4, gen, shard_tiles=shard_tiles)

    def linears(self) -> List[AnalogLinear]:
        return [self.qkv, self.proj, self.fc, self.fc_out]

    def __call__(self, h: torch.Tensor, timer=None) -> torch.Tensor:
        b, s, d = h.shape
        a = F.layer_norm(h, (d,), self.ln1_w, self.ln1_b)
        q, k, v = timed(timer, self.qkv, a).split(d, dim=-1)
        shape = (b, s, self.n_head, d // self.n_head)
        q, k, v = (t.reshape(shape).transpose(1, 2) for t in (q, k, v))
        att = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        h = h + timed(timer, self.proj, att.transpose(1, 2).reshape(b, s, d))
        a = F.layer_norm(h, (d,), self.ln2_w, self.ln2_b)
        return h + timed(timer, self.fc_out, F.gelu(timed(timer, self.fc, a)))


def timed(timer, fn, x):
    """Run ``fn(x)``; with a timer, bracket it with CUDA events on the current stream."""
    if timer is None:
        return fn(x)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    y = fn(x)
    e1.record()
    timer.append((e0, e1))
    return y


class AnalogGPT2:
    def __init__(self, n_layer: int = 12, d_model: int = 768, n_head: int = 12, device: int = 0,
                 seed: int = 4, shard_tiles: bool = False):
        gen = torch.Generator().manual_seed(seed)
        dev = f"cuda:{device}"
        self.device = dev
        self.d_model = d_model
        self.wte = (torch.randn(VOCAB, d_model, generator=gen) * 0.02).to(dev)
        self.wpe = (torch.randn(N_POS, d_model, generator=gen) * 0.01).to(dev)
        self.blocks = [Block(d_model, n_head, device, seed * 1000 + 10 * i, gen, shard_tiles)
                       for i in range(n_layer)]
        self.lnf_w, self.lnf_b = torch.ones(d_model, device=dev), torch.zeros(d_model, device=dev)

    def forward(self, ids: torch.Tensor, timer=None) -> torch.Tensor:
        """``ids`` [batch, seq] on the device -> id of the most likely next token per position."""
        b, s = ids.shape
        h = self.wte[ids] + self.wpe[:s]
        for blk in self.blocks:
            h = blk(h, timer)
        h = F.layer_norm(h, (self.d_model,), self.lnf_w, self.lnf_b)
        out = torch.empty(b, s, dtype=torch.long, device=ids.device)
        # vocabulary projection in row chunks: the full logits would be 3.3 GB per 16384 tokens
        flat = h.reshape(-1, self.d_model)
        chunk = 4096
        for r0 in range(0, flat.size(0), chunk):
            out.view(-1)[r0 : r0 + chunk] = (flat[r0 : r0 + chunk] @ self.wte.t()).argmax(dim=-1)
        return out

    def analog_flops_per_token(self) -> float:
        return sum(2.0 * lin.in_features * lin.out_features for blk in self.blocks for lin in blk.linears())

    def n_tiles(self) -> int:
        return sum(lin.n_tiles for blk in self.blocks for lin in blk.linears())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--shard", default="sequences", choices=["sequences", "tiles"],
                    help="N > 1: split the sequences over the ranks, or the tiles of every analog layer")
    args = ap.parse_args(argv)

    import torch.distributed as dist

    from . import _cabi

    if not torch.cuda.is_available():
        raise RuntimeError("needs a CUDA device: the analog tiles have no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    shard_tiles = world > 1 and args.shard == "tiles"
    if args.batch % world and not shard_tiles:
        raise SystemExit("--batch must be a multiple of the number of ranks")
    local_batch = args.batch if shard_tiles else args.batch // world
    model = AnalogGPT2(args.layers, device=local_rank, seed=4, shard_tiles=shard_tiles)
    k = 0
    for blk in model.blocks:  # independent noise per layer (and per rank when ranks hold replicas)
        for lin in blk.linears():
            lin.array.set_seed((1 if shard_tiles else 100003 * (rank + 1)) + k)
            k += 1
    g = torch.Generator().manual_seed(4 + (0 if shard_tiles else rank))
    ids_host = torch.randint(0, VOCAB, (local_batch, args.seq), generator=g).pin_memory()
    out_host = torch.empty(local_batch, args.seq, dtype=torch.long).pin_memory()
    ids = ids_host.to(model.device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_loop(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=model.device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps

    with torch.no_grad():
        for _ in range(args.warmup):
            model.forward(ids)
        launches0 = _cabi.lib().ab200_kernel_launch_count()
        ms = timed_loop(lambda: model.forward(ids), args.steps)
        launches = (_cabi.lib().ab200_kernel_launch_count() - launches0) // args.steps

        def e2e():
            d = ids_host.to(model.device, non_blocking=True)
            out_host.copy_(model.forward(d), non_blocking=True)

        e2e()
        ms_e2e = timed_loop(e2e, args.steps)
        timer = []
        torch.cuda.synchronize()
        model.forward(ids, timer)
        torch.cuda.synchronize()
        analog_ms = sum(a.elapsed_time(b) for a, b in timer)
    tokens = args.batch * args.seq
    if rank == 0:
        flops = model.analog_flops_per_token() * local_batch * args.seq / (world if shard_tiles else 1)
        print(json.dumps({
            "metric": "analog_inference_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "dtype": "f32 (analog layers: DAC codes x split-bf16 weights, f32 accumulate)",
            "data": "synthetic",
            "config": {"workload": f"GPT-2-small-shaped forward, {args.layers} blocks, batch {args.batch} x seq {args.seq}",
                       "analog_tiles": model.n_tiles(), "parallelism": (f"tiles of every analog layer over {world} rank(s), all-reduce of the "
                                       "partial outputs, digital parts replicated" if shard_tiles
                                       else f"sequences over {world} rank(s)")},
            "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": ids_host.numel() * 8 * (1 if shard_tiles else world),
                    "d2h_bytes_per_step": out_host.numel() * 8 * (1 if shard_tiles else world)},
            "analog_layers": {"ms_per_step": analog_ms, "share": analog_ms / ms,
                              "logical_tflops": flops / (analog_ms * 1e-3) / 1e12},
            "gpu_launches": int(launches),
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
