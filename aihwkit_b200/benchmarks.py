"""Training-step timings of the analog tile on one GPU: forward + backward + pulsed update.

    python -m aihwkit_b200.benchmarks --config 0|2|3 [--steps K] [--warmup W] [--indexed]

Configurations (seeded synthetic inputs with the stated shapes and distributions):
  0  single tile 256 x 256, batch 64, ConstantStep device, 7-bit DAC / 9-bit ADC, out_noise 0.06,
     ABS_MAX noise management, ITERATIVE bound management, StochasticCompressed BL 31, UM + UBLM
  2  Tiki-Taka: 1024 x 1024 TransferCompound of two SoftBoundsReference devices, batch 256,
     transfer every 2 batches, one column per transfer
  3  convolution-shaped tile 256 x 2304 (3x3x256), 131072 input columns per step, SoftBounds device
     (default: the activations are fed as an already unfolded [columns, 2304] matrix; with
     --indexed the step goes through forward_indexed / backward_indexed / update_indexed on
     [128, 256, 32, 32] images and the index array of a padded 3x3 convolution, as a convolution
     layer calls the tile)

Prints one JSON line: columns/s for the whole step and per phase, and for the update kernel the
achieved HBM bandwidth on its algorithmic bytes `x*d*(8+P) + 4*m*(x+d)` against the measured copy
bandwidth (P = per-element parameter bytes: 16 ConstantStep, 24 SoftBounds / SoftBoundsReference).
For large batches the update is bound by the coincidence arithmetic (x*d*m AND+popc), not by HBM;
the line then also reports coincidence pairs per second.
"""

from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path, "r", encoding="utf-8") as f:
            p = json.load(f)
        return p["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def build(config: int):
    from .rpu_base import devices as D

    p = D.AnalogTileParameter()
    for io in (p.forward_io, p.backward_io):
        io.inp_res, io.out_res = 1.0 / 126.0, 1.0 / 510.0
        io.out_noise, io.out_bound, io.inp_bound = 0.06, 12.0, 1.0
        io.noise_management = D.NoiseManagementType.AbsMax
    p.forward_io.bound_management = D.BoundManagementType.Iterative
    p.update.pulse_type = D.PulseType.StochasticCompressed
    p.update.desired_bl = 31
    if config == 0:
        dp = D.ConstantStepResistiveDeviceParameter()
        dp.dw_min, dp.dw_min_dtod, dp.dw_min_std = 0.001, 0.3, 0.3
        dp.up_down, dp.up_down_dtod, dp.w_max, dp.w_min = 0.0, 0.01, 0.6, -0.6
        dp.enforce_consistency = True
        dp.construction_seed = 1
        return p, dp, dict(x=256, d=256, m=64, lr=0.01, par_bytes=16, xdist="uniform", dstd=0.1,
                           winit="uniform")
    if config == 2:
        dp = D.TransferResistiveDeviceParameter()
        for _ in range(2):
            u = D.SoftBoundsReferenceResistiveDeviceParameter()
            u.dw_min, u.w_max, u.w_min, u.reference_std = 0.002, 1.0, -1.0, 0.05
            u.enforce_consistency = True
            dp.append_parameter(u)
        dp.construction_seed = 2
        dp.gamma, dp.transfer_every, dp.units_in_mbatch = 0.0, 2.0, True
        dp.n_reads_per_transfer, dp.transfer_lr, dp.fast_lr = 1, 0.01, 1.0
        dp.transfer_forward.bound_management = D.BoundManagementType.Iterative
        return p, dp, dict(x=1024, d=1024, m=256, lr=0.01, par_bytes=24, xdist="uniform",
                           dstd=0.05, winit="zero")
    if config == 3:
        dp = D.SoftBoundsResistiveDeviceParameter()
        dp.dw_min, dp.w_max, dp.w_min, dp.dw_min_dtod = 0.001, 0.6, -0.6, 0.3
        dp.enforce_consistency = True
        dp.construction_seed = 3
        return p, dp, dict(x=2304, d=256, m=131072, lr=0.01, par_bytes=24, xdist="relu",
                           dstd=0.01, winit="uniform")
    raise SystemExit("config must be 0, 2 or 3")


def _bf16_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)["bf16_tflops"], "measured"
    return 1590.0, "fallback"


def launch_floor_us(lib, n: int = 300) -> float:
    """Time per launch of a chain of dependent, near-empty kernels of the library on the current
    stream: the floor a phase made of L launches cannot go below (L times this)."""
    import torch

    a = torch.zeros(2, 4, device="cuda")
    o = torch.zeros(4, device="cuda")
    for _ in range(20):
        lib.ab200_sum_slots(a.data_ptr(), 2, 4, o.data_ptr(), None)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n):
        lib.ab200_sum_slots(a.data_ptr(), 2, 4, o.data_ptr(), None)
    e1.record()
    torch.cuda.synchronize()
    return 1e3 * e0.elapsed_time(e1) / n


def run(config: int, steps: int = 20, warmup: int = 3, batch: int = 0, indexed: bool = False,
        on_line=None, update_path: int = 0) -> dict:
    """One benchmark line (a dict) for configuration 0, 2 or 3.  ``on_line(line, cfg, x, d, lr)``,
    when given, may extend it (``bench.py --config N`` adds the CPU baseline of the compiled
    reference there)."""
    import ctypes as C

    import torch

    from . import _cabi
    from .rpu_base import tiles as T

    if not torch.cuda.is_available():
        raise RuntimeError("needs a CUDA device: the analog tile has no CPU path")
    lib = _cabi.lib()
    _cabi.check(lib.ab200_set_update_path(int(update_path)))
    p, dp, w = build(config)
    x_size, d_size = w["x"], w["d"]
    m = batch or w["m"]
    cfg = p._config(x_size, d_size, dp, seed=100 + config)
    tile = T.AnalogTile(cfg, cuda_device=0)
    g = torch.Generator().manual_seed(config)
    if w["winit"] == "uniform":
        tile.set_weights(torch.rand(d_size, x_size, generator=g) - 0.5)
    tile.set_learning_rate(w["lr"])
    if w["xdist"] == "uniform":
        x = torch.rand(m, x_size, generator=g) * 2 - 1
    else:
        x = torch.relu(torch.randn(m, x_size, generator=g))
    d = torch.randn(m, d_size, generator=g) * w["dstd"]
    x, d = x.cuda(), d.cuda()
    fwd = lambda: tile.forward(x, non_blocking=True)  # noqa: E731
    bwd = lambda: tile.backward(d, non_blocking=True)  # noqa: E731
    upd = lambda: tile.update(x, d, non_blocking=True)  # noqa: E731
    if indexed:
        if config != 3:
            raise SystemExit("--indexed applies to config 3")
        c, hw = 256, 32
        n_img = m // (hw * hw)
        m = n_img * hw * hw
        img = torch.relu(torch.randn(n_img, c, hw, hw, generator=g)).cuda()
        err = (torch.randn(n_img, d_size, hw, hw, generator=g) * w["dstd"]).cuda()
        idx = torch.nn.functional.unfold(
            torch.arange(2, c * hw * hw + 2, dtype=torch.float64).reshape(1, c, hw, hw),
            kernel_size=3, padding=1).flatten().round().to(torch.int32).cuda()
        tile.set_matrix_indices(idx)
        y_img, g_img = torch.empty_like(err), torch.empty_like(img)
        fwd = lambda: tile.forward_indexed(img, y_img, non_blocking=True)  # noqa: E731
        bwd = lambda: tile.backward_indexed(err, g_img, non_blocking=True)  # noqa: E731
        upd = lambda: tile.update_indexed(img, err, non_blocking=True)  # noqa: E731

    def ev():
        return torch.cuda.Event(enable_timing=True)

    for _ in range(warmup):
        fwd()
        bwd()
        upd()
    torch.cuda.synchronize()
    # launches per phase (the library counts its own)
    launches = []
    for fn in (fwd, bwd, upd):
        n0 = lib.ab200_kernel_launch_count()
        fn()
        launches.append(int(lib.ab200_kernel_launch_count() - n0))
    torch.cuda.synchronize()
    t_f = t_b = t_u = 0.0
    e = [ev() for _ in range(4)]
    t0 = time.perf_counter()
    for _ in range(steps):
        e[0].record()
        fwd()
        e[1].record()
        bwd()
        e[2].record()
        upd()
        e[3].record()
        torch.cuda.synchronize()
        t_f += e[0].elapsed_time(e[1])
        t_b += e[1].elapsed_time(e[2])
        t_u += e[2].elapsed_time(e[3])
    wall = time.perf_counter() - t0
    # the same step without a host synchronisation between steps: what a training loop sees
    e0, e1 = ev(), ev()
    e0.record()
    th0 = time.perf_counter()
    for _ in range(steps):
        fwd()
        bwd()
        upd()
    host_ms = 1e3 * (time.perf_counter() - th0) / steps  # time the host needs to enqueue a step
    e1.record()
    torch.cuda.synchronize()
    stream_ms = e0.elapsed_time(e1) / steps
    k = steps
    t_f, t_b, t_u = t_f / k, t_b / k, t_u / k
    step_ms = t_f + t_b + t_u
    hbm, src = _peaks()
    bf16, bf16_src = _bf16_peak()
    floor_us = launch_floor_us(lib)
    upd_bytes = x_size * d_size * (8 + w["par_bytes"]) + 4 * m * (x_size + d_size)
    mvm_bytes = 4 * m * (x_size + d_size) + 4 * x_size * d_size
    flops = 2.0 * m * x_size * d_size
    pairs = float(x_size) * d_size * m
    popc = C.c_double(0.0)
    _cabi.check(lib.ab200_measure_popc_peak(0, C.byref(popc)))

    def mvm_roofline(t_ms, n_launch):
        tf = flops / (t_ms * 1e-3) / 1e12
        gbs = mvm_bytes / (t_ms * 1e-3) / 1e9
        # whichever ceiling is nearer bounds the pass: the split-bf16 tensor rate or the HBM copy rate
        t_tensor = flops / (bf16 / 2 * 1e12)
        t_hbm = mvm_bytes / (hbm * 1e9)
        bound = "tensor" if t_tensor >= t_hbm else "hbm"
        return {"bound": bound, "logical_tflops": tf, "tensor_peak": bf16, "terms": 2,
                "frac_of_split_bf16_peak": tf / (bf16 / 2), "algorithmic_gbs": gbs,
                "frac_of_hbm": gbs / hbm, "launches": n_launch,
                "launch_floor_ms": n_launch * floor_us * 1e-3,
                "frac_of_time_above_launch_floor": max(0.0, 1.0 - n_launch * floor_us * 1e-3 / t_ms)}

    line = {
        "metric": "analog_tile_fwd_bwd_update_columns_per_s",
        "config": config, "indexed": bool(indexed), "x_size": x_size, "d_size": d_size, "batch": m,
        "value": m / (stream_ms * 1e-3), "unit": "columns/s",
        "ms": {"forward": t_f, "backward": t_b, "update": t_u, "step_sum_of_phases": step_ms,
               "step_back_to_back": stream_ms, "host_enqueue_per_step": host_ms, "wall_per_step": 1e3 * wall / k},
        "launch_floor_us_per_launch": floor_us,
        "forward_roofline": mvm_roofline(t_f, launches[0]),
        "backward_roofline": mvm_roofline(t_b, launches[1]),
        "update_roofline": {
            "bound": "integer" if pairs / (popc.value or 1.0) > upd_bytes / (hbm * 1e9) else "hbm",
            "algorithmic_bytes": upd_bytes,
            "achieved": upd_bytes / (t_u * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
            "frac": upd_bytes / (t_u * 1e-3) / 1e9 / hbm, "peak_source": src,
            "coincidence_pairs_per_s": pairs / (t_u * 1e-3),
            "popc_pairs_per_s_peak": popc.value,
            "frac_of_popc_peak": pairs / (t_u * 1e-3) / (popc.value or 1.0),
            "launches": launches[2], "launch_floor_ms": launches[2] * floor_us * 1e-3,
        },
        "peak_sources": {"hbm": src, "bf16": bf16_src},
    }
    if on_line is not None:
        on_line(line, cfg, x, d, w["lr"])
    return line


def main(argv=None, on_line=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=0)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=0, help="override the batch size")
    ap.add_argument("--indexed", action="store_true", help="config 3 through the indexed interface")
    ap.add_argument("--update-path", type=int, default=0, choices=[0, 1, 2],
                    help="kernel of the pulsed update: 0 automatic, 1 staged, 2 streaming")
    args = ap.parse_args(argv)
    print(json.dumps(run(args.config, args.steps, args.warmup, args.batch, args.indexed, on_line,
                         args.update_path)))


if __name__ == "__main__":
    main()
