#!/usr/bin/env python
"""Benchmark of the analog-tile hot path.

Workload (N GPUs): "analog inference MVM" — a logical 4096 x 4096 weight (~N(0, 1/64)) mapped onto
64 physical 512 x 512 tiles, batch of 8192 rows ~N(0, 1), forward only, 8-bit DAC / ADC,
out_noise 0.04, additive-constant weight noise 0.0175, out_bound 10, ABS_MAX noise management,
no bound management.  A step is one forward pass of the whole batch through all tiles; with N > 1
the in-splits are sharded over the ranks and the partial outputs are summed to rank 0 with one
NCCL reduce (strong scaling: the total work is fixed).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

`--impl reference` times the reference's own CPU tile (oracle/_ref, built from the reference's
sources) on a bounded sample of the same workload on the host cores.

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(out_size=4096, in_size=4096, max_tile=512, batch=8192)
METRIC = "analog_inference_rows_per_s"
UNIT = "rows/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path, "r", encoding="utf-8") as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def inference_config(seed: int):
    from aihwkit_b200.rpu_base import devices as D

    p = D.AnalogTileParameter()
    io = p.forward_io
    io.inp_res = 1.0 / 254.0
    io.out_res = 1.0 / 254.0
    io.out_noise = 0.04
    io.w_noise = 0.0175
    io.w_noise_type = D.WeightNoiseType.AdditiveConstant
    io.out_bound = 10.0
    io.inp_bound = 1.0
    io.noise_management = D.NoiseManagementType.AbsMax
    io.bound_management = D.BoundManagementType.None_
    p.update.pulse_type = D.PulseType.None_
    return p._config(512, 512, D.IdealResistiveDeviceParameter(), seed=seed)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def wait_first(self, timeout=8.0):
        """Block until nvidia-smi has printed its first sample (its start-up takes a second or
        more on a multi-GPU host), so that a short run is not over before sampling begins."""
        t0 = time.time()
        while self.proc is not None and not self.lines and time.time() - t0 < timeout:
            time.sleep(0.02)

    def samples_in(self, window):
        return sum(1 for l in self.lines if window[0] <= l[0] <= window[1] + 0.02)

    def stop(self, window=None, scope_if_window="timed region"):
        """`window` = (t0, t1) wall-clock bounds of the timed region: samples inside it are used;
        if the region was shorter than the sampling period, all samples taken under load (from
        the warm-up on) are used instead and the result says so."""
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power, masks = [], [], set(), [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = self.lines
        scope = "warm-up + timed region"
        if window is not None:
            inside = [l for l in lines if window[0] <= l[0] <= window[1] + 0.02]
            if inside:
                lines, scope = inside, scope_if_window
        for _, line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            try:
                power.append(float(parts[3]))
            except ValueError:
                pass
            masks.add(parts[4])
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None,
                    sm_max_mhz=max(smax) if smax else None, reasons=sorted(reasons),
                    samples=len(sm), scope=scope, power_w_max=max(power) if power else None,
                    reasons_mask=sorted(masks))


# --------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CPU tile on a bounded sample
# --------------------------------------------------------------------------------------------
def _ref_worker(args):
    """Runs `rows` input rows through the tiles `tile_ids` of the mapped layer with the reference
    CPU tile (one C++ forward call per tile, as TileModuleArray does)."""
    tile_ids, rows, seed, reps = args
    from oracle import ref

    cfg = inference_config(seed)
    rng = np.random.default_rng(seed)
    tiles = []
    for tid in tile_ids:
        t = ref.RefTile(cfg)
        t.set_weights(rng.normal(0, 1.0 / 64.0, (512, 512)).astype(np.float32))
        tiles.append(t)
    x = rng.normal(0, 1, (rows, 512)).astype(np.float32)
    for t in tiles[:1]:
        t.forward(x[: max(1, rows // 8)], is_test=True)  # warm-up
    t0 = time.perf_counter()
    for _ in range(reps):
        for t in tiles:
            t.forward(x, is_test=True)
    return time.perf_counter() - t0


def cpu_reference_rate(rows: int, reps: int = 1, workers=None):
    """rows/s of the reference CPU tile for the full 64-tile layer, all host cores: the 64 tiles
    are independent, so they are spread over `workers` processes (the analog CPU path itself is a
    serial per-sample loop, src/rpucuda/rpu_pulsed.h:107)."""
    from concurrent.futures import ProcessPoolExecutor
    from oracle import ref

    if not ref.available():
        return None
    n_tiles = (WORKLOAD["out_size"] // WORKLOAD["max_tile"]) * (WORKLOAD["in_size"] // WORKLOAD["max_tile"])
    workers = workers or min(os.cpu_count() or 1, n_tiles)
    os.environ.setdefault("OPENBLAS_NUM_THREADS", "1")
    os.environ.setdefault("OMP_NUM_THREADS", "1")
    chunks = [list(range(n_tiles))[i::workers] for i in range(workers)]
    t0 = time.perf_counter()
    with ProcessPoolExecutor(max_workers=workers) as ex:
        times = list(ex.map(_ref_worker, [(c, rows, 17 + i, reps) for i, c in enumerate(chunks)]))
    wall = time.perf_counter() - t0
    busy = max(times)
    return dict(value=rows * reps / busy, unit=UNIT, cores=workers, kind="reference",
                sample=f"{rows} of {WORKLOAD['batch']} rows through all {n_tiles} tiles x {reps} "
                       f"(reference CPU RPUPulsed, BLAS {ref.blas_name()}, 1 BLAS thread per "
                       f"process, tiles spread over {workers} processes; wall {wall:.1f} s)",
                seconds=busy)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_reference_rate(rows=args.ref_rows, reps=1)
    if base is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/librpu_ref.so is not built or does not load on this box"}))
        return
    # K timed steps of the bounded sample (W warm-up steps are the worker's own warm-up call)
    vals = [base["value"]]
    for _ in range(max(0, min(args.steps, 3) - 1)):
        vals.append(cpu_reference_rate(rows=args.ref_rows, reps=1)["value"])
    v = statistics.median(vals)
    base["value"] = v
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(vals), "warmup": args.warmup, "ms_per_step": 1e3 * WORKLOAD["batch"] / v,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "cfg1: 4096x4096 analog inference MVM, 64 tiles of 512x512, batch 8192",
                   "timed": f"bounded sample of {args.ref_rows} rows per step, extrapolated linearly"},
        "cpu_baseline": base,
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def owned_blocks(m: int, rank: int, world: int, blk: int = 256):
    """(first row of the batch, first row in the owner's buffer, rows) of the 256-row blocks of a
    batch that are dealt to ``rank``."""
    out = []
    for b in range(rank, (m + blk - 1) // blk, world):
        out.append((b * blk, (b // world) * blk, min(blk, m - b * blk)))
    return out


def other_configurations(args):
    """Short one-GPU runs of the other benchmark configurations (GPU part only), so that their
    lines are measured in the same run: 0, 2, 3 = training step of a single tile, 4 = the
    GPT-2-small-shaped forward."""
    import io
    import contextlib

    from aihwkit_b200 import benchmarks, gpt2_inference

    out = {}
    for c, steps in ((0, 50), (2, 30), (3, 4)):
        try:
            line = benchmarks.run(c, steps=steps, warmup=3)
            out[f"cfg{c}"] = {k: line[k] for k in ("value", "unit", "batch", "ms", "forward_roofline",
                                                   "backward_roofline", "update_roofline",
                                                   "launch_floor_us_per_launch")}
        except Exception as exc:  # a failing side run must not lose the contract line
            out[f"cfg{c}"] = {"error": str(exc)[:200]}
    try:
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            gpt2_inference.main(["--steps", "2", "--warmup", "2"])
        g = json.loads(buf.getvalue().strip().splitlines()[-1])
        out["cfg4"] = {k: g[k] for k in ("value", "unit", "ms_per_step", "config", "e2e", "analog_layers",
                                         "gpu_launches")}
    except Exception as exc:
        out["cfg4"] = {"error": str(exc)[:200]}
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    from aihwkit_b200 import _cabi, hostmem
    from aihwkit_b200.rpu_base import tiles as T
    from aihwkit_b200.sharded import ShardedTileArray, column_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the analog tile has no CPU path")
    if args.mvm_path:
        _cabi.check(_cabi.lib().ab200_set_mvm_path(args.mvm_path))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # page-locked staging buffers on the CPU socket this GPU hangs off (before they are allocated)
    numa_cpus = hostmem.bind_to_gpu_numa(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _cabi.lib()

    W = WORKLOAD
    m = W["batch"]
    cfg = inference_config(seed=1234)
    arr = ShardedTileArray(
        W["out_size"], W["in_size"], W["max_tile"], W["max_tile"],
        lambda b, e: T.TileArray(cfg, W["out_size"], W["in_size"], W["max_tile"], W["max_tile"],
                                 cuda_device=local_rank, in_split_range=(b, e)))
    g = torch.Generator().manual_seed(1)
    weight = torch.randn(W["out_size"], W["in_size"], generator=g) / 64.0
    arr.local.set_weights(weight)
    x_host = torch.randn(m, W["in_size"], generator=g).pin_memory()
    x = x_host.to(dev)

    scatter = world > 1 and args.collective == "scatter"
    c0, c1 = column_range(W["in_size"], W["max_tile"], rank, world)
    x_local_dev = x[:, c0:c1].contiguous() if world > 1 else x
    if scatter:
        # partial sums are pushed to the owners of the row blocks by the MVM kernel itself
        # (peer stores over NVLink), the result stays sharded by rows
        try:
            arr.enable_scatter(m, codes={"auto": None, "on": True, "off": False}[args.scatter_codes],
                               cyclic=True, buffers=4 if args.step_pipeline else 2)
        except RuntimeError as exc:  # raised on every rank alike: fall back to the NCCL reduce
            if rank == 0:
                print(f"bench: {exc}; using --collective reduce", file=sys.stderr)
            scatter = False
            args.collective = "reduce"

    def step():
        if scatter:
            return arr.forward_reduce_scatter(x_local_dev, pipelined=bool(args.step_pipeline))
        if world > 1 and args.reduce_chunks > 1:
            return arr.forward_overlapped(x, dst=0, n_chunks=args.reduce_chunks, is_test=True)
        y = arr.forward_partial(x, is_test=True, non_blocking=True)
        return arr.reduce(y, dst=0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- the fused data plane against NCCL, same noise (the call counters restart with the seed)
    check = None
    if scatter:
        arr.local.set_seed(4242)
        mine = arr.forward_reduce_scatter(x_local_dev).clone()
        arr.local.set_seed(4242)
        full = arr.local.forward_local(x_local_dev)
        dist.all_reduce(full)
        diff = torch.zeros(2, device=dev)
        for r0, l0, n in owned_blocks(m, rank, world):
            diff[0] = torch.maximum(diff[0], (mine[l0:l0 + n] - full[r0:r0 + n]).abs().max())
        diff[1] = full.abs().max()
        dist.all_reduce(diff, op=dist.ReduceOp.MAX)
        tol = 2e-5 * float(diff[1])
        check = {"against": "NCCL all-reduce of the ranks' partial sums, same noise draws",
                 "max_abs_diff": float(diff[0]), "max_abs_value": float(diff[1]), "tolerance": tol,
                 "ok": bool(float(diff[0]) <= tol)}
        arr.local.set_seed(1234)
        del mine, full

    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_first()
    for _ in range(args.warmup):
        step()
    barrier()
    t_wall0 = time.time()
    launches0 = lib.ab200_kernel_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    if scatter:
        arr.scatter_flush()  # the owner's sums of the last steps (side stream) belong to the region
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = lib.ab200_kernel_launch_count() - launches0
    window = (t_wall0, time.time())

    # ---- the same load for at least a second, with the clock samples taken inside it
    n_sus = max(args.steps, int(args.sustain_s / max(ms * 1e-3 / args.steps, 1e-6)))
    n_sus_t = torch.tensor([n_sus], device=dev)
    if world > 1:
        dist.all_reduce(n_sus_t, op=dist.ReduceOp.MAX)  # every rank runs the same count
    n_sus = int(n_sus_t)
    barrier()
    t_sus0 = time.time()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(n_sus):
        step()
    if scatter:
        arr.scatter_flush()
    s1.record()
    barrier()
    sus_ms = s0.elapsed_time(s1)
    sus_window = (t_sus0, time.time())
    if sampler.samples_in(window) >= 3:
        clocks = sampler.stop(window, "timed region")
        sus_clocks = None
    else:
        # the timed region is shorter than a few sampling periods: the clocks are those of the
        # sustained loop of the same step that followed it
        clocks = sampler.stop(sus_window, "sustained loop of the same step right after the timed region")
        sus_clocks = clocks

    # ---- phases of the step (N > 1): kernel with its stores / owner's wait + sum
    phases = None
    mvm_ms = ms / args.steps
    if scatter:
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        acc = [0.0, 0.0]
        for _ in range(args.steps):
            arr.forward_reduce_scatter(x_local_dev, events=evs)
            torch.cuda.synchronize()
            acc[0] += evs[0].elapsed_time(evs[1])
            acc[1] += evs[1].elapsed_time(evs[2])
        t = torch.tensor(acc, device=dev) / args.steps
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        phases = {"dac_mvm_and_peer_stores_ms": float(t[0]),
                  "wait_for_senders_and_owner_sum_ms": float(t[1]),
                  "note": "max over ranks, one step at a time (host synchronisation between steps)"}
        mvm_ms = float(t[0])

    # ---- end to end through the public API with host buffers: this rank's input columns come
    # from page-locked host memory every step, its rows of the result go back to the host
    x_local_host = x_host[:, c0:c1].contiguous().pin_memory() if world > 1 else x_host
    if scatter:
        y_rows_host = torch.empty(arr.scatter_rows, W["out_size"]).pin_memory()

        def e2e_step():
            arr.forward_reduce_scatter_host(x_local_host, y_rows_host, chunk_rows=args.e2e_chunk_rows)
    else:
        y_host = torch.empty(m, W["out_size"]).pin_memory() if rank == 0 else None

        def e2e_step():
            # ShardedTileArray.forward_host: chunked host->device copies overlapped with the
            # kernels (inside the library for one rank), result back to the host on rank 0
            arr.forward_host(x_local_host, y_host, dst=0)

    for _ in range(max(1, args.warmup // 2)):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = min(args.steps, 50)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # ---- what the host link of this box gives for the same bytes: this rank's input columns in
    # and its rows out as plain page-locked copies on two streams at once (no kernels), so that
    # the end-to-end figure can be read as a fraction of a measured copy rate
    out_host_probe = y_rows_host if scatter else (y_host if y_host is not None else None)
    copy_ms = None
    if out_host_probe is not None:
        xd_probe = torch.empty_like(x_local_host, device=dev)
        yd_probe = torch.empty_like(out_host_probe, device=dev)
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        torch.cuda.synchronize()
        c0e, c1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for it in range(4):
            if it == 1:
                c0e.record()
                s_in.wait_event(c0e)
                s_out.wait_event(c0e)
            with torch.cuda.stream(s_in):
                xd_probe.copy_(x_local_host, non_blocking=True)
            with torch.cuda.stream(s_out):
                out_host_probe.copy_(yd_probe, non_blocking=True)
        torch.cuda.current_stream().wait_stream(s_in)
        torch.cuda.current_stream().wait_stream(s_out)
        c1e.record()
        torch.cuda.synchronize()
        copy_ms = c0e.elapsed_time(c1e) / 3
        del xd_probe, yd_probe
    barrier()

    if world > 1:
        t = torch.tensor([ms, e2e_ms, sus_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, sus_ms = (float(v) for v in t.tolist())
        tl = torch.tensor([launches], device=dev, dtype=torch.int64)
        dist.all_reduce(tl)
        launches = int(tl.item())

    if rank == 0:
        peaks = measured_peaks()
        n_local = arr.n_local_tiles
        flops = 2.0 * m * 512 * 512 * n_local  # algorithmic: one multiply-add per weight per row
        achieved = flops / (mvm_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]
        value = m * args.steps / (ms * 1e-3)
        pcie = 2.0 * m * W["in_size"] * 4 / world / (e2e_ms * 1e-3) / 1e9  # both directions, per rank
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {
                "workload": "cfg1: 4096x4096 analog inference MVM, 64 tiles of 512x512, batch 8192",
                "sharding": (f"in-splits over {world} rank(s), "
                             + ("signed-byte ADC codes of every in-split"
                                if getattr(arr, "_sc_codes", False) else "fp32 partial sums")
                             + " stored by the kernel into the row-block owners' memory over NVLink, "
                             "arrival flags, owner's sum (reduce-scatter, no collective call; the "
                             "256-row blocks are dealt to the ranks in turn and stay there)"
                             + ("; consecutive steps pipelined two deep: the owner's sum of step j runs "
                                "on a side stream beside the kernels of step j + 1, four slot sets"
                                if args.step_pipeline else ""))
                if scatter else (f"in-splits over {world} rank(s), NCCL reduce to rank 0"
                                 if world > 1 else "one rank, all 64 tiles"),
                "l2": "input (134 MB) and output (134 MB) per step exceed the 126 MB L2",
                "host_numa_cpus": numa_cpus,
            },
            "clocks": clocks,
            "e2e": {"value": m / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": int(m * W["in_size"] * 4),  # summed over the ranks
                    "d2h_bytes_per_step": int(m * W["out_size"] * 4),
                    "ms_per_step": e2e_ms, "pcie_gbs_per_rank_both_directions": pcie,
                    # the same bytes of rank 0 as bare copies, both directions at once
                    "copies_only_ms": copy_ms,
                    "frac_of_copies_only": (copy_ms / e2e_ms) if copy_ms else None},
            "gpu_launches": int(launches),
            "sustained": {"value": m * n_sus / (sus_ms * 1e-3), "unit": UNIT, "steps": n_sus,
                          "seconds": sus_ms * 1e-3, "ms_per_step": sus_ms / n_sus,
                          "clocks": sus_clocks if sus_clocks is not None else "see clocks (timed region)"},
            "roofline": {
                "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak,
                "terms": 2, "frac_of_split_bf16_peak": achieved / (peak / 2),
                # dram__bytes_read.sum + dram__bytes_write.sum of the step's two kernels on one
                # GPU (dacQuantizeRowKernel 173 MB + mvmTcKernel 419 MB), from the two ncu captures
                # of this command summarised in profiles/mvmTcKernel_cfg1_inference_4096x4096_b8192.md;
                # algorithmic bytes of the step are 536 MB (input 134, codes 67 written + 67 read,
                # bf16 hi / lo operands 134, output 134)
                "traffic": 592.0e6 if world == 1 else None,
                "peak_source": f"bf16_tflops (burst), {peaks['source']}",
                "kernel": ("DAC + IO-managed MVM of this rank's tiles: the timed step itself"
                           if world == 1 else "DAC + MVM + peer stores phase of the step (max over ranks)"),
                "kernel_ms_per_step": mvm_ms, "tiles_per_launch_group": n_local,
            },
        }
        if check is not None:
            line["check"] = check
        if phases is not None:
            line["phases"] = phases
        if world == 1 and not args.no_other_configs:
            line["other_configs"] = other_configurations(args)
        if world == 1 and not args.no_cpu_baseline:
            base = cpu_reference_rate(rows=args.ref_rows)
            if base is not None:
                line["cpu_baseline"] = base
            else:
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference",
                                        "sample": "oracle/_ref not available on this box"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if check is not None and not check["ok"]:
        sys.exit(3)


def run_training_config(args):
    """Configurations 0, 2, 3: GPU timing by the package's benchmark module; the compiled
    reference CPU tile runs a bounded sample of the same step on one host thread."""
    from aihwkit_b200 import benchmarks

    def add_cpu_baseline(line, cfg, x, d, lr):
        if args.no_cpu_baseline:
            return
        from oracle import ref

        if not ref.available():
            line["cpu_baseline"] = {"value": None, "kind": "reference", "sample": "oracle/_ref not built"}
            return
        rt = ref.RefTile(cfg)
        m = x.size(0)
        mc = min(m, 512)
        xc, dc = x[:mc].cpu().numpy(), d[:mc].cpu().numpy()
        rt.set_learning_rate(lr)
        rt.forward(xc[:8])
        t0 = time.perf_counter()
        rt.forward(xc)
        rt.backward(dc)
        rt.update(xc, dc)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": mc / dt, "unit": "columns/s", "cores": 1, "kind": "reference",
                                "sample": f"{mc} of {m} columns, 1 thread"}

    argv = ["--config", str(args.config)]
    if args.steps != 200:
        argv += ["--steps", str(args.steps)]
    if args.warmup != 10:
        argv += ["--warmup", str(args.warmup)]
    benchmarks.main(argv, on_line=add_cpu_baseline)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-rows", type=int, default=4096,
                    help="rows of the bounded CPU sample (reference arm / cpu_baseline)")
    ap.add_argument("--mvm-path", type=int, default=0, choices=[0, 1, 2, 3],
                    help="kernel selection of the library (ab200_set_mvm_path); 0 = automatic")
    ap.add_argument("--scatter-codes", default="auto", choices=["auto", "on", "off"],
                    help="N > 1 with --collective scatter: send the signed-byte ADC codes of every "
                         "in-split instead of fp32 partial sums (auto: when a rank holds at most "
                         "three in-splits)")
    ap.add_argument("--step-pipeline", type=int, default=0, choices=[0, 1],
                    help="N > 1 with --collective scatter: 1 = overlap the owner's sum of a step with the "
                         "kernels of the next one (side stream, four slot sets); measured slower than "
                         "one stream (the sum's CTAs delay the persistent MVM kernel's), so off")
    ap.add_argument("--collective", default="scatter", choices=["scatter", "reduce"],
                    help="N > 1: 'scatter' = the MVM kernel stores its partial sums into the row-block "
                         "owners' memory (reduce-scatter fused with the compute); 'reduce' = local "
                         "partial sums + NCCL reduce to rank 0")
    ap.add_argument("--reduce-chunks", type=int, default=1,
                    help="N > 1: row blocks whose partial-sum reduce overlaps the next block's kernels")
    ap.add_argument("--no-cpu-baseline", action="store_true",
                    help="skip the CPU baseline leg (used for profiler captures)")
    ap.add_argument("--no-other-configs", action="store_true",
                    help="N = 1: skip the short runs of configurations 0, 2, 3, 4")
    ap.add_argument("--sustain-s", type=float, default=1.2,
                    help="length of the sustained loop of the same step (clock samples inside it)")
    ap.add_argument("--e2e-chunk-rows", type=int, default=2048,
                    help="N > 1: rows per part of the pipelined end-to-end path")
    ap.add_argument("--config", type=int, default=1, choices=[0, 1, 2, 3, 4],
                    help="1 = the mapped inference layer (the contract line); 0, 2, 3 = training "
                         "step of a single tile (aihwkit_b200.benchmarks) with the reference CPU "
                         "tile timed beside it; 4 = forward of the GPT-2-small-shaped stack "
                         "(aihwkit_b200.gpt2_inference), under torchrun with --shard")
    ap.add_argument("--shard", default="tiles", choices=["tiles", "sequences"],
                    help="--config 4, N > 1: deal the tiles of every analog layer to the ranks "
                         "(all-reduce of the activations per layer) or the sequences (no collective)")
    args = ap.parse_args()
    if args.config == 4:
        from aihwkit_b200 import gpt2_inference
        argv = ["--shard", args.shard]
        if args.steps != 200:
            argv += ["--steps", str(args.steps)]
        if args.warmup != 10:
            argv += ["--warmup", str(args.warmup)]
        gpt2_inference.main(argv)
    elif args.config != 1:
        run_training_config(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
