"""Shared builders for the parity tests: tile configurations (the five benchmark configurations
at reduced and full size), seeded inputs and comparison utilities."""

from __future__ import annotations

import numpy as np

from aihwkit_b200.rpu_base import devices as D

KINDS = {
    "cs": D.ConstantStepResistiveDeviceParameter,
    "ls": D.LinearStepResistiveDeviceParameter,
    "sb": D.SoftBoundsResistiveDeviceParameter,
    "sbr": D.SoftBoundsReferenceResistiveDeviceParameter,
    "es": D.ExpStepResistiveDeviceParameter,
    "ps": D.PowStepResistiveDeviceParameter,
    "pw": D.PiecewiseStepResistiveDeviceParameter,
}


def training_params(noise: bool, pulse_det: bool, bm: bool = True, out_bound: float = 12.0,
                    adc: bool = True) -> D.AnalogTileParameter:
    """IO of benchmark configuration 0: 7-bit DAC, 9-bit ADC, out_noise 0.06, ABS_MAX noise
    management, ITERATIVE bound management; StochasticCompressed BL=31 with UM + UBLM."""
    p = D.AnalogTileParameter()
    for io in (p.forward_io, p.backward_io):
        io.inp_res = 1.0 / 126.0
        io.out_res = 1.0 / 510.0 if adc else -1.0
        io.out_noise = 0.06 if noise else 0.0
        io.out_bound = out_bound
        io.inp_bound = 1.0
        io.noise_management = D.NoiseManagementType.AbsMax
    p.forward_io.bound_management = (
        D.BoundManagementType.Iterative if bm else D.BoundManagementType.None_
    )
    p.update.pulse_type = (
        D.PulseType.DeterministicImplicit if pulse_det else D.PulseType.StochasticCompressed
    )
    p.update.desired_bl = 31
    p.update.update_management = True
    p.update.update_bl_management = True
    return p


def inference_params(noise: bool) -> D.AnalogTileParameter:
    """IO of benchmark configuration 1: 8-bit DAC / ADC, out_noise 0.04, additive-constant weight
    noise 0.0175, out_bound 10, ABS_MAX, no bound management."""
    p = D.AnalogTileParameter()
    io = p.forward_io
    io.inp_res = 1.0 / 254.0
    io.out_res = 1.0 / 254.0
    io.out_noise = 0.04 if noise else 0.0
    io.w_noise = 0.0175 if noise else 0.0
    io.w_noise_type = D.WeightNoiseType.AdditiveConstant
    io.out_bound = 10.0
    io.noise_management = D.NoiseManagementType.AbsMax
    io.bound_management = D.BoundManagementType.None_
    p.update.pulse_type = D.PulseType.None_
    return p


def device(kind: str, noise: bool, seed: int = 11, **kw):
    dp = KINDS[kind]()
    dp.construction_seed = seed
    dp.enforce_consistency = True  # Python-side default of the reference (configs/devices.py:188)
    if not noise:
        dp.dw_min_std = 0.0
    if kind == "sbr":
        dp.reference_std = 0.05
    for k, v in kw.items():
        setattr(dp, k, v)
    return dp


PIECEWISE_UP = [1.2, 1.0, 0.8, 0.55, 0.4, 0.3]
PIECEWISE_DOWN = [0.25, 0.5, 0.7, 0.9, 1.0, 1.3]


def piecewise_device(noise: bool, **kw):
    """PiecewiseStep with six nodes per direction: steps up shrink towards the upper bound, steps
    down towards the lower one."""
    return device("pw", noise, piecewise_up=list(PIECEWISE_UP), piecewise_down=list(PIECEWISE_DOWN),
                  dw_min=0.002, dw_min_dtod=0.2, up_down=0.05, up_down_dtod=0.02, **kw)


def transfer_device(noise: bool, seed: int = 21, transfer_every: float = 2.0,
                    units_in_mbatch: bool = True, n_reads: int = 1, transfer_lr: float = 0.01,
                    det: bool = False):
    """Benchmark configuration 2: TransferCompound of two SoftBoundsReference devices."""
    dp = D.TransferResistiveDeviceParameter()
    for _ in range(2):
        dp.append_parameter(device("sbr", noise, dw_min=0.002, w_max=1.0, w_min=-1.0))
    dp.construction_seed = seed
    dp.gamma = 0.0
    dp.transfer_every = transfer_every
    dp.units_in_mbatch = units_in_mbatch
    dp.n_reads_per_transfer = n_reads
    dp.transfer_lr = transfer_lr
    dp.fast_lr = 1.0
    # Python defaults of TransferCompound: IOParameters() / UpdateParameters()
    tf = dp.transfer_forward
    tf.bound_management = D.BoundManagementType.Iterative
    tf.out_noise = 0.06 if noise else 0.0
    if det:
        dp.transfer_update.pulse_type = D.PulseType.DeterministicImplicit
    return dp


def lsb_report(a: np.ndarray, b: np.ndarray, lsb: np.ndarray):
    """Fraction of elements that differ and the largest difference in units of `lsb`."""
    diff = np.abs(a.astype(np.float64) - b.astype(np.float64))
    rel = diff / np.maximum(lsb, 1e-30)
    return float((rel > 1e-3).mean()), float(rel.max(initial=0.0))


def assert_moments_agree(a: np.ndarray, b: np.ndarray, z_max: float = 5.0, std_tol: float = 0.1):
    """Two sets of repeats `[reps, ...]` agree in their first two moments: every element's mean
    difference is within `z_max` standard errors (the reference's own tests use 2/sqrt(nloop) on
    unit-scale data, src/rpucuda/cuda/rpucuda_pulsed_test.cpp:1050-1131) and the average
    per-element standard deviations agree within `std_tol`."""
    ra, rb = a.shape[0], b.shape[0]
    se = np.sqrt(a.var(axis=0) / ra + b.var(axis=0) / rb)
    floor = 1e-3 * max(float(a.std()), float(b.std()), 1e-30) / np.sqrt(min(ra, rb))
    z = np.abs(a.mean(axis=0) - b.mean(axis=0)) / np.maximum(se, floor)
    assert float(z.max()) < z_max, f"max z-score {float(z.max()):.2f}"
    sa, sb = float(a.std(axis=0).mean()), float(b.std(axis=0).mean())
    assert sb > 0 and abs(sa / sb - 1.0) < std_tol, f"std ratio {sa / sb:.3f}"


def buffered_transfer_device(seed: int = 21, transfer_every: float = 1.0, n_reads: int = 2,
                             thres_scale: float = 1.0, momentum: float = 0.0,
                             forget_buffer: bool = True, transfer_lr: float = 1.0):
    """Tiki-Taka v2: BufferedTransferCompound of two noise-free SoftBoundsReference devices; the
    gradient update of the fast tile uses deterministic pulses, the write of the slow tile the
    device's default of exactly one pulse per whole step in the buffer."""
    dp = D.BufferedTransferResistiveDeviceParameter()
    for _ in range(2):
        dp.append_parameter(device("sbr", False, dw_min=0.002, w_max=1.0, w_min=-1.0))
    dp.construction_seed = seed
    dp.gamma = 0.0
    dp.transfer_every = transfer_every
    dp.units_in_mbatch = False
    dp.n_reads_per_transfer = n_reads
    dp.transfer_lr = transfer_lr
    dp.fast_lr = 1.0
    dp.thres_scale, dp.momentum, dp.forget_buffer = thres_scale, momentum, forget_buffer
    dp.transfer_forward.out_noise = 0.0
    dp.transfer_forward.bound_management = D.BoundManagementType.Iterative
    return dp


def chopped_transfer_device(seed: int = 21, transfer_every: float = 1.0, in_chop_prob: float = 1.0,
                            in_chop_random: bool = True, out_chop_prob: float = 0.0,
                            momentum: float = 0.0, forget_buffer: bool = True,
                            transfer_lr: float = 1.0, buffer_granularity: float = 1.0,
                            correct_gradient_magnitudes: bool = False, auto_granularity: float = 0.0):
    """Tiki-Taka with choppers: ChoppedTransferCompound of two noise-free SoftBoundsReference
    devices, one read per transfer."""
    dp = D.ChoppedTransferResistiveDeviceParameter()
    for _ in range(2):
        dp.append_parameter(device("sbr", False, dw_min=0.002, w_max=1.0, w_min=-1.0))
    dp.construction_seed = seed
    dp.gamma = 0.0
    dp.transfer_every = transfer_every
    dp.units_in_mbatch = False
    dp.transfer_lr = transfer_lr
    dp.fast_lr = 1.0
    dp.momentum, dp.forget_buffer = momentum, forget_buffer
    dp.in_chop_prob, dp.in_chop_random, dp.out_chop_prob = in_chop_prob, in_chop_random, out_chop_prob
    dp.buffer_granularity = buffer_granularity
    dp.correct_gradient_magnitudes = correct_gradient_magnitudes
    dp.auto_granularity = auto_granularity
    dp.transfer_forward.out_noise = 0.0
    dp.transfer_forward.bound_management = D.BoundManagementType.Iterative
    return dp


def dynamic_transfer_device(in_chop_prob: float = 0.5, tail_weightening: float = 1.0,
                            buffer_cap: float = 10.0, correct_accumulation: bool = False, **kw):
    """Tiki-Taka with choppers and a running-mean reference: DynamicTransferCompound of two
    noise-free SoftBoundsReference devices, regular in-chopper schedule."""
    base = chopped_transfer_device(in_chop_prob=in_chop_prob, in_chop_random=False, **kw)
    dp = D.DynamicTransferResistiveDeviceParameter()
    for k, v in vars(base).items():
        setattr(dp, k, v)
    dp.tail_weightening, dp.buffer_cap = tail_weightening, buffer_cap
    dp.experimental_correct_accumulation = correct_accumulation
    return dp


def mixed_precision_device(kind: str = "sb", n_x_bins: int = 9, n_d_bins: int = 5, transfer_every: int = 1,
                           n_rows_per_transfer: int = -1, granularity: float = 0.0,
                           transfer_lr: float = 1.0, seed: int = 21, **kw):
    """MixedPrecisionCompound: a digital rank-update accumulator in front of one noise-free
    analog device."""
    dp = D.MixedPrecResistiveDeviceParameter()
    assert dp.set_device_parameter(device(kind, False, dw_min=0.002, **kw))
    dp.construction_seed = seed
    dp.n_x_bins, dp.n_d_bins = n_x_bins, n_d_bins
    dp.transfer_every, dp.n_rows_per_transfer = transfer_every, n_rows_per_transfer
    dp.granularity, dp.transfer_lr = granularity, transfer_lr
    return dp
