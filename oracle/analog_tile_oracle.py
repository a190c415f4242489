"""TEST INFRASTRUCTURE — numpy restatement of the reference's analog-tile hot path.

This module restates, in fp32 numpy, what the reference CPU tile computes for
  * the IO-managed forward / backward MVM
    (src/rpucuda/rpu_forward_backward_pass.cpp:113-178, 571-719, 901-1027),
  * the pulsed update: update management, pulse generation, coincidences
    (src/rpucuda/rpu_pulsed_meta_parameter.cpp:153-236,
     src/rpucuda/sparse_bit_line_maker.cpp:200-353,
     src/rpucuda/dense_bit_line_maker.cpp:210-331,
     src/rpucuda/rpu_weight_updater.cpp:198-294),
  * the device rules ConstantStep / LinearStep(SoftBounds) / SoftBoundsReference
    (src/rpucuda/rpu_constantstep_device.cpp:28-78, rpu_linearstep_device.cpp:113-164,
     rpu_softbounds_reference_device.cpp:107-175),
  * the Tiki-Taka sequencing of TransferRPUDevice (src/rpucuda/rpu_transfer_device.cpp:366-557).

Parity pin: tests/test_oracle_vs_reference.py checks every function here against the compiled
reference (oracle/_ref, built from the reference's own sources) where that library is present,
and against the golden vectors in tests/golden/ (generated from the compiled reference by
tests/golden/make_golden.py) everywhere else.

It is a checker only.  The product (aihwkit_b200) never imports it.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Tuple

import numpy as np

f32 = np.float32

# enum values: src/rpucuda/rpu_pulsed_meta_parameter.h:146-178
NM_NONE, NM_ABS_MAX, NM_ABS_MAX_NP_SUM, NM_MAX, NM_CONSTANT = 0, 1, 2, 3, 4
BM_NONE, BM_ITERATIVE, BM_ITERATIVE_WORST_CASE = 0, 1, 2
WN_NONE, WN_ADDITIVE_CONSTANT, WN_PCM_READ = 0, 1, 2
PULSE_NONE, PULSE_STOCHASTIC_COMPRESSED, PULSE_DETERMINISTIC_IMPLICIT = 0, 1, 5
PULSE_MEAN_COUNT = 4
DEV_IDEAL, DEV_CONSTANT_STEP, DEV_LINEAR_STEP, DEV_SOFT_BOUNDS, DEV_SOFT_BOUNDS_REFERENCE = range(5)
DEV_TRANSFER = 5
DEV_EXP_STEP = 6
DEV_POW_STEP = 7
DEV_PIECEWISE_STEP = 8


def _check_res(res: float) -> np.float32:
    """detail::checkRes (rpu_pulsed_meta_parameter.cpp:26-29)."""
    r = f32(0.0) if res < 0 else f32(res)
    return f32(1.0) / r if r > f32(1.0) else r


@dataclass
class IO:
    """Effective IO parameters after initializeForForward/Backward
    (rpu_pulsed_meta_parameter.cpp:40-128)."""

    is_perfect: bool = False
    noise_management: int = NM_ABS_MAX
    bound_management: int = BM_NONE
    w_noise_type: int = WN_NONE
    bm_test_negative_bound: bool = True
    max_bm_factor: int = 1000
    max_bm_res: float = 0.25
    inp_bound: float = 1.0
    inp_res: float = 1.0 / 126.0
    out_bound: float = 12.0
    out_res: float = 1.0 / 510.0
    out_noise: float = 0.06
    out_scale: float = 1.0
    w_noise: float = 0.0
    nm_thres: float = 0.0
    nm_assumed_wmax: float = 0.6
    inp_noise: float = 0.0
    inp_asymmetry: float = 0.0
    out_asymmetry: float = 0.0
    inp_sto_round: bool = False
    out_sto_round: bool = False
    res_in: np.float32 = field(default=f32(0), init=False)
    res_out: np.float32 = field(default=f32(0), init=False)

    _finalized: bool = field(default=False, init=False)

    def __post_init__(self) -> None:
        self.finalize()

    def finalize(self, backward: bool = False) -> "IO":
        if backward:
            self.bound_management = BM_NONE
        if self.noise_management == NM_NONE:
            self.nm_thres = 0.0
        if self._finalized:
            return self
        self._finalized = True
        self.res_out = f32(_check_res(self.out_res) * f32(2.0) * f32(self.out_bound))
        self.res_in = f32(_check_res(self.inp_res) * f32(2.0) * f32(self.inp_bound))
        if self.noise_management == NM_NONE:
            self.nm_thres = 0.0
        if self.out_bound <= 0:
            self.out_bound = math.inf
        if self.inp_bound <= 0:
            self.inp_bound = math.inf
        if backward:
            self.bound_management = BM_NONE
        return self

    @staticmethod
    def from_c(c, backward: bool = False) -> "IO":
        """Build from an ``ab200_io_params`` ctypes struct."""
        io = IO(
            is_perfect=bool(c.is_perfect),
            noise_management=int(c.noise_management),
            bound_management=int(c.bound_management),
            w_noise_type=int(c.w_noise_type),
            bm_test_negative_bound=bool(c.bm_test_negative_bound),
            max_bm_factor=int(c.max_bm_factor),
            max_bm_res=float(c.max_bm_res),
            inp_bound=float(c.inp_bound),
            inp_res=float(c.inp_res),
            out_bound=float(c.out_bound),
            out_res=float(c.out_res),
            out_noise=float(c.out_noise),
            out_scale=float(c.out_scale),
            w_noise=float(c.w_noise),
            nm_thres=float(c.nm_thres),
            nm_assumed_wmax=float(c.nm_assumed_wmax),
            inp_noise=float(c.inp_noise),
            inp_asymmetry=float(c.inp_asymmetry),
            out_asymmetry=float(c.out_asymmetry),
            inp_sto_round=bool(c.inp_sto_round),
            out_sto_round=bool(c.out_sto_round),
        )
        return io.finalize(backward)


def quantize(v: np.ndarray, res: np.float32) -> np.ndarray:
    """getDiscretizedValueSR<false> (utility_functions.h:204-210); rint = ties-to-even."""
    if res <= 0:
        return v
    return (np.rint((v / f32(res)).astype(f32)).astype(f32) * f32(res)).astype(f32)


def quantize_sto(v: np.ndarray, res: np.float32, rng: np.random.Generator) -> np.ndarray:
    """getDiscretizedValue with sto_round (utility_functions.h:186-193):
    rint(v / res + (u - 0.5)) * res with u uniform in [0, 1)."""
    if res <= 0:
        return v
    u = rng.random(v.shape).astype(f32)
    q = ((v / f32(res)).astype(f32) + (u - f32(0.5)).astype(f32)).astype(f32)
    return (np.rint(q).astype(f32) * f32(res)).astype(f32)


def _nm_scale(v: np.ndarray, io: IO, nm_type: Optional[int] = None) -> np.ndarray:
    """computeNoiseManagement, per sample (rpu_forward_backward_pass.cpp:113-178)."""
    m = v.shape[0]
    nm_type = io.noise_management if nm_type is None else nm_type
    if nm_type == NM_NONE:
        return np.ones(m, f32)
    if nm_type == NM_ABS_MAX:
        s = np.abs(v).max(axis=1).astype(f32)
        return np.minimum(s, f32(io.nm_thres)) if io.nm_thres > 0 else s
    if nm_type == NM_MAX:
        s = v.max(axis=1).astype(f32)
        return np.minimum(s, f32(io.nm_thres)) if io.nm_thres > 0 else s
    if nm_type == NM_CONSTANT:
        return np.full(m, io.nm_thres if io.nm_thres > 0 else 1.0, f32)
    if nm_type == NM_ABS_MAX_NP_SUM:
        amax = np.abs(v).max(axis=1).astype(f32)
        bound = f32(1.0) if np.isinf(io.out_bound) else f32(io.out_bound)
        # sequential fp32 sums like the reference's loop
        psum = np.zeros(m, f32)
        nsum = np.zeros(m, f32)
        for j in range(v.shape[1]):
            col = v[:, j]
            psum = (psum + np.where(col > 0, col, f32(0))).astype(f32)
            nsum = (nsum + np.where(col < 0, col, f32(0))).astype(f32)
        tot = np.maximum(psum, -nsum)
        if io.nm_thres > 0:
            amax = np.minimum(amax, f32(io.nm_thres))
        np_scale = (tot * f32(io.nm_assumed_wmax) / bound).astype(f32)
        if io.res_in > 0:
            np_scale = np.minimum((amax / io.res_in * f32(io.max_bm_res)).astype(f32), np_scale)
        return np.maximum(amax, np_scale).astype(f32)
    raise NotImplementedError("noise management type")


def _analog_mv(
    w_op: np.ndarray, v_in: np.ndarray, scale: np.ndarray, scaling: np.ndarray, io: IO, bm: bool,
    rng: Optional[np.random.Generator],
) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """computeAnalogMV, OnePass (rpu_forward_backward_pass.cpp:795-829) for a batch of rows.

    ``w_op`` is [out, in]. Returns (output, bound_test_passed per row, pre-ADC value).
    """
    # prepareInput (:571-604)
    v = np.where(scaling[:, None], (v_in * scale[:, None]).astype(f32), v_in).astype(f32)
    v = quantize_sto(v, io.res_in, rng) if (io.inp_sto_round and rng is not None) else quantize(v, io.res_in)
    bound = f32(io.inp_bound) if io.inp_bound > 0 else f32(np.inf)
    v = np.clip(v, -bound, bound).astype(f32)
    if io.inp_noise > 0 and rng is not None:  # after the clip, as in the reference
        v = (v + f32(io.inp_noise) * rng.standard_normal(v.shape).astype(f32)).astype(f32)
    if io.inp_asymmetry != 0:
        v = np.where(v < 0, (v * f32(f32(1.0) - f32(io.inp_asymmetry))).astype(f32), v).astype(f32)
    # gemv
    y = (v @ w_op.T).astype(f32)
    # applyOutputWeightNoise (:326-352)
    if io.w_noise_type == WN_ADDITIVE_CONSTANT and io.w_noise > 0 and rng is not None:
        nrm = np.sqrt((v.astype(np.float64) ** 2).sum(axis=1)).astype(f32)
        y = (y + (f32(io.w_noise) * nrm)[:, None] * rng.standard_normal(y.shape).astype(f32)).astype(f32)
    if io.w_noise_type == WN_PCM_READ and io.w_noise > 0 and rng is not None:
        # :353-381: std-dev w_noise * sqrt(sum_j |w_ij| v_j^2) per output
        var = ((v.astype(np.float64) ** 2) @ np.abs(w_op.astype(np.float64)).T)
        y = (y + f32(io.w_noise) * np.sqrt(var).astype(f32) * rng.standard_normal(y.shape).astype(f32)).astype(f32)
    # finalizeOutput (:673-719): asymmetry, noise, ADC, clip
    if io.out_asymmetry != 0:
        y = np.where(y < 0, (y * f32(f32(1.0) - f32(io.out_asymmetry))).astype(f32), y).astype(f32)
    if io.out_noise > 0 and rng is not None:
        y = (y + f32(io.out_noise) * rng.standard_normal(y.shape).astype(f32)).astype(f32)
    pre_adc = y.copy()
    y = quantize_sto(y, io.res_out, rng) if (io.out_sto_round and rng is not None) else quantize(y, io.res_out)
    ob = f32(io.out_bound) if io.out_bound > 0 else f32(np.inf)
    passed = np.ones(y.shape[0], bool)
    if bm:
        hi = y > ob
        lo = y < -ob
        passed &= ~hi.any(axis=1)
        if io.bm_test_negative_bound:
            passed &= ~lo.any(axis=1)
    y = np.clip(y, -ob, ob).astype(f32)
    return y, passed, pre_adc


def forward(
    w: np.ndarray, x: np.ndarray, io: IO, rng: Optional[np.random.Generator] = None,
    alpha: float = 1.0, return_pre_adc: bool = False,
):
    """ForwardBackwardPassIOManaged::forwardVector for every row of ``x``
    (rpu_forward_backward_pass.cpp:901-988).  ``w`` is [d, x]; ``x`` is [m, x_size].
    ``rng`` None = all noise off (deterministic regime)."""
    w = np.asarray(w, f32)
    x = np.asarray(x, f32)
    m = x.shape[0]
    if io.is_perfect:
        return ((x @ w.T) * f32(io.out_scale * alpha)).astype(f32)
    s = _nm_scale(x, io)
    nm = io.noise_management != NM_NONE
    bm = io.bound_management != BM_NONE
    out = np.zeros((m, w.shape[0]), f32)
    pre = np.zeros((m, w.shape[0]), f32)
    reductions = np.ones(m, f32)
    # all-zero rows give zero, unless input noise is on (:924-933)
    zero_rows = nm & (s <= 0) & (not (io.inp_noise > 0 and rng is not None))
    todo = ~zero_rows
    red = f32(0.5)
    out_scale = f32(io.out_scale) * f32(alpha)
    final_scale = np.ones(m, f32)
    scaling_any = np.zeros(m, bool)
    bm_round = 0
    s = s.copy()
    while todo.any():
        red = f32(red * f32(2.0))
        idx = np.nonzero(todo)[0]
        if (bm_round == 1 and io.bound_management == BM_ITERATIVE_WORST_CASE
                and io.noise_management != NM_ABS_MAX_NP_SUM):
            # the first re-run switches to the AbsMaxNPSum scale and restarts the halving (:945-950)
            s[idx] = _nm_scale(x[idx], io, NM_ABS_MAX_NP_SUM)
            red = f32(1.0)
        bm_round += 1
        scale = np.ones(len(idx), f32)
        scaling = np.zeros(len(idx), bool)
        if nm:
            pos = s[idx] > 0
            safe = np.where(pos, s[idx], f32(1.0)).astype(f32)
            scale = np.where(pos, (f32(1.0) / safe).astype(f32), scale).astype(f32)
            scaling |= pos
        if bm:
            scale = (scale / red).astype(f32)
            scaling[:] = True
        y, passed, pre_adc = _analog_mv(w, x[idx], scale, scaling, io, bm, rng)
        out[idx] = y
        pre[idx] = pre_adc
        final_scale[idx] = scale
        scaling_any[idx] = scaling
        reductions[idx] = red
        if bm:
            stop = (int(red) > io.max_bm_factor) or (io.res_in > 0 and red > f32(io.max_bm_res) / io.res_in)
            passed = passed | stop
        else:
            passed[:] = True
        todo[idx[passed]] = False
    apply = scaling_any | (out_scale != f32(1.0))
    fac = (out_scale / final_scale).astype(f32)
    out = np.where(apply[:, None], (out * fac[:, None]).astype(f32), out).astype(f32)
    out[zero_rows] = 0
    if return_pre_adc:
        return out, pre, final_scale, reductions
    return out


def backward(
    w: np.ndarray, d: np.ndarray, io: IO, rng: Optional[np.random.Generator] = None,
    alpha: float = 1.0, return_pre_adc: bool = False,
):
    """ForwardBackwardPassIOManaged::backwardVector (rpu_forward_backward_pass.cpp:991-1027).
    ``d`` is [m, d_size]; result [m, x_size]."""
    w = np.asarray(w, f32)
    d = np.asarray(d, f32)
    if io.is_perfect:
        return ((d @ w) * f32(io.out_scale * alpha)).astype(f32)
    s = _nm_scale(d, io)
    nm = io.noise_management != NM_NONE
    scaling = np.full(d.shape[0], nm) & (s > 0)
    zero_rows = nm & (s <= 0)
    safe = np.where(s > 0, s, f32(1.0)).astype(f32)
    scale = (f32(1.0) / safe).astype(f32)
    y, _, pre = _analog_mv(w.T, d, scale, scaling, io, False, rng)
    out_scale = f32(io.out_scale) * f32(alpha)
    apply = scaling | (out_scale != f32(1.0))
    fac = (out_scale * s).astype(f32)
    y = np.where(apply[:, None], (y * fac[:, None]).astype(f32), y).astype(f32)
    y[zero_rows] = 0
    if return_pre_adc:
        return y, pre, scale
    return y


# ------------------------------------------------------------------------------------------
# update
# ------------------------------------------------------------------------------------------


@dataclass
class Up:
    """PulsedUpdateMetaParameter after initialize() (rpu_pulsed_meta_parameter.cpp:134-151)."""

    pulse_type: int = PULSE_STOCHASTIC_COMPRESSED
    desired_bl: int = 31
    fixed_bl: bool = True
    update_management: bool = True
    update_bl_management: bool = True
    um_grad_scale: float = 1.0
    res: float = 0.0
    x_res_implicit: float = 0.0
    d_res_implicit: float = 0.0

    def __post_init__(self) -> None:
        self.update_management = self.update_management or self.update_bl_management

    @staticmethod
    def from_c(c) -> "Up":
        return Up(
            int(c.pulse_type), int(c.desired_bl), bool(c.fixed_bl), bool(c.update_management),
            bool(c.update_bl_management), float(c.um_grad_scale), float(c.res),
            float(c.x_res_implicit), float(c.d_res_implicit),
        )


def bl_a_b(up: Up, lr: float, dw_min: float, xm: float, dm: float) -> Tuple[int, np.float32, np.float32]:
    """calculateBlAB + performUpdateManagement in fp32
    (rpu_pulsed_meta_parameter.cpp:153-236). Returns (BL, A, B); BL == 0 means no update."""
    lr, dw_min = f32(lr), f32(dw_min)
    if lr == 0:
        return 0, f32(0), f32(0)
    if up.fixed_bl or up.update_bl_management:
        bl = up.desired_bl
        a = f32(np.sqrt(f32(lr / f32(dw_min * f32(bl)))))
        b = a
    else:
        if f32(dw_min * f32(up.desired_bl)) < lr:
            a = b = f32(1.0)
            bl = max(int(math.ceil(f32(lr / dw_min))), 1)
        else:
            bl = up.desired_bl
            a = f32(np.sqrt(f32(lr / f32(dw_min * f32(bl)))))
            b = a
    if up.update_bl_management or up.update_management:
        xm, dm = f32(xm), f32(dm)
        if xm == 0 or dm == 0:
            return 0, f32(1), f32(1)
        x_val = xm
        d_val = f32(f32(up.um_grad_scale) * dm)
        k_val = f32(f32(f32(lr * x_val) * d_val) / dw_min)
        if up.update_bl_management:
            bl = int(np.ceil(k_val))
            bl = min(bl, up.desired_bl)
            a = f32(np.sqrt(f32(lr / f32(dw_min * f32(bl))))) if bl > 0 else f32(np.inf)
            b = a
        if up.update_management:
            if k_val > f32(up.desired_bl):
                d_val = f32(d_val * f32(f32(up.desired_bl) / k_val))
            a = f32(a * f32(np.sqrt(f32(x_val / d_val))))
            b = f32(b * f32(np.sqrt(f32(d_val / x_val))))
    return bl, a, b


def coincidences_det_implicit(x: np.ndarray, d: np.ndarray, lr: float, dw_min: float, up: Up) -> np.ndarray:
    """DenseBitLineMaker::makeCoincidences, DeterministicImplicit, one sample
    (dense_bit_line_maker.cpp:210-264, 266-331). Signed int32 [d, x]; positive = weight decreases."""
    x = np.asarray(x, f32)
    d = np.asarray(d, f32)
    alr = abs(lr)
    bl, a, b = bl_a_b(up, alr, dw_min, np.abs(x).max(initial=0), np.abs(d).max(initial=0))

    def implicit(v, p, res):
        vv = -v if lr < 0 else v
        pp = quantize((np.abs(vv) * f32(p)).astype(f32), f32(res))
        pp = np.clip(pp, f32(0), f32(1)).astype(f32)
        return np.where(vv >= 0, pp, -pp).astype(f32)

    xv = implicit(x, b, up.x_res_implicit)
    dv = implicit(d, a, up.d_res_implicit)
    dc = (dv * f32(bl)).astype(f32)
    n = np.rint((dc[:, None] * xv[None, :]).astype(f32)).astype(np.int32)
    n[dv == 0, :] = 0
    return n


def coincidences_mean_count(x: np.ndarray, d: np.ndarray, lr: float, dw_min: float, up: Up) -> np.ndarray:
    """DenseBitLineMaker::makeCoincidences, MeanCount, one sample (dense_bit_line_maker.cpp:142-204,
    266-312): the mean number of pulses per line, coincidences rint(d_count / BL * x_count).
    Signed int32 [d, x]; positive = weight decreases."""
    x = np.asarray(x, f32)
    d = np.asarray(d, f32)
    alr = abs(lr)
    bl, a, b = bl_a_b(up, alr, dw_min, np.abs(x).max(initial=0), np.abs(d).max(initial=0))
    if bl <= 0:
        return np.zeros((d.size, x.size), np.int32)

    def counts(v, p):
        vv = -v if lr < 0 else v
        pp = quantize((np.abs(vv) * f32(p)).astype(f32), f32(up.res))
        nt = np.clip(np.rint((f32(bl) * pp).astype(f32)), 0, bl).astype(np.int32)
        nt = np.where(pp == 0, 0, nt)
        return np.where(vv >= 0, nt, -nt).astype(np.int32)

    xc = counts(x, b)
    dc = (counts(d, a).astype(f32) / f32(bl)).astype(f32)
    n = np.rint((dc[:, None] * xc[None, :].astype(f32)).astype(f32)).astype(np.int32)
    n[dc == 0, :] = 0
    return n


def coincidences_stochastic_compressed(
    x: np.ndarray, d: np.ndarray, lr: float, dw_min: float, up: Up, rng: np.random.Generator
) -> np.ndarray:
    """SparseBitLineMaker::makeCounts (StochasticCompressed) + the coincidence loop of
    updateVectorWithDevice (sparse_bit_line_maker.cpp:200-238, 288-353;
    rpu_weight_updater.cpp:236-283), one sample. Signed int32 [d, x]; positive = decrease."""
    x = np.asarray(x, f32)
    d = np.asarray(d, f32)
    alr = abs(lr)
    lr_sign = -1 if lr < 0 else 1
    bl, a, b = bl_a_b(up, alr, dw_min, np.abs(x).max(initial=0), np.abs(d).max(initial=0))
    if bl <= 0:
        return np.zeros((d.size, x.size), np.int32)
    px = quantize((np.abs(x) * b).astype(f32), f32(up.res))
    pd = quantize((np.abs(d) * a).astype(f32), f32(up.res))
    xb = px[None, :] > rng.random((bl, x.size), dtype=np.float32)
    db = pd[None, :] > rng.random((bl, d.size), dtype=np.float32)
    n = db.T.astype(np.int32) @ xb.astype(np.int32)
    sx = np.where(x > 0, 1, -1)
    sd = np.where(d > 0, 1, -1) * lr_sign
    return (n * (sd[:, None] * sx[None, :])).astype(np.int32)


@dataclass
class DeviceArrays:
    """Per-element device parameters, all [d, x] fp32 (PulsedRPUDevice members,
    rpu_pulsed_device.cpp:594-733; names as in getDPNames :235-253)."""

    kind: int
    max_bound: np.ndarray
    min_bound: np.ndarray
    dwmin_up: np.ndarray
    dwmin_down: np.ndarray
    slope_up: Optional[np.ndarray] = None
    slope_down: Optional[np.ndarray] = None
    reference: Optional[np.ndarray] = None
    gamma_up: Optional[np.ndarray] = None  # PowStep exponents
    gamma_down: Optional[np.ndarray] = None
    dw_min_std: float = 0.0
    mult_noise: bool = True
    # ExpStep globals: (a, b, A_up, A_down, gamma_up, gamma_down, dw_min_std_add, dw_min_std_slope)
    es: Optional[tuple] = None
    # PiecewiseStep: (up factors, down factors) at equally spaced nodes over [min_bound, max_bound]
    pw: Optional[tuple] = None

    @staticmethod
    def from_hidden(kind: int, names, hp: np.ndarray, dw_min_std: float, mult_noise: bool, suffix=""):
        g = {n: hp[i] for i, n in enumerate(names)}
        kw = dict(
            kind=kind,
            max_bound=g["max_bound" + suffix],
            min_bound=g["min_bound" + suffix],
            dwmin_up=g["dwmin_up" + suffix],
            dwmin_down=g["dwmin_down" + suffix],
            dw_min_std=dw_min_std,
            mult_noise=mult_noise,
        )
        if "slope_up" + suffix in g:
            kw["slope_up"] = g["slope_up" + suffix]
            kw["slope_down"] = g["slope_down" + suffix]
        if "reference" + suffix in g:
            kw["reference"] = g["reference" + suffix]
        if "gamma_up" + suffix in g:
            kw["gamma_up"] = g["gamma_up" + suffix]
            kw["gamma_down"] = g["gamma_down" + suffix]
        return DeviceArrays(**kw)


def apply_pulses(w: np.ndarray, n_signed: np.ndarray, dev: DeviceArrays,
                 rng: Optional[np.random.Generator] = None) -> np.ndarray:
    """Apply |n| pulses of direction sign(n) to every element, one pulse at a time with the clip
    after each pulse (PULSED_UPDATE_W_LOOP[_DENSE], rpu_pulsed_device.h:450-474).  In place."""
    n_abs = np.abs(n_signed)
    down = n_signed > 0
    std = f32(dev.dw_min_std)
    for it in range(int(n_abs.max(initial=0))):
        act = n_abs > it
        if not act.any():
            break
        if std > 0 and rng is not None:
            xi = (std * rng.standard_normal(w.shape).astype(f32)).astype(f32)
        else:
            xi = np.zeros_like(w)
        if dev.kind == DEV_CONSTANT_STEP:
            # rpu_constantstep_device.cpp:28-78
            dw_down = ((f32(1.0) + xi) * dev.dwmin_down).astype(f32)
            dw_up = ((f32(1.0) + xi) * dev.dwmin_up).astype(f32)
            wn = np.where(down, w - dw_down, w + dw_up).astype(f32)
            wn = np.maximum(np.minimum(wn, dev.max_bound), dev.min_bound)
        elif dev.kind in (DEV_LINEAR_STEP, DEV_SOFT_BOUNDS):
            # rpu_linearstep_device.cpp:113-164
            if dev.mult_noise:
                dn = ((dev.slope_down * w + dev.dwmin_down).astype(f32) * (f32(1.0) + xi)).astype(f32)
                up_ = ((dev.slope_up * w + dev.dwmin_up).astype(f32) * (f32(1.0) + xi)).astype(f32)
            else:
                dn = (dev.slope_down * w + dev.dwmin_down * (f32(1.0) + xi)).astype(f32)
                up_ = (dev.slope_up * w + dev.dwmin_up * (f32(1.0) + xi)).astype(f32)
            wn = np.where(down, w - dn, w + up_).astype(f32)
            wn = np.minimum(np.maximum(wn, dev.min_bound), dev.max_bound)
        elif dev.kind == DEV_SOFT_BOUNDS_REFERENCE:
            # rpu_softbounds_reference_device.cpp:107-175
            wr = (w + dev.reference).astype(f32)
            with np.errstate(divide="ignore", invalid="ignore"):
                a_dn = np.where(dev.min_bound < 0, wr / dev.min_bound, f32(0)).astype(f32)
                a_up = np.where(dev.max_bound > 0, wr / dev.max_bound, f32(0)).astype(f32)
            if dev.mult_noise:
                dn = (dev.dwmin_down * (f32(1.0) - a_dn) * (f32(1.0) + xi)).astype(f32)
                up_ = (dev.dwmin_up * (f32(1.0) - a_up) * (f32(1.0) + xi)).astype(f32)
            else:
                dn = (dev.dwmin_down * (f32(1.0) - a_dn + xi)).astype(f32)
                up_ = (dev.dwmin_up * (f32(1.0) - a_up + xi)).astype(f32)
            wn = np.where(down, wr - dn, wr + up_).astype(f32)
            wn = np.minimum(np.maximum(wn, dev.min_bound), dev.max_bound)
            wn = (wn - dev.reference).astype(f32)
        elif dev.kind == DEV_EXP_STEP:
            # rpu_expstep_device.cpp:18-100 (expf in fp32)
            a, b, A_up, A_dn, g_up, g_dn, s_add, s_slope = (f32(v) for v in dev.es)
            b_diff = (dev.max_bound - dev.min_bound).astype(f32)
            with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
                z = ((f32(2.0) * w / b_diff).astype(f32) * a + b).astype(f32)
                y_dn = np.maximum(f32(1.0) - A_dn * np.exp((g_dn * (-z)).astype(f32)).astype(f32), f32(0))
                y_up = np.maximum(f32(1.0) - A_up * np.exp((g_up * z).astype(f32)).astype(f32), f32(0))
            if std > 0 and (s_add != 0 or s_slope != 0):
                dw = np.where(down, -(y_dn * dev.dwmin_down), y_up * dev.dwmin_up).astype(f32)
                # the oracle's xi already carries dw_min_std
                spread = (np.abs(dw) + s_add + s_slope * np.abs(w)).astype(f32)
                wn = (w + (dw + spread * xi)).astype(f32)
            else:
                dn = ((y_dn * (f32(1.0) + xi)).astype(f32) * dev.dwmin_down).astype(f32)
                up_ = ((y_up * (f32(1.0) + xi)).astype(f32) * dev.dwmin_up).astype(f32)
                wn = np.where(down, w - dn, w + up_).astype(f32)
            wn = np.maximum(np.minimum(wn, dev.max_bound), dev.min_bound)
            wn = np.where(b_diff > 0, wn, w)
        elif dev.kind == DEV_POW_STEP:
            # rpu_powstep_device.cpp:91-121 (powf in fp32)
            rng_w = (dev.max_bound - dev.min_bound).astype(f32)
            with np.errstate(divide="ignore", invalid="ignore"):
                f_dn = np.power(((w - dev.min_bound) / rng_w).astype(f32), dev.gamma_down).astype(f32)
                f_up = np.power(((dev.max_bound - w) / rng_w).astype(f32), dev.gamma_up).astype(f32)
            dn = ((dev.dwmin_down * f_dn).astype(f32) * (f32(1.0) + xi)).astype(f32)
            up_ = ((dev.dwmin_up * f_up).astype(f32) * (f32(1.0) + xi)).astype(f32)
            wn = np.where(down, w - dn, w + up_).astype(f32)
            wn = np.minimum(np.maximum(wn, dev.min_bound), dev.max_bound)
            wn = np.where(rng_w == 0, w, wn)
        elif dev.kind == DEV_PIECEWISE_STEP:
            # rpu_piecewisestep_device.cpp:30-80
            up_t, dn_t = (np.asarray(t, f32) for t in dev.pw)
            n_sec = len(up_t) - 1
            rng_w = (dev.max_bound - dev.min_bound).astype(f32)
            if n_sec <= 0:
                f_up = np.full_like(w, up_t[0])
                f_dn = np.full_like(w, dn_t[0])
            else:
                with np.errstate(divide="ignore", invalid="ignore"):
                    ws = np.maximum((((w - dev.min_bound) / rng_w).astype(f32) * f32(n_sec)).astype(f32), f32(0))
                ws = np.where(rng_w > 0, ws, f32(0)).astype(f32)
                idx = np.minimum(np.floor(ws).astype(np.int64), n_sec - 1)
                t = np.minimum((ws - idx.astype(f32)).astype(f32), f32(1))
                t1 = (f32(1) - t).astype(f32)
                f_up = ((t1 * up_t[idx]).astype(f32) + (t * up_t[idx + 1]).astype(f32)).astype(f32)
                f_dn = ((t1 * dn_t[idx]).astype(f32) + (t * dn_t[idx + 1]).astype(f32)).astype(f32)
                f_up = np.where(rng_w > 0, f_up, up_t[0]).astype(f32)
                f_dn = np.where(rng_w > 0, f_dn, dn_t[0]).astype(f32)
            dn = ((dev.dwmin_down * f_dn).astype(f32) * (f32(1.0) + xi)).astype(f32)
            up_ = ((dev.dwmin_up * f_up).astype(f32) * (f32(1.0) + xi)).astype(f32)
            wn = np.where(down, w - dn, w + up_).astype(f32)
            wn = np.minimum(np.maximum(wn, dev.min_bound), dev.max_bound)
        else:
            raise NotImplementedError("device kind")
        w[act] = wn[act]
    return w


def update(
    w: np.ndarray, x: np.ndarray, d: np.ndarray, lr: float, dw_min: float, up: Up,
    dev: DeviceArrays, rng: Optional[np.random.Generator] = None,
) -> np.ndarray:
    """RPUPulsed::updateMatrix -> updateVectorWithDevice per sample, in batch order
    (rpu_pulsed.cpp:559-585; rpu_weight_updater.cpp:198-294).  ``w`` [d, x] is modified in
    place.  Returns the summed signed coincidence counts (diagnostics)."""
    total = np.zeros(w.shape, np.int64)
    if lr == 0:
        return total
    for s in range(x.shape[0]):
        if up.pulse_type == PULSE_DETERMINISTIC_IMPLICIT:
            n = coincidences_det_implicit(x[s], d[s], lr, dw_min, up)
        elif up.pulse_type == PULSE_MEAN_COUNT:
            n = coincidences_mean_count(x[s], d[s], lr, dw_min, up)
        elif up.pulse_type == PULSE_STOCHASTIC_COMPRESSED:
            assert rng is not None
            n = coincidences_stochastic_compressed(x[s], d[s], lr, dw_min, up, rng)
        else:
            raise NotImplementedError("pulse type")
        apply_pulses(w, n, dev, rng)
        total += n
    return total


class TransferOracle:
    """TransferRPUDevice with two devices and gamma = 0 (fully hidden fast tile):
    rpu_transfer_device.cpp:366-383 (fast LR), :396-516 (transfer), :522-557 (update hooks)."""

    def __init__(self, w_visible, dev_fast: DeviceArrays, dev_slow: DeviceArrays, tp, up: Up,
                 dw_min_fast: float, dw_min_slow: float, x_size: int, d_size: int):
        self.c = w_visible  # slow device == visible weights
        self.a = np.zeros_like(w_visible)
        self.dev_fast, self.dev_slow = dev_fast, dev_slow
        self.tp, self.up = tp, up
        self.t_io = IO.from_c(tp.transfer_io)
        self.t_io.noise_management = NM_NONE
        self.t_io.bound_management = BM_NONE
        self.t_io.finalize()
        self.t_up = Up.from_c(tp.transfer_up)
        self.dw_min_fast, self.dw_min_slow = dw_min_fast, dw_min_slow
        self.x_size, self.d_size = x_size, d_size
        self.update_idx = 0
        self.slice_idx = 0
        self.h = np.zeros_like(w_visible)  # digital buffer of the buffered variant (Tiki-Taka v2)

    def update(self, x, d, lr, rng=None):
        m = x.shape[0]
        tp = self.tp
        pc_lr = (f32(tp.fast_lr) * f32(lr) if tp.scale_fast_lr else f32(tp.fast_lr)) if tp.fast_lr > 0 else f32(lr)
        if tp.units_in_mbatch:
            every = max(int(math.ceil(f32(tp.transfer_every) * f32(m))), 0)
        else:
            every = max(int(round(tp.transfer_every)), 0)
        for s in range(m):
            update(self.a, x[s : s + 1], d[s : s + 1], float(pc_lr), self.dw_min_fast, self.up,
                   self.dev_fast, rng)
            self.update_idx += 1
            if every > 0 and self.update_idx % every == 0:
                self.transfer(lr, rng)

    def transfer(self, lr, rng=None):
        tp = self.tp
        t_lr = f32(tp.transfer_lr) * f32(lr) if tp.scale_transfer_lr else f32(tp.transfer_lr)
        n = min(tp.n_reads_per_transfer, self.x_size)
        for k in range(n):
            col = (self.slice_idx + k) % self.x_size
            e = np.zeros((1, self.x_size), f32)
            e[0, col] = 1
            if getattr(tp, "buffered", 0):
                # BufferedTransferRPUDevice::readAndUpdate (rpu_buffered_transfer_device.cpp:142-212)
                r = forward(self.a, e, self.t_io, rng, alpha=1.0)[0]
                bg = f32(tp.thres_scale) * f32(self.dw_min_slow)
                omega = (self.h[:, col] + r * abs(t_lr)).astype(f32)
                max_steps = f32(self.t_up.desired_bl)
                n_steps = np.clip(np.trunc((omega / bg).astype(f32)), -max_steps, max_steps).astype(f32)
                mom = f32(tp.momentum)
                if tp.forget_buffer:
                    keep = (omega * mom).astype(f32)
                else:
                    sub = f32(1.0) - min(max(mom, f32(0)), f32(1))
                    keep = (omega - (sub * n_steps).astype(f32) * bg).astype(f32)
                self.h[:, col] = np.where(n_steps != 0, keep, omega)
                if (n_steps != 0).any():
                    update(self.c, e, (-n_steps)[None, :], float(f32(tp.step) * f32(self.dw_min_slow)),
                           self.dw_min_slow, self.t_up, self.dev_slow, rng)
                continue
            r = forward(self.a, e, self.t_io, rng, alpha=-1.0)
            update(self.c, e, r, float(t_lr), self.dw_min_slow, self.t_up, self.dev_slow, rng)
        self.slice_idx = (self.slice_idx + n) % self.x_size


# ---------------------------------------------------------------------------------------------
# Indexed (im2col-free) convolution interface
# ---------------------------------------------------------------------------------------------
def conv_indices(in_shape, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1),
                 analog_bias: bool = False) -> np.ndarray:
    """Index array of a 2-D convolution, as ``AnalogConv2d._calculate_indexes`` builds it
    (src/aihwkit/nn/modules/conv.py:534-571): the unfold of ``arange(2, C*H*W + 2)`` with zero
    padding, flattened ``[C*kh*kw][H_out*W_out]``; 0 marks padding, 1 (appended row) the constant
    input of an analog bias.  ``in_shape`` = (C, H, W)."""
    c, h, w = in_shape
    kh, kw = kernel
    ho = (h + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    wo = (w + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    idx = np.zeros((c * kh * kw, ho * wo), np.int32)
    for ci in range(c):
        for ki in range(kh):
            for kj in range(kw):
                r = (ci * kh + ki) * kw + kj
                for oy in range(ho):
                    y = oy * stride[0] - padding[0] + ki * dilation[0]
                    if y < 0 or y >= h:
                        continue
                    xs = np.arange(wo) * stride[1] - padding[1] + kj * dilation[1]
                    ok = (xs >= 0) & (xs < w)
                    row = np.where(ok, 2 + ci * h * w + y * w + xs, 0)
                    idx[r, oy * wo:(oy + 1) * wo] = row
    flat = idx.reshape(-1)
    if analog_bias:
        flat = np.concatenate([flat, np.ones(ho * wo, np.int32)])
    return flat


def indexed_input(x: np.ndarray, indices: np.ndarray, size: int, m_batch: int, dim3: int,
                  trans: bool) -> np.ndarray:
    """``RPUSimple::copyIndexedInput`` (src/rpucuda/rpu.cpp:846-941, no batch slice), returned as
    the sample-major matrix ``[dim3 * m_batch][size]``: sample ``n * m_batch + l`` is position
    ``l`` of image ``n``.  The index array is ``[size][m_batch]`` if ``trans`` else
    ``[m_batch][size]``; entries 0 and 1 give the constants 0.0 and 1.0, ``j >= 2`` reads element
    ``j - 2`` of the image."""
    x = np.asarray(x, np.float32).reshape(dim3, -1)
    idx = np.asarray(indices, np.int64).reshape((size, m_batch) if trans else (m_batch, size))
    if trans:
        idx = idx.T  # [m_batch][size]
    src = np.concatenate([np.zeros((dim3, 1), np.float32), np.ones((dim3, 1), np.float32), x], 1)
    return src[:, idx].reshape(dim3 * m_batch, size)


def indexed_output(x_cols: np.ndarray, indices: np.ndarray, size: int, m_batch: int, dim3: int,
                   trans: bool, total_output_size: int) -> np.ndarray:
    """``RPUSimple::copyIndexedOutput`` (src/rpucuda/rpu.cpp:943-1013): scatter-add of the
    sample-major matrix ``[dim3 * m_batch][size]`` into zeroed images ``[dim3][total / dim3]``."""
    idx = np.asarray(indices, np.int64).reshape((size, m_batch) if trans else (m_batch, size))
    if trans:
        idx = idx.T
    out = np.zeros((dim3, total_output_size // dim3), np.float32)
    cols = np.asarray(x_cols, np.float32).reshape(dim3, m_batch, size)
    sel = idx > 1
    for n in range(dim3):
        np.add.at(out[n], idx[sel] - 2, cols[n][sel])
    return out


def to_sample_major(t: np.ndarray, size: int, m_batch: int, dim3: int, trans: bool) -> np.ndarray:
    """Output-side tensor ``[dim3][size][m_batch]`` (``trans``) or ``[dim3][m_batch][size]`` as the
    sample-major matrix ``[dim3 * m_batch][size]`` (the ``permute132`` of rpu.cpp:1136-1139)."""
    t = np.asarray(t, np.float32)
    if trans:
        return t.reshape(dim3, size, m_batch).transpose(0, 2, 1).reshape(dim3 * m_batch, size)
    return t.reshape(dim3 * m_batch, size)


def from_sample_major(a: np.ndarray, size: int, m_batch: int, dim3: int, trans: bool) -> np.ndarray:
    a = np.asarray(a, np.float32)
    if trans:
        return np.ascontiguousarray(a.reshape(dim3, m_batch, size).transpose(0, 2, 1))
    return a.reshape(dim3, m_batch, size)


# ---------------------------------------------------------------------------------------------
# Weight operations between updates
# ---------------------------------------------------------------------------------------------
def _hidden(names, hp, name):
    return np.asarray(hp[list(names).index(name)], np.float32)


def decay_weights(w: np.ndarray, names, hp: np.ndarray, alpha: float = 1.0,
                  bias_no_decay: bool = False) -> np.ndarray:
    """``PulsedRPUDevice::decayWeights(weights, alpha, bias_no_decay)``
    (src/rpucuda/rpu_pulsed_device.cpp:391-420): ``w = (w - b) * (1 + alpha * (wd - 1)) + b``,
    clipped to the element's bounds; weights are ``[d][x]``."""
    f = np.float32
    wd, b = _hidden(names, hp, "decay_scales"), _hidden(names, hp, "reset_bias")
    s = f(1.0) + f(alpha) * (wd - f(1.0))
    if bias_no_decay:
        s = s.copy()
        s[:, -1] = f(1.0)
    out = (np.asarray(w, f) - b) * s + b
    out = np.minimum(out, _hidden(names, hp, "max_bound"))
    return np.maximum(out, _hidden(names, hp, "min_bound")).astype(f)


def decay_weights_simple(w: np.ndarray, lifetime: float, alpha: float = 1.0) -> np.ndarray:
    """``RPUSimple::decayWeights`` (src/rpucuda/rpu.cpp:1556-1575)."""
    f = np.float32
    rate = f(1.0) / f(lifetime) if lifetime > 1.0 else f(0.0)
    scale = f(1.0) - f(alpha) * rate
    return (np.asarray(w, f) * scale).astype(f) if 0.0 < scale < 1.0 else np.asarray(w, f).copy()


def clip_to_device(w: np.ndarray, names, hp: np.ndarray, clip: float = -1.0) -> np.ndarray:
    """``PulsedRPUDevice::clipWeights`` (src/rpucuda/rpu_pulsed_device.cpp:451-470)."""
    hi, lo = _hidden(names, hp, "max_bound"), _hidden(names, hp, "min_bound")
    if clip >= 0:
        hi, lo = np.minimum(hi, np.float32(clip)), np.maximum(lo, np.float32(-clip))
    return np.maximum(np.minimum(np.asarray(w, np.float32), hi), lo)


def clip_value(w: np.ndarray, clip_type: int, fixed_value: float = -1.0, sigma: float = 2.5) -> float:
    """Clip value of ``WeightClipper::apply`` (src/rpucuda/weight_clipper.cpp:38-112) for the
    types 1 FixedValue, 2 LayerGaussian, 3 AverageChannelMax; <= 0 means no clipping."""
    w = np.asarray(w, np.float32)
    if clip_type == 1:
        return float(fixed_value)
    if clip_type == 2:
        c = float(np.std(w.astype(np.float64), ddof=1)) * sigma
    elif clip_type == 3:
        c = float(np.abs(w).max(axis=1).astype(np.float64).mean())
    else:
        return -1.0
    return min(c, fixed_value) if fixed_value > 0 else c
