"""Mirror of ``aihwkit.simulator.rpu_base.devices`` for the analog-tile hot path.

Class and attribute names are the ones bound in
``src/aihwkit/simulator/rpu_base_src/rpu_base_devices.cpp:436-960`` and the enums of
``rpu_base_utils.cpp:55-91``; default values are the C++ member initialisers of the
reference's meta-parameter structs (``src/rpucuda/rpu_pulsed_meta_parameter.h:180-279``,
``rpu_pulsed_device.h:60-110``, ``rpu_linearstep_device.h``, ``rpu_softbounds_reference_device.h``,
``rpu_transfer_device.h:52-75``).  ``AnalogTileParameter.create_array`` is the factory the
reference exposes at ``rpu_base_devices.cpp:453-467``.

Also provided: ExpStep, PowStep, PiecewiseStep and the buffered, chopped and dynamic transfer
compounds (Tiki-Taka v2 to v4).  Other devices (MixedPrec, OneSided, Vector, ...) are not; there
is no class for them here.
"""

from __future__ import annotations

import enum
from typing import List

from .. import _cabi


class NoiseManagementType(enum.IntEnum):
    """rpu_pulsed_meta_parameter.h:146-156 (``None`` spelt ``None_``)."""

    None_ = 0
    AbsMax = 1
    AbsMaxNPSum = 2
    Max = 3
    Constant = 4
    AverageAbsMax = 5


class BoundManagementType(enum.IntEnum):
    None_ = 0
    Iterative = 1
    IterativeWorstCase = 2


class WeightNoiseType(enum.IntEnum):
    None_ = 0
    AdditiveConstant = 1
    PCMRead = 2


class PulseType(enum.IntEnum):
    None_ = 0
    StochasticCompressed = 1
    Stochastic = 2
    NoneWithDevice = 3
    MeanCount = 4
    DeterministicImplicit = 5


class AnalogMVType(enum.IntEnum):
    Ideal = 0
    OnePass = 1
    PosNegSeparate = 2
    PosNegSeparateDigitalSum = 3


for _e in (NoiseManagementType, BoundManagementType, WeightNoiseType, PulseType):
    # the binding spells the first member "None"; keep that name reachable via getattr
    _e._member_map_["None"] = _e(0)  # type: ignore[attr-defined]
    type.__setattr__(_e, "None", _e(0))


DEVICE_IDEAL = 0
DEVICE_CONSTANT_STEP = 1
DEVICE_LINEAR_STEP = 2
DEVICE_SOFT_BOUNDS = 3
DEVICE_SOFT_BOUNDS_REFERENCE = 4
DEVICE_TRANSFER = 5
DEVICE_EXP_STEP = 6
DEVICE_POW_STEP = 7
DEVICE_PIECEWISE_STEP = 8


class AnalogTileInputOutputParameter:
    """IOMetaParameter (rpu_base_devices.cpp:485-519)."""

    _unsupported = {
        "w_read_asymmetry_dtod": 0.0,
    }

    def __init__(self) -> None:
        self.is_perfect = False
        self.mv_type = AnalogMVType.OnePass
        self.noise_management = NoiseManagementType.AbsMax
        self.bound_management = BoundManagementType.None_
        self.w_noise_type = WeightNoiseType.None_
        self.bm_test_negative_bound = True
        self.max_bm_factor = 1000
        self.max_bm_res = 0.25
        self.inp_sto_round = False
        self.out_sto_round = False
        self.inp_bound = 1.0
        self.inp_res = 1.0 / (2.0**7 - 2.0)
        self.inp_noise = 0.0
        self.out_bound = 12.0
        self.out_res = 1.0 / (2.0**9 - 2.0)
        self.out_noise = 0.06
        self.out_noise_std = 0.0
        self.out_scale = 1.0
        self.w_noise = 0.0
        self.nm_thres = 0.0
        self.nm_assumed_wmax = 0.6
        self.nm_decay = 1e-3
        self.inp_asymmetry = 0.0
        self.out_asymmetry = 0.0
        self.ir_drop = 0.0
        self.ir_drop_g_ratio = 5.7143e5
        self.out_nonlinearity = 0.0
        self.out_nonlinearity_std = 0.0
        self.slope_calibration = 0.5
        self.r_series = 0.0
        self.v_offset_std = 0.0
        self.v_offset_w_min = 0.0
        self.w_read_asymmetry_dtod = 0.0

    def _to_c(self) -> _cabi.IOParams:
        for name, off in self._unsupported.items():
            if getattr(self, name) != off:
                raise RuntimeError(
                    f"IO parameter '{name}' is not implemented by the B200 analog tile"
                )
        if (self.v_offset_std > 0 or self.r_series > 0) and self.v_offset_w_min != 0.0:
            # the reference term of the offsets, - 2 vo_i g_ref sum_j x_j
            # (rpu_forward_backward_pass.cpp:471-503); without offsets the value is not read
            raise RuntimeError(
                "IO parameter 'v_offset_w_min' (with voltage offsets on) is not implemented by the "
                "B200 analog tile"
            )
        mv = int(self.mv_type)
        if mv not in (0, 1, 2, 3):
            raise RuntimeError("AnalogMVType not implemented.")
        nm = int(self.noise_management)
        if nm not in (0, 1, 2, 3, 4, 5, 6):
            raise RuntimeError("Noise Management type not implemented!")
        c = _cabi.IOParams()
        c.is_perfect = int(bool(self.is_perfect) or mv == int(AnalogMVType.Ideal))
        c.mv_type = max(mv - 1, 0)  # ab200_mv_type: one pass, pos / neg separate, digital sum
        c.noise_management = nm
        c.bound_management = int(self.bound_management)
        c.w_noise_type = int(self.w_noise_type)
        c.bm_test_negative_bound = int(bool(self.bm_test_negative_bound))
        c.max_bm_factor = int(self.max_bm_factor)
        c.inp_sto_round = int(bool(self.inp_sto_round))
        c.out_sto_round = int(bool(self.out_sto_round))
        for name in (
            "inp_bound", "inp_res", "inp_noise", "out_bound", "out_res", "out_noise", "out_scale",
            "w_noise", "nm_thres", "max_bm_res", "inp_asymmetry", "out_asymmetry", "nm_assumed_wmax",
            "out_noise_std", "nm_decay", "ir_drop", "ir_drop_g_ratio", "v_offset_std", "r_series",
            "out_nonlinearity", "out_nonlinearity_std", "slope_calibration",
        ):
            setattr(c, name, float(getattr(self, name)))
        return c


class AnalogTileUpdateParameter:
    """PulsedUpdateMetaParameter (rpu_base_devices.cpp:469-483)."""

    def __init__(self) -> None:
        self.fixed_bl = True
        self.desired_bl = 31
        self.pulse_type = PulseType.StochasticCompressed
        self.res = 0.0
        self.x_res_implicit = 0.0
        self.d_res_implicit = 0.0
        self.sto_round = False
        self.um_reg_scale = 1.0
        self.um_grad_scale = 1.0
        self.d_sparsity = False
        self.update_management = True
        self.update_bl_management = True

    def _to_c(self) -> _cabi.UpdateParams:
        pt = int(self.pulse_type)
        c = _cabi.UpdateParams()
        c.pulse_type = pt
        c.desired_bl = int(self.desired_bl)
        c.fixed_bl = int(bool(self.fixed_bl))
        c.update_management = int(bool(self.update_management))
        c.update_bl_management = int(bool(self.update_bl_management))
        c.sto_round = int(bool(self.sto_round))
        c.um_grad_scale = float(self.um_grad_scale)
        c.res = float(self.res)
        c.x_res_implicit = float(self.x_res_implicit)
        c.d_res_implicit = float(self.d_res_implicit)
        return c


class DriftParameter:
    """DriftParameter (rpu_base_devices.cpp:521-533): power-law drift of the weights over time,
    ``w(t) = w0 (t / t_0)^(-nu)`` for weights that were not written since (weight_drifter.cpp:111-157)."""

    def __init__(self) -> None:
        self.nu = 0.0
        self.nu_dtod = 0.0
        self.nu_std = 0.0
        self.wg_ratio = 1.0
        self.g_offset = 0.0
        self.w_offset = 0.0
        self.nu_k = 0.0
        self.log_g0 = 0.0
        self.t_0 = 1.0
        self.reset_tol = 1e-7
        self.w_noise_std = 0.0

    def _active(self) -> bool:
        return self.nu != 0.0 or self.nu_dtod != 0.0 or self.nu_std != 0.0 or self.nu_k != 0.0

    def _to_c(self, simple: bool = False) -> "_cabi.DriftParams":
        c = _cabi.DriftParams()
        c.nu = float(self.nu)
        c.nu_dtod = 0.0 if simple else float(self.nu_dtod)  # setSimpleDrift (weight_drifter.h:51-54)
        c.nu_std = float(self.nu_std)
        c.wg_ratio = float(self.wg_ratio)
        c.g_offset = float(self.g_offset)
        c.w_offset = float(self.w_offset)
        c.nu_k = float(self.nu_k)
        c.log_g0 = float(self.log_g0)
        c.t0 = float(self.t_0)
        c.reset_tol = float(self.reset_tol)
        c.w_read_std = float(self.w_noise_std)
        return c


class FloatingPointTileParameter:
    """SimpleMetaParameter (rpu_base_devices.cpp:436-451): the floating-point tile's own
    parameters and its factory."""

    def __init__(self) -> None:
        self.diffusion = 0.0
        self.lifetime = 0.0
        self.drift = DriftParameter()

    def create_array(self, x_size: int, d_size: int):
        """``createRPUArray`` of the floating-point tile (src/rpucuda/rpu.cpp)."""
        from .tiles import FloatingPointTile

        return FloatingPointTile(x_size, d_size, lifetime=float(self.lifetime),
                                 diffusion=float(self.diffusion), drift=self.drift)

    def __str__(self) -> str:
        return f"FloatingPointTileParameter(diffusion={self.diffusion}, lifetime={self.lifetime})"


class AbstractResistiveDeviceParameter:
    """AbstractRPUDeviceMetaParameter (rpu_base_devices.cpp:536-539), derived from the
    floating-point tile's parameters as in the reference."""

    _kind = -1

    def __init__(self) -> None:
        self.construction_seed = 0
        self.diffusion = 0.0
        self.lifetime = 0.0
        self.drift = DriftParameter()

    def calc_weight_granularity(self) -> float:
        raise RuntimeError("Needs implementation.")


def __getattr__(name):
    # WeightClipType / WeightClipParameter belong to the tiles module in the reference's binding
    # (rpu_base_utils.cpp:18-53); earlier callers of this package found them here
    if name in ("WeightClipType", "WeightClipParameter"):
        from . import tiles

        return getattr(tiles, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


class IdealResistiveDeviceParameter(AbstractResistiveDeviceParameter):
    """SimpleRPUDeviceMetaParameter: floating-point update (rpu_base_devices.cpp:545-552)."""

    _kind = DEVICE_IDEAL

    def __init__(self) -> None:
        super().__init__()
        self.reset_std = 0.0


class PulsedResistiveDeviceParameter(AbstractResistiveDeviceParameter):
    """PulsedRPUDeviceMetaParameter (rpu_base_devices.cpp:554-581)."""

    def __init__(self) -> None:
        super().__init__()
        self.dw_min = 0.001
        self.dw_min_dtod = 0.3
        self.dw_min_std = 0.3
        self.dw_min_dtod_log_normal = False
        self.w_min = -0.6
        self.w_min_dtod = 0.3
        self.w_max = 0.6
        self.w_max_dtod = 0.3
        self.up_down = 0.0
        self.up_down_dtod = 0.01
        self.lifetime_dtod = 0.0
        self.diffusion_dtod = 0.0
        self.enforce_consistency = False
        self.perfect_bias = False
        self.corrupt_devices_prob = 0.0
        self.corrupt_devices_range = 3.4028234663852886e38
        self.reset = 0.0
        self.reset_std = 0.0
        self.reset_dtod = 0.0
        self.count_pulses = False

    def calc_weight_granularity(self) -> float:
        return float(self.dw_min)

    def _fill_base(self, c: _cabi.DeviceParams) -> None:
        if self.corrupt_devices_prob != 0.0:
            raise RuntimeError(
                "device parameter 'corrupt_devices_prob' is not implemented by the B200 analog tile"
            )
        c.count_pulses = int(bool(self.count_pulses))
        c.kind = self._kind
        c.construction_seed = int(self.construction_seed) & 0xFFFFFFFF
        c.enforce_consistency = int(bool(self.enforce_consistency))
        c.dw_min_dtod_log_normal = int(bool(self.dw_min_dtod_log_normal))
        c.perfect_bias = int(bool(self.perfect_bias))
        for name in (
            "dw_min", "dw_min_dtod", "dw_min_std", "w_min", "w_min_dtod", "w_max", "w_max_dtod",
            "up_down", "up_down_dtod", "lifetime", "lifetime_dtod", "diffusion", "diffusion_dtod",
            "reset", "reset_dtod", "reset_std",
        ):
            setattr(c, name, float(getattr(self, name)))
        c.drift = self.drift._to_c()

    def _to_c(self) -> _cabi.DeviceParams:
        c = _cabi.DeviceParams()
        self._fill_base(c)
        return c


class ConstantStepResistiveDeviceParameter(PulsedResistiveDeviceParameter):
    """rpu_base_devices.cpp:583-600."""

    _kind = DEVICE_CONSTANT_STEP


class PiecewiseStepResistiveDeviceParameter(PulsedResistiveDeviceParameter):
    """rpu_base_devices.cpp:857-870 (PiecewiseStepRPUDeviceMetaParameter,
    rpu_piecewisestep_device.h:17-50): the step is ``dw_min`` times a factor interpolated linearly
    between equally spaced nodes over the weight range of the element, one table per direction."""

    _kind = DEVICE_PIECEWISE_STEP
    MAX_NODES = 32

    def __init__(self) -> None:
        super().__init__()
        self.piecewise_up = [1.0]
        self.piecewise_down = [1.0]
        self.write_noise_std = 0.0
        self.apply_write_noise_on_set = True

    def calc_weight_granularity(self) -> float:
        """PiecewiseStepRPUDeviceMetaParameter::calcWeightGranularity
        (rpu_piecewisestep_device.h:34-39)."""
        up = list(self.piecewise_up)
        if up and len(self.piecewise_down) > 0:
            return float(self.dw_min) * float(up[len(up) // 2])
        return float(self.dw_min)

    def _to_c(self) -> _cabi.DeviceParams:
        if self.write_noise_std != 0.0:
            raise RuntimeError("write noise is not implemented by the B200 analog tile")
        up, down = list(self.piecewise_up), list(self.piecewise_down)
        if not up or not down:
            raise RuntimeError("piecewise_up_vec and piecewise_down_vec needs to have some contents.")
        if len(up) != len(down):
            raise RuntimeError("piecewise_up_vec and piecewise_down_vec needs to have some size.")
        if len(up) > self.MAX_NODES:
            raise RuntimeError(
                f"PiecewiseStep: at most {self.MAX_NODES} nodes per direction are implemented"
            )
        c = _cabi.DeviceParams()
        self._fill_base(c)
        c.pw_n = len(up)
        for i, (u, d) in enumerate(zip(up, down)):
            c.pw_up[i] = float(u)
            c.pw_down[i] = float(d)
        return c


class PowStepResistiveDeviceParameter(PulsedResistiveDeviceParameter):
    """rpu_base_devices.cpp:806-813 (PowStepRPUDeviceMetaParameter, rpu_powstep_device.h:22-25):
    the step shrinks with a power of the distance to the bound."""

    _kind = DEVICE_POW_STEP

    def __init__(self) -> None:
        super().__init__()
        self.pow_gamma = 1.0
        self.pow_gamma_dtod = 0.1
        self.pow_up_down = 0.0
        self.pow_up_down_dtod = 0.0
        self.write_noise_std = 0.0
        self.apply_write_noise_on_set = True

    def calc_weight_granularity(self) -> float:
        """PowStepRPUDeviceMetaParameter::calcWeightGranularity (rpu_powstep_device.h:33)."""
        return float(self.dw_min) * 0.5 ** float(self.pow_gamma)

    def _to_c(self) -> _cabi.DeviceParams:
        if self.write_noise_std != 0.0:
            raise RuntimeError("write noise is not implemented by the B200 analog tile")
        c = _cabi.DeviceParams()
        self._fill_base(c)
        c.ps_gamma, c.ps_gamma_dtod = float(self.pow_gamma), float(self.pow_gamma_dtod)
        c.ps_gamma_up_down, c.ps_gamma_up_down_dtod = float(self.pow_up_down), float(self.pow_up_down_dtod)
        return c


class ExpStepResistiveDeviceParameter(PulsedResistiveDeviceParameter):
    """rpu_base_devices.cpp:658-683 (ExpStepRPUDeviceMetaParameter, rpu_expstep_device.h:22-29)."""

    _kind = DEVICE_EXP_STEP

    def __init__(self) -> None:
        super().__init__()
        self.A_up = 0.00081
        self.A_down = 0.36833
        self.gamma_up = 12.44625
        self.gamma_down = 12.78785
        self.a = 0.244
        self.b = 0.2425
        self.write_noise_std = 0.0
        self.apply_write_noise_on_set = True
        self.dw_min_std_add = 0.0
        self.dw_min_std_slope = 0.0

    def calc_weight_granularity(self) -> float:
        """ExpStepRPUDeviceMetaParameter::calcWeightGranularity (rpu_expstep_device.h:43-55)."""
        import math

        down_bias = -self.up_down if self.up_down > 0 else 0.0
        dw_down = (down_bias + 1.0) * self.dw_min * max(
            1.0 - self.A_down * math.exp(self.gamma_down * (-self.b)), 0.0)
        return dw_down if dw_down > 0 else float(self.dw_min)

    def _to_c(self) -> _cabi.DeviceParams:
        if self.write_noise_std != 0.0:
            raise RuntimeError("write noise is not implemented by the B200 analog tile")
        c = _cabi.DeviceParams()
        self._fill_base(c)
        c.es_A_up, c.es_A_down = float(self.A_up), float(self.A_down)
        c.es_gamma_up, c.es_gamma_down = float(self.gamma_up), float(self.gamma_down)
        c.es_a, c.es_b = float(self.a), float(self.b)
        c.dw_min_std_add, c.dw_min_std_slope = float(self.dw_min_std_add), float(self.dw_min_std_slope)
        return c


class LinearStepResistiveDeviceParameter(PulsedResistiveDeviceParameter):
    """rpu_base_devices.cpp:602-631 (``gamma_*`` are the ``ls_decrease_*`` fields)."""

    _kind = DEVICE_LINEAR_STEP

    def __init__(self) -> None:
        super().__init__()
        self.gamma_up = 0.0
        self.gamma_down = 0.0
        self.gamma_up_dtod = 0.05
        self.gamma_down_dtod = 0.05
        self.allow_increasing = False
        self.mean_bound_reference = True
        self.mult_noise = True
        self.write_noise_std = 0.0
        self.apply_write_noise_on_set = True
        self.reverse_up = False
        self.reverse_down = False
        self.reverse_offset = 0.01

    def _to_c(self) -> _cabi.DeviceParams:
        if self.write_noise_std != 0.0 or self.reverse_up or self.reverse_down:
            raise RuntimeError("write noise / reversed slopes are not implemented")
        c = _cabi.DeviceParams()
        self._fill_base(c)
        c.ls_mult_noise = int(bool(self.mult_noise))
        c.ls_allow_increasing_slope = int(bool(self.allow_increasing))
        c.ls_mean_bound_reference = int(bool(self.mean_bound_reference))
        c.ls_decrease_up = float(self.gamma_up)
        c.ls_decrease_down = float(self.gamma_down)
        c.ls_decrease_up_dtod = float(self.gamma_up_dtod)
        c.ls_decrease_down_dtod = float(self.gamma_down_dtod)
        return c


class SoftBoundsResistiveDeviceParameter(LinearStepResistiveDeviceParameter):
    """SoftBounds = LinearStep with slopes tied to the bounds (rpu_linearstep_device.h:70-83)."""

    _kind = DEVICE_SOFT_BOUNDS

    def __init__(self) -> None:
        super().__init__()
        self.gamma_up = 1.0
        self.gamma_down = 1.0
        self.gamma_up_dtod = 0.0
        self.gamma_down_dtod = 0.0
        self.allow_increasing = False
        self.mean_bound_reference = False


class SoftBoundsReferenceResistiveDeviceParameter(PulsedResistiveDeviceParameter):
    """rpu_base_devices.cpp:926-950."""

    _kind = DEVICE_SOFT_BOUNDS_REFERENCE

    def __init__(self) -> None:
        super().__init__()
        self.slope_up_dtod = 0.0
        self.slope_down_dtod = 0.0
        self.reference_mean = 0.0
        self.reference_std = 0.0
        self.subtract_symmetry_point = False
        self.mult_noise = False
        self.write_noise_std = 0.0
        self.apply_write_noise_on_set = True

    def _to_c(self) -> _cabi.DeviceParams:
        if self.write_noise_std != 0.0:
            raise RuntimeError("write noise is not implemented")
        c = _cabi.DeviceParams()
        self._fill_base(c)
        c.mult_noise = int(bool(self.mult_noise))
        c.subtract_symmetry_point = int(bool(self.subtract_symmetry_point))
        c.slope_up_dtod = float(self.slope_up_dtod)
        c.slope_down_dtod = float(self.slope_down_dtod)
        c.reference_mean = float(self.reference_mean)
        c.reference_std = float(self.reference_std)
        return c


class VectorResistiveDeviceParameter(AbstractResistiveDeviceParameter):
    """VectorRPUDeviceMetaParameter (rpu_base_devices.cpp:686-714); container only."""

    def __init__(self) -> None:
        super().__init__()
        self.gamma_vec: List[float] = []
        self._vec_par: List[PulsedResistiveDeviceParameter] = []

    def append_parameter(self, parameter: PulsedResistiveDeviceParameter) -> bool:
        if not isinstance(parameter, PulsedResistiveDeviceParameter):
            raise RuntimeError("Only pulsed devices can be appended")
        self._vec_par.append(parameter)
        return True

    def calc_weight_granularity(self) -> float:
        return self._vec_par[0].calc_weight_granularity() if self._vec_par else 0.0


class TransferResistiveDeviceParameter(VectorResistiveDeviceParameter):
    """TransferRPUDeviceMetaParameter (rpu_base_devices.cpp:742-776)."""

    _kind = DEVICE_TRANSFER

    def __init__(self) -> None:
        super().__init__()
        self.gamma = 0.0
        self.transfer_every = 1.0
        self.no_self_transfer = True
        self.transfer_every_vec: List[float] = []
        self.units_in_mbatch = False
        self.n_reads_per_transfer = 1
        self.with_reset_prob = 0.0
        self.random_selection = False
        self.transfer_columns = True
        self.transfer_lr = 1.0
        self.fast_lr = 0.0
        self.transfer_lr_vec: List[float] = []
        self.scale_transfer_lr = True
        self.scale_fast_lr = True
        self.transfer_forward = AnalogTileInputOutputParameter()
        self.transfer_update = AnalogTileUpdateParameter()

    def _to_c(self) -> _cabi.TransferParams:
        if len(self._vec_par) != 2:
            raise RuntimeError("The B200 analog tile implements Transfer with exactly 2 devices")
        if self.gamma != 0.0 or self.gamma_vec:
            raise RuntimeError("Only gamma = 0 (fully hidden fast tile) is implemented")
        if self.with_reset_prob != 0.0 or self.random_selection or not self.transfer_columns:
            raise RuntimeError("reset / random selection / row transfer are not implemented")
        if self.transfer_every_vec or self.transfer_lr_vec:
            raise RuntimeError("per-device transfer vectors are not implemented")
        c = _cabi.TransferParams()
        c.gamma = float(self.gamma)
        c.transfer_every = float(self.transfer_every)
        c.units_in_mbatch = int(bool(self.units_in_mbatch))
        c.n_reads_per_transfer = int(self.n_reads_per_transfer)
        c.fast_lr = float(self.fast_lr)
        c.transfer_lr = float(self.transfer_lr)
        c.scale_transfer_lr = int(bool(self.scale_transfer_lr))
        c.scale_fast_lr = int(bool(self.scale_fast_lr))
        c.transfer_columns = 1
        c.transfer_io = self.transfer_forward._to_c()
        c.transfer_up = self.transfer_update._to_c()
        c.buffered = 0
        c.thres_scale, c.step, c.momentum, c.forget_buffer = 1.0, 1.0, 0.0, 1
        return c


class BufferedTransferResistiveDeviceParameter(TransferResistiveDeviceParameter):
    """BufferedTransferRPUDeviceMetaParameter, Tiki-Taka v2 (rpu_base_devices.cpp
    ``BufferedTransferResistiveDeviceParameter``; defaults of ``initDefaults``,
    src/rpucuda/rpu_buffered_transfer_device.h:54-68)."""

    def __init__(self) -> None:
        super().__init__()
        self.thres_scale = 1.0
        self.step = 1.0
        self.momentum = 0.0
        self.forget_buffer = True
        self.transfer_lr = 1.0
        self.scale_transfer_lr = True
        self.transfer_update.update_bl_management = False
        self.transfer_update.update_management = False
        self.transfer_update.desired_bl = 1
        self.transfer_update.fixed_bl = True

    def _to_c(self) -> _cabi.TransferParams:
        c = super()._to_c()
        c.buffered = 1
        c.thres_scale, c.step = float(self.thres_scale), float(self.step)
        c.momentum, c.forget_buffer = float(self.momentum), int(bool(self.forget_buffer))
        return c


class ChoppedTransferResistiveDeviceParameter(BufferedTransferResistiveDeviceParameter):
    """ChoppedTransferRPUDeviceMetaParameter, Tiki-Taka with choppers (rpu_base_devices.cpp:893-910;
    src/rpucuda/rpu_chopped_transfer_device.h:22-60)."""

    def __init__(self) -> None:
        super().__init__()
        self.in_chop_prob = 1.0
        self.in_chop_random = True
        self.out_chop_prob = 0.0
        self.auto_scale = False
        self.correct_gradient_magnitudes = False
        self.auto_momentum = 0.99
        self.auto_granularity = 0.0
        self.buffer_granularity = 1.0
        self.no_buffer = False
        self.n_reads_per_transfer = 1

    def _to_c(self) -> _cabi.TransferParams:
        if self.auto_scale:
            raise RuntimeError("ChoppedTransfer: auto_scale is not implemented by the B200 analog tile")
        if float(self.transfer_every) < 0:
            raise RuntimeError("ChoppedTransfer: the automatic transfer period (transfer_every < 0) is "
                               "not implemented by the B200 analog tile")
        if int(self.n_reads_per_transfer) != 1:
            # ChoppedTransferRPUDeviceMetaParameter::checkSupported (rpu_chopped_transfer_device.cpp:66-88)
            raise RuntimeError("In / out chopper not implemented the given parameters. \nRequired: "
                               "n_devices==2, n_reads_per_transfer==1, random_selection=false).\n")
        c = super()._to_c()
        c.chopped = 1
        c.in_chop_random = int(bool(self.in_chop_random))
        c.correct_gradient_magnitudes = int(bool(self.correct_gradient_magnitudes))
        c.no_buffer = int(bool(self.no_buffer))
        c.in_chop_prob = float(self.in_chop_prob)
        c.out_chop_prob = float(self.out_chop_prob)
        c.auto_granularity = float(self.auto_granularity)
        c.buffer_granularity = float(self.buffer_granularity)
        return c


class MixedPrecResistiveDeviceParameter:
    """MixedPrecRPUDeviceMetaParameter (rpu_base_devices.cpp:778-804): a digital rank-update
    accumulator in front of one pulsed analog device, set with ``set_device_parameter``."""

    def __init__(self) -> None:
        # SimpleRPUDeviceMetaParameter part (src/rpucuda/rpu.h:140-175)
        self.construction_seed = 0
        self.transfer_every = 1
        self.n_rows_per_transfer = -1
        self.random_row = False
        self.granularity = 0.0
        self.compute_sparsity = False
        self.n_x_bins = 0
        self.n_d_bins = 0
        self.stoc_round_x = False
        self.stoc_round_d = False
        self.transfer_lr = 1.0
        self._device = None

    def set_device_parameter(self, parameter) -> bool:
        kind = getattr(parameter, "_kind", -1)
        if kind in (-1, DEVICE_IDEAL, DEVICE_TRANSFER):
            return False  # setDevicePar accepts pulsed devices only
        self._device = parameter
        return True

    @property
    def _kind(self) -> int:
        return -1 if self._device is None else self._device._kind

    def _to_c_mixed(self) -> _cabi.MixedPrecParams:
        if (int(self.n_x_bins) > 0) != (int(self.n_d_bins) > 0):
            raise RuntimeError("MixedPrec: quantising only one of x and d is not implemented by the "
                               "B200 analog tile")
        c = _cabi.MixedPrecParams()
        c.enabled = 1
        c.transfer_every = int(self.transfer_every)
        c.n_rows_per_transfer = int(self.n_rows_per_transfer)
        c.random_row = int(bool(self.random_row))
        c.granularity = float(self.granularity)
        c.n_x_bins, c.n_d_bins = int(self.n_x_bins), int(self.n_d_bins)
        c.stoc_round_x, c.stoc_round_d = int(bool(self.stoc_round_x)), int(bool(self.stoc_round_d))
        c.transfer_lr = float(self.transfer_lr)
        return c


class DynamicTransferResistiveDeviceParameter(ChoppedTransferResistiveDeviceParameter):
    """DynamicTransferRPUDeviceMetaParameter, Tiki-Taka with choppers and a running-mean reference
    (rpu_base_devices.cpp:912-924; src/rpucuda/rpu_dynamic_transfer_device.h:26-62)."""

    def __init__(self) -> None:
        super().__init__()
        self.in_chop_random = False  # initDefaults (rpu_dynamic_transfer_device.h:61)
        self.tail_weightening = 1.0
        self.buffer_cap = 10.0
        self.experimental_correct_accumulation = False

    def _to_c(self) -> _cabi.TransferParams:
        if float(self.in_chop_prob) <= 0.0:
            # DynamicTransferRPUDeviceMetaParameter::checkSupported (rpu_dynamic_transfer_device.cpp:38-49)
            raise RuntimeError("In chopper prob needs to be positive.")
        if not 0.0 < float(self.auto_momentum) < 1.0:
            raise RuntimeError("Auto-momentum needs to be smaller than 1 and larger than 0.")
        c = super()._to_c()
        c.dynamic = 1
        c.correct_accumulation = int(bool(self.experimental_correct_accumulation))
        c.tail_weightening = float(self.tail_weightening)
        c.buffer_cap = float(self.buffer_cap)
        return c


class AnalogTileParameter:
    """PulsedMetaParameter (rpu_base_devices.cpp:453-467)."""

    def __init__(self) -> None:
        self.forward_io = AnalogTileInputOutputParameter()
        self.backward_io = AnalogTileInputOutputParameter()
        self.update = AnalogTileUpdateParameter()

    def _config(self, x_size: int, d_size: int, device_par, seed: int = 0) -> _cabi.TileConfig:
        cfg = _cabi.TileConfig()
        cfg.x_size = int(x_size)
        cfg.d_size = int(d_size)
        cfg.forward_io = self.forward_io._to_c()
        cfg.backward_io = self.backward_io._to_c()
        cfg.update = self.update._to_c()
        cfg.seed = int(seed)
        kind = getattr(device_par, "_kind", -1)
        if kind < 0:
            raise RuntimeError(
                f"{type(device_par).__name__} is not implemented by the B200 analog tile"
            )
        cfg.device_kind = kind
        if kind == DEVICE_TRANSFER:
            cfg.transfer = device_par._to_c()
            cfg.device[0] = device_par._vec_par[0]._to_c()
            cfg.device[1] = device_par._vec_par[1]._to_c()
            if device_par.construction_seed:
                cfg.device[0].construction_seed = int(device_par.construction_seed)
        elif kind == DEVICE_IDEAL:
            cfg.device[0].kind = DEVICE_IDEAL
            cfg.device[0].lifetime = float(device_par.lifetime)
            cfg.device[0].diffusion = float(device_par.diffusion)
            cfg.device[0].reset_std = float(device_par.reset_std)
            cfg.device[0].construction_seed = int(device_par.construction_seed)
            # SimpleMetaParameter: one exponent for all weights (src/rpucuda/rpu.h:165)
            cfg.device[0].drift = device_par.drift._to_c(simple=True)
        elif isinstance(device_par, MixedPrecResistiveDeviceParameter):
            cfg.device[0] = device_par._device._to_c()
            cfg.mixed = device_par._to_c_mixed()
            if device_par.construction_seed:
                cfg.device[0].construction_seed = int(device_par.construction_seed)
        else:
            cfg.device[0] = device_par._to_c()
        return cfg

    def create_array(self, x_size: int, d_size: int, device_par):
        """Factory for an analog tile (``createRPUArray``, src/rpucuda/rpu_pulsed.cpp:49-56)."""
        from .tiles import AnalogTile

        tile = AnalogTile(self._config(x_size, d_size, device_par))
        tile._meta = self
        return tile
