"""ctypes view of the C ABI declared in ``include/aihwkit_b200.h``.

The shared library ``aihwkit_b200/csrc/libaihwkit_b200.so`` is built in-tree by
``aihwkit_b200.build`` (nvcc, sm_100a).  There is no CPU compute path and no
fallback: if the library is missing, :func:`lib` raises and every tile call fails.
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libaihwkit_b200.so")


class IOParams(C.Structure):
    """``ab200_io_params`` (IOMetaParameter, src/rpucuda/rpu_pulsed_meta_parameter.h:180-226)."""

    _fields_ = [
        ("is_perfect", C.c_int32),
        ("noise_management", C.c_int32),
        ("bound_management", C.c_int32),
        ("w_noise_type", C.c_int32),
        ("bm_test_negative_bound", C.c_int32),
        ("max_bm_factor", C.c_int32),
        ("inp_sto_round", C.c_int32),
        ("out_sto_round", C.c_int32),
        ("inp_bound", C.c_float),
        ("inp_res", C.c_float),
        ("inp_noise", C.c_float),
        ("out_bound", C.c_float),
        ("out_res", C.c_float),
        ("out_noise", C.c_float),
        ("out_scale", C.c_float),
        ("w_noise", C.c_float),
        ("nm_thres", C.c_float),
        ("max_bm_res", C.c_float),
        ("inp_asymmetry", C.c_float),
        ("out_asymmetry", C.c_float),
        ("nm_assumed_wmax", C.c_float),
        ("out_noise_std", C.c_float),
        ("nm_decay", C.c_float),
        ("ir_drop", C.c_float),
        ("ir_drop_g_ratio", C.c_float),
        ("v_offset_std", C.c_float),
        ("r_series", C.c_float),
        ("r_series_max_total", C.c_float),
        ("out_nonlinearity", C.c_float),
        ("out_nonlinearity_std", C.c_float),
        ("slope_calibration", C.c_float),
        ("mv_type", C.c_int32),
    ]


class UpdateParams(C.Structure):
    """``ab200_update_params`` (PulsedUpdateMetaParameter, rpu_pulsed_meta_parameter.h:248-279)."""

    _fields_ = [
        ("pulse_type", C.c_int32),
        ("desired_bl", C.c_int32),
        ("fixed_bl", C.c_int32),
        ("update_management", C.c_int32),
        ("update_bl_management", C.c_int32),
        ("sto_round", C.c_int32),
        ("um_grad_scale", C.c_float),
        ("res", C.c_float),
        ("x_res_implicit", C.c_float),
        ("d_res_implicit", C.c_float),
    ]


class WeightModifierParams(C.Structure):
    """``ab200_weight_modifier_params`` (WeightModifierParameter, src/rpucuda/weight_modifier.h:28-50)."""

    _fields_ = [
        ("type", C.c_int32),
        ("sto_round", C.c_int32),
        ("enable_during_test", C.c_int32),
        ("copy_last_column", C.c_int32),
        ("rel_to_actual_wmax", C.c_int32),
        ("n_coeffs", C.c_int32),
        ("std_dev", C.c_float),
        ("res", C.c_float),
        ("dorefa_clip", C.c_float),
        ("pdrop", C.c_float),
        ("assumed_wmax", C.c_float),
        ("g_max", C.c_float),
        ("coeffs", C.c_float * 8),
    ]


class DriftParams(C.Structure):
    """``ab200_drift_params`` (DriftParameter, src/rpucuda/weight_drifter.h:17-60)."""

    _fields_ = [(n, C.c_float) for n in (
        "nu", "nu_dtod", "nu_std", "wg_ratio", "g_offset", "w_offset", "nu_k", "log_g0", "t0",
        "reset_tol", "w_read_std")]


class DeviceParams(C.Structure):
    """``ab200_device_params`` (PulsedRPUDeviceMetaParameter, rpu_pulsed_device.h:60-110)."""

    _fields_ = [
        ("kind", C.c_int32),
        ("construction_seed", C.c_uint32),
        ("enforce_consistency", C.c_int32),
        ("dw_min_dtod_log_normal", C.c_int32),
        ("perfect_bias", C.c_int32),
        ("count_pulses", C.c_int32),
        ("dw_min", C.c_float),
        ("dw_min_dtod", C.c_float),
        ("dw_min_std", C.c_float),
        ("w_min", C.c_float),
        ("w_min_dtod", C.c_float),
        ("w_max", C.c_float),
        ("w_max_dtod", C.c_float),
        ("up_down", C.c_float),
        ("up_down_dtod", C.c_float),
        ("ls_mult_noise", C.c_int32),
        ("ls_allow_increasing_slope", C.c_int32),
        ("ls_mean_bound_reference", C.c_int32),
        ("ls_decrease_up", C.c_float),
        ("ls_decrease_down", C.c_float),
        ("ls_decrease_up_dtod", C.c_float),
        ("ls_decrease_down_dtod", C.c_float),
        ("mult_noise", C.c_int32),
        ("subtract_symmetry_point", C.c_int32),
        ("slope_up_dtod", C.c_float),
        ("slope_down_dtod", C.c_float),
        ("reference_mean", C.c_float),
        ("reference_std", C.c_float),
        ("lifetime", C.c_float),
        ("lifetime_dtod", C.c_float),
        ("diffusion", C.c_float),
        ("diffusion_dtod", C.c_float),
        ("reset", C.c_float),
        ("reset_dtod", C.c_float),
        ("reset_std", C.c_float),
        ("es_A_up", C.c_float),
        ("es_A_down", C.c_float),
        ("es_gamma_up", C.c_float),
        ("es_gamma_down", C.c_float),
        ("es_a", C.c_float),
        ("es_b", C.c_float),
        ("dw_min_std_add", C.c_float),
        ("dw_min_std_slope", C.c_float),
        ("ps_gamma", C.c_float),
        ("ps_gamma_dtod", C.c_float),
        ("ps_gamma_up_down", C.c_float),
        ("ps_gamma_up_down_dtod", C.c_float),
        ("pw_n", C.c_int32),
        ("pw_up", C.c_float * 32),
        ("pw_down", C.c_float * 32),
        ("drift", DriftParams),
    ]


class TransferParams(C.Structure):
    """``ab200_transfer_params`` (TransferRPUDeviceMetaParameter, rpu_transfer_device.h:52-75)."""

    _fields_ = [
        ("gamma", C.c_float),
        ("transfer_every", C.c_float),
        ("units_in_mbatch", C.c_int32),
        ("n_reads_per_transfer", C.c_int32),
        ("fast_lr", C.c_float),
        ("transfer_lr", C.c_float),
        ("scale_transfer_lr", C.c_int32),
        ("scale_fast_lr", C.c_int32),
        ("transfer_columns", C.c_int32),
        ("transfer_io", IOParams),
        ("transfer_up", UpdateParams),
        ("buffered", C.c_int32),
        ("forget_buffer", C.c_int32),
        ("thres_scale", C.c_float),
        ("step", C.c_float),
        ("momentum", C.c_float),
        ("chopped", C.c_int32),
        ("in_chop_random", C.c_int32),
        ("correct_gradient_magnitudes", C.c_int32),
        ("no_buffer", C.c_int32),
        ("in_chop_prob", C.c_float),
        ("out_chop_prob", C.c_float),
        ("auto_granularity", C.c_float),
        ("buffer_granularity", C.c_float),
        ("dynamic", C.c_int32),
        ("correct_accumulation", C.c_int32),
        ("tail_weightening", C.c_float),
        ("buffer_cap", C.c_float),
    ]


class MixedPrecParams(C.Structure):
    """``ab200_mixedprec_params``."""

    _fields_ = [
        ("enabled", C.c_int32),
        ("transfer_every", C.c_int32),
        ("n_rows_per_transfer", C.c_int32),
        ("random_row", C.c_int32),
        ("granularity", C.c_float),
        ("n_x_bins", C.c_int32),
        ("n_d_bins", C.c_int32),
        ("stoc_round_x", C.c_int32),
        ("stoc_round_d", C.c_int32),
        ("transfer_lr", C.c_float),
    ]


class TileConfig(C.Structure):
    """``ab200_tile_config``."""

    _fields_ = [
        ("x_size", C.c_int32),
        ("d_size", C.c_int32),
        ("forward_io", IOParams),
        ("backward_io", IOParams),
        ("update", UpdateParams),
        ("device_kind", C.c_int32),
        ("device", DeviceParams * 2),
        ("transfer", TransferParams),
        ("mixed", MixedPrecParams),
        ("seed", C.c_uint64),
    ]


class ScatterPlan(C.Structure):
    """``ab200_scatter_plan``."""

    _fields_ = [
        ("out_table_dev", C.c_void_p),
        ("code_table_dev", C.c_void_p),
        ("fac_table_dev", C.c_void_p),
        ("flag_table_dev", C.c_void_p),
        ("n_owners", C.c_int32),
        ("rows_per_owner", C.c_int32),
        ("rotate_rows", C.c_int32),
        ("row_base", C.c_int32),
        ("owner_block_rows", C.c_int32),
        ("epoch", C.c_int32),
    ]


_lib: Optional[C.CDLL] = None

_VP = C.c_void_p
_FP = C.c_void_p  # float pointers are passed as raw addresses (host or device)
_I = C.c_int


def _declare(lib: C.CDLL) -> None:
    cfgp = C.POINTER(TileConfig)
    sig = {
        "ab200_last_error": (C.c_char_p, []),
        "ab200_version": (C.c_char_p, []),
        "ab200_default_io_params": (None, [C.POINTER(IOParams)]),
        "ab200_default_update_params": (None, [C.POINTER(UpdateParams)]),
        "ab200_default_device_params": (None, [C.POINTER(DeviceParams), C.c_int32]),
        "ab200_default_transfer_params": (None, [C.POINTER(TransferParams)]),
        "ab200_default_mixedprec_params": (None, [C.POINTER(MixedPrecParams)]),
        "ab200_tile_create": (_I, [cfgp, _I, C.POINTER(_VP)]),
        "ab200_tile_destroy": (_I, [_VP]),
        "ab200_tile_to_device": (_I, [_VP, _I]),
        "ab200_tile_get_x_size": (_I, [_VP]),
        "ab200_tile_get_d_size": (_I, [_VP]),
        "ab200_tile_set_learning_rate": (_I, [_VP, C.c_float]),
        "ab200_tile_get_learning_rate": (_I, [_VP, C.POINTER(C.c_float)]),
        "ab200_tile_set_weights": (_I, [_VP, _FP]),
        "ab200_tile_get_weights": (_I, [_VP, _FP]),
        "ab200_tile_set_weights_device": (_I, [_VP, _FP, _VP]),
        "ab200_tile_get_weights_device": (_I, [_VP, _FP, _VP]),
        "ab200_tile_set_shared_weights": (_I, [_VP, _FP, C.c_uint64]),
        "ab200_tile_set_delta_weights": (_I, [_VP, _FP]),
        "ab200_tile_hidden_parameter_count": (_I, [_VP]),
        "ab200_tile_hidden_parameter_name": (C.c_char_p, [_VP, _I]),
        "ab200_tile_get_hidden_parameters": (_I, [_VP, _FP]),
        "ab200_tile_set_hidden_parameters": (_I, [_VP, _FP]),
        "ab200_tile_forward": (_I, [_VP, _FP, _FP, _I, _I, _I, _I, _I, _VP]),
        "ab200_tile_backward": (_I, [_VP, _FP, _FP, _I, _I, _I, _I, _VP]),
        "ab200_tile_update": (_I, [_VP, _FP, _FP, _I, _I, _I, _I, _VP]),
        "ab200_tile_forward_host": (_I, [_VP, _FP, _FP, _I, _I, _I, _I, _I, _VP]),
        "ab200_tile_backward_host": (_I, [_VP, _FP, _FP, _I, _I, _I, _I, _VP]),
        "ab200_tile_update_host": (_I, [_VP, _FP, _FP, _I, _I, _I, _I, _VP]),
        "ab200_tile_coincidences": (_I, [_VP, _FP, _FP, _FP, _VP]),
        "ab200_tile_set_matrix_indices": (_I, [_VP, _FP, C.c_longlong, _VP]),
        "ab200_tile_has_matrix_indices": (_I, [_VP]),
        "ab200_tile_forward_indexed": (_I, [_VP, _FP, _FP, C.c_longlong, _I, _I, _I, _I, _VP]),
        "ab200_tile_backward_indexed": (_I, [_VP, _FP, _FP, C.c_longlong, _I, _I, _I, _VP]),
        "ab200_tile_update_indexed": (_I, [_VP, _FP, _FP, C.c_longlong, _I, _I, _I, _VP]),
        "ab200_sizeof": (C.c_size_t, [_I]),
        "ab200_tile_extra_count": (_I, []),
        "ab200_tile_extra_name": (C.c_char_p, [_I]),
        "ab200_tile_dump_extra": (_I, [_VP, C.POINTER(C.c_double)]),
        "ab200_tile_extra_vector_count": (_I, [_VP]),
        "ab200_tile_extra_vector_name": (C.c_char_p, [_VP, _I]),
        "ab200_tile_extra_vector_size": (_I, [_VP, _I]),
        "ab200_tile_get_extra_vector": (_I, [_VP, _I, C.POINTER(C.c_double)]),
        "ab200_tile_set_extra_vector": (_I, [_VP, _I, C.POINTER(C.c_double), _I]),
        "ab200_tile_load_extra": (_I, [_VP, C.POINTER(C.c_char_p), C.POINTER(C.c_double), _I, _I]),
        "ab200_tile_decay_weights": (_I, [_VP, C.c_float, _I, _VP]),
        "ab200_tile_drift_weights": (_I, [_VP, C.c_float, _VP]),
        "ab200_tile_modify_weights": (_I, [_VP, C.POINTER(WeightModifierParams), _VP]),
        "ab200_tile_get_io_vector": (_I, [_VP, _I, _I, _VP, _I]),
        "ab200_tile_set_io_vector": (_I, [_VP, _I, _I, _VP, _I]),
        "ab200_tile_diffuse_weights": (_I, [_VP, _VP]),
        "ab200_tile_clip_weights": (_I, [_VP, _I, C.c_float, C.c_float, _VP]),
        "ab200_tile_reset_columns": (_I, [_VP, _I, _I, C.c_float, _VP]),
        "ab200_tile_set_weights_uniform_random": (_I, [_VP, C.c_float, C.c_float, _VP]),
        "ab200_tile_last_bm_stats": (_I, [_VP, C.POINTER(C.c_int32), C.POINTER(C.c_float)]),
        "ab200_tile_get_pulse_counters": (_I, [_VP, _VP]),
        "ab200_tile_counts_pulses": (_I, [_VP]),
        "ab200_tile_set_seed": (_I, [_VP, C.c_uint64]),
        "ab200_array_create": (_I, [cfgp, _I, _I, _I, _I, _I, _I, _I, C.POINTER(_VP)]),
        "ab200_array_create_block": (_I, [cfgp, _I, _I, _I, _I, _I, _I, _I, _I, _I, C.POINTER(_VP)]),
        "ab200_array_destroy": (_I, [_VP]),
        "ab200_array_num_in_splits": (_I, [_VP]),
        "ab200_array_num_out_splits": (_I, [_VP]),
        "ab200_array_set_weights": (_I, [_VP, _FP]),
        "ab200_array_forward_scatter": (_I, [_VP, _FP, _I, _VP, _I, _I, _I, _VP]),
        "ab200_sum_slots": (_I, [_FP, _I, C.c_longlong, _FP, _VP]),
        "ab200_array_scatter_codes_supported": (_I, [_VP]),
        "ab200_array_forward_scatter_codes": (_I, [_VP, _FP, _I, _VP, _VP, _I, _I, _I, _VP]),
        "ab200_sum_code_slots": (_I, [_VP, C.c_longlong, _VP, C.c_longlong, _I, C.POINTER(_I), _I, _I, _I,
                                      _FP, _VP]),
        "ab200_array_forward_scatter_plan": (_I, [_VP, _FP, _I, C.POINTER(ScatterPlan), _VP]),
        "ab200_sum_slots_wait": (_I, [_FP, _I, C.c_longlong, _I, _I, _I, _FP, _VP, _I, _I, C.c_float, _VP]),
        "ab200_sum_code_slots_wait": (_I, [_VP, C.c_longlong, _VP, C.c_longlong, _I, C.POINTER(_I), _I, _I,
                                           _I, _I, _FP, _VP, _I, _I, C.c_float, _VP]),
        "ab200_wait_status": (_I, [_I, C.POINTER(_I)]),
        "ab200_peer_alloc": (_I, [C.c_size_t, _I, C.POINTER(_VP), C.c_char_p]),
        "ab200_peer_open": (_I, [C.c_char_p, _I, C.POINTER(_VP)]),
        "ab200_peer_close": (_I, [_VP]),
        "ab200_peer_free": (_I, [_VP]),
        "ab200_array_backward": (_I, [_VP, _FP, _FP, _I, _VP]),
        "ab200_array_update": (_I, [_VP, _FP, _FP, _I, _VP]),
        "ab200_array_set_learning_rate": (_I, [_VP, C.c_float]),
        "ab200_array_set_weights_scaled": (_I, [_VP, _FP, C.c_float]),
        "ab200_array_get_tile_scales": (_I, [_VP, _FP]),
        "ab200_array_set_bias": (_I, [_VP, _FP]),
        "ab200_array_get_weights": (_I, [_VP, _FP]),
        "ab200_array_forward": (_I, [_VP, _FP, _FP, _I, _I, _VP]),
        "ab200_array_forward_host": (_I, [_VP, _FP, _FP, _I, _I, _VP]),
        "ab200_array_forward_local": (_I, [_VP, _FP, _FP, _I, _I, _VP]),
        "ab200_array_local_in_size": (_I, [_VP]),
        "ab200_array_set_seed": (_I, [_VP, C.c_uint64]),
        "ab200_mvm_forward_noalloc": (
            _I, [C.POINTER(IOParams), _FP, _I, _I, _FP, _FP, _I, C.c_uint64, C.c_uint32, _VP]
        ),
        "ab200_set_mvm_path": (_I, [_I]),
        "ab200_set_update_path": (_I, [_I]),
        "ab200_measure_popc_peak": (_I, [_I, C.POINTER(C.c_double)]),
        "ab200_kernel_launch_count": (C.c_uint64, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


#: every symbol ``include/aihwkit_b200.h`` declares (checked by the CPU test-suite)
def declared_symbols() -> list:
    import re

    header = os.path.join(os.path.dirname(_HERE), "include", "aihwkit_b200.h")
    with open(header, "r", encoding="utf-8") as f:
        text = f.read()
    return sorted(set(re.findall(r"\b(ab200_[a-z0-9_]+)\s*\(", text)))


def lib() -> C.CDLL:
    """Load the CUDA library; raise loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `python -m aihwkit_b200.build` "
                "(nvcc, sm_100a). There is no CPU fallback for the analog tile."
            )
        loaded = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        _declare(loaded)
        _lib = loaded
    return _lib


def check(code: int) -> None:
    """Turn a non-zero return code into the RuntimeError the reference binding raises."""
    if code != 0:
        msg = lib().ab200_last_error()
        raise RuntimeError(msg.decode("utf-8", "replace") if msg else f"ab200 error {code}")
