"""TEST INFRASTRUCTURE — ctypes access to the compiled reference CPU tile.

``oracle/_ref/librpu_ref.so`` is the UNMODIFIED reference (``RPU::RPUPulsed<float>``,
src/rpucuda/rpu_pulsed.h:23-125) behind the thin C wrapper ``oracle/ref_capi.cpp``; it is
built by ``make -C oracle``.  Only tests, ``smoke()`` and bench.py's CPU-baseline legs may
import this module; the product never does.
"""

from __future__ import annotations

import ctypes as C
import glob
import os
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(_HERE))
from aihwkit_b200 import _cabi  # noqa: E402  (struct layouts of include/aihwkit_b200.h)

REF_LIB = os.path.join(_HERE, "_ref", "librpu_ref.so")
_lib = None


def blas_name() -> str:
    """Which BLAS the reference was linked against when ``_ref`` was built."""
    path = os.path.join(_HERE, "_ref", "blas.txt")
    if os.path.exists(path):
        with open(path, "r", encoding="utf-8") as f:
            return f.read().strip()
    return "unknown"


def available() -> bool:
    try:
        load()
        return True
    except OSError:
        return False


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(REF_LIB):
        raise OSError(f"{REF_LIB} not built (run `make -C oracle` where the reference is present)")
    # the bundled OpenBLAS needs its sibling libgfortran / libquadmath, which carry hashed names
    try:
        import sysconfig

        libs = os.path.join(sysconfig.get_paths()["purelib"], "opencv_python_headless.libs")
        for pat in ("libquadmath*.so*", "libgfortran*.so*"):
            for p in sorted(glob.glob(os.path.join(libs, pat))):
                C.CDLL(p, mode=C.RTLD_GLOBAL)
    except OSError:
        pass
    lib = C.CDLL(REF_LIB)
    vp, fp, i = C.c_void_p, C.c_void_p, C.c_int
    sig = {
        "ref_last_error": (C.c_char_p, []),
        "ref_tile_create": (i, [C.POINTER(_cabi.TileConfig), C.POINTER(vp)]),
        "ref_tile_destroy": (i, [vp]),
        "ref_tile_set_seed": (i, [vp, C.c_uint64]),
        "ref_tile_set_learning_rate": (i, [vp, C.c_float]),
        "ref_tile_set_weights": (i, [vp, fp]),
        "ref_tile_get_weights": (i, [vp, fp]),
        "ref_tile_hidden_parameter_count": (i, [vp]),
        "ref_tile_hidden_parameter_name": (C.c_char_p, [vp, i]),
        "ref_tile_get_hidden_parameters": (i, [vp, fp]),
        "ref_tile_set_hidden_parameters": (i, [vp, fp]),
        "ref_tile_forward": (i, [vp, fp, fp, i, i, i, i, i]),
        "ref_tile_backward": (i, [vp, fp, fp, i, i, i, i]),
        "ref_tile_update": (i, [vp, fp, fp, i, i, i, i]),
        "ref_tile_coincidences": (i, [vp, fp, fp, C.c_float, C.c_float, fp]),
        "ref_tile_decay_weights": (i, [vp, C.c_float, i]),
        "ref_tile_diffuse_weights": (i, [vp]),
        "ref_tile_drift_weights": (i, [vp, C.c_float]),
        "ref_tile_modify_weights": (i, [vp, vp]),
        "ref_tile_get_io_vector": (i, [vp, i, i, fp, i]),
        "ref_tile_clip_weights": (i, [vp, i, C.c_float, C.c_float]),
        "ref_tile_reset_columns": (i, [vp, i, i, C.c_float]),
        "ref_tile_set_matrix_indices": (i, [vp, fp, C.c_longlong]),
        "ref_tile_forward_indexed": (i, [vp, fp, fp, C.c_longlong, i, i, i, i]),
        "ref_tile_backward_indexed": (i, [vp, fp, fp, C.c_longlong, i, i, i]),
        "ref_tile_update_indexed": (i, [vp, fp, fp, C.c_longlong, i, i, i]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class RefTile:
    """The reference CPU analog tile, driven through plain numpy arrays."""

    def __init__(self, cfg: _cabi.TileConfig):
        self._lib = load()
        self.x_size, self.d_size = int(cfg.x_size), int(cfg.d_size)
        h = C.c_void_p()
        self._ck(self._lib.ref_tile_create(C.byref(cfg), C.byref(h)))
        self._h = h

    def _ck(self, code: int) -> None:
        if code:
            raise RuntimeError(self._lib.ref_last_error().decode())

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.ref_tile_destroy(self._h)
            self._h = None

    def set_seed(self, seed: int) -> None:
        self._ck(self._lib.ref_tile_set_seed(self._h, seed))

    def set_learning_rate(self, lr: float) -> None:
        self._ck(self._lib.ref_tile_set_learning_rate(self._h, lr))

    def set_weights(self, w) -> None:
        w = _f32(w)
        assert w.shape == (self.d_size, self.x_size)
        self._ck(self._lib.ref_tile_set_weights(self._h, w.ctypes.data))

    def get_weights(self) -> np.ndarray:
        w = np.empty((self.d_size, self.x_size), np.float32)
        self._ck(self._lib.ref_tile_get_weights(self._h, w.ctypes.data))
        return w

    def hidden_parameter_names(self) -> list:
        n = self._lib.ref_tile_hidden_parameter_count(self._h)
        return [self._lib.ref_tile_hidden_parameter_name(self._h, k).decode() for k in range(n)]

    def get_hidden_parameters(self) -> np.ndarray:
        n = self._lib.ref_tile_hidden_parameter_count(self._h)
        out = np.empty((n, self.d_size, self.x_size), np.float32)
        if n:
            self._ck(self._lib.ref_tile_get_hidden_parameters(self._h, out.ctypes.data))
        return out

    def set_hidden_parameters(self, hp) -> None:
        hp = _f32(hp)
        self._ck(self._lib.ref_tile_set_hidden_parameters(self._h, hp.ctypes.data))

    def forward(self, x, bias=False, x_trans=False, d_trans=False, is_test=False) -> np.ndarray:
        x = _f32(x)
        in_size = x.shape[0] if x_trans else x.shape[-1]
        m = x.size // in_size
        out = np.empty((self.d_size, m) if d_trans else (m, self.d_size), np.float32)
        self._ck(
            self._lib.ref_tile_forward(
                self._h, x.ctypes.data, out.ctypes.data, int(bias), m, int(x_trans), int(d_trans),
                int(is_test),
            )
        )
        return out

    def backward(self, d, bias=False, d_trans=False, x_trans=False) -> np.ndarray:
        d = _f32(d)
        dsz = d.shape[0] if d_trans else d.shape[-1]
        m = d.size // dsz
        xs = self.x_size - (1 if bias else 0)
        out = np.empty((xs, m) if x_trans else (m, xs), np.float32)
        self._ck(
            self._lib.ref_tile_backward(
                self._h, d.ctypes.data, out.ctypes.data, int(bias), m, int(d_trans), int(x_trans)
            )
        )
        return out

    def update(self, x, d, bias=False, x_trans=False, d_trans=False) -> None:
        x, d = _f32(x), _f32(d)
        in_size = x.shape[0] if x_trans else x.shape[-1]
        m = x.size // in_size
        self._ck(
            self._lib.ref_tile_update(
                self._h, x.ctypes.data, d.ctypes.data, int(bias), m, int(x_trans), int(d_trans)
            )
        )

    def coincidences(self, x, d, lr: float, dw_min: float) -> np.ndarray:
        """Signed coincidence counts [d, x] of one sample (deterministic pulse types)."""
        x, d = _f32(x), _f32(d)
        out = np.empty((self.d_size, self.x_size), np.int32)
        self._ck(
            self._lib.ref_tile_coincidences(
                self._h, x.ctypes.data, d.ctypes.data, lr, dw_min, out.ctypes.data
            )
        )
        return out

    # indexed convolution interface (src/rpucuda/rpu.cpp:1117-1239); images are [N, C, H, W]
    # (`trans=True`, the layout the Python binding always uses) or [N, H*W, C] (`trans=False`)
    def set_matrix_indices(self, indices) -> None:
        idx = np.ascontiguousarray(indices, dtype=np.int32)
        self._ck(self._lib.ref_tile_set_matrix_indices(self._h, idx.ctypes.data, idx.size))

    def forward_indexed(self, x, d_shape, trans=True, is_test=False) -> np.ndarray:
        x = _f32(x)
        out = np.zeros(d_shape, np.float32)
        n = x.shape[0]
        m_batch = out.size // (n * self.d_size)
        self._ck(
            self._lib.ref_tile_forward_indexed(
                self._h, x.ctypes.data, out.ctypes.data, x.size, m_batch, n, int(trans), int(is_test)
            )
        )
        return out

    def backward_indexed(self, d, x_shape, trans=True) -> np.ndarray:
        d = _f32(d)
        out = np.zeros(x_shape, np.float32)
        n = d.shape[0]
        m_batch = d.size // (n * self.d_size)
        self._ck(
            self._lib.ref_tile_backward_indexed(
                self._h, d.ctypes.data, out.ctypes.data, out.size, m_batch, n, int(trans)
            )
        )
        return out

    def update_indexed(self, x, d, trans=True) -> None:
        x, d = _f32(x), _f32(d)
        n = d.shape[0]
        m_batch = d.size // (n * self.d_size)
        self._ck(
            self._lib.ref_tile_update_indexed(
                self._h, x.ctypes.data, d.ctypes.data, x.size, m_batch, n, int(trans)
            )
        )

    # weight operations between updates (src/rpucuda/rpu_pulsed.cpp:189-284)
    def decay_weights(self, alpha: float = 1.0, bias_no_decay: bool = False) -> None:
        self._ck(self._lib.ref_tile_decay_weights(self._h, alpha, int(bias_no_decay)))

    def get_io_vector(self, backward: bool, which: int, n: int) -> np.ndarray:
        """The per-line IO vector the reference drew (0 v_offset, 1 out_nonlinearity,
        2 out_noise_values); empty when it is not in use."""
        out = np.zeros(n, np.float32)
        cnt = self._lib.ref_tile_get_io_vector(self._h, int(backward), int(which),
                                               out.ctypes.data_as(C.POINTER(C.c_float)), n)
        if cnt < 0:
            raise RuntimeError("ref_tile_get_io_vector failed")
        return out[:cnt]

    def modify_weights(self, weight_modifier_params) -> None:
        """``weight_modifier_params``: a ``WeightModifierParameter`` of aihwkit_b200.rpu_base.tiles."""
        c = weight_modifier_params._to_c()
        self._ck(self._lib.ref_tile_modify_weights(self._h, C.byref(c)))

    def drift_weights(self, time_since_last_call: float) -> None:
        self._ck(self._lib.ref_tile_drift_weights(self._h, time_since_last_call))

    def diffuse_weights(self) -> None:
        self._ck(self._lib.ref_tile_diffuse_weights(self._h))

    def clip_weights(self, clip_type: int, fixed_value: float = -1.0, sigma: float = 2.5) -> None:
        self._ck(self._lib.ref_tile_clip_weights(self._h, int(clip_type), fixed_value, sigma))

    def reset_columns(self, start_col: int = 0, n_cols: int = 1, reset_prob: float = 1.0) -> None:
        self._ck(self._lib.ref_tile_reset_columns(self._h, start_col, n_cols, reset_prob))
