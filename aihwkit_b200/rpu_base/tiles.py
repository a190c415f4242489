"""Mirror of ``aihwkit.simulator.rpu_base.tiles`` for the analog-tile hot path.

Method names, argument order and error behaviour follow the reference's binding
(``src/aihwkit/simulator/rpu_base_src/rpu_base_tiles.cpp:53-886`` and the CUDA overrides in
``rpu_base_tiles_cuda.cpp:45-543``).  Every compute call goes through the C ABI of
``include/aihwkit_b200.h`` into the sm_100a kernels; there is no CPU compute path.  torch is
used only for device memory and streams.

Differences from the reference binding, all forced by "GPU only":
  * a tile created by ``AnalogTileParameter.create_array`` carries configuration, weights and the
    host-drawn device parameters but cannot compute until ``.cuda()`` (or ``CudaAnalogTile(tile)``)
    has moved it to a device;
  * CUDA tensors are processed in place on the current torch stream; CPU tensors are accepted
    too and are staged through pinned memory by the library (host -> device -> host per call).
"""

from __future__ import annotations

import ctypes as C
import enum
from typing import List, Optional

import numpy as np
import torch

from .. import _cabi
from .._cabi import check


class WeightClipType(enum.IntEnum):
    """rpu_base_utils.cpp:49-53 (src/rpucuda/weight_clipper.h:14-19); ``None`` spelt ``None_``."""

    None_ = 0
    FixedValue = 1
    LayerGaussian = 2
    AverageChannelMax = 3


class WeightRemapType(enum.IntEnum):
    """rpu_base_utils.cpp:44-47 (src/rpucuda/weight_remapper.h)."""

    None_ = 0
    LayerwiseSymmetric = 1
    ChannelwiseSymmetric = 2


class WeightModifierType(enum.IntEnum):
    """rpu_base_utils.cpp:31-42 (src/rpucuda/weight_modifier.h)."""

    Copy = 0
    Discretize = 1
    MultNormal = 2
    AddNormal = 3
    DiscretizeAddNormal = 4
    DoReFa = 5
    Poly = 6
    PCMNoise = 7
    DropConnect = 8
    ProgNoise = 9


for _e in (WeightClipType, WeightRemapType):
    _e._member_map_["None"] = _e(0)  # type: ignore[attr-defined]
    type.__setattr__(_e, "None", _e(0))
WeightModifierType._member_map_["None"] = WeightModifierType.Copy  # type: ignore[attr-defined]
type.__setattr__(WeightModifierType, "None", WeightModifierType.Copy)


class WeightClipParameter:
    """``WeightClipParameter`` (rpu_base_utils.cpp:18-22; src/rpucuda/weight_clipper.h:22-27)."""

    def __init__(self) -> None:
        self.type = WeightClipType.None_
        self.fixed_value = -1.0
        self.sigma = 2.5


class WeightRemapParameter:
    """``WeightRemapParameter`` (rpu_base_utils.cpp:24-29; src/rpucuda/weight_remapper.h)."""

    def __init__(self) -> None:
        self.type = WeightRemapType.None_
        self.remapped_wmax = 1.0
        self.max_scale_range = 0.0
        self.max_scale_ref = 0.0


class WeightModifierParameter:
    """``WeightModifierParameter`` (rpu_base_tiles.cpp:31-51; src/rpucuda/weight_modifier.h)."""

    def __init__(self) -> None:
        self.std_dev = 0.0
        self.per_batch_sample = False
        self.res = 0.1
        self.sto_round = False
        self.dorefa_clip = 0.6
        self.pdrop = 0.0
        self.enable_during_test = False
        self.copy_last_column = False
        self.rel_to_actual_wmax = True
        self.assumed_wmax = 1.0
        self.type = WeightModifierType.Copy
        self.coeffs = [0.26348 / 25.0, 0.0768, -0.001877 * 25.0]  # weight_modifier.h:49
        self.pcm_zero_thres = 0.0
        self.pcm_t_inference = 0.0
        self.pcm_prob_at_reset = 0.0
        self.pcm_prob_at_gmax = 0.0
        self.pcm_prob_at_random = 0.0
        self.pcm_t0 = 20.0
        self.g_max = 25.0

    def _to_c(self) -> "_cabi.WeightModifierParams":
        coeffs = [float(v) for v in self.coeffs]
        if len(coeffs) > 8:
            raise RuntimeError("modify_weights: at most 8 polynomial coefficients are implemented")
        c = _cabi.WeightModifierParams()
        c.type = int(self.type)
        c.sto_round = int(bool(self.sto_round))
        c.enable_during_test = int(bool(self.enable_during_test))
        c.copy_last_column = int(bool(self.copy_last_column))
        c.rel_to_actual_wmax = int(bool(self.rel_to_actual_wmax))
        c.n_coeffs = len(coeffs)
        for name in ("std_dev", "res", "dorefa_clip", "pdrop", "assumed_wmax", "g_max"):
            setattr(c, name, float(getattr(self, name)))
        for k, v in enumerate(coeffs):
            c.coeffs[k] = v
        return c


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(t: torch.Tensor) -> int:
    """The ``cudaStream_t`` torch currently launches on for the tensor's device."""
    if _raw_stream is not None:
        # the handle itself, without building a torch.cuda.Stream object around it (a few
        # microseconds per call, which count for a tile whose whole step takes 75)
        return int(_raw_stream(t.device.index if t.device.index is not None else torch.cuda.current_device()))
    return int(torch.cuda.current_stream(t.device).cuda_stream)


def _check_input(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be a float32 tensor")
    return t.contiguous()


class AnalogTile:
    """``tiles.AnalogTile`` / ``tiles.CudaAnalogTile`` (RPUPulsed / RPUCudaPulsed)."""

    def __init__(self, config: _cabi.TileConfig, cuda_device: int = -1):
        self._lib = _cabi.lib()
        self._cfg = config
        handle = C.c_void_p()
        check(self._lib.ab200_tile_create(C.byref(config), int(cuda_device), C.byref(handle)))
        self._h = handle
        self._device_index = int(cuda_device)
        self._shared: Optional[torch.Tensor] = None
        self._shared_version = -1
        self._delta: Optional[torch.Tensor] = None
        self._meta = None  # the AnalogTileParameter the tile was created from
        self._hidden_update_index = 0

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ab200_tile_destroy(h)

    # -- placement -------------------------------------------------------------------------
    def cuda(self, device=None) -> "AnalogTile":
        """Move the tile to a CUDA device (``CudaAnalogTile(cpu_tile)``,
        rpu_base_tiles_cuda.cpp:532-538)."""
        if device is None:
            index = torch.cuda.current_device() if torch.cuda.is_available() else 0
        else:
            index = torch.device(device).index if not isinstance(device, int) else device
            index = 0 if index is None else index
        check(self._lib.ab200_tile_to_device(self._h, int(index)))
        self._device_index = int(index)
        return self

    @property
    def is_cuda(self) -> bool:
        return self._device_index >= 0

    # -- sizes / learning rate ---------------------------------------------------------------
    def get_x_size(self) -> int:
        return int(self._cfg.x_size)

    def get_d_size(self) -> int:
        return int(self._cfg.d_size)

    def set_learning_rate(self, learning_rate: float) -> None:
        check(self._lib.ab200_tile_set_learning_rate(self._h, float(learning_rate)))

    def get_learning_rate(self) -> float:
        out = C.c_float()
        check(self._lib.ab200_tile_get_learning_rate(self._h, C.byref(out)))
        return float(out.value)

    def set_seed(self, seed: int) -> None:
        check(self._lib.ab200_tile_set_seed(self._h, int(seed)))

    # -- weights ---------------------------------------------------------------------------
    def set_weights(self, weights: torch.Tensor) -> None:
        """``[d_size, x_size]`` (rpu_base_tiles.cpp:150-178)."""
        w = weights.detach().to(torch.float32).cpu().contiguous()
        if tuple(w.shape) != (self.get_d_size(), self.get_x_size()):
            raise RuntimeError(
                f"Invalid weights dimensions: expected [{self.get_d_size()},{self.get_x_size()}] array"
            )
        check(self._lib.ab200_tile_set_weights(self._h, w.data_ptr()))
        if self._device_index < 0 and self._shared is not None:
            # a tile without a device keeps the caller's host tensor in step (the reference CPU
            # tile writes through the shared memory)
            self._shared.copy_(self._get_weights_c())

    def _get_weights_c(self) -> torch.Tensor:
        w = torch.empty(self.get_d_size(), self.get_x_size(), dtype=torch.float32)
        check(self._lib.ab200_tile_get_weights(self._h, w.data_ptr()))
        return w

    def get_weights(self) -> torch.Tensor:
        """CPU tensor ``[d_size, x_size]`` (rpu_base_tiles.cpp:130-148)."""
        if self._device_index < 0 and self._shared is not None:
            return self._shared.detach().clone()
        return self._get_weights_c()

    def __getattr__(self, name):
        # ``get_weights_cuda`` / ``set_weights_cuda`` exist on tiles that sit on a device only:
        # the reference's Python probes for them with hasattr (tiles/base.py:452-453,
        # tiles/periphery.py:164-171, 225-226) and falls back to the host accessors otherwise
        if name in ("get_weights_cuda", "set_weights_cuda") and \
                self.__dict__.get("_device_index", -1) >= 0:
            return getattr(self, "_" + name)
        raise AttributeError(f"'{type(self).__name__}' object has no attribute '{name}'")

    def _set_weights_cuda(self, weights_xd: torch.Tensor) -> None:
        """Device tensor ``[x_size, d_size]`` (probed by tiles/base.py:452-453)."""
        w = _check_input(weights_xd, "weights")
        if not w.is_cuda or tuple(w.shape) != (self.get_x_size(), self.get_d_size()):
            raise RuntimeError("set_weights_cuda expects a CUDA [x_size, d_size] tensor")
        check(self._lib.ab200_tile_set_weights_device(self._h, w.data_ptr(), _stream_ptr(w)))

    def _get_weights_cuda(self) -> torch.Tensor:
        dev = torch.device("cuda", self._device_index)
        w = torch.empty(self.get_x_size(), self.get_d_size(), dtype=torch.float32, device=dev)
        check(self._lib.ab200_tile_get_weights_device(self._h, w.data_ptr(), _stream_ptr(w)))
        return w

    def set_shared_weights(self, weights_xd: torch.Tensor) -> None:
        """Alias caller-owned memory as the tile's weights: ``[x_size, d_size]`` CUDA memory for a
        tile on a device (rpu_base_tiles_cuda.cpp:96-124; src/rpucuda/cuda/rpucuda.cu:322-334; the
        buffer is NOT filled, the caller copies the weights in, tiles/base.py:413-417), ``[d_size,
        x_size]`` host memory for a tile without a device (rpu_base_tiles.cpp:216-229: filled with
        the current weights)."""
        if weights_xd.dtype != torch.float32:
            raise RuntimeError("set_shared_weights expects a float32 tensor")
        if not weights_xd.is_contiguous() or weights_xd.numel() != self.get_x_size() * self.get_d_size():
            raise RuntimeError("Shared weights need to be contiguous and of the tile's size")
        if self._device_index < 0:
            if weights_xd.is_cuda:
                raise RuntimeError("set_shared_weights: a tile without a device takes host memory")
            if self._shared is None or self._shared.data_ptr() != weights_xd.data_ptr():
                weights_xd.copy_(self._get_weights_c().reshape(weights_xd.shape))
            self._shared = weights_xd
            return
        if not weights_xd.is_cuda:
            raise RuntimeError("set_shared_weights expects a float32 CUDA tensor")
        self._shared = weights_xd
        self._shared_version = int(weights_xd._version)
        check(
            self._lib.ab200_tile_set_shared_weights(
                self._h, weights_xd.data_ptr(), self._shared_version
            )
        )

    def _sync_shared(self) -> None:
        """The caller may have written into the shared tensor since it was set (the reason to
        share it): tell the tile, so that operand copies derived from the weights are rebuilt."""
        if self._shared is not None and self._device_index >= 0 and \
                int(self._shared._version) != self._shared_version:
            self.set_shared_weights(self._shared)

    def get_shared_weights_if(self) -> bool:
        return self._shared is not None

    def set_delta_weights(self, delta_weights: torch.Tensor) -> None:
        """rpu_base_tiles_cuda.cpp ``set_delta_weights`` (rpu_base_tiles.cpp:231-245): the
        floating-point update writes the gradient into this ``[x_size, d_size]`` CUDA tensor
        instead of changing the weights, until :meth:`reset_delta_weights`."""
        if not delta_weights.is_cuda or delta_weights.dtype != torch.float32 or \
                not delta_weights.is_contiguous() or \
                delta_weights.numel() != self.get_x_size() * self.get_d_size():
            raise RuntimeError("Delta weights need to be a contiguous float32 CUDA tensor of the tile's size")
        self._delta = delta_weights
        check(self._lib.ab200_tile_set_delta_weights(self._h, delta_weights.data_ptr()))

    def reset_delta_weights(self) -> None:
        """rpu_base_tiles.cpp:246-252."""
        self._delta = None
        check(self._lib.ab200_tile_set_delta_weights(self._h, None))

    # -- hidden parameters ---------------------------------------------------------------------
    def get_hidden_parameter_names(self) -> List[str]:
        n = self._lib.ab200_tile_hidden_parameter_count(self._h)
        return [self._lib.ab200_tile_hidden_parameter_name(self._h, i).decode() for i in range(n)]

    def get_hidden_parameters(self) -> torch.Tensor:
        """``[n, d_size, x_size]`` CPU tensor (rpu_base_tiles.cpp:764-789)."""
        n = self._lib.ab200_tile_hidden_parameter_count(self._h)
        if n == 0:
            return torch.empty(0, dtype=torch.float32)
        out = torch.empty(n, self.get_d_size(), self.get_x_size(), dtype=torch.float32)
        check(self._lib.ab200_tile_get_hidden_parameters(self._h, out.data_ptr()))
        return out

    def set_hidden_parameters(self, hidden_parameters: torch.Tensor) -> None:
        n = self._lib.ab200_tile_hidden_parameter_count(self._h)
        if n == 0:
            return
        hp = hidden_parameters.detach().to(torch.float32).cpu().contiguous()
        if tuple(hp.shape) != (n, self.get_d_size(), self.get_x_size()):
            raise RuntimeError("Hidden parameter shape mismatch!")
        check(self._lib.ab200_tile_set_hidden_parameters(self._h, hp.data_ptr()))

    # -- the hot path ------------------------------------------------------------------------
    def forward(
        self, x_input: torch.Tensor, bias: bool = False, x_trans: bool = False,
        d_trans: bool = False, is_test: bool = False, non_blocking: bool = False,
    ) -> torch.Tensor:
        """rpu_base_tiles.cpp:405-445 / rpu_base_tiles_cuda.cpp:160-205."""
        x = _check_input(x_input, "x_input")
        if x.dim() < 1:
            raise RuntimeError("Invalid x_input dimensions: expected at least 1 dimensional tensor")
        in_size = x.size(0) if x_trans else x.size(-1)
        expected = self.get_x_size() - (1 if bias else 0)
        if in_size != expected:
            shape = f"[*, {expected}]" if x_trans else f"[{expected},*]"
            raise RuntimeError(f"Invalid x_input dimensions: expected {shape} tensor")
        m = x.numel() // in_size if in_size else 0
        dims = list(x.shape)
        if x_trans != d_trans:
            # mixed layouts: the reference binding keeps the input's leading dims, which only
            # fits when both flags agree; give the batch its own dimension instead
            dims = [self.get_d_size(), m] if d_trans else [m, self.get_d_size()]
        elif d_trans:
            dims[0] = self.get_d_size()
        else:
            dims[-1] = self.get_d_size()
        out = torch.empty(dims, dtype=torch.float32, device=x.device)
        self._sync_shared()
        if x.is_cuda:
            check(
                self._lib.ab200_tile_forward(
                    self._h, x.data_ptr(), out.data_ptr(), int(bias), m, int(x_trans), int(d_trans),
                    int(is_test), _stream_ptr(x),
                )
            )
            if not non_blocking:
                torch.cuda.current_stream(x.device).synchronize()
        else:
            check(
                self._lib.ab200_tile_forward_host(
                    self._h, x.data_ptr(), out.data_ptr(), int(bias), m, int(x_trans), int(d_trans),
                    int(is_test), None,
                )
            )
        return out

    def backward(
        self, d_input: torch.Tensor, bias: bool = False, d_trans: bool = False,
        x_trans: bool = False, non_blocking: bool = False,
    ) -> torch.Tensor:
        """rpu_base_tiles.cpp:473-512."""
        d = _check_input(d_input, "d_input")
        if d.dim() < 1:
            raise RuntimeError("Invalid d_input dimensions: expected at least 1 dimensional tensor")
        dsz = d.size(0) if d_trans else d.size(-1)
        if dsz != self.get_d_size():
            shape = f"[*, {self.get_d_size()}]" if d_trans else f"[{self.get_d_size()},*]"
            raise RuntimeError(f"Invalid d_input dimensions: expected {shape} tensor")
        m = d.numel() // dsz if dsz else 0
        x_out = self.get_x_size() - (1 if bias else 0)
        dims = list(d.shape)
        if x_trans != d_trans:
            dims = [x_out, m] if x_trans else [m, x_out]
        elif x_trans:
            dims[0] = x_out
        else:
            dims[-1] = x_out
        out = torch.empty(dims, dtype=torch.float32, device=d.device)
        self._sync_shared()
        if d.is_cuda:
            check(
                self._lib.ab200_tile_backward(
                    self._h, d.data_ptr(), out.data_ptr(), int(bias), m, int(d_trans), int(x_trans),
                    _stream_ptr(d),
                )
            )
            if not non_blocking:
                torch.cuda.current_stream(d.device).synchronize()
        else:
            check(
                self._lib.ab200_tile_backward_host(
                    self._h, d.data_ptr(), out.data_ptr(), int(bias), m, int(d_trans), int(x_trans), None
                )
            )
        return out

    def update(
        self, x_input: torch.Tensor, d_input: torch.Tensor, bias: bool = False,
        x_trans: bool = False, d_trans: bool = False, non_blocking: bool = False,
    ) -> None:
        """rpu_base_tiles.cpp:541-598 (4th / 5th positional arguments are x_trans, d_trans)."""
        x = _check_input(x_input, "x_input")
        d = _check_input(d_input, "d_input")
        in_size = x.size(0) if x_trans else x.size(-1)
        expected = self.get_x_size() - (1 if bias else 0)
        dsz = d.size(0) if d_trans else d.size(-1)
        if in_size != expected or dsz != self.get_d_size():
            raise RuntimeError("Invalid x_input / d_input dimensions for update")
        m = x.numel() // in_size if in_size else 0
        if m != (d.numel() // dsz if dsz else 0):
            raise RuntimeError("x_input and d_input need the same batch size")
        if x.is_cuda != d.is_cuda:
            raise RuntimeError("x_input and d_input need to live on the same device")
        if x.is_cuda:
            check(
                self._lib.ab200_tile_update(
                    self._h, x.data_ptr(), d.data_ptr(), int(bias), m, int(x_trans), int(d_trans),
                    _stream_ptr(x),
                )
            )
            if not non_blocking:
                torch.cuda.current_stream(x.device).synchronize()
        else:
            check(
                self._lib.ab200_tile_update_host(
                    self._h, x.data_ptr(), d.data_ptr(), int(bias), m, int(x_trans), int(d_trans), None
                )
            )

    # -- extra state, copies ---------------------------------------------------------------------
    def dump_extra(self) -> dict:
        """rpu_base_tiles.cpp ``dump_extra``: state besides weights and hidden parameters as
        ``{name: [values]}`` (learning rate, compound counters, noise key and call counters, and
        the chopper vectors of the chopped / dynamic transfer compounds)."""
        n = self._lib.ab200_tile_extra_count()
        values = (C.c_double * n)()
        check(self._lib.ab200_tile_dump_extra(self._h, values))
        out = {self._lib.ab200_tile_extra_name(k).decode(): [float(values[k])] for k in range(n)}
        for k in range(self._lib.ab200_tile_extra_vector_count(self._h)):
            size = self._lib.ab200_tile_extra_vector_size(self._h, k)
            vec = (C.c_double * size)()
            check(self._lib.ab200_tile_get_extra_vector(self._h, k, vec))
            out[self._lib.ab200_tile_extra_vector_name(self._h, k).decode()] = [float(v) for v in vec]
        return out

    def load_extra(self, extra: dict, strict: bool = False) -> None:
        """rpu_base_tiles.cpp ``load_extra``; with ``strict`` unknown or missing keys raise."""
        vectors = {self._lib.ab200_tile_extra_vector_name(self._h, k).decode(): k
                   for k in range(self._lib.ab200_tile_extra_vector_count(self._h))}
        names = [k for k in extra.keys() if k not in vectors]
        n = len(names)
        c_names = (C.c_char_p * max(n, 1))(*[k.encode() for k in names])
        c_vals = (C.c_double * max(n, 1))(*[float(extra[k][0] if isinstance(extra[k], (list, tuple)) else extra[k])
                                            for k in names])
        check(self._lib.ab200_tile_load_extra(self._h, c_names, c_vals, n, int(strict)))
        for name, k in vectors.items():
            if name not in extra:
                if strict:
                    raise RuntimeError(f"load_extra: key '{name}' is missing")
                continue
            vals = [float(v) for v in extra[name]]
            vec = (C.c_double * max(len(vals), 1))(*vals)
            check(self._lib.ab200_tile_set_extra_vector(self._h, k, vec, len(vals)))

    def __copy__(self):
        """A new tile with the same configuration, device parameters, weights and state
        (rpu_base_tiles.cpp ``__copy__`` / ``__deepcopy__``)."""
        other = type(self).__new__(type(self))
        AnalogTile.__init__(other, self._cfg, cuda_device=self._device_index)
        other._meta = self._meta
        # weights first: setting them resets a compound device's hidden tiles and counters
        other.set_weights(self.get_weights())
        if self.get_hidden_parameter_names():
            other.set_hidden_parameters(self.get_hidden_parameters())
        other.load_extra(self.dump_extra(), strict=True)
        return other

    def __deepcopy__(self, memo):
        return self.__copy__()

    # -- weight operations between updates -------------------------------------------------------
    def _op_stream(self):
        if self._device_index < 0:
            return None  # the library raises: no CPU compute path
        return int(torch.cuda.current_stream(torch.device("cuda", self._device_index)).cuda_stream)

    def decay_weights(self, alpha: float = 1.0) -> None:
        """rpu_base_tiles.cpp:277-292: ``W = (W - b) * (1 + alpha * (decay_scale - 1)) + b`` per
        element, clipped to the device bounds (floating-point tile: ``W *= 1 - alpha / lifetime``)."""
        check(self._lib.ab200_tile_decay_weights(self._h, float(alpha), 0, self._op_stream()))

    def diffuse_weights(self) -> None:
        """rpu_base_tiles.cpp:373-386: ``W += diffusion_rate * N(0, 1)`` per element, clipped."""
        check(self._lib.ab200_tile_diffuse_weights(self._h, self._op_stream()))

    def clip_weights(self, weight_clipper_params) -> None:
        """rpu_base_tiles.cpp:316-330; ``weight_clipper_params`` is a ``WeightClipParameter``."""
        check(self._lib.ab200_tile_clip_weights(
            self._h, int(weight_clipper_params.type), float(weight_clipper_params.fixed_value),
            float(weight_clipper_params.sigma), self._op_stream()))

    def reset_columns(self, start_column_idx: int = 0, num_columns: int = 1,
                      reset_prob: float = 1.0) -> None:
        """rpu_base_tiles.cpp:388-410: ``W_ij = xi * reset_std + reset_bias_ij`` for the given
        input columns (wrapping around), each element with probability ``reset_prob``."""
        check(self._lib.ab200_tile_reset_columns(self._h, int(start_column_idx), int(num_columns),
                                                 float(reset_prob), self._op_stream()))

    def set_weights_uniform_random(self, min_value: float, max_value: float) -> None:
        """rpu_base_tiles.cpp:263-275."""
        check(self._lib.ab200_tile_set_weights_uniform_random(self._h, float(min_value),
                                                              float(max_value), self._op_stream()))

    # -- indexed convolution interface ---------------------------------------------------------
    def set_matrix_indices(self, indices: torch.Tensor) -> None:
        """rpu_base_tiles.cpp ``set_matrix_indices``: int32 index tensor of a convolution
        (``AnalogConv2d._calculate_indexes``, nn/modules/conv.py:534-571).  The tile keeps its
        own copy."""
        if indices.dtype != torch.int32:
            raise RuntimeError("indices must be an int32 tensor")
        idx = indices.contiguous()
        stream = _stream_ptr(idx) if idx.is_cuda else None
        check(self._lib.ab200_tile_set_matrix_indices(self._h, idx.data_ptr(), idx.numel(), stream))

    def has_matrix_indices(self) -> bool:
        return bool(self._lib.ab200_tile_has_matrix_indices(self._h))

    def _indexed_dims(self, d: torch.Tensor):
        n = d.size(0)
        return n, d.numel() // (d.size(0) * d.size(1))

    def forward_indexed(self, x_input: torch.Tensor, d_tensor: torch.Tensor, is_test: bool = False,
                        non_blocking: bool = False) -> torch.Tensor:
        """rpu_base_tiles_cuda.cpp:399-432: ``x_input`` is ``[N, C, H, W]``, ``d_tensor`` the
        preallocated ``[N, d_size, H_out, W_out]`` result, which is filled and returned."""
        x = _check_input(x_input, "x_input")
        if not (x.is_cuda and d_tensor.is_cuda and d_tensor.is_contiguous()):
            raise RuntimeError("forward_indexed expects contiguous CUDA tensors")
        if d_tensor.size(1) != self.get_d_size() or d_tensor.size(0) != x.size(0):
            raise RuntimeError("d_tensor must be [N, d_size, ...]")
        n, d_image = self._indexed_dims(d_tensor)
        self._sync_shared()
        check(self._lib.ab200_tile_forward_indexed(
            self._h, x.data_ptr(), d_tensor.data_ptr(), x.numel(), d_image, n, 1, int(is_test),
            _stream_ptr(x)))
        if not non_blocking:
            torch.cuda.current_stream(x.device).synchronize()
        return d_tensor

    def backward_indexed(self, d_input: torch.Tensor, x_tensor: torch.Tensor,
                         non_blocking: bool = False) -> torch.Tensor:
        """rpu_base_tiles_cuda.cpp:444-477: ``d_input`` is ``[N, d_size, H_out, W_out]``,
        ``x_tensor`` the preallocated ``[N, C, H, W]`` result."""
        d = _check_input(d_input, "d_input")
        if not (d.is_cuda and x_tensor.is_cuda and x_tensor.is_contiguous()):
            raise RuntimeError("backward_indexed expects contiguous CUDA tensors")
        if d.size(1) != self.get_d_size() or d.size(0) != x_tensor.size(0):
            raise RuntimeError("d_input must be [N, d_size, ...]")
        n, d_image = self._indexed_dims(d)
        self._sync_shared()
        check(self._lib.ab200_tile_backward_indexed(
            self._h, d.data_ptr(), x_tensor.data_ptr(), x_tensor.numel(), d_image, n, 1,
            _stream_ptr(d)))
        if not non_blocking:
            torch.cuda.current_stream(d.device).synchronize()
        return x_tensor

    def update_indexed(self, x_input: torch.Tensor, d_input: torch.Tensor,
                       non_blocking: bool = False) -> None:
        """rpu_base_tiles_cuda.cpp:489-516."""
        x = _check_input(x_input, "x_input")
        d = _check_input(d_input, "d_input")
        if not (x.is_cuda and d.is_cuda):
            raise RuntimeError("update_indexed expects CUDA tensors")
        if d.size(1) != self.get_d_size() or d.size(0) != x.size(0):
            raise RuntimeError("d_input must be [N, d_size, ...]")
        n, d_image = self._indexed_dims(d)
        check(self._lib.ab200_tile_update_indexed(
            self._h, x.data_ptr(), d.data_ptr(), x.numel(), d_image, n, 1, _stream_ptr(x)))
        if not non_blocking:
            torch.cuda.current_stream(x.device).synchronize()

    # -- diagnostics -------------------------------------------------------------------------
    def coincidences(self, x: torch.Tensor, d: torch.Tensor) -> torch.Tensor:
        """Signed coincidence counts ``[d_size, x_size]`` (int32) of one sample."""
        x = _check_input(x, "x").reshape(-1)
        d = _check_input(d, "d").reshape(-1)
        if x.numel() != self.get_x_size() or d.numel() != self.get_d_size() or not x.is_cuda:
            raise RuntimeError("coincidences expects CUDA vectors of size x_size and d_size")
        out = torch.empty(self.get_d_size(), self.get_x_size(), dtype=torch.int32, device=x.device)
        check(
            self._lib.ab200_tile_coincidences(
                self._h, x.data_ptr(), d.data_ptr(), out.data_ptr(), _stream_ptr(x)
            )
        )
        torch.cuda.current_stream(x.device).synchronize()
        return out

    def last_bm_stats(self):
        n = C.c_int32()
        r = C.c_float()
        check(self._lib.ab200_tile_last_bm_stats(self._h, C.byref(n), C.byref(r)))
        return int(n.value), float(r.value)

    def get_brief_info(self) -> str:
        return f"{type(self).__name__}(B200, {self.get_d_size()}x{self.get_x_size()})"

    def get_info(self) -> str:
        """rpu_base_tiles.cpp:71-78: a printable summary of the tile's parameters."""
        lines = [self.get_brief_info(), f"  learning_rate: {self.get_learning_rate()}"]
        if self._meta is not None:
            for part in ("forward_io", "backward_io", "update"):
                sub = getattr(self._meta, part, None)
                if sub is not None:
                    lines.append(f"  {part}: " + ", ".join(
                        f"{k}={getattr(v, 'name', v)}" for k, v in vars(sub).items() if not k.startswith("_")))
        return "\n".join(lines) + "\n"

    __str__ = get_brief_info

    def get_meta_parameters(self):
        """rpu_base_tiles.cpp:258 / :886: the meta parameters the tile was created from."""
        if self._meta is None:
            from . import devices

            return devices.AnalogTileParameter()
        return self._meta

    def set_verbosity_level(self, verbose: int) -> None:
        """rpu_base_tiles.cpp:115: the B200 tile prints nothing at any level."""
        self._verbose = int(verbose)

    def get_hidden_update_index(self) -> int:
        """rpu_base_tiles.cpp:838-845: which device of a compound receives the gradient update;
        the Transfer compound updates its first (fast) device, single devices have index 0."""
        return int(self._hidden_update_index)

    def set_hidden_update_index(self, index: int) -> None:
        """rpu_base_tiles.cpp:827-837."""
        if int(index) != 0:
            raise RuntimeError("hidden update index: only the first device of a compound is updated "
                               "by the B200 analog tile")
        self._hidden_update_index = 0

    def get_pulse_counters(self) -> torch.Tensor:
        """rpu_base_tiles.cpp:846-868: int64 ``[2, d_size, x_size]`` (pulses up, pulses down) of a
        device made with ``count_pulses``; empty otherwise."""
        if not self._lib.ab200_tile_counts_pulses(self._h):
            return torch.zeros(0, dtype=torch.int64)
        out = torch.empty(2, self.get_d_size(), self.get_x_size(), dtype=torch.int64)
        check(self._lib.ab200_tile_get_pulse_counters(self._h, out.data_ptr()))
        return out

    def drift_weights(self, time_since_last_call: float) -> None:
        """rpu_base_tiles.cpp:294-314 (power-law drift, src/rpucuda/rpu.cpp:1581-1587,
        rpu_pulsed.cpp:226-229)."""
        check(self._lib.ab200_tile_drift_weights(self._h, float(time_since_last_call),
                                                 self._op_stream()))

    def remap_weights(self, weight_remap_params, scales: torch.Tensor,
                      biases: Optional[torch.Tensor] = None) -> torch.Tensor:
        """rpu_base_tiles.cpp:331-356 (WeightRemapper::apply, src/rpucuda/weight_remapper.cpp):
        rescale the weights so that their largest magnitude - of the whole tile, or per output
        row - becomes ``remapped_wmax``, and move the factor into ``scales`` (one per output)."""
        kind = int(weight_remap_params.type)
        if kind == int(WeightRemapType.None_):
            return scales
        if biases is not None:
            raise RuntimeError("remap_weights with biases is not implemented")
        if self._device_index < 0:
            raise RuntimeError("remap_weights: the analog tile has no CPU compute path")
        dev = torch.device("cuda", self._device_index)
        w = self._shared if self._shared is not None else self.get_weights_cuda()  # [x, d]
        scales_dev = scales.to(dev, torch.float32)
        amax = w.abs().amax(dim=0)  # per output row
        max_range = float(weight_remap_params.max_scale_range)
        if kind == int(WeightRemapType.LayerwiseSymmetric):
            amax = (amax.max() / float(weight_remap_params.remapped_wmax)).expand_as(amax)
            max_range = 0.0
        elif max_range <= 0:
            amax = amax / float(weight_remap_params.remapped_wmax)
        elif float(weight_remap_params.remapped_wmax) != 1.0:
            raise RuntimeError("For max_scales set, expect wrmpar.remapped_wmax to be 1.")
        factor = torch.where(amax > 0, amax, torch.ones_like(amax))
        new_scales = scales_dev * factor
        if max_range > 0:
            # the range of the scales is limited relative to the smallest old scale
            # (weight_remapper.cpp: min_scale, max_scale_ref)
            min_scale = max(float(scales_dev.min()), 0.0)
            ref = float(weight_remap_params.max_scale_ref)
            if min_scale > 0 and ref:
                min_scale = max(min_scale, ref)
            if min_scale > 0:
                new_scales = torch.minimum(new_scales, torch.full_like(new_scales, min_scale * max_range))
            factor = new_scales / scales_dev
        w_new = w / factor[None, :]
        if self._shared is not None:
            self._shared.copy_(w_new)
            self._sync_shared()
        else:
            self.set_weights_cuda(w_new.contiguous())
        scales.copy_(new_scales.to(scales.device))
        return scales

    def get_io_vector(self, backward: bool, which: int) -> torch.Tensor:
        """Per-line values of one IO direction: 0 voltage offsets, 1 output non-linearities,
        2 output-noise values (part of ``dump_extra`` in the reference as ``fwd.v_offset`` ...,
        src/rpucuda/rpu_forward_backward_pass.cpp:63-82). Device tiles only."""
        n = self.get_x_size() if backward else self.get_d_size()
        out = torch.empty(n, dtype=torch.float32)
        check(self._lib.ab200_tile_get_io_vector(self._h, int(bool(backward)), int(which), out.data_ptr(), n))
        return out

    def set_io_vector(self, backward: bool, which: int, values: torch.Tensor) -> None:
        v = values.detach().to(dtype=torch.float32, device="cpu").contiguous()
        check(self._lib.ab200_tile_set_io_vector(self._h, int(bool(backward)), int(which), v.data_ptr(),
                                                 v.numel()))

    def modify_weights(self, weight_modifier_params) -> None:
        """rpu_base_tiles.cpp:358-371 (WeightModifier, src/rpucuda/weight_modifier.cpp)."""
        if int(weight_modifier_params.type) != int(WeightModifierType.Copy) and \
                bool(weight_modifier_params.per_batch_sample):
            raise RuntimeError("Per batch sample is not implemented in RPUCuda")  # weight_modifier.cpp:36-38
        c = weight_modifier_params._to_c()
        check(self._lib.ab200_tile_modify_weights(self._h, C.byref(c), self._op_stream()))


class FloatingPointTile(AnalogTile):
    """``tiles.FloatingPointTile`` (RPUSimple): perfect IO and floating-point update."""

    def __init__(self, x_size: int, d_size: int, cuda_device: int = -1, lifetime: float = 0.0,
                 diffusion: float = 0.0, drift=None):
        from . import devices

        par = devices.AnalogTileParameter()
        par.forward_io.is_perfect = True
        par.backward_io.is_perfect = True
        par.update.pulse_type = devices.PulseType.None_
        dev = devices.IdealResistiveDeviceParameter()
        dev.lifetime, dev.diffusion = lifetime, diffusion
        if drift is not None:
            dev.drift = drift
        cfg = par._config(x_size, d_size, dev)
        super().__init__(cfg, cuda_device)
        self._meta = par


def _device_index(device) -> int:
    if device is None:
        return torch.cuda.current_device() if torch.cuda.is_available() else 0
    if isinstance(device, int):
        return device
    index = torch.device(device).index
    return torch.cuda.current_device() if index is None else index


def _take_over(new: AnalogTile, tile: AnalogTile, device) -> None:
    """Build ``new`` as the device copy of the host tile ``tile``: same configuration, weights
    (from the shared host tensor when there is one), per-element parameters and extra state."""
    if not isinstance(tile, AnalogTile):
        raise RuntimeError("a CUDA tile is constructed from a host tile of this module")
    AnalogTile.__init__(new, tile._cfg, cuda_device=_device_index(device))
    new._meta = tile._meta
    new.set_weights(tile.get_weights())
    if tile.get_hidden_parameter_names():
        new.set_hidden_parameters(tile.get_hidden_parameters())
    new.load_extra(tile.dump_extra(), strict=True)


class CudaAnalogTile(AnalogTile):
    """``tiles.CudaAnalogTile(cpu_tile)`` (rpu_base_tiles_cuda.cpp:524-543): the tile on the
    current CUDA device, built from a host tile that carries configuration, weights and the
    host-drawn per-element parameters."""

    def __init__(self, tile: AnalogTile, device=None):
        _take_over(self, tile, device)


class CudaFloatingPointTile(FloatingPointTile):
    """``tiles.CudaFloatingPointTile(cpu_tile)`` (rpu_base_tiles_cuda.cpp:45-58)."""

    def __init__(self, tile: AnalogTile, device=None):
        _take_over(self, tile, device)


class TileArray:
    """Native mapped-tile layer (``TileModuleArray``, src/aihwkit/simulator/tiles/array.py:30-198).

    ``in_split_range`` / ``out_split_range`` select the in-splits and out-splits this process
    materialises (a shard of the layer: the partial sums of the shards add up to the layer's
    output; a shard writes zeros outside its own output columns)."""

    def __init__(self, config: _cabi.TileConfig, out_size: int, in_size: int,
                 max_output_size: int, max_input_size: int, cuda_device: int = 0,
                 in_split_range=None, out_split_range=None):
        self._lib = _cabi.lib()
        self.out_size, self.in_size = int(out_size), int(in_size)
        begin, end = (0, -1) if in_split_range is None else in_split_range
        obegin, oend = (0, -1) if out_split_range is None else out_split_range
        h = C.c_void_p()
        check(
            self._lib.ab200_array_create_block(
                C.byref(config), self.out_size, self.in_size, int(max_output_size),
                int(max_input_size), int(begin), int(end), int(obegin), int(oend),
                int(cuda_device), C.byref(h),
            )
        )
        self._h = h
        self._n_local_in = None if in_split_range is None else max(0, int(end) - int(begin))
        self.device = torch.device("cuda", int(cuda_device))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ab200_array_destroy(h)

    @property
    def num_in_splits(self) -> int:
        return int(self._lib.ab200_array_num_in_splits(self._h))

    @property
    def num_out_splits(self) -> int:
        return int(self._lib.ab200_array_num_out_splits(self._h))

    def set_seed(self, seed: int) -> None:
        check(self._lib.ab200_array_set_seed(self._h, int(seed)))

    def set_weights(self, weight: torch.Tensor, weight_scaling_omega: float = 0.0) -> None:
        """Logical ``[out_size, in_size]`` weights.  With ``weight_scaling_omega > 0`` every tile
        stores ``w / alpha`` with ``alpha = max|w_tile| / omega`` and applies ``alpha`` to its
        output in digital, inside the layer's kernels (the layer-wise weight scaling of
        ``TileWithPeriphery.apply_weight_scaling``, tiles/periphery.py:437-500)."""
        w = weight.detach().to(torch.float32).cpu().reshape(self.out_size, self.in_size).contiguous()
        check(self._lib.ab200_array_set_weights_scaled(self._h, w.data_ptr(), float(weight_scaling_omega)))

    def set_learning_rate(self, lr: float) -> None:
        check(self._lib.ab200_array_set_learning_rate(self._h, float(lr)))

    def backward(self, d_input: torch.Tensor, non_blocking: bool = False) -> torch.Tensor:
        """Gradient with respect to the layer input, ``[m, in_size]``: every tile's IO-managed
        backward MVM on its block of ``d_input`` (``[m, out_size]``, times the tile's mapping
        scale), summed over the out-splits."""
        d = _check_input(d_input, "d_input")
        if not d.is_cuda or d.size(-1) != self.out_size:
            raise RuntimeError(f"expected a CUDA [*, {self.out_size}] tensor")
        m = d.numel() // self.out_size
        out = torch.zeros(list(d.shape[:-1]) + [self.in_size], dtype=torch.float32, device=d.device)
        check(self._lib.ab200_array_backward(self._h, d.data_ptr(), out.data_ptr(), m, _stream_ptr(d)))
        if not non_blocking:
            torch.cuda.current_stream(d.device).synchronize()
        return out

    def update(self, x_input: torch.Tensor, d_input: torch.Tensor, non_blocking: bool = False) -> None:
        """Pulsed (or floating-point) update of every tile with its block of the activations and
        of the gradients (divided by the tile's mapping scale)."""
        x = _check_input(x_input, "x_input")
        d = _check_input(d_input, "d_input")
        if not (x.is_cuda and d.is_cuda) or x.size(-1) != self.in_size or d.size(-1) != self.out_size:
            raise RuntimeError("expected CUDA tensors [*, in_size] and [*, out_size]")
        m = x.numel() // self.in_size
        if m != d.numel() // self.out_size:
            raise RuntimeError("x_input and d_input need the same batch size")
        check(self._lib.ab200_array_update(self._h, x.data_ptr(), d.data_ptr(), m, _stream_ptr(x)))
        if not non_blocking:
            torch.cuda.current_stream(x.device).synchronize()

    def get_tile_scales(self) -> torch.Tensor:
        """Digital output scales of the locally owned tiles ``[in-splits, out-splits]``."""
        n_in = self.num_in_splits if self._n_local_in is None else self._n_local_in
        sc = torch.ones(max(n_in, 1) * self.num_out_splits, dtype=torch.float32)
        check(self._lib.ab200_array_get_tile_scales(self._h, sc.data_ptr()))
        return sc.reshape(-1, self.num_out_splits)[:n_in]

    def set_bias(self, bias: Optional[torch.Tensor]) -> None:
        """Digital bias ``[out_size]`` added after the sum over in-splits
        (``TileModuleArray.forward``, tiles/array.py:178-181); ``None`` removes it."""
        if bias is None:
            check(self._lib.ab200_array_set_bias(self._h, None))
            return
        b = bias.detach().to(torch.float32).cpu().reshape(self.out_size).contiguous()
        check(self._lib.ab200_array_set_bias(self._h, b.data_ptr()))

    def get_weights(self) -> torch.Tensor:
        w = torch.zeros(self.out_size, self.in_size, dtype=torch.float32)
        check(self._lib.ab200_array_get_weights(self._h, w.data_ptr()))
        return w

    @property
    def local_in_size(self) -> int:
        """Number of input columns covered by the in-splits this object owns."""
        return int(self._lib.ab200_array_local_in_size(self._h))

    def forward_local(self, x_local: torch.Tensor, out: Optional[torch.Tensor] = None,
                      is_test: bool = True) -> torch.Tensor:
        """Forward on a CUDA input that holds only this object's own input columns
        ``[m, local_in_size]``; asynchronous on the current stream."""
        x = _check_input(x_local, "x_local")
        if not x.is_cuda or x.dim() != 2 or x.size(1) != self.local_in_size:
            raise RuntimeError(f"expected a CUDA [m, {self.local_in_size}] tensor")
        if out is None:
            out = torch.empty(x.size(0), self.out_size, dtype=torch.float32, device=x.device)
        check(self._lib.ab200_array_forward_local(self._h, x.data_ptr(), out.data_ptr(), x.size(0),
                                                  int(is_test), _stream_ptr(x)))
        return out

    def forward_scatter(self, x_local: torch.Tensor, out_table: torch.Tensor, rows_per_owner: int,
                        rotate_rows: int = 0) -> None:
        """Forward on this object's own input columns with the output rows written straight to
        the buffers of their owners: ``out_table`` is a CUDA int64 tensor of device pointers (one
        per owner, local or peer memory, row pitch ``out_size``); row ``r`` goes to owner
        ``r // rows_per_owner``.  Asynchronous on the current stream."""
        x = _check_input(x_local, "x_local")
        if not x.is_cuda or x.dim() != 2 or x.size(1) != self.local_in_size:
            raise RuntimeError(f"expected a CUDA [m, {self.local_in_size}] tensor")
        if not out_table.is_cuda or out_table.dtype != torch.int64 or not out_table.is_contiguous():
            raise RuntimeError("out_table must be a contiguous CUDA int64 tensor of device pointers")
        check(self._lib.ab200_array_forward_scatter(
            self._h, x.data_ptr(), x.size(0), out_table.data_ptr(), out_table.numel(),
            int(rows_per_owner), int(rotate_rows), _stream_ptr(x)))

    def forward_scatter_plan(self, x_local: torch.Tensor, plan) -> None:
        """General scatter forward (``ab200_array_forward_scatter_plan``): ``plan`` is an
        ``aihwkit_b200._cabi.ScatterPlan`` with the owners' buffer tables, the row of the whole
        batch this launch starts at, the owner layout (contiguous or dealt in blocks) and the
        completion flags.  Asynchronous on the current stream."""
        import ctypes as C

        x = _check_input(x_local, "x_local")
        if not x.is_cuda or x.dim() != 2 or x.size(1) != self.local_in_size:
            raise RuntimeError(f"expected a CUDA [m, {self.local_in_size}] tensor")
        check(self._lib.ab200_array_forward_scatter_plan(self._h, x.data_ptr(), x.size(0),
                                                         C.byref(plan), _stream_ptr(x)))

    def scatter_codes_supported(self) -> bool:
        """Whether :meth:`forward_scatter_codes` can be used: noisy inference settings whose ADC
        codes fit a signed byte, no bound management, out-splits in multiples of 128, no mapping
        scales or bias on this object."""
        return bool(self._lib.ab200_array_scatter_codes_supported(self._h))

    def forward_scatter_codes(self, x_local: torch.Tensor, code_table: torch.Tensor,
                              fac_table: torch.Tensor, rows_per_owner: int,
                              rotate_rows: int = 0) -> None:
        """Like :meth:`forward_scatter`, but every in-split's integer ADC code (one byte per
        element) is written to the owners instead of the fp32 sum over the in-splits, together
        with the per-row factors; the owner multiplies and sums
        (``ab200_sum_code_slots``).  ``code_table`` / ``fac_table``: CUDA int64 tensors of device
        pointers, one per owner."""
        x = _check_input(x_local, "x_local")
        if not x.is_cuda or x.dim() != 2 or x.size(1) != self.local_in_size:
            raise RuntimeError(f"expected a CUDA [m, {self.local_in_size}] tensor")
        for t in (code_table, fac_table):
            if not t.is_cuda or t.dtype != torch.int64 or not t.is_contiguous():
                raise RuntimeError("pointer tables must be contiguous CUDA int64 tensors")
        if code_table.numel() != fac_table.numel():
            raise RuntimeError("code_table and fac_table need one pointer per owner each")
        check(self._lib.ab200_array_forward_scatter_codes(
            self._h, x.data_ptr(), x.size(0), code_table.data_ptr(), fac_table.data_ptr(),
            code_table.numel(), int(rows_per_owner), int(rotate_rows), _stream_ptr(x)))

    def forward(self, x_input: torch.Tensor, is_test: bool = True, non_blocking: bool = False,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x_input`` on the GPU: kernels only.  ``x_input`` on the CPU: the library pipelines
        host->device copies, kernels and device->host copies over row chunks; page-locked
        tensors (``pin_memory()``) are copied directly, and ``out`` lets the caller provide a
        page-locked result tensor."""
        x = _check_input(x_input, "x_input")
        if x.size(-1) != self.in_size:
            raise RuntimeError(f"Invalid x_input dimensions: expected [{self.in_size},*] tensor")
        m = x.numel() // self.in_size
        shape = list(x.shape[:-1]) + [self.out_size]
        if out is None:
            out = torch.empty(shape, dtype=torch.float32, device=x.device)
        elif (list(out.shape) != shape or out.dtype != torch.float32 or out.device != x.device
              or not out.is_contiguous()):
            raise RuntimeError("out must be a contiguous float32 tensor of the result shape on x's device")
        if x.is_cuda:
            check(self._lib.ab200_array_forward(self._h, x.data_ptr(), out.data_ptr(), m, int(is_test), _stream_ptr(x)))
            if not non_blocking:
                torch.cuda.current_stream(x.device).synchronize()
        else:
            check(self._lib.ab200_array_forward_host(self._h, x.data_ptr(), out.data_ptr(), m, int(is_test), None))
        return out
