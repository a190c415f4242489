"""The compiled pybind11 / torch binding over the C ABI (aihwkit_b200/csrc/pybind_module.cpp: the
stub a maintainer of the reference links in place of its own tile classes) against the ctypes
mirror of the same library: one training step of benchmark configuration 0's tile, bit for bit."""

import importlib.util
import os

import numpy as np
import pytest
import torch

from tests import helpers as H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _module():
    so = os.path.join(ROOT, "aihwkit_b200", "csrc", "build_pybind", "ab200_pybind.so")
    if os.path.exists(so):
        spec = importlib.util.spec_from_file_location("ab200_pybind", so)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    from aihwkit_b200 import build as b

    return b.build_pybind()


def test_binding_is_built_and_links_the_library():
    mod = _module()
    assert mod.version().startswith("aihwkit_b200")
    for name in ("forward", "backward", "update", "set_weights", "get_weights", "get_hidden_parameters",
                 "set_hidden_parameters", "set_learning_rate"):
        assert hasattr(mod.CudaAnalogTile, name)
    p = H.training_params(noise=False, pulse_det=True)
    with pytest.raises(RuntimeError, match="size mismatch"):
        mod.CudaAnalogTile(b"too short", 0)
    if not torch.cuda.is_available():
        cfg = p._config(8, 4, H.device("cs", False), seed=1)
        with pytest.raises(RuntimeError):
            mod.CudaAnalogTile(bytes(cfg), 0)  # no device: the library refuses, it has no CPU path


@pytest.mark.gpu
@pytest.mark.parametrize("noise", [False, True])
def test_binding_equals_ctypes_mirror(noise):
    from aihwkit_b200.rpu_base import tiles as T

    mod = _module()
    rng = np.random.default_rng(3)
    x_size, d_size, m = 256, 256, 64
    p = H.training_params(noise=noise, pulse_det=not noise)
    cfg = p._config(x_size, d_size, H.device("cs", noise), seed=7)
    a = mod.CudaAnalogTile(bytes(cfg), 0)
    b = T.AnalogTile(cfg, cuda_device=0)
    assert (a.get_x_size(), a.get_d_size()) == (x_size, d_size)
    assert a.get_hidden_parameter_names() == b.get_hidden_parameter_names()
    assert torch.equal(a.get_hidden_parameters(), b.get_hidden_parameters())
    W = torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    a.set_weights(W)
    b.set_weights(W)
    x = torch.from_numpy(rng.uniform(-1, 1, (m, x_size)).astype(np.float32)).cuda()
    d = torch.from_numpy(rng.normal(0, 0.1, (m, d_size)).astype(np.float32)).cuda()
    # same seed, same call counters: the two front ends drive the same kernels
    assert torch.equal(a.forward(x), b.forward(x))
    assert torch.equal(a.backward(d), b.backward(d))
    assert torch.equal(a.forward(x.t().contiguous(), x_trans=True, d_trans=True),
                       b.forward(x.t().contiguous(), False, True, True))
    a.set_learning_rate(0.01)
    b.set_learning_rate(0.01)
    assert a.get_learning_rate() == pytest.approx(0.01)
    a.update(x, d)
    b.update(x, d)
    wa, wb = a.get_weights(), b.get_weights()
    assert torch.equal(wa, wb) and float((wa - torch.clamp(W, -0.6, 0.6)).abs().max()) > 0
    with pytest.raises(RuntimeError, match="size mismatch"):
        a.forward(x[:, :10].contiguous())
