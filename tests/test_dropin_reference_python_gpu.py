"""The reference's own Python package (``aihwkit.nn``, ``aihwkit.optim``, ``aihwkit.simulator.tiles``,
staged unmodified under oracle/_ref/python by ``make -C oracle python``) running on top of this
repository's tiles registered as ``aihwkit.simulator.rpu_base``: AnalogLinear / AnalogConv2d /
AnalogSGD drive the sm_100a kernels through the reference's wrappers, and the numbers are checked
against the oracle and against digital torch layers."""

import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_PY = os.path.join(ROOT, "oracle", "_ref", "python")


@pytest.fixture(scope="module")
def aihwkit():
    if not os.path.isdir(os.path.join(REF_PY, "aihwkit")):
        pytest.skip("the reference's Python package is not staged (make -C oracle python)")
    import aihwkit_b200.dropin

    aihwkit_b200.dropin.install()
    if REF_PY not in sys.path:
        sys.path.insert(0, REF_PY)
    import aihwkit as pkg
    import aihwkit.simulator  # noqa: F401  (the parent package first: its rpu_base is the registered one)
    from aihwkit.simulator import rpu_base as rb

    assert rb.__name__ == "aihwkit_b200.rpu_base" and rb.cuda.is_compiled()
    return pkg


def _quiet_io(io, adc=True):
    io.out_noise = 0.0
    io.w_noise = 0.0
    io.inp_noise = 0.0
    if not adc:
        io.inp_res = io.out_res = -1.0


def test_analog_linear_trains_with_analog_sgd(aihwkit):
    """SingleRPUConfig / ConstantStep, the training configuration of the benchmarks at 256 x 256:
    the reference's AnalogLinear forward equals the oracle on the tile's weights, its backward and
    pulsed update run through AnalogSGD, and the loss of a small regression falls."""
    from aihwkit.nn import AnalogLinear
    from aihwkit.optim import AnalogSGD
    from aihwkit.simulator.configs import SingleRPUConfig, ConstantStepDevice
    from aihwkit.simulator.parameters.enums import BoundManagementType, NoiseManagementType
    from oracle import analog_tile_oracle as O

    torch.manual_seed(0)
    cfg = SingleRPUConfig(device=ConstantStepDevice(dw_min=0.001, dw_min_dtod=0.3, dw_min_std=0.3,
                                                    up_down_dtod=0.01, w_max=0.6, w_min=-0.6))
    for io in (cfg.forward, cfg.backward):
        _quiet_io(io)
        io.noise_management = NoiseManagementType.ABS_MAX
    cfg.forward.bound_management = BoundManagementType.ITERATIVE
    cfg.mapping.weight_scaling_omega = 0.0
    cfg.mapping.learn_out_scaling = False
    model = AnalogLinear(256, 256, bias=False, rpu_config=cfg).cuda()
    tile_module = next(model.analog_tiles())
    assert type(tile_module.tile).__name__ == "CudaAnalogTile"
    x = torch.rand(64, 256, device="cuda") * 2 - 1
    y = model(x)
    w = tile_module.tile.get_weights().numpy()
    from aihwkit_b200.rpu_base import devices as D

    io_c = tile_module.tile.get_meta_parameters().forward_io._to_c()
    y_or, _, scale, _ = O.forward(w, x.cpu().numpy(), O.IO.from_c(io_c), return_pre_adc=True)
    lsb = (O.IO.from_c(io_c).res_out / scale)[:, None]
    diff = np.abs(y.detach().cpu().numpy() - y_or)
    assert (diff > 1e-3 * lsb).mean() <= 2e-3 and diff.max() <= 1.001 * lsb.max()

    teacher = torch.randn(256, 256, device="cuda") * 0.1
    target = x @ teacher.t()
    opt = AnalogSGD(model.parameters(), lr=0.1)
    opt.regroup_param_groups(model)
    losses = []
    for _ in range(30):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(model(x), target)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < 0.95 * losses[0] and losses[-1] < losses[10] < losses[0], losses
    w_after = tile_module.tile.get_weights().numpy()
    assert np.abs(w_after - w).max() > 0 and np.abs(w_after).max() <= 0.6 * 3  # bounds vary per device


def test_inference_layer_mapped_forward_and_hwa_update(aihwkit):
    """InferenceRPUConfig on a 1024 x 1024 layer mapped to four 512 x 512 tiles by the reference's
    TileModuleArray: forward against the array oracle; one hardware-aware training step (the
    gradient goes through set_delta_weights + floating-point update into torch's grad) against a
    digital linear layer with the same weights."""
    from aihwkit.nn import AnalogLinear
    from aihwkit.optim import AnalogSGD
    from aihwkit.simulator.configs import InferenceRPUConfig
    from aihwkit.simulator.parameters.enums import BoundManagementType, NoiseManagementType
    from oracle import analog_tile_oracle as O
    from aihwkit_b200.sharded import split_sizes

    torch.manual_seed(1)
    cfg = InferenceRPUConfig()
    _quiet_io(cfg.forward)
    cfg.forward.inp_res = cfg.forward.out_res = 1.0 / 254.0
    cfg.forward.out_bound = 10.0
    cfg.forward.noise_management = NoiseManagementType.ABS_MAX
    cfg.forward.bound_management = BoundManagementType.NONE
    cfg.mapping.max_input_size = cfg.mapping.max_output_size = 512
    cfg.mapping.weight_scaling_omega = 0.0
    cfg.mapping.learn_out_scaling = False
    cfg.mapping.digital_bias = True
    model = AnalogLinear(1024, 1024, bias=True, rpu_config=cfg).cuda()
    assert len(list(model.analog_tiles())) == 4
    w, b = model.get_weights()
    x = torch.randn(300, 1024, device="cuda")
    model.eval()
    y = model(x).detach().cpu().numpy()
    # the array oracle: per-tile analog MVM, sum over in-splits after each tile's ADC, digital bias
    tile0 = next(model.analog_tiles()).tile
    io = O.IO.from_c(tile0.get_meta_parameters().forward_io._to_c())
    w, b = w.cpu(), b.cpu()
    W, X = w.numpy(), x.cpu().numpy()
    y_or = np.zeros((300, 1024), np.float32)
    lsb = np.zeros_like(y_or)
    c0 = 0
    for isz in split_sizes(1024, 512):
        r0 = 0
        for osz in split_sizes(1024, 512):
            yt, _, scale, _ = O.forward(W[r0:r0 + osz, c0:c0 + isz], X[:, c0:c0 + isz], io, return_pre_adc=True)
            y_or[:, r0:r0 + osz] += yt
            lsb[:, r0:r0 + osz] = np.maximum(lsb[:, r0:r0 + osz], (io.res_out / scale)[:, None])
            r0 += osz
        c0 += isz
    y_or += b.numpy()[None, :]
    diff = np.abs(y - y_or)
    assert (diff > 1e-3 * lsb).mean() <= 4e-3 and (diff <= 2.002 * lsb).all()

    # hardware-aware training step: perfect backward, gradient d^T x into the shared weights' grad
    model.train()
    ref = torch.nn.Linear(1024, 1024, bias=True).cuda()
    with torch.no_grad():
        ref.weight.copy_(w.cuda())
        ref.bias.copy_(b.cuda())
    opt = AnalogSGD(model.parameters(), lr=0.05)
    opt.regroup_param_groups(model)
    xs = torch.randn(64, 1024, device="cuda")
    target = torch.randn(64, 1024, device="cuda")
    opt.zero_grad()
    out = model(xs)
    grad_out = 2.0 * (out.detach() - target) / out.numel()
    torch.nn.functional.mse_loss(out, target).backward()
    opt.step()
    w2, b2 = model.get_weights()
    # the same step on the digital layer with the analog layer's output gradient
    expected_w = w.cuda() - 0.05 * grad_out.t() @ xs
    expected_b = b.cuda() - 0.05 * grad_out.sum(0)
    assert torch.allclose(w2.cuda(), expected_w, atol=2e-5, rtol=1e-4)
    assert torch.allclose(b2.cuda(), expected_b, atol=2e-5, rtol=1e-4)
    assert float((w2.cpu() - w).abs().max()) > 0


def test_analog_conv2d_indexed_path(aihwkit):
    """AnalogConv2d of the reference feeds the tile through set_matrix_indices / forward_indexed /
    backward_indexed / update_indexed; with perfect IO and a floating-point device the layer equals
    torch's convolution and an SGD step on it."""
    from aihwkit.nn import AnalogConv2d
    from aihwkit.optim import AnalogSGD
    from aihwkit.simulator.configs import FloatingPointRPUConfig

    torch.manual_seed(2)
    cfg = FloatingPointRPUConfig()
    cfg.mapping.weight_scaling_omega = 0.0
    cfg.mapping.learn_out_scaling = False
    conv = AnalogConv2d(8, 16, 3, padding=1, bias=False, rpu_config=cfg, use_indexed=True).cuda()
    w, _ = conv.get_weights()
    ref = torch.nn.Conv2d(8, 16, 3, padding=1, bias=False).cuda()
    with torch.no_grad():
        ref.weight.copy_(w.reshape(16, 8, 3, 3).cuda())
    x = torch.randn(4, 8, 12, 12, device="cuda")
    tf32 = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        y, y_ref = conv(x), ref(x)
        assert torch.allclose(y, y_ref, atol=1e-4, rtol=1e-4)
        opt = AnalogSGD(conv.parameters(), lr=0.1)
        opt.regroup_param_groups(conv)
        opt_ref = torch.optim.SGD(ref.parameters(), lr=0.1)
        x2 = x.clone().requires_grad_(True)
        x3 = x.clone().requires_grad_(True)
        opt.zero_grad()
        opt_ref.zero_grad()
        conv(x2).square().mean().backward()
        ref(x3).square().mean().backward()
        assert torch.allclose(x2.grad, x3.grad, atol=1e-5, rtol=1e-3)
        opt.step()
        opt_ref.step()
    finally:
        torch.backends.cudnn.allow_tf32 = tf32
    w_new, _ = conv.get_weights()
    assert torch.allclose(w_new.reshape(16, 8, 3, 3).cuda(), ref.weight.detach(), atol=1e-5, rtol=1e-4)


def test_tiki_taka_tile_through_reference_wrappers(aihwkit):
    """UnitCellRPUConfig with a TransferCompound of two SoftBoundsReference devices: the wrappers
    build the tile, expose its hidden parameters by the reference's names and update it."""
    from aihwkit.nn import AnalogLinear
    from aihwkit.optim import AnalogSGD
    from aihwkit.simulator.configs import UnitCellRPUConfig
    from aihwkit.simulator.configs.compounds import TransferCompound
    from aihwkit.simulator.configs.devices import SoftBoundsReferenceDevice

    torch.manual_seed(3)
    dev = TransferCompound(
        unit_cell_devices=[SoftBoundsReferenceDevice(dw_min=0.002, w_max=1.0, w_min=-1.0, reference_std=0.05)
                           for _ in range(2)],
        transfer_every=2, n_reads_per_transfer=1, transfer_lr=0.01, gamma=0.0)
    cfg = UnitCellRPUConfig(device=dev)
    cfg.mapping.weight_scaling_omega = 0.0
    cfg.mapping.learn_out_scaling = False
    model = AnalogLinear(64, 32, bias=False, rpu_config=cfg).cuda()
    tm = next(model.analog_tiles())
    hidden = tm.get_hidden_parameters()
    assert "hidden_weights_0" in hidden and "max_bound_1" in hidden
    opt = AnalogSGD(model.parameters(), lr=0.1)
    opt.regroup_param_groups(model)
    x = torch.rand(16, 64, device="cuda")
    for _ in range(4):
        opt.zero_grad()
        model(x).square().mean().backward()
        opt.step()
    fast = tm.get_hidden_parameters()["hidden_weights_0"]
    assert float(fast.abs().max()) > 0
    # state dict round trip through the reference's own serialisation
    state = model.state_dict()
    model2 = AnalogLinear(64, 32, bias=False, rpu_config=cfg).cuda()
    model2.load_state_dict(state)
    # set_weights clips to the plain device bounds (PulsedRPUDevice::onSetWeights,
    # src/rpucuda/rpu_pulsed_device.cpp:545-556), so an element the reference device held beyond
    # them by its reference offset comes back clipped - as it does in the reference
    diff = (model2.get_weights()[0].cpu() - model.get_weights()[0].cpu()).abs()
    # (a handful of the 2048 elements, depending on the noise of the training steps above)
    assert int((diff > 1e-6).sum()) <= 0.01 * diff.numel() and float(diff.max()) <= 0.3


@pytest.mark.parametrize("which", ["chopped", "dynamic", "mixed"])
def test_later_compounds_through_reference_wrappers(aihwkit, which):
    """ChoppedTransferCompound (Tiki-Taka v3), DynamicTransferCompound (v4) and
    MixedPrecisionCompound of the reference's own configuration classes: `as_bindings` fills this
    module's parameter classes by the binding's attribute names, the tile trains with AnalogSGD,
    and its extra hidden planes carry the reference's names."""
    from aihwkit.nn import AnalogLinear
    from aihwkit.optim import AnalogSGD
    from aihwkit.simulator.configs import DigitalRankUpdateRPUConfig, UnitCellRPUConfig
    from aihwkit.simulator.configs.compounds import (ChoppedTransferCompound, DynamicTransferCompound,
                                                     MixedPrecisionCompound)
    from aihwkit.simulator.configs.devices import SoftBoundsReferenceDevice

    torch.manual_seed(5)
    unit = lambda: SoftBoundsReferenceDevice(dw_min=0.002, w_max=1.0, w_min=-1.0)  # noqa: E731
    if which == "chopped":
        cfg = UnitCellRPUConfig(device=ChoppedTransferCompound(
            unit_cell_devices=[unit(), unit()], in_chop_prob=0.1, transfer_every=1.0, units_in_mbatch=False))
        planes = ["buffered_FP_weight_0"]
    elif which == "dynamic":
        cfg = UnitCellRPUConfig(device=DynamicTransferCompound(
            unit_cell_devices=[unit(), unit()], in_chop_prob=0.5, transfer_every=1.0, units_in_mbatch=False))
        planes = ["buffered_FP_weight", "running_mean_weight", "past_mean_weight"]
    else:
        cfg = DigitalRankUpdateRPUConfig(device=MixedPrecisionCompound(device=unit(), n_x_bins=9, n_d_bins=5))
        planes = ["hidden_weights_chi"]
    cfg.mapping.weight_scaling_omega = 0.0
    cfg.mapping.learn_out_scaling = False
    model = AnalogLinear(24, 16, bias=False, rpu_config=cfg).cuda()
    tm = next(model.analog_tiles())
    hidden = tm.get_hidden_parameters()
    for name in planes:
        assert name in hidden, (name, list(hidden))
    w0 = model.get_weights()[0].clone()
    opt = AnalogSGD(model.parameters(), lr=0.2)
    opt.regroup_param_groups(model)
    x = torch.rand(8, 24, device="cuda")
    for _ in range(12):
        opt.zero_grad()
        model(x).square().mean().backward()
        opt.step()
    hidden = tm.get_hidden_parameters()
    # (with the default forgetting buffer and a transfer scale of 1 / granularity every read
    # empties its buffer element again: the chopped case is judged by its fast tile)
    moved = [n for n in planes + ["hidden_weights_0"] if n in hidden and float(hidden[n].abs().max()) > 0]
    assert moved, list(hidden)
    assert float((model.get_weights()[0] - w0).abs().max()) > 0
