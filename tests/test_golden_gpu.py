"""The CUDA path against the golden vectors recorded from the compiled reference CPU tile
(tests/golden/*.npz), through the C ABI."""

import glob
import os

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DET = sorted(glob.glob(os.path.join(GOLD, "det_*.npz")))


def _gpu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("path", DET, ids=[os.path.basename(p)[:-4] for p in DET])
def test_deterministic_case(path):
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import analog_tile_oracle as O

    g = np.load(path)
    kind = os.path.basename(path).split("_")[1]
    d_size, x_size = g["w0"].shape
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=float(g["out_bound"]))
    dp = H.device(kind, False)
    cfg = p._config(x_size, d_size, dp, seed=1)
    t = T.AnalogTile(cfg, cuda_device=0)
    t.set_hidden_parameters(torch.from_numpy(g["hidden"]))
    t.set_weights(torch.from_numpy(g["w0"]))
    assert np.array_equal(t.get_weights().numpy(), g["w0"])
    fio, bio = O.IO.from_c(cfg.forward_io), O.IO.from_c(cfg.backward_io, backward=True)
    # ADC step in output units: res_out / input scale (per row; bound management may halve it)
    _, _, scale, _ = O.forward(g["w0"], g["x"], fio, return_pre_adc=True)
    y = t.forward(_gpu(g["x"])).cpu().numpy()
    frac, worst = H.lsb_report(y, g["y"], (fio.res_out / scale)[:, None])
    assert frac <= 2e-3 and worst <= 1.001, (frac, worst)
    gb = t.backward(_gpu(g["d"])).cpu().numpy()
    frac, worst = H.lsb_report(gb, g["g"], (bio.res_out * np.abs(g["d"]).max(axis=1))[:, None])
    assert frac <= 2e-3 and worst <= 1.001, (frac, worst)
    t.set_learning_rate(float(g["lr"]))
    for s in range(g["counts"].shape[0]):
        c = t.coincidences(_gpu(g["x"][s]), _gpu(g["d"][s])).cpu().numpy()
        assert np.array_equal(c, g["counts"][s])  # pulse counts: bit-exact
    t.update(_gpu(g["x"]), _gpu(g["d"]))
    assert np.abs(t.get_weights().numpy() - g["w1"]).max() <= 1e-6


def test_noisy_forward_against_reference_samples():
    from scipy import stats
    from aihwkit_b200.rpu_base import tiles as T

    g = np.load(os.path.join(GOLD, "noisy_forward.npz"))
    p = H.training_params(noise=True, pulse_det=False, bm=True)
    t = T.AnalogTile(p._config(64, 32, H.device("cs", True), seed=11), cuda_device=0)
    t.set_weights(torch.from_numpy(g["w0"]))
    xg = _gpu(g["x"])
    ys = np.stack([t.forward(xg).cpu().numpy() for _ in range(g["ys"].shape[0])])
    H.assert_moments_agree(ys, g["ys"], std_tol=0.05)
    mu = g["ys"].mean(axis=0)
    assert stats.ks_2samp((ys - mu).ravel(), (g["ys"] - mu).ravel()).pvalue > 0.01


def test_noisy_inference_against_reference_samples():
    from scipy import stats
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    g = np.load(os.path.join(GOLD, "noisy_inference.npz"))
    p = H.inference_params(noise=True)
    t = T.AnalogTile(p._config(128, 24, D.IdealResistiveDeviceParameter(), seed=12), cuda_device=0)
    t.set_weights(torch.from_numpy(g["w0"]))
    xg = _gpu(g["x"])
    ys = np.stack([t.forward(xg, is_test=True).cpu().numpy() for _ in range(g["ys"].shape[0])])
    H.assert_moments_agree(ys, g["ys"], std_tol=0.05)
    mu = g["ys"].mean(axis=0)
    assert stats.ks_2samp((ys - mu).ravel(), (g["ys"] - mu).ravel()).pvalue > 0.01


@pytest.mark.parametrize("kind", ["cs", "sbr"])
def test_noisy_update_against_reference_samples(kind):
    from scipy import stats
    from aihwkit_b200.rpu_base import tiles as T

    g = np.load(os.path.join(GOLD, f"noisy_update_{kind}.npz"))
    p = H.training_params(noise=True, pulse_det=False)
    t = T.AnalogTile(p._config(16, 12, H.device(kind, True), seed=13), cuda_device=0)
    t.set_hidden_parameters(torch.from_numpy(g["hidden"]))
    t.set_learning_rate(float(g["lr"]))
    xg, dg = _gpu(g["x"]), _gpu(g["d"])
    dws = []
    for _ in range(g["dws"].shape[0]):
        t.set_weights(torch.from_numpy(g["w"]))
        w0 = t.get_weights().numpy()
        t.update(xg, dg)
        dws.append(t.get_weights().numpy() - w0)
    dws = np.stack(dws)
    H.assert_moments_agree(dws, g["dws"])
    assert stats.ks_2samp(dws.sum(axis=(1, 2)), g["dws"].sum(axis=(1, 2))).pvalue > 0.01


def test_transfer_sequence_against_reference():
    from aihwkit_b200.rpu_base import tiles as T

    g = np.load(os.path.join(GOLD, "transfer_det.npz"))
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.transfer_device(noise=False, det=True, transfer_every=2.0, units_in_mbatch=True,
                           n_reads=2, transfer_lr=1.0)
    t = T.AnalogTile(p._config(20, 12, dp, seed=1), cuda_device=0)
    assert np.array_equal(t.get_hidden_parameters().numpy(), g["hidden0"])
    t.set_learning_rate(float(g["lr"]))
    ia = t.get_hidden_parameter_names().index("hidden_weights_0")
    for k in range(g["xs"].shape[0]):
        t.update(_gpu(g["xs"][k]), _gpu(g["ds"][k]))
        assert np.abs(t.get_hidden_parameters().numpy()[ia] - g["a"][k]).max() <= 1e-6, k
        assert np.abs(t.get_weights().numpy() - g["ws"][k]).max() <= 1e-6, k


def test_extensions_against_reference_vectors():
    """PiecewiseStep update, non-idealities of the output lines, power-law drift, weight modifiers,
    running-average noise management and the NoneWithDevice update against vectors recorded from
    the compiled reference (tests/golden/make_golden.py extensions_case)."""
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.rpu_base import tiles as T
    from tests.golden.make_golden import LINE_ALL  # the settings the vectors were made with

    g = np.load(os.path.join(GOLD, "extensions_det.npz"))

    # PiecewiseStep
    d_size, x_size = g["pw_w0"].shape
    p = H.training_params(noise=False, pulse_det=True)
    t = T.AnalogTile(p._config(x_size, d_size, H.piecewise_device(False), seed=1), cuda_device=0)
    t.set_hidden_parameters(torch.from_numpy(g["pw_hidden"]))
    t.set_weights(torch.from_numpy(g["pw_w0"]))
    t.set_learning_rate(0.01)
    t.update(_gpu(g["pw_x"]), _gpu(g["pw_d"]))
    assert np.abs(t.get_weights().numpy() - g["pw_w1"]).max() <= 1e-6
    assert np.abs(g["pw_w1"] - g["pw_w0"]).max() > 1e-3

    # output-line non-idealities, bound management with out_bound 2
    d_size, x_size = g["line_w0"].shape
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
    for io in (p.forward_io, p.backward_io):
        for k, v in LINE_ALL.items():
            setattr(io, k, v)
    t = T.AnalogTile(p._config(x_size, d_size, H.device("cs", False), seed=1), cuda_device=0)
    t.set_weights(torch.from_numpy(g["line_w0"]))
    for backward, which, key in ((False, 0, "line_voff_f"), (False, 1, "line_nl_f"),
                                 (True, 0, "line_voff_b"), (True, 1, "line_nl_b")):
        t.set_io_vector(backward, which, torch.from_numpy(g[key]))
    y = t.forward(_gpu(g["line_x"])).cpu().numpy()
    lsb = (2.0 * 2.0 / 510.0) * np.abs(g["line_x"]).max(axis=1, keepdims=True) * t.last_bm_stats()[1]
    frac, worst = H.lsb_report(y, g["line_y"], lsb)
    assert frac <= 5e-3 and worst <= 1.001, (frac, worst)
    gb = t.backward(_gpu(g["line_d"])).cpu().numpy()
    frac, worst = H.lsb_report(gb, g["line_g"], (2.0 * 12.0 / 510.0) * np.abs(g["line_d"]).max(axis=1, keepdims=True))
    assert frac <= 5e-3 and worst <= 1.001, (frac, worst)

    # drift
    d_size, x_size = g["drift_w0"].shape
    dp = H.device("cs", False)
    dp.drift.nu, dp.drift.nu_dtod, dp.drift.nu_k, dp.drift.g_offset, dp.drift.wg_ratio = 0.1, 0.3, 0.05, 0.2, 0.6
    p = H.training_params(noise=False, pulse_det=True)
    t = T.AnalogTile(p._config(x_size, d_size, dp, seed=1), cuda_device=0)
    t.set_hidden_parameters(torch.from_numpy(g["drift_hidden"]))
    t.set_weights(torch.from_numpy(g["drift_w0"]))
    t.drift_weights(5.0)
    assert np.abs(t.get_weights().numpy() - g["drift_w1"]).max() <= 2e-6
    t.set_weights(torch.from_numpy(g["drift_w2"]))
    t.drift_weights(40.0)
    assert np.abs(t.get_weights().numpy() - g["drift_w3"]).max() <= 2e-6
    assert np.abs(g["drift_w3"] - g["drift_w2"]).max() > 0.01

    # weight modifiers
    d_size, x_size = g["mod_w0"].shape
    pp = D.AnalogTileParameter()
    pp.forward_io.is_perfect = True
    pp.backward_io.is_perfect = True
    pp.update.pulse_type = D.PulseType.None_
    t = T.AnalogTile(pp._config(x_size, d_size, D.IdealResistiveDeviceParameter(), seed=1), cuda_device=0)
    t.set_weights(torch.from_numpy(g["mod_w0"]))
    eye = torch.eye(x_size, device="cuda")
    for name, kw in (("disc", dict(type=T.WeightModifierType.Discretize, res=0.1)),
                     ("dorefa", dict(type=T.WeightModifierType.DoReFa, res=0.08, dorefa_clip=0.6))):
        wm = T.WeightModifierParameter()
        for k, v in kw.items():
            setattr(wm, k, v)
        t.modify_weights(wm)
        fb = t.forward(eye).cpu().numpy().T
        assert (np.abs(fb - g["mod_" + name]) > 1e-6).mean() <= 0.005, name

    # running-average noise management over two calls
    d_size, x_size = g["nm_w0"].shape
    p = H.training_params(noise=False, pulse_det=True, bm=False)
    p.forward_io.noise_management = D.NoiseManagementType.AverageAbsMax
    p.forward_io.nm_decay = 0.1
    t = T.AnalogTile(p._config(x_size, d_size, H.device("cs", False), seed=1), cuda_device=0)
    t.set_weights(torch.from_numpy(g["nm_w0"]))
    for k in range(2):
        y = t.forward(_gpu(g["nm_xs"][k])).cpu().numpy()
        lsb = (2.0 * 12.0 / 510.0) * np.abs(g["nm_xs"][0]).max()
        frac, worst = H.lsb_report(y, g["nm_ys"][k], np.full((y.shape[0], 1), lsb))
        assert frac <= 5e-3 and worst <= 1.001, (k, frac, worst)

    # NoneWithDevice
    d_size, x_size = g["nwd_w0"].shape
    p = H.training_params(noise=False, pulse_det=True)
    p.update.pulse_type = D.PulseType.NoneWithDevice
    t = T.AnalogTile(p._config(x_size, d_size, H.device("cs", False, w_max=0.3, w_min=-0.3), seed=1),
                     cuda_device=0)
    t.set_hidden_parameters(torch.from_numpy(g["nwd_hidden"]))
    t.set_weights(torch.from_numpy(g["nwd_w0"]))
    t.set_learning_rate(0.2)
    t.update(_gpu(g["nwd_x"]), _gpu(g["nwd_d"]))
    assert np.abs(t.get_weights().numpy() - g["nwd_w1"]).max() <= 2e-6


def test_compounds_against_reference_vectors():
    """The two-pass MV types and the chopped / dynamic transfer and mixed-precision compounds
    against vectors recorded from the compiled reference (tests/golden/make_golden.py
    compounds_case): outputs within one ADC step (two for the digital sum), weights and hidden
    planes through eight updates."""
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.rpu_base import tiles as T
    from tests.golden.make_golden import COMPOUND_CASES, LINE_ALL

    g = np.load(os.path.join(GOLD, "compounds_det.npz"))
    d_size, x_size = g["pn_w0"].shape
    for mv in ("PosNegSeparate", "PosNegSeparateDigitalSum"):
        for lines in (False, True):
            key = f"pn_{mv}_{int(lines)}"
            p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
            for io in (p.forward_io, p.backward_io):
                io.mv_type = getattr(D.AnalogMVType, mv)
                if lines:
                    for k, v in LINE_ALL.items():
                        setattr(io, k, v)
            t = T.AnalogTile(p._config(x_size, d_size, H.device("cs", False), seed=1), cuda_device=0)
            t.set_weights(torch.from_numpy(g[key + "_w"]))
            if lines:
                for backward, tag in ((False, "f"), (True, "b")):
                    t.set_io_vector(backward, 0, torch.from_numpy(g[f"{key}_voff_{tag}"]))
                    t.set_io_vector(backward, 1, torch.from_numpy(g[f"{key}_nl_{tag}"]))
            steps = 2.002 if mv.endswith("DigitalSum") else 1.001
            y = t.forward(_gpu(g["pn_x"])).cpu().numpy()
            lsb = (2.0 * 2.0 / 510.0) * np.abs(g["pn_x"]).max(axis=1, keepdims=True) * t.last_bm_stats()[1]
            frac, worst = H.lsb_report(y, g[key + "_y"], lsb)
            assert frac <= 1e-2 and worst <= steps, (key, frac, worst)
            gb = t.backward(_gpu(g["pn_d"])).cpu().numpy()
            lsb_b = (2.0 * 12.0 / 510.0) * np.abs(g["pn_d"]).max(axis=1, keepdims=True)
            frac, worst = H.lsb_report(gb, g[key + "_g"], lsb_b)
            assert frac <= 1e-2 and worst <= steps, (key, "backward", frac, worst)

    m, x_size = g["cp_x"].shape[1:]
    d_size = g["cp_d"].shape[2]
    for name, (helper, kw) in COMPOUND_CASES.items():
        p = H.training_params(noise=False, pulse_det=True)
        t = T.AnalogTile(p._config(x_size, d_size, getattr(H, helper)(**kw), seed=3), cuda_device=0)
        assert np.array_equal(t.get_hidden_parameters().numpy(), g[f"cp_{name}_hidden0"]), name
        names = t.get_hidden_parameter_names()
        state = [k for k, n in enumerate(names)
                 if n.startswith(("hidden_weights", "buffered_FP", "running_mean", "past_mean"))]
        t.set_learning_rate(0.1)
        for k in range(8):
            t.update(_gpu(g["cp_x"][k]), _gpu(g["cp_d"][k]))
            assert np.abs(t.get_weights().numpy() - g[f"cp_{name}_w"][k]).max() <= 1e-6, (name, k)
            hp = t.get_hidden_parameters().numpy()
            for q in state:
                assert np.abs(hp[q] - g[f"cp_{name}_hidden"][k][q]).max() <= 1e-4, (name, names[q], k)
        assert np.abs(g[f"cp_{name}_w"][-1]).max() > 0
