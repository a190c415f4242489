"""The numpy oracle against the golden vectors recorded from the compiled reference
(tests/golden/*.npz, made by tests/golden/make_golden.py).  CPU only."""

import glob
import os

import numpy as np
import pytest

from oracle import analog_tile_oracle as O
from tests import helpers as H

GOLD = os.path.join(os.path.dirname(__file__), "golden")
KIND = {"cs": O.DEV_CONSTANT_STEP, "ls": O.DEV_LINEAR_STEP, "sb": O.DEV_SOFT_BOUNDS,
        "sbr": O.DEV_SOFT_BOUNDS_REFERENCE}
BASE_NAMES = ["max_bound", "min_bound", "dwmin_up", "dwmin_down", "decay_scales",
              "diffusion_rates", "reset_bias", "drift_nu"]


def names_for(kind):
    extra = {"ls": ["slope_up", "slope_down"], "sb": ["slope_up", "slope_down"], "sbr": ["reference"]}
    return BASE_NAMES + extra.get(kind, [])


DET = sorted(glob.glob(os.path.join(GOLD, "det_*.npz")))


def test_fixtures_present():
    assert len(DET) == 8
    for n in ("noisy_forward", "noisy_inference", "noisy_update_cs", "noisy_update_sbr", "transfer_det"):
        assert os.path.exists(os.path.join(GOLD, n + ".npz"))


@pytest.mark.parametrize("path", DET, ids=[os.path.basename(p)[:-4] for p in DET])
def test_deterministic_case(path):
    g = np.load(path)
    kind = os.path.basename(path).split("_")[1]
    d_size, x_size = g["w0"].shape
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=float(g["out_bound"]))
    dp = H.device(kind, False)
    cfg = p._config(x_size, d_size, dp, seed=1)
    fio, bio = O.IO.from_c(cfg.forward_io), O.IO.from_c(cfg.backward_io, backward=True)
    y = O.forward(g["w0"], g["x"], fio)
    assert np.array_equal(y, g["y"])
    assert np.all(y[1] == 0)
    gb = O.backward(g["w0"], g["d"], bio)
    assert np.array_equal(gb, g["g"])
    up = O.Up.from_c(cfg.update)
    lr = float(g["lr"])
    for s in range(g["counts"].shape[0]):
        c = O.coincidences_det_implicit(g["x"][s], g["d"][s], lr, dp.dw_min, up)
        assert np.array_equal(c, g["counts"][s])
    dev = O.DeviceArrays.from_hidden(KIND[kind], names_for(kind), g["hidden"], 0.0,
                                     getattr(dp, "mult_noise", True))
    w = g["w0"].copy()
    O.update(w, g["x"], g["d"], lr, dp.dw_min, up, dev)
    assert np.abs(w - g["w1"]).max() <= 1e-7


def test_bound_management_really_reran():
    g = np.load(os.path.join(GOLD, "det_cs_70x33_ob2.npz"))
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
    cfg = p._config(70, 33, H.device("cs", False), seed=1)
    _, _, _, red = O.forward(g["w0"], g["x"], O.IO.from_c(cfg.forward_io), return_pre_adc=True)
    assert (red > 1).any()


def test_noisy_forward_moments_and_ks():
    from scipy import stats

    g = np.load(os.path.join(GOLD, "noisy_forward.npz"))
    p = H.training_params(noise=True, pulse_det=False, bm=True)
    cfg = p._config(64, 32, H.device("cs", True), seed=1)
    fio = O.IO.from_c(cfg.forward_io)
    rng = np.random.default_rng(0)
    reps = g["ys"].shape[0]
    yo = np.stack([O.forward(g["w0"], g["x"], fio, rng) for _ in range(reps)])
    H.assert_moments_agree(yo, g["ys"], std_tol=0.05)
    mu = g["ys"].mean(axis=0)
    assert stats.ks_2samp((yo - mu).ravel(), (g["ys"] - mu).ravel()).pvalue > 0.01


def test_noisy_inference_moments():
    from aihwkit_b200.rpu_base import devices as D

    g = np.load(os.path.join(GOLD, "noisy_inference.npz"))
    p = H.inference_params(noise=True)
    cfg = p._config(128, 24, D.IdealResistiveDeviceParameter(), seed=1)
    fio = O.IO.from_c(cfg.forward_io)
    rng = np.random.default_rng(0)
    reps = g["ys"].shape[0]
    yo = np.stack([O.forward(g["w0"], g["x"], fio, rng) for _ in range(reps)])
    H.assert_moments_agree(yo, g["ys"], std_tol=0.05)


@pytest.mark.parametrize("kind", ["cs", "sbr"])
def test_noisy_update_moments(kind):
    from scipy import stats

    g = np.load(os.path.join(GOLD, f"noisy_update_{kind}.npz"))
    p = H.training_params(noise=True, pulse_det=False)
    dp = H.device(kind, True)
    cfg = p._config(16, 12, dp, seed=1)
    up = O.Up.from_c(cfg.update)
    dev = O.DeviceArrays.from_hidden(KIND[kind], names_for(kind), g["hidden"], dp.dw_min_std,
                                     getattr(dp, "mult_noise", True))
    rng = np.random.default_rng(3)
    reps = g["dws"].shape[0]
    dwo = []
    for _ in range(reps):
        w = g["w0"].copy()
        O.update(w, g["x"], g["d"], float(g["lr"]), dp.dw_min, up, dev, rng)
        dwo.append(w - g["w0"])
    dwo = np.stack(dwo)
    H.assert_moments_agree(dwo, g["dws"])
    assert stats.ks_2samp(dwo.sum(axis=(1, 2)), g["dws"].sum(axis=(1, 2))).pvalue > 0.01


def test_transfer_sequence():
    g = np.load(os.path.join(GOLD, "transfer_det.npz"))
    x_size, d_size = 20, 12
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.transfer_device(noise=False, det=True, transfer_every=2.0, units_in_mbatch=True,
                           n_reads=2, transfer_lr=1.0)
    cfg = p._config(x_size, d_size, dp, seed=1)
    names = []
    for k in range(2):
        names += [f"{n}_{k}" for n in names_for("sbr")] + [f"hidden_weights_{k}"]
    fast = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS_REFERENCE, names, g["hidden0"], 0.0, False, "_0")
    slow = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS_REFERENCE, names, g["hidden0"], 0.0, False, "_1")
    orc = O.TransferOracle(np.zeros((d_size, x_size), np.float32), fast, slow, cfg.transfer,
                           O.Up.from_c(cfg.update), 0.002, 0.002, x_size, d_size)
    for k in range(g["xs"].shape[0]):
        orc.update(g["xs"][k], g["ds"][k], float(g["lr"]))
        assert np.abs(orc.a - g["a"][k]).max() <= 1e-7, k
        assert np.abs(orc.c - g["ws"][k]).max() <= 1e-7, k
    assert np.abs(g["ws"][-1]).max() > 0


def test_indexed_conv_fixture():
    """The numpy restatement of the indexed interface against the vectors of the compiled
    reference (tests/golden/indexed_conv.npz)."""
    g = np.load(os.path.join(GOLD, "indexed_conv.npz"))
    n, c, h, w = g["x"].shape
    c_out, x_size = g["w0"].shape
    m_batch = g["indices"].size // x_size
    assert np.array_equal(g["indices"], O.conv_indices((c, h, w), (3, 3), (2, 1), (1, 1), (1, 1), True))
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=float(g["out_bound"]))
    dp = H.device("sb", False)
    cfg = p._config(x_size, c_out, dp, seed=1)
    cols = O.indexed_input(g["x"], g["indices"], x_size, m_batch, n, True)
    y = O.forward(g["w0"], cols, O.IO.from_c(cfg.forward_io))
    assert np.array_equal(O.from_sample_major(y, c_out, m_batch, n, True).reshape(g["y"].shape), g["y"])
    d_cols = O.to_sample_major(g["d"], c_out, m_batch, n, True)
    xg = O.backward(g["w0"], d_cols, O.IO.from_c(cfg.backward_io, backward=True))
    xo = O.indexed_output(xg, g["indices"], x_size, m_batch, n, True, g["x"].size)
    assert np.abs(xo.reshape(g["g"].shape) - g["g"]).max() <= 1e-5
    w1 = g["w0"].copy()
    dev = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS, names_for("sb"), g["hidden"], 0.0, True)
    O.update(w1, cols, d_cols, float(g["lr"]), dp.dw_min, O.Up.from_c(cfg.update), dev)
    assert np.abs(w1 - g["w1"]).max() <= 1e-7
