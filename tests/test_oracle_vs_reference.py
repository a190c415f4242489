"""The numpy oracle against the compiled reference CPU tile (oracle/_ref), on fresh seeded
inputs.  Skipped where the reference library is not present."""

import numpy as np
import pytest

from oracle import analog_tile_oracle as O
from oracle import ref
from tests import helpers as H

pytestmark = pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built")

KIND = {"cs": O.DEV_CONSTANT_STEP, "ls": O.DEV_LINEAR_STEP, "sb": O.DEV_SOFT_BOUNDS,
        "sbr": O.DEV_SOFT_BOUNDS_REFERENCE}


@pytest.mark.parametrize("kind", ["cs", "ls", "sb", "sbr"])
@pytest.mark.parametrize("shape", [(96, 64, 32), (33, 70, 5)])
def test_noise_off_exact(kind, shape):
    x_size, d_size, m = shape
    rng = np.random.default_rng(x_size)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
    dp = H.device(kind, False)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = ref.RefTile(cfg)
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    W = t.get_weights()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    X[m // 2] = 0
    Dm = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    assert np.array_equal(t.forward(X), O.forward(W, X, O.IO.from_c(cfg.forward_io)))
    assert np.array_equal(t.backward(Dm), O.backward(W, Dm, O.IO.from_c(cfg.backward_io, backward=True)))
    up = O.Up.from_c(cfg.update)
    lr = 0.01
    assert np.array_equal(t.coincidences(X[0], Dm[0], lr, dp.dw_min),
                          O.coincidences_det_implicit(X[0], Dm[0], lr, dp.dw_min, up))
    dev = O.DeviceArrays.from_hidden(KIND[kind], t.hidden_parameter_names(),
                                     t.get_hidden_parameters(), 0.0, getattr(dp, "mult_noise", True))
    t.set_learning_rate(lr)
    t.update(X, Dm)
    Wo = W.copy()
    O.update(Wo, X, Dm, lr, dp.dw_min, up, dev)
    assert np.abs(t.get_weights() - Wo).max() <= 1e-7


def test_transposed_and_bias_layouts():
    rng = np.random.default_rng(1)
    x_size, d_size, m = 21, 10, 6
    p = H.training_params(noise=False, pulse_det=True, bm=False)
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=3)
    t = ref.RefTile(cfg)
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    W = t.get_weights()
    X = rng.uniform(-1, 1, (m, x_size - 1)).astype(np.float32)
    Xb = np.concatenate([X, np.ones((m, 1), np.float32)], axis=1)
    y = t.forward(np.ascontiguousarray(X.T), bias=True, x_trans=True, d_trans=True)
    assert np.array_equal(y.T, O.forward(W, Xb, O.IO.from_c(cfg.forward_io)))


def test_noisy_stochastic_update_moments():
    rng = np.random.default_rng(2)
    x_size, d_size, m, reps = 16, 12, 8, 120
    p = H.training_params(noise=True, pulse_det=False)
    dp = H.device("sb", True)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = ref.RefTile(cfg)
    t.set_seed(5)
    w = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    lr = 0.05
    t.set_learning_rate(lr)
    up = O.Up.from_c(cfg.update)
    dev = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS, t.hidden_parameter_names(),
                                     t.get_hidden_parameters(), dp.dw_min_std, True)
    org = np.random.default_rng(9)
    dr, do = [], []
    for _ in range(reps):
        t.set_weights(w)
        w0 = t.get_weights()
        t.update(X, Dm)
        dr.append(t.get_weights() - w0)
        wo = w0.copy()
        O.update(wo, X, Dm, lr, dp.dw_min, up, dev, org)
        do.append(wo - w0)
    dr, do = np.stack(dr), np.stack(do)
    H.assert_moments_agree(do, dr)
