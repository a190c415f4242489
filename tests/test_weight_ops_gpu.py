"""Weight operations between updates on the GPU (decay, diffusion, clipping, column reset,
uniform re-initialisation) against the numpy oracle (which is pinned to the compiled reference in
tests/test_oracle_vs_reference.py) and, where it is built, against the compiled reference."""

import numpy as np
import pytest
import torch

from oracle import analog_tile_oracle as O
from oracle import ref
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _device(kind="sb"):
    dp = H.device(kind, False)
    dp.lifetime, dp.lifetime_dtod = 50.0, 0.2
    dp.diffusion, dp.diffusion_dtod = 0.01, 0.3
    dp.reset, dp.reset_dtod, dp.reset_std = 0.05, 0.1, 0.02
    dp.w_max_dtod = dp.w_min_dtod = 0.2
    return dp


def _tile(cfg):
    from aihwkit_b200.rpu_base import tiles as T

    return T.AnalogTile(cfg, cuda_device=0)


@pytest.mark.parametrize("kind", ["cs", "sbr"])
def test_decay_and_clip_exact(kind):
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(5)
    x_size, d_size = 70, 33
    p = H.training_params(noise=False, pulse_det=True)
    cfg = p._config(x_size, d_size, _device(kind), seed=3)
    t = _tile(cfg)
    t.set_weights(torch.from_numpy(rng.uniform(-0.7, 0.7, (d_size, x_size)).astype(np.float32)))
    names, hp = t.get_hidden_parameter_names(), t.get_hidden_parameters().numpy()
    w = t.get_weights().numpy()
    for alpha in (1.0, 0.3):
        t.decay_weights(alpha)
        w = O.decay_weights(w, names, hp, alpha)
        assert np.array_equal(t.get_weights().numpy(), w)
    # bias column kept (C ABI only; the binding always passes bias_no_decay = False)
    from aihwkit_b200 import _cabi

    _cabi.check(_cabi.lib().ab200_tile_decay_weights(t._h, 0.5, 1, None))
    w = O.decay_weights(w, names, hp, 0.5, True)
    assert np.array_equal(t.get_weights().numpy(), w)
    wc = D.WeightClipParameter()
    wc.type, wc.fixed_value = D.WeightClipType.FixedValue, 0.25
    t.clip_weights(wc)
    w = O.clip_to_device(w, names, hp, 0.25)
    assert np.array_equal(t.get_weights().numpy(), w)
    wc.type = D.WeightClipType.LayerGaussian
    with pytest.raises(RuntimeError, match="Sophisticated clipping"):
        t.clip_weights(wc)
    if ref.available():
        rt = ref.RefTile(cfg)
        rt.set_weights(w)
        rt.decay_weights(0.7)
        t.decay_weights(0.7)
        assert np.array_equal(t.get_weights().numpy(), rt.get_weights())


def test_floating_point_tile_ops():
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(6)
    x_size, d_size = 130, 40
    ideal = D.IdealResistiveDeviceParameter()
    ideal.lifetime, ideal.diffusion, ideal.reset_std = 20.0, 0.05, 0.1
    p = H.training_params(noise=False, pulse_det=True)
    t = _tile(p._config(x_size, d_size, ideal, seed=3))
    w = rng.normal(0, 0.3, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(w))
    t.decay_weights(0.5)
    w = O.decay_weights_simple(w, 20.0, 0.5)
    assert np.array_equal(t.get_weights().numpy(), w)
    wc = D.WeightClipParameter()
    for ctype, fixed in ((D.WeightClipType.LayerGaussian, -1.0), (D.WeightClipType.AverageChannelMax, -1.0),
                         (D.WeightClipType.AverageChannelMax, 0.4), (D.WeightClipType.FixedValue, 0.2)):
        wc.type, wc.fixed_value, wc.sigma = ctype, fixed, 1.5
        c = O.clip_value(w, int(ctype), fixed, 1.5)
        t.clip_weights(wc)
        w = np.clip(w, -np.float32(c), np.float32(c))
        assert np.abs(t.get_weights().numpy() - w).max() <= 2e-6
    # diffusion: one global rate, no bounds
    before = t.get_weights().numpy()
    t.diffuse_weights()
    mid = t.get_weights().numpy()
    delta = mid - before
    assert abs(delta.std() / 0.05 - 1) < 0.05 and abs(delta.mean()) < 4 * 0.05 / np.sqrt(delta.size)
    # reset: N(0, reset_std) in the chosen columns only
    t.reset_columns(128, 5, 1.0)  # 128, 129, 0, 1, 2
    after = t.get_weights().numpy()
    cols = [128, 129, 0, 1, 2]
    assert abs(after[:, cols].std() / 0.1 - 1) < 0.15
    keep = [c for c in range(x_size) if c not in cols]
    assert np.array_equal(after[:, keep], mid[:, keep])
    t.set_weights_uniform_random(-0.3, 0.5)
    u = t.get_weights().numpy()
    assert u.min() >= -0.3 and u.max() <= 0.5 and abs(u.mean() - 0.1) < 0.01
    assert abs(u.std() - 0.8 / np.sqrt(12)) < 0.01


def test_diffusion_and_reset_moments_against_reference():
    """Per-element diffusion rates and reset biases: the GPU samples and the reference's samples
    have the same element-wise means and standard deviations."""
    x_size, d_size, reps = 12, 10, 300
    p = H.training_params(noise=False, pulse_det=True)
    dp = _device()
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = _tile(cfg)
    names, hp = t.get_hidden_parameter_names(), t.get_hidden_parameters().numpy()
    rate, bias = hp[names.index("diffusion_rates")], hp[names.index("reset_bias")]
    hi, lo = hp[names.index("max_bound")], hp[names.index("min_bound")]
    w0 = torch.zeros(d_size, x_size)
    diffs, resets, partial = [], [], []
    for _ in range(reps):
        t.set_weights(w0)
        t.diffuse_weights()
        diffs.append(t.get_weights().numpy())
        t.reset_columns(10, 4, 1.0)
        resets.append(t.get_weights().numpy())
        t.set_weights(w0 + 0.3)
        t.reset_columns(0, -1, 0.25)  # every column, a quarter of the elements
        partial.append(t.get_weights().numpy())
    diffs, resets, partial = np.stack(diffs), np.stack(resets), np.stack(partial)
    assert np.abs(diffs.std(0) / rate - 1).mean() < 0.06
    assert (diffs <= hi).all() and (diffs >= lo).all()
    cols = [10, 11, 0, 1]
    assert np.abs(resets[:, :, cols].mean(0) - bias[:, cols]).max() < 5 * dp.reset_std / np.sqrt(reps) + 1e-3
    assert abs(resets[:, :, cols].std(0).mean() / dp.reset_std - 1) < 0.08
    assert np.array_equal(resets[:, :, 2:10], diffs[:, :, 2:10])
    untouched = np.isclose(partial, np.minimum(0.3, hi)[None])
    assert abs((~untouched).mean() - 0.25) < 0.02
    if ref.available():
        rt = ref.RefTile(cfg)
        rt.set_seed(7)
        rd = []
        for _ in range(reps):
            rt.set_weights(w0.numpy())
            rt.diffuse_weights()
            rd.append(rt.get_weights())
        H.assert_moments_agree(diffs, np.stack(rd))


@pytest.mark.skipif(not ref.available(), reason="compiled reference not built")
def test_weight_ops_on_a_transfer_compound_against_reference():
    """Decay, clip and column reset of a Tiki-Taka tile (TransferRPUDevice with a fully hidden fast
    tile, src/rpucuda/rpu_transfer_device.cpp:612-651): decay and clip act on the fast tile with
    device 0 and on the visible weights with device 1, the reset on the fast tile only."""
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(21)
    x_size, d_size, m = 48, 36, 24
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.transfer_device(noise=False, det=True, transfer_every=2.0, units_in_mbatch=True,
                           n_reads=1, transfer_lr=1.0)
    for sub in dp._vec_par:
        sub.lifetime, sub.lifetime_dtod = 30.0, 0.2
        sub.reset, sub.reset_dtod, sub.reset_std = 0.02, 0.1, 0.0
    cfg = p._config(x_size, d_size, dp, seed=9)
    t = _tile(cfg)
    rt = ref.RefTile(cfg)
    names = t.get_hidden_parameter_names()
    assert np.array_equal(t.get_hidden_parameters().numpy(), rt.get_hidden_parameters())
    ia = names.index("hidden_weights_0")
    W0 = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W0))
    rt.set_weights(W0)
    t.set_learning_rate(0.05)
    rt.set_learning_rate(0.05)
    for _ in range(3):
        X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        Dm = rng.normal(0, 0.05, (m, d_size)).astype(np.float32)
        t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
        rt.update(X, Dm)

    def same(what):
        a, a_r = t.get_hidden_parameters().numpy()[ia], rt.get_hidden_parameters()[ia]
        c, c_r = t.get_weights().numpy(), rt.get_weights()
        assert np.abs(a - a_r).max() <= 1e-6, what
        assert np.abs(c - c_r).max() <= 1e-6, what
        return a, c

    a0, c0 = same("after the updates")
    assert np.abs(a0).max() > 0
    t.decay_weights(0.7)
    rt.decay_weights(0.7)
    a1, c1 = same("decay")
    assert np.abs(a1 - a0).max() > 1e-4 and np.abs(c1 - c0).max() > 1e-4
    wc = D.WeightClipParameter()
    wc.type, wc.fixed_value = D.WeightClipType.FixedValue, 0.1
    t.clip_weights(wc)
    rt.clip_weights(int(wc.type), 0.1)
    a2, c2 = same("clip")
    assert np.abs(c2).max() <= 0.1 + 1e-6 and np.abs(a2).max() <= 0.1 + 1e-6
    t.reset_columns(3, 5, 1.0)
    rt.reset_columns(3, 5, 1.0)
    a3, c3 = same("reset of the fast tile's columns")
    assert np.array_equal(c3, c2) and np.abs(a3[:, 3:8] - a2[:, 3:8]).max() > 0


def _drift(dp, **kw):
    dp.drift.nu, dp.drift.nu_dtod = 0.1, 0.3
    for k, v in kw.items():
        setattr(dp.drift, k, v)
    return dp


@pytest.mark.skipif(not ref.available(), reason="compiled reference not built")
@pytest.mark.parametrize("extra", [{}, {"nu_k": 0.05, "g_offset": 0.2, "wg_ratio": 0.6, "w_offset": -0.1,
                                        "log_g0": -0.3, "t_0": 2.0}])
def test_power_law_drift_against_reference(extra):
    """WeightDrifter::apply + saturate (src/rpucuda/weight_drifter.cpp:101-157) on a pulsed device:
    per-element exponents drawn as the reference draws them, clocks restarted for the elements
    written between two calls, conductance-offset term and weight-dependent exponent."""
    rng = np.random.default_rng(8)
    x_size, d_size = 70, 33
    p = H.training_params(noise=False, pulse_det=True)
    dp = _drift(H.device("cs", False), **extra)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t, rt = _tile(cfg), ref.RefTile(cfg)
    names = t.get_hidden_parameter_names()
    hp = t.get_hidden_parameters().numpy()
    assert np.array_equal(hp, rt.get_hidden_parameters())
    nu = hp[names.index("drift_nu")]
    assert abs(nu.mean() - 0.1) < 0.002 and abs(nu.std() / 0.03 - 1) < 0.1
    W = rng.uniform(0.05, 0.5, (d_size, x_size)).astype(np.float32)  # G > 0 for the log term
    t.set_weights(torch.from_numpy(W))
    rt.set_weights(W)
    for step, dt in enumerate((5.0, 20.0, 300.0)):
        if step == 1:
            # write a block of weights between the calls: their clocks restart
            W2 = t.get_weights().numpy().copy()
            W2[:10, :20] = rng.uniform(0.05, 0.5, (10, 20)).astype(np.float32)
            t.set_weights(torch.from_numpy(W2))
            rt.set_weights(W2)
        t.drift_weights(dt)
        rt.drift_weights(dt)
        a, b = t.get_weights().numpy(), rt.get_weights()
        assert np.abs(a - b).max() <= 2e-6 * np.abs(b).max(), (step, np.abs(a - b).max())
    assert np.abs(a - W2).max() > 0.01  # the weights did drift


@pytest.mark.skipif(not ref.available(), reason="compiled reference not built")
def test_power_law_drift_floating_point_tile_and_noise():
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(9)
    x_size, d_size = 64, 48
    ideal = _drift(D.IdealResistiveDeviceParameter())
    ideal.construction_seed = 13
    p = H.training_params(noise=False, pulse_det=True)
    cfg = p._config(x_size, d_size, ideal, seed=3)
    t, rt = _tile(cfg), ref.RefTile(cfg)
    W = rng.normal(0, 0.3, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    rt.set_weights(W)
    for dt in (3.0, 40.0):
        t.drift_weights(dt)
        rt.drift_weights(dt)
        a, b = t.get_weights().numpy(), rt.get_weights()
        assert np.abs(a - b).max() <= 2e-6 * np.abs(b).max()
    # the floating-point tile proper: one exponent for all weights (RPUSimple::driftWeights)
    fp = D.FloatingPointTileParameter()
    fp.drift.nu, fp.drift.nu_dtod = 0.2, 0.5
    ft = fp.create_array(x_size, d_size)
    from aihwkit_b200.rpu_base import tiles as T

    ft = T.CudaFloatingPointTile(ft)
    ft.set_weights(torch.from_numpy(W))
    ft.drift_weights(10.0)
    assert np.allclose(ft.get_weights().cpu().numpy(), W * np.float32(10.0) ** np.float32(-0.2), rtol=3e-6)
    # read noise and exponent noise: moments against the reference
    noisy = _drift(H.device("cs", False), nu_std=0.2, w_noise_std=0.01)
    cfg = p._config(x_size, d_size, noisy, seed=3)
    t, rt = _tile(cfg), ref.RefTile(cfg)
    W = rng.uniform(-0.4, 0.4, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    rt.set_weights(W)
    t.drift_weights(50.0)
    rt.drift_weights(50.0)
    da, db = t.get_weights().numpy() - W, rt.get_weights() - W
    assert abs(da.mean() - db.mean()) < 5 * db.std() / np.sqrt(db.size)
    assert abs(da.std() / db.std() - 1) < 0.05
    ra = (t.get_weights().numpy() / W)[np.abs(W) > 0.1]
    rb = (rt.get_weights() / W)[np.abs(W) > 0.1]
    assert abs(ra.std() / rb.std() - 1) < 0.1
