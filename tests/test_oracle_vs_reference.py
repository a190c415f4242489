"""The numpy oracle against the compiled reference CPU tile (oracle/_ref), on fresh seeded
inputs.  Skipped where the reference library is not present."""

import numpy as np
import pytest

from oracle import analog_tile_oracle as O
from oracle import ref
from tests import helpers as H

pytestmark = pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built")

KIND = {"cs": O.DEV_CONSTANT_STEP, "ls": O.DEV_LINEAR_STEP, "sb": O.DEV_SOFT_BOUNDS,
        "sbr": O.DEV_SOFT_BOUNDS_REFERENCE, "es": O.DEV_EXP_STEP}


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


@pytest.mark.parametrize("trans", [True, False])
@pytest.mark.parametrize("analog_bias", [False, True])
def test_indexed_interface(trans, analog_bias):
    """forward/backward/update through the index array of a padded, strided 3x3 convolution."""
    rng = np.random.default_rng(4)
    n, c, h, w, c_out = 3, 4, 7, 6, 5
    idx_t = O.conv_indices((c, h, w), (3, 3), (2, 1), (1, 1), (1, 1), analog_bias)
    x_size = c * 9 + (1 if analog_bias else 0)
    m_batch = idx_t.size // x_size
    idx = idx_t if trans else np.ascontiguousarray(idx_t.reshape(x_size, m_batch).T).reshape(-1)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
    dp = H.device("sb", False)
    cfg = p._config(x_size, c_out, dp, seed=3)
    t = ref.RefTile(cfg)
    t.set_weights(rng.uniform(-0.5, 0.5, (c_out, x_size)).astype(np.float32))
    t.set_matrix_indices(idx)
    W = t.get_weights()
    # image layout: [N][C*H*W]; the gather only sees flat images
    X = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
    d_shape = (n, c_out, m_batch) if trans else (n, m_batch, c_out)
    Dm = rng.normal(0, 0.1, d_shape).astype(np.float32)

    cols = O.indexed_input(X, idx, x_size, m_batch, n, trans)
    y = O.forward(W, cols, O.IO.from_c(cfg.forward_io))
    assert np.array_equal(t.forward_indexed(X, d_shape, trans),
                          O.from_sample_major(y, c_out, m_batch, n, trans).reshape(d_shape))

    d_cols = O.to_sample_major(Dm, c_out, m_batch, n, trans)
    xg = O.backward(W, d_cols, O.IO.from_c(cfg.backward_io, backward=True))
    xo = O.indexed_output(xg, idx, x_size, m_batch, n, trans, X.size)
    got = t.backward_indexed(Dm, X.shape, trans).reshape(n, -1)
    assert np.abs(got - xo).max() <= 1e-5 * max(1.0, np.abs(xo).max())

    lr = 0.01
    t.set_learning_rate(lr)
    dev = O.DeviceArrays.from_hidden(KIND["sb"], t.hidden_parameter_names(),
                                     t.get_hidden_parameters(), 0.0, True)
    t.update_indexed(X, Dm, trans)
    Wo = W.copy()
    O.update(Wo, cols, d_cols, lr, dp.dw_min, O.Up.from_c(cfg.update), dev)
    assert np.abs(t.get_weights() - Wo).max() <= 1e-7


def _decay_device(kind="sb"):
    dp = H.device(kind, False)
    dp.lifetime, dp.lifetime_dtod = 50.0, 0.2
    dp.diffusion, dp.diffusion_dtod = 0.01, 0.3
    dp.reset, dp.reset_dtod, dp.reset_std = 0.05, 0.1, 0.02
    dp.w_max_dtod = dp.w_min_dtod = 0.2
    return dp


def test_weight_ops_deterministic():
    """Decay and clipping against the compiled reference (exact), and the per-element decay /
    diffusion / reset parameters the host draws."""
    rng = np.random.default_rng(5)
    x_size, d_size = 23, 11
    p = H.training_params(noise=False, pulse_det=True)
    cfg = p._config(x_size, d_size, _decay_device(), seed=3)
    t = ref.RefTile(cfg)
    t.set_weights(rng.uniform(-0.7, 0.7, (d_size, x_size)).astype(np.float32))
    names, hp = t.hidden_parameter_names(), t.get_hidden_parameters()
    assert np.ptp(hp[names.index("decay_scales")]) > 0 and np.ptp(hp[names.index("reset_bias")]) > 0
    w = t.get_weights()
    for alpha, bnd in ((1.0, False), (0.3, True)):
        t.decay_weights(alpha, bnd)
        w = O.decay_weights(w, names, hp, alpha, bnd)
        assert np.array_equal(t.get_weights(), w)
    t.clip_weights(1, fixed_value=0.3)
    w = O.clip_to_device(w, names, hp, 0.3)
    assert np.array_equal(t.get_weights(), w)
    # floating-point tile: scalar decay and the data-dependent clip values
    from aihwkit_b200.rpu_base import devices as D

    ideal = D.IdealResistiveDeviceParameter()
    ideal.lifetime = 20.0
    t2 = ref.RefTile(p._config(x_size, d_size, ideal, seed=3))
    w2 = rng.normal(0, 0.3, (d_size, x_size)).astype(np.float32)
    t2.set_weights(w2)
    t2.decay_weights(0.5)
    w2 = O.decay_weights_simple(w2, 20.0, 0.5)
    assert np.array_equal(t2.get_weights(), w2)
    for ctype, fixed in ((2, -1.0), (3, -1.0), (3, 0.4)):
        c = O.clip_value(w2, ctype, fixed, 1.5)
        t2.clip_weights(ctype, fixed, 1.5)
        w2 = np.clip(w2, -np.float32(c), np.float32(c))
        assert np.abs(t2.get_weights() - w2).max() <= 1e-6


def test_weight_ops_stochastic_moments():
    """Diffusion and column reset of the reference: per-element standard deviations follow the
    hidden diffusion rates / reset_std, means the reset bias."""
    x_size, d_size, reps = 12, 10, 400
    p = H.training_params(noise=False, pulse_det=True)
    dp = _decay_device()
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = ref.RefTile(cfg)
    t.set_seed(7)
    names, hp = t.hidden_parameter_names(), t.get_hidden_parameters()
    rate, bias = hp[names.index("diffusion_rates")], hp[names.index("reset_bias")]
    w0 = np.zeros((d_size, x_size), np.float32)
    diffs, resets = [], []
    for _ in range(reps):
        t.set_weights(w0)
        t.diffuse_weights()
        diffs.append(t.get_weights())
        t.reset_columns(10, 4, 1.0)  # columns 10, 11, 0, 1
        resets.append(t.get_weights())
    diffs, resets = np.stack(diffs), np.stack(resets)
    assert np.abs(diffs.std(0) / rate - 1).mean() < 0.05
    cols = [10, 11, 0, 1]
    assert np.abs(resets[:, :, cols].mean(0) - bias[:, cols]).max() < 5 * dp.reset_std / np.sqrt(reps) + 1e-3
    assert abs(resets[:, :, cols].std(0).mean() / dp.reset_std - 1) < 0.08
    assert np.array_equal(resets[:, :, 2:10], diffs[:, :, 2:10])


@pytest.mark.parametrize("kind", ["cs", "sb", "sbr"])
def test_host_parameter_draw_with_decay_diffusion_reset(kind):
    """The library's host-side draw of decay scales, diffusion rates and reset biases equals the
    reference's for the same construction seed (needs no GPU: the tile stays on the host)."""
    from aihwkit_b200.rpu_base import tiles as T

    p = H.training_params(noise=False, pulse_det=True)
    cfg = p._config(17, 9, _decay_device(kind), seed=3)
    ours = T.AnalogTile(cfg)
    t = ref.RefTile(cfg)
    assert ours.get_hidden_parameter_names() == t.hidden_parameter_names()
    assert np.array_equal(ours.get_hidden_parameters().numpy(), t.get_hidden_parameters())


def _es_tuple(dp):
    return (dp.a, dp.b, dp.A_up, dp.A_down, dp.gamma_up, dp.gamma_down, dp.dw_min_std_add,
            dp.dw_min_std_slope)


@pytest.mark.parametrize("shape", [(96, 64, 32), (33, 70, 5)])
def test_exp_step_device_noise_off(shape):
    """ExpStep device: granularity, host parameter draw and the weights after a deterministic
    update (expf of numpy vs glibc: last-bit differences allowed)."""
    from aihwkit_b200.rpu_base import tiles as T

    x_size, d_size, m = shape
    rng = np.random.default_rng(x_size)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
    dp = H.device("es", False, A_up=0.1, A_down=0.3, gamma_up=3.0, gamma_down=2.5)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = ref.RefTile(cfg)
    ours = T.AnalogTile(cfg)
    assert np.array_equal(ours.get_hidden_parameters().numpy(), t.get_hidden_parameters())
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    W = t.get_weights()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    lr = 0.01
    gran = dp.calc_weight_granularity()
    up = O.Up.from_c(cfg.update)
    assert np.array_equal(t.coincidences(X[0], Dm[0], lr, gran),
                          O.coincidences_det_implicit(X[0], Dm[0], lr, gran, up))
    dev = O.DeviceArrays.from_hidden(O.DEV_EXP_STEP, t.hidden_parameter_names(),
                                     t.get_hidden_parameters(), 0.0, True)
    dev.es = _es_tuple(dp)
    t.set_learning_rate(lr)
    t.update(X, Dm)
    Wo = W.copy()
    O.update(Wo, X, Dm, lr, gran, up, dev)
    assert np.abs(t.get_weights() - Wo).max() <= 2e-6
    assert np.abs(t.get_weights() - W).max() > 1e-3  # the update did something


@pytest.mark.parametrize("nm,bm", [("Max", "Iterative"), ("AbsMaxNPSum", "Iterative"),
                                   ("AbsMax", "IterativeWorstCase"), ("None_", "IterativeWorstCase")])
def test_noise_and_bound_management_variants(nm, bm):
    """Max and AbsMaxNPSum noise management, IterativeWorstCase bound management: the oracle
    equals the compiled reference with noise off, rows that clip and re-run included."""
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(7)
    x_size, d_size, m = 96, 40, 24
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=1.5)
    p.forward_io.noise_management = getattr(D.NoiseManagementType, nm)
    p.forward_io.bound_management = getattr(D.BoundManagementType, bm)
    p.forward_io.nm_assumed_wmax = 0.5
    if nm == "None_":
        p.forward_io.inp_bound = 1.0
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=3)
    t = ref.RefTile(cfg)
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    W = t.get_weights()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    X[3] = -np.abs(X[3])  # Max noise management: no positive input => zero output
    X[5] *= 0.05
    io = O.IO.from_c(cfg.forward_io)
    y_ref = t.forward(X)
    y, _, _, red = O.forward(W, X, io, return_pre_adc=True)
    assert np.array_equal(y_ref, y)
    if nm == "Max":
        assert (red > 1).any()  # some rows re-ran with a halved input
        assert (y[3] == 0).all()
    if bm == "IterativeWorstCase":
        # the re-run really happened: without bound management the clipped rows differ
        io_plain = O.IO.from_c(cfg.forward_io)
        io_plain.bound_management = O.BM_NONE
        assert not np.array_equal(O.forward(W, X, io_plain), y)


@pytest.mark.parametrize("forget,momentum", [(True, 0.0), (False, 0.3), (True, 0.5)])
def test_buffered_transfer_sequence(forget, momentum):
    """Tiki-Taka v2 (BufferedTransfer): fast tile, digital buffer and slow tile of the oracle
    follow the compiled reference update by update."""
    rng = np.random.default_rng(13)
    x_size, d_size, m = 12, 10, 4
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.buffered_transfer_device(thres_scale=2.0, momentum=momentum, forget_buffer=forget,
                                    transfer_lr=4.0)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = ref.RefTile(cfg)
    lr = 0.1
    t.set_learning_rate(lr)
    names, hp = t.hidden_parameter_names(), t.get_hidden_parameters()
    assert names[-1] == "buffered_FP_weight_0"
    fast = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS_REFERENCE, names, hp, 0.0, False, "_0")
    slow = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS_REFERENCE, names, hp, 0.0, False, "_1")
    orc = O.TransferOracle(np.zeros((d_size, x_size), np.float32), fast, slow, cfg.transfer,
                           O.Up.from_c(cfg.update), 0.002, 0.002, x_size, d_size)
    moved = False
    # the write uses stochastic trains with probability exactly 1 per line (one pulse per whole
    # step): the generator is consulted but cannot change the outcome
    org = np.random.default_rng(0)
    for _ in range(10):
        x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        d = rng.normal(0, 0.5, (m, d_size)).astype(np.float32)
        t.update(x, d)
        orc.update(x, d, lr, org)
        hp = t.get_hidden_parameters()
        assert np.abs(hp[names.index("hidden_weights_0")] - orc.a).max() <= 1e-7
        assert np.abs(hp[names.index("buffered_FP_weight_0")] - orc.h).max() <= 1e-6
        assert np.abs(t.get_weights() - orc.c).max() <= 1e-7
        moved = moved or np.abs(orc.c).max() > 0
    assert moved
    if momentum > 0 or not forget:
        assert np.abs(orc.h).max() > 0


def test_io_asymmetries_exact():
    """inp_asymmetry / out_asymmetry (negative DAC outputs and negative pre-ADC values scaled by
    1 - asymmetry): deterministic, the oracle equals the compiled reference, forward and backward."""
    rng = np.random.default_rng(17)
    x_size, d_size, m = 70, 33, 20
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=4.0)
    for io in (p.forward_io, p.backward_io):
        io.inp_asymmetry, io.out_asymmetry = 0.1, 0.2
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=3)
    t = ref.RefTile(cfg)
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    W = t.get_weights()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
    y = O.forward(W, X, O.IO.from_c(cfg.forward_io))
    assert np.array_equal(t.forward(X), y)
    g = O.backward(W, Dm, O.IO.from_c(cfg.backward_io, backward=True))
    assert np.array_equal(t.backward(Dm), g)
    plain = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=4.0)
    y0 = O.forward(W, X, O.IO.from_c(plain._config(x_size, d_size, H.device("cs", False), seed=3).forward_io))
    assert np.abs(y - y0).max() > 1e-2  # the asymmetries did something


@pytest.mark.parametrize("what", ["inp_noise", "inp_sto_round", "out_sto_round"])
def test_io_random_input_stage_moments(what):
    """Input noise and stochastic DAC / ADC rounding: the oracle's samples and the compiled
    reference's samples agree in their element-wise means and standard deviations."""
    rng = np.random.default_rng(19)
    x_size, d_size, m, reps = 40, 12, 6, 300
    p = H.training_params(noise=False, pulse_det=True)
    if what == "inp_noise":
        p.forward_io.inp_noise = 0.1
    else:
        p.forward_io.inp_res, p.forward_io.out_res = 1 / 14.0, 1 / 30.0  # coarse: rounding matters
        setattr(p.forward_io, what, True)
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=3)
    t = ref.RefTile(cfg)
    t.set_seed(5)
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    W = t.get_weights()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    X[2] = 0.0  # zero row: zero output without input noise, pure noise with it
    io = O.IO.from_c(cfg.forward_io)
    org = np.random.default_rng(1)
    ys_ref = np.stack([t.forward(X) for _ in range(reps)])
    ys = np.stack([O.forward(W, X, io, org) for _ in range(reps)])
    assert ys.std(axis=0).max() > 0  # something random happened
    if what == "inp_noise":
        assert ys_ref[:, 2].std() > 0 and ys[:, 2].std() > 0
    else:
        assert (ys_ref[:, 2] == 0).all() and (ys[:, 2] == 0).all()
    H.assert_moments_agree(ys, ys_ref)


@pytest.mark.parametrize("shape", [(96, 64, 32), (33, 70, 5)])
def test_pow_step_device_noise_off(shape):
    """PowStep device: granularity, host parameter draw (per-element exponents included) and the
    weights after a deterministic update (powf of numpy vs glibc: last-bit differences allowed)."""
    from aihwkit_b200.rpu_base import tiles as T

    x_size, d_size, m = shape
    rng = np.random.default_rng(x_size)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
    dp = H.device("ps", False, pow_gamma=1.3, pow_gamma_dtod=0.2, pow_up_down=0.1, pow_up_down_dtod=0.05)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = ref.RefTile(cfg)
    ours = T.AnalogTile(cfg)
    names = t.hidden_parameter_names()
    assert names == ours.get_hidden_parameter_names() and names[-2:] == ["gamma_up", "gamma_down"]
    assert np.array_equal(ours.get_hidden_parameters().numpy(), t.get_hidden_parameters())
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    W = t.get_weights()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    lr = 0.01
    gran = dp.calc_weight_granularity()
    up = O.Up.from_c(cfg.update)
    assert np.array_equal(t.coincidences(X[0], Dm[0], lr, gran),
                          O.coincidences_det_implicit(X[0], Dm[0], lr, gran, up))
    dev = O.DeviceArrays.from_hidden(O.DEV_POW_STEP, names, t.get_hidden_parameters(), 0.0, True)
    t.set_learning_rate(lr)
    t.update(X, Dm)
    Wo = W.copy()
    O.update(Wo, X, Dm, lr, gran, up, dev)
    assert np.abs(t.get_weights() - Wo).max() <= 2e-6
    assert np.abs(t.get_weights() - W).max() > 1e-3  # the update did something


@pytest.mark.parametrize("shape", [(96, 64, 32), (33, 70, 5)])
@pytest.mark.parametrize("nodes", [6, 1])
def test_piecewise_step_device_noise_off(shape, nodes):
    """PiecewiseStep device (rpu_piecewisestep_device.cpp:30-80): granularity, host parameter draw
    and the weights after a deterministic update; one node = the short-cut without interpolation."""
    from aihwkit_b200.rpu_base import tiles as T

    x_size, d_size, m = shape
    rng = np.random.default_rng(x_size + nodes)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
    dp = H.piecewise_device(False)
    if nodes == 1:
        dp.piecewise_up, dp.piecewise_down = [0.7], [1.1]
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = ref.RefTile(cfg)
    ours = T.AnalogTile(cfg)
    names = t.hidden_parameter_names()
    assert names == ours.get_hidden_parameter_names()
    assert np.array_equal(ours.get_hidden_parameters().numpy(), t.get_hidden_parameters())
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    W = t.get_weights()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    lr = 0.01
    gran = dp.calc_weight_granularity()
    assert gran == pytest.approx(dp.dw_min * dp.piecewise_up[len(dp.piecewise_up) // 2])
    up = O.Up.from_c(cfg.update)
    assert np.array_equal(t.coincidences(X[0], Dm[0], lr, gran),
                          O.coincidences_det_implicit(X[0], Dm[0], lr, gran, up))
    dev = O.DeviceArrays.from_hidden(O.DEV_PIECEWISE_STEP, names, t.get_hidden_parameters(), 0.0, True)
    dev.pw = (dp.piecewise_up, dp.piecewise_down)
    t.set_learning_rate(lr)
    t.update(X, Dm)
    Wo = W.copy()
    O.update(Wo, X, Dm, lr, gran, up, dev)
    assert np.abs(t.get_weights() - Wo).max() <= 1e-6
    assert np.abs(t.get_weights() - W).max() > 1e-3  # the update did something


@pytest.mark.parametrize("kind,bl,ubl", [("cs", 31, True), ("sb", 100, True), ("cs", 20, False)])
def test_mean_count_pulse_type(kind, bl, ubl):
    """PulseType.MeanCount (the mean number of pulses per line, no fluctuation; pulse trains
    longer than 31 allowed): coincidences and weights after an update equal the compiled
    reference's."""
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(29)
    x_size, d_size, m = 40, 24, 12
    p = H.training_params(noise=False, pulse_det=True)
    p.update.pulse_type = D.PulseType.MeanCount
    p.update.desired_bl = bl
    p.update.update_bl_management = ubl
    p.update.update_management = ubl
    dp = H.device(kind, False)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = ref.RefTile(cfg)
    t.set_weights(rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32))
    W = t.get_weights()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.2, (m, d_size)).astype(np.float32)
    up = O.Up.from_c(cfg.update)
    lr = 0.02
    for s in range(3):
        for sign in (1.0, -1.0):
            c_ref = t.coincidences(X[s], Dm[s], sign * lr, dp.dw_min)
            c = O.coincidences_mean_count(X[s], Dm[s], sign * lr, dp.dw_min, up)
            assert np.array_equal(c_ref, c)
            assert np.abs(c).max() > 0
    dev = O.DeviceArrays.from_hidden(KIND[kind], t.hidden_parameter_names(), t.get_hidden_parameters(),
                                     0.0, bool(getattr(dp, "mult_noise", True)))
    t.set_learning_rate(lr)
    t.update(X, Dm)
    Wo = W.copy()
    O.update(Wo, X, Dm, lr, dp.dw_min, up, dev)
    assert np.abs(t.get_weights() - Wo).max() <= 1e-6
    assert np.abs(t.get_weights() - W).max() > 1e-3
