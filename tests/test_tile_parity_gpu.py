"""GPU parity of the single analog tile against the oracle, through the C ABI.

Deterministic regime (noise off, DeterministicImplicit pulses): coincidence counts bit-exact;
forward / backward within 1e-5 (relative to the output range) before the ADC and at most 0.1 %
of the elements off by one ADC step after it; weights after an update within 1e-6.
Noisy regime: first two moments within 4 sigma of their sampling error and a two-sample
Kolmogorov-Smirnov test with p > 0.01."""

import numpy as np
import pytest
import torch

from oracle import analog_tile_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

REL_TOL_PRE_ADC = 1e-5
MAX_LSB_FLIP_FRACTION = 1e-3
KS_P = 0.01


def _tile(p, dp, x, d, seed=5):
    from aihwkit_b200.rpu_base import tiles as T

    cfg = p._config(x, d, dp, seed=seed)
    return T.AnalogTile(cfg, cuda_device=0), cfg


def _inputs(rng, m, x, d):
    X = rng.uniform(-1, 1, (m, x)).astype(np.float32)
    Dm = rng.normal(0, 0.1, (m, d)).astype(np.float32)
    return X, Dm


SHAPES = [(64, 48, 17), (256, 256, 64), (100, 36, 33), (512, 512, 96)]


@pytest.mark.parametrize("x_size,d_size,m", SHAPES)
def test_forward_backward_pre_adc(x_size, d_size, m):
    """ADC off, noise off: only the MVM arithmetic differs from the oracle's fp32 product."""
    rng = np.random.default_rng(x_size + m)
    p = H.training_params(noise=False, pulse_det=True, bm=False, adc=False, out_bound=0.0)
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().numpy()
    X, Dm = _inputs(rng, m, x_size, d_size)
    X[1] = 0.0  # all-zero row: output is identically zero
    y = t.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    y_or = O.forward(W, X, O.IO.from_c(cfg.forward_io))
    assert np.abs(y - y_or).max() <= REL_TOL_PRE_ADC * np.abs(y_or).max()
    assert np.all(y[1] == 0)
    g = t.backward(torch.from_numpy(Dm).cuda()).cpu().numpy()
    g_or = O.backward(W, Dm, O.IO.from_c(cfg.backward_io, backward=True))
    assert np.abs(g - g_or).max() <= REL_TOL_PRE_ADC * np.abs(g_or).max()


@pytest.mark.parametrize("x_size,d_size,m", SHAPES)
@pytest.mark.parametrize("out_bound", [12.0, 2.0])
def test_forward_backward_post_adc(x_size, d_size, m, out_bound):
    """Full IO chain, noise off; out_bound = 2 forces iterative bound management to re-run."""
    rng = np.random.default_rng(7 * x_size + m)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=out_bound)
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().numpy()
    X, Dm = _inputs(rng, m, x_size, d_size)
    fio = O.IO.from_c(cfg.forward_io)
    y = t.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    y_or, _, scale, red = O.forward(W, X, fio, return_pre_adc=True)
    lsb = (fio.res_out / scale)[:, None]
    frac, worst = H.lsb_report(y, y_or, lsb)
    assert frac <= MAX_LSB_FLIP_FRACTION and worst <= 1.001, (frac, worst)
    n_rerun, max_red = t.last_bm_stats()
    assert n_rerun == int((red > 1).sum())
    assert max_red == float(red.max())
    if out_bound == 2.0:
        assert n_rerun > 0
    bio = O.IO.from_c(cfg.backward_io, backward=True)
    g = t.backward(torch.from_numpy(Dm).cuda()).cpu().numpy()
    g_or = O.backward(W, Dm, bio)
    s = np.abs(Dm).max(axis=1)
    frac, worst = H.lsb_report(g, g_or, (bio.res_out * s)[:, None])
    assert frac <= MAX_LSB_FLIP_FRACTION and worst <= 1.001, (frac, worst)


@pytest.mark.parametrize("trans", [(True, False), (False, True), (True, True)])
def test_transposed_layouts_and_bias(trans):
    """`batch first iff *_trans` layouts and the appended bias column give the same numbers."""
    x_trans, d_trans = trans
    rng = np.random.default_rng(3)
    x_size, d_size, m = 65, 40, 24
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=3.0)
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().numpy()
    X = rng.uniform(-1, 1, (m, x_size - 1)).astype(np.float32)  # bias=True: one feature less
    Xb = np.concatenate([X, np.ones((m, 1), np.float32)], axis=1)
    fio = O.IO.from_c(cfg.forward_io)
    y_or, _, scale, _ = O.forward(W, Xb, fio, return_pre_adc=True)
    xin = torch.from_numpy(np.ascontiguousarray(X.T if x_trans else X)).cuda()
    y = t.forward(xin, bias=True, x_trans=x_trans, d_trans=d_trans).cpu().numpy()
    y = y.T if d_trans else y
    frac, worst = H.lsb_report(y, y_or, (fio.res_out / scale)[:, None])
    assert frac <= 2e-3 and worst <= 1.001
    Dm = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    bio = O.IO.from_c(cfg.backward_io, backward=True)
    g_or = O.backward(W, Dm, bio)[:, : x_size - 1]
    din = torch.from_numpy(np.ascontiguousarray(Dm.T if d_trans else Dm)).cuda()
    g = t.backward(din, bias=True, d_trans=d_trans, x_trans=x_trans).cpu().numpy()
    g = g.T if x_trans else g
    assert g.shape == g_or.shape
    frac, worst = H.lsb_report(g, g_or, (bio.res_out * np.abs(Dm).max(axis=1))[:, None])
    assert frac <= 2e-3 and worst <= 1.001


@pytest.mark.parametrize("kind", ["cs", "ls", "sb", "sbr"])
@pytest.mark.parametrize("x_size,d_size,m", [(64, 48, 17), (256, 256, 64), (70, 130, 9)])
def test_deterministic_update_bit_exact_counts(kind, x_size, d_size, m):
    rng = np.random.default_rng(11 + x_size)
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.device(kind, False)
    t, cfg = _tile(p, dp, x_size, d_size)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().numpy()
    X, Dm = _inputs(rng, m, x_size, d_size)
    X[2] = 0.0  # no update for this sample
    up = O.Up.from_c(cfg.update)
    lr = 0.01
    t.set_learning_rate(lr)
    # pulse counts per element, sample by sample: bit-exact
    for s in (0, 2, m - 1):
        c = t.coincidences(torch.from_numpy(X[s]).cuda(), torch.from_numpy(Dm[s]).cuda()).cpu().numpy()
        c_or = O.coincidences_det_implicit(X[s], Dm[s], lr, dp.dw_min, up)
        assert np.array_equal(c, c_or)
    names = t.get_hidden_parameter_names()
    hp = t.get_hidden_parameters().numpy()
    dev = O.DeviceArrays.from_hidden(
        {"cs": O.DEV_CONSTANT_STEP, "ls": O.DEV_LINEAR_STEP, "sb": O.DEV_SOFT_BOUNDS,
         "sbr": O.DEV_SOFT_BOUNDS_REFERENCE}[kind], names, hp, 0.0, getattr(dp, "mult_noise", True))
    W_or = W.copy()
    O.update(W_or, X, Dm, lr, dp.dw_min, up, dev)
    t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
    W_new = t.get_weights().numpy()
    assert np.abs(W_new - W).max() > 0
    assert np.abs(W_new - W_or).max() <= 1e-6


def test_forward_noise_statistics():
    """Noise on: per-element mean / std of the output over repeats, and a KS test of the
    standardised residuals against the oracle's."""
    from scipy import stats

    rng = np.random.default_rng(5)
    x_size, d_size, m, reps = 128, 64, 8, 200
    p = H.training_params(noise=True, pulse_det=False, bm=True)
    t, cfg = _tile(p, H.device("cs", True), x_size, d_size)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().numpy()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    xg = torch.from_numpy(X).cuda()
    ys = np.stack([t.forward(xg).cpu().numpy() for _ in range(reps)])
    fio = O.IO.from_c(cfg.forward_io)
    org = np.random.default_rng(99)
    yo = np.stack([O.forward(W, X, fio, org) for _ in range(reps)])
    H.assert_moments_agree(ys, yo, std_tol=0.05)
    # successive calls must not repeat the noise
    assert not np.array_equal(ys[0], ys[1])
    ks = stats.ks_2samp((ys - yo.mean(axis=0)).ravel(), (yo - yo.mean(axis=0)).ravel())
    assert ks.pvalue > KS_P, ks


@pytest.mark.parametrize("kind", ["cs", "sb", "sbr"])
def test_stochastic_update_statistics(kind):
    """Noise on, StochasticCompressed pulses: mean and std of the weight change per element over
    repeats agree with the oracle (the reference's own test criterion, 2/sqrt(nloop) scaled)."""
    from scipy import stats

    rng = np.random.default_rng(17)
    x_size, d_size, m, reps = 32, 24, 10, 150
    p = H.training_params(noise=True, pulse_det=False)
    dp = H.device(kind, True)
    t, cfg = _tile(p, dp, x_size, d_size)
    W0 = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    X, Dm = _inputs(rng, m, x_size, d_size)
    up = O.Up.from_c(cfg.update)
    names = t.get_hidden_parameter_names()
    hp = t.get_hidden_parameters().numpy()
    dev = O.DeviceArrays.from_hidden(
        {"cs": O.DEV_CONSTANT_STEP, "sb": O.DEV_SOFT_BOUNDS, "sbr": O.DEV_SOFT_BOUNDS_REFERENCE}[kind],
        names, hp, dp.dw_min_std, getattr(dp, "mult_noise", True))
    lr = 0.05
    t.set_learning_rate(lr)
    xg, dg = torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda()
    dws, dwo = [], []
    org = np.random.default_rng(123)
    for _ in range(reps):
        t.set_weights(torch.from_numpy(W0))
        Wc = t.get_weights().numpy()
        t.update(xg, dg)
        dws.append(t.get_weights().numpy() - Wc)
        Wo = Wc.copy()
        O.update(Wo, X, Dm, lr, dp.dw_min, up, dev, org)
        dwo.append(Wo - Wc)
    dws, dwo = np.stack(dws), np.stack(dwo)
    H.assert_moments_agree(dws, dwo)
    # gradient direction: expected change follows -lr * d^T x
    grad = -(Dm.T @ X).ravel()
    corr = np.corrcoef(dws.mean(axis=0).ravel(), grad)[0, 1]
    corr_or = np.corrcoef(dwo.mean(axis=0).ravel(), grad)[0, 1]
    assert corr > 0.5 and abs(corr - corr_or) < 0.1
    ks = stats.ks_2samp(dws.sum(axis=(1, 2)), dwo.sum(axis=(1, 2)))
    assert ks.pvalue > KS_P, ks


def test_floating_point_tile_mimics_mac():
    """Perfect IO + floating-point update equal numpy (tests/test_bindings_tiles.py:138-177)."""
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(1)
    x_size, d_size, m = 30, 20, 12
    t = T.FloatingPointTile(x_size, d_size).cuda(0)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    X, Dm = _inputs(rng, m, x_size, d_size)
    y = t.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    np.testing.assert_allclose(y, X @ W.T, atol=1e-5)
    g = t.backward(torch.from_numpy(Dm).cuda()).cpu().numpy()
    np.testing.assert_allclose(g, Dm @ W, atol=1e-5)
    t.set_learning_rate(0.1)
    t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
    np.testing.assert_allclose(t.get_weights().numpy(), W - 0.1 * Dm.T @ X, atol=1e-5)


def test_host_buffer_entry_points_match_device_path():
    """CPU tensors go through the *_host entry points (pinned staging inside the library)."""
    rng = np.random.default_rng(2)
    x_size, d_size, m = 96, 80, 20
    p = H.training_params(noise=False, pulse_det=True)
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    X, Dm = _inputs(rng, m, x_size, d_size)
    y_dev = t.forward(torch.from_numpy(X).cuda()).cpu()
    y_host = t.forward(torch.from_numpy(X))
    assert not y_host.is_cuda and torch.equal(y_dev, y_host)
    g_dev = t.backward(torch.from_numpy(Dm).cuda()).cpu()
    g_host = t.backward(torch.from_numpy(Dm))
    assert torch.equal(g_dev, g_host)


def test_empty_batch_and_errors():
    p = H.training_params(noise=False, pulse_det=True)
    t, _ = _tile(p, H.device("cs", False), 16, 8)
    y = t.forward(torch.empty(0, 16).cuda())
    assert tuple(y.shape) == (0, 8)
    with pytest.raises(RuntimeError):
        t.forward(torch.zeros(4, 15).cuda())
    with pytest.raises(RuntimeError):
        t.set_weights(torch.zeros(3, 3))
    t.set_learning_rate(0.0)  # lr == 0: update is a no-op (rpu_weight_updater.cpp:206-208)
    w0 = t.get_weights()
    t.update(torch.ones(4, 16).cuda(), torch.ones(4, 8).cuda())
    assert torch.equal(w0, t.get_weights())


def _exp_step_device(noise, **kw):
    return H.device("es", noise, A_up=0.1, A_down=0.3, gamma_up=3.0, gamma_down=2.5, **kw)


def _es_arrays(t, dp, std):
    dev = O.DeviceArrays.from_hidden(O.DEV_EXP_STEP, t.get_hidden_parameter_names(),
                                     t.get_hidden_parameters().numpy(), std, True)
    dev.es = (dp.a, dp.b, dp.A_up, dp.A_down, dp.gamma_up, dp.gamma_down, dp.dw_min_std_add,
              dp.dw_min_std_slope)
    return dev


@pytest.mark.parametrize("x_size,d_size,m", [(64, 48, 17), (70, 130, 9)])
def test_exp_step_deterministic_update(x_size, d_size, m):
    """ExpStep device (rpu_expstep_device.cpp): bit-exact pulse counts with the device's own weight
    granularity, weights after the update within the expf rounding of the two platforms."""
    rng = np.random.default_rng(3 + x_size)
    p = H.training_params(noise=False, pulse_det=True)
    dp = _exp_step_device(False)
    t, cfg = _tile(p, dp, x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    X, Dm = _inputs(rng, m, x_size, d_size)
    up = O.Up.from_c(cfg.update)
    lr, gran = 0.01, dp.calc_weight_granularity()
    t.set_learning_rate(lr)
    c = t.coincidences(torch.from_numpy(X[0]).cuda(), torch.from_numpy(Dm[0]).cuda()).cpu().numpy()
    assert np.array_equal(c, O.coincidences_det_implicit(X[0], Dm[0], lr, gran, up))
    W_or = W.copy()
    O.update(W_or, X, Dm, lr, gran, up, _es_arrays(t, dp, 0.0))
    t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
    W_new = t.get_weights().numpy()
    assert np.abs(W_new - W).max() > 1e-3
    assert np.abs(W_new - W_or).max() <= 2e-6


@pytest.mark.parametrize("complex_noise", [False, True])
def test_exp_step_stochastic_update_statistics(complex_noise):
    rng = np.random.default_rng(19)
    x_size, d_size, m, reps = 32, 24, 10, 150
    p = H.training_params(noise=True, pulse_det=False)
    kw = dict(dw_min_std_add=0.5, dw_min_std_slope=0.3) if complex_noise else {}
    dp = _exp_step_device(True, **kw)
    t, cfg = _tile(p, dp, x_size, d_size)
    W0 = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    X, Dm = _inputs(rng, m, x_size, d_size)
    up = O.Up.from_c(cfg.update)
    dev = _es_arrays(t, dp, dp.dw_min_std)
    lr, gran = 0.05, dp.calc_weight_granularity()
    t.set_learning_rate(lr)
    xg, dg = torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda()
    dws, dwo = [], []
    org = np.random.default_rng(123)
    for _ in range(reps):
        t.set_weights(torch.from_numpy(W0))
        Wc = t.get_weights().numpy()
        t.update(xg, dg)
        dws.append(t.get_weights().numpy() - Wc)
        Wo = Wc.copy()
        O.update(Wo, X, Dm, lr, gran, up, dev, org)
        dwo.append(Wo - Wc)
    H.assert_moments_agree(np.stack(dws), np.stack(dwo))


@pytest.mark.parametrize("nm,bm", [("Max", "Iterative"), ("AbsMaxNPSum", "Iterative"),
                                   ("AbsMax", "IterativeWorstCase"), ("AbsMaxNPSum", "None_")])
@pytest.mark.parametrize("m", [24, 300])
def test_noise_and_bound_management_variants(nm, bm, m):
    """Max / AbsMaxNPSum noise management and IterativeWorstCase bound management against the
    oracle (pinned to the compiled reference in tests/test_oracle_vs_reference.py)."""
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(7)
    x_size, d_size = 96, 40
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=1.5)
    p.forward_io.noise_management = getattr(D.NoiseManagementType, nm)
    p.forward_io.bound_management = getattr(D.BoundManagementType, bm)
    p.forward_io.nm_assumed_wmax = 0.5
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    X[3] = -np.abs(X[3])
    X[5] *= 0.05
    fio = O.IO.from_c(cfg.forward_io)
    y_or, _, scale, _ = O.forward(W, X, fio, return_pre_adc=True)
    y = t.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    lsb = (fio.res_out / np.maximum(scale, 1e-30))[:, None]
    frac, worst = H.lsb_report(y, y_or, lsb)
    assert frac <= 3e-3 and worst <= 1.001, (frac, worst)
    if nm == "Max":
        assert (y[3] == 0).all()


def test_io_asymmetries():
    """inp_asymmetry / out_asymmetry on the GPU against the oracle, forward and backward, a batch
    small enough for the per-sample kernels and one large enough for the tiled ones."""
    rng = np.random.default_rng(17)
    x_size, d_size = 70, 33
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=4.0)
    for io in (p.forward_io, p.backward_io):
        io.inp_asymmetry, io.out_asymmetry = 0.1, 0.2
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    fio, bio = O.IO.from_c(cfg.forward_io), O.IO.from_c(cfg.backward_io, backward=True)
    for m in (20, 300):
        X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        Dm = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
        y_or, _, scale, _ = O.forward(W, X, fio, return_pre_adc=True)
        y = t.forward(torch.from_numpy(X).cuda()).cpu().numpy()
        frac, worst = H.lsb_report(y, y_or, (fio.res_out / scale)[:, None])
        assert frac <= 3e-3 and worst <= 1.001, (frac, worst)
        g_or = O.backward(W, Dm, bio)
        g = t.backward(torch.from_numpy(Dm).cuda()).cpu().numpy()
        frac, worst = H.lsb_report(g, g_or, (bio.res_out * np.abs(Dm).max(axis=1))[:, None])
        assert frac <= 3e-3 and worst <= 1.001, (frac, worst)


@pytest.mark.parametrize("what", ["inp_noise", "inp_sto_round", "out_sto_round"])
def test_io_random_input_stage_moments(what):
    """Input noise and stochastic DAC / ADC rounding: the GPU's samples and the oracle's (pinned to
    the compiled reference in tests/test_oracle_vs_reference.py) agree in their element-wise means
    and standard deviations; a zero row stays zero unless input noise is on."""
    rng = np.random.default_rng(19)
    x_size, d_size, m, reps = 40, 12, 6, 300
    p = H.training_params(noise=False, pulse_det=True)
    if what == "inp_noise":
        p.forward_io.inp_noise = 0.1
    else:
        p.forward_io.inp_res, p.forward_io.out_res = 1 / 14.0, 1 / 30.0
        setattr(p.forward_io, what, True)
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    X[2] = 0.0
    io = O.IO.from_c(cfg.forward_io)
    org = np.random.default_rng(1)
    xg = torch.from_numpy(X).cuda()
    ys = np.stack([t.forward(xg).cpu().numpy() for _ in range(reps)])
    ys_or = np.stack([O.forward(W, X, io, org) for _ in range(reps)])
    assert ys.std(axis=0).max() > 0
    if what == "inp_noise":
        assert ys[:, 2].std() > 0
    else:
        assert (ys[:, 2] == 0).all()
    H.assert_moments_agree(ys, ys_or)


def _pow_step_device(noise):
    return H.device("ps", noise, pow_gamma=1.3, pow_gamma_dtod=0.2, pow_up_down=0.1, pow_up_down_dtod=0.05)


@pytest.mark.parametrize("x_size,d_size,m", [(64, 48, 17), (70, 130, 9)])
def test_pow_step_deterministic_update(x_size, d_size, m):
    """PowStep device (rpu_powstep_device.cpp): bit-exact pulse counts with the device's own weight
    granularity, weights after the update within the powf rounding of the two platforms."""
    rng = np.random.default_rng(5 + x_size)
    p = H.training_params(noise=False, pulse_det=True)
    dp = _pow_step_device(False)
    t, cfg = _tile(p, dp, x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    X, Dm = _inputs(rng, m, x_size, d_size)
    up = O.Up.from_c(cfg.update)
    lr, gran = 0.01, dp.calc_weight_granularity()
    t.set_learning_rate(lr)
    c = t.coincidences(torch.from_numpy(X[0]).cuda(), torch.from_numpy(Dm[0]).cuda()).cpu().numpy()
    assert np.array_equal(c, O.coincidences_det_implicit(X[0], Dm[0], lr, gran, up))
    dev = O.DeviceArrays.from_hidden(O.DEV_POW_STEP, t.get_hidden_parameter_names(),
                                     t.get_hidden_parameters().numpy(), 0.0, True)
    W_or = W.copy()
    O.update(W_or, X, Dm, lr, gran, up, dev)
    t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
    W_new = t.get_weights().numpy()
    assert np.abs(W_new - W).max() > 1e-3
    assert np.abs(W_new - W_or).max() <= 3e-6


def test_pow_step_stochastic_update_statistics():
    rng = np.random.default_rng(23)
    x_size, d_size, m, reps = 32, 24, 10, 150
    p = H.training_params(noise=True, pulse_det=False)
    dp = _pow_step_device(True)
    t, cfg = _tile(p, dp, x_size, d_size)
    W0 = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    X, Dm = _inputs(rng, m, x_size, d_size)
    up = O.Up.from_c(cfg.update)
    dev = O.DeviceArrays.from_hidden(O.DEV_POW_STEP, t.get_hidden_parameter_names(),
                                     t.get_hidden_parameters().numpy(), dp.dw_min_std, True)
    lr, gran = 0.05, dp.calc_weight_granularity()
    t.set_learning_rate(lr)
    xg, dg = torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda()
    dws, dwo = [], []
    org = np.random.default_rng(123)
    for _ in range(reps):
        t.set_weights(torch.from_numpy(W0))
        Wc = t.get_weights().numpy()
        t.update(xg, dg)
        dws.append(t.get_weights().numpy() - Wc)
        Wo = Wc.copy()
        O.update(Wo, X, Dm, lr, gran, up, dev, org)
        dwo.append(Wo - Wc)
    H.assert_moments_agree(np.stack(dws), np.stack(dwo))


def _piecewise_arrays(t, dp, std):
    dev = O.DeviceArrays.from_hidden(O.DEV_PIECEWISE_STEP, t.get_hidden_parameter_names(),
                                     t.get_hidden_parameters().numpy(), std, True)
    dev.pw = (dp.piecewise_up, dp.piecewise_down)
    return dev


@pytest.mark.parametrize("x_size,d_size,m", [(64, 48, 17), (70, 130, 9), (256, 256, 300)])
def test_piecewise_step_deterministic_update(x_size, d_size, m):
    """PiecewiseStep device (rpu_piecewisestep_device.cpp:30-80): bit-exact pulse counts with the
    device's own granularity, weights after the update within 1e-6 of the oracle (which equals the
    compiled reference for this device, tests/test_oracle_vs_reference.py)."""
    rng = np.random.default_rng(5 + x_size)
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.piecewise_device(False)
    t, cfg = _tile(p, dp, x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    X, Dm = _inputs(rng, m, x_size, d_size)
    up = O.Up.from_c(cfg.update)
    lr, gran = 0.01, dp.calc_weight_granularity()
    t.set_learning_rate(lr)
    c = t.coincidences(torch.from_numpy(X[0]).cuda(), torch.from_numpy(Dm[0]).cuda()).cpu().numpy()
    assert np.array_equal(c, O.coincidences_det_implicit(X[0], Dm[0], lr, gran, up))
    W_or = W.copy()
    O.update(W_or, X, Dm, lr, gran, up, _piecewise_arrays(t, dp, 0.0))
    t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
    W_new = t.get_weights().numpy()
    assert np.abs(W_new - W).max() > 1e-3
    assert np.abs(W_new - W_or).max() <= 1e-6


def test_piecewise_step_stochastic_update_statistics():
    rng = np.random.default_rng(23)
    x_size, d_size, m, reps = 32, 24, 10, 150
    p = H.training_params(noise=True, pulse_det=False)
    dp = H.piecewise_device(True)
    t, cfg = _tile(p, dp, x_size, d_size)
    W0 = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    X, Dm = _inputs(rng, m, x_size, d_size)
    up = O.Up.from_c(cfg.update)
    dev = _piecewise_arrays(t, dp, dp.dw_min_std)
    lr, gran = 0.05, dp.calc_weight_granularity()
    t.set_learning_rate(lr)
    xg, dg = torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda()
    dws, dwo = [], []
    org = np.random.default_rng(123)
    for _ in range(reps):
        t.set_weights(torch.from_numpy(W0))
        Wc = t.get_weights().numpy()
        t.update(xg, dg)
        dws.append(t.get_weights().numpy() - Wc)
        Wo = Wc.copy()
        O.update(Wo, X, Dm, lr, gran, up, dev, org)
        dwo.append(Wo - Wc)
    H.assert_moments_agree(np.stack(dws), np.stack(dwo))


def test_piecewise_step_stream_kernel_equals_staged():
    """Both update kernels apply the same pulses in the same per-weight order."""
    from aihwkit_b200 import _cabi

    rng = np.random.default_rng(41)
    x_size, d_size, m = 96, 64, 1100
    p = H.training_params(noise=True, pulse_det=False)
    dp = H.piecewise_device(False)
    W0 = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    X, Dm = _inputs(rng, m, x_size, d_size)
    res = []
    lib = _cabi.lib()
    try:
        for path in (1, 2):
            lib.ab200_set_update_path(path)
            t, _ = _tile(p, dp, x_size, d_size)
            t.set_weights(torch.from_numpy(W0))
            t.set_learning_rate(0.05)
            t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
            res.append(t.get_weights().numpy())
    finally:
        lib.ab200_set_update_path(0)
    assert np.abs(res[0] - W0).max() > 1e-3
    assert np.array_equal(res[0], res[1])


@pytest.mark.parametrize("kind,bl,ubl", [("cs", 31, True), ("sb", 100, True), ("cs", 20, False)])
def test_mean_count_pulse_type(kind, bl, ubl):
    """PulseType.MeanCount on the GPU: bit-exact coincidence counts (pulse trains longer than 31
    included) and the weights after the update against the oracle."""
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(29)
    x_size, d_size, m = 70, 40, 40
    p = H.training_params(noise=False, pulse_det=True)
    p.update.pulse_type = D.PulseType.MeanCount
    p.update.desired_bl = bl
    p.update.update_bl_management = ubl
    p.update.update_management = ubl
    dp = H.device(kind, False)
    t, cfg = _tile(p, dp, x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    X, Dm = _inputs(rng, m, x_size, d_size)
    up = O.Up.from_c(cfg.update)
    lr = 0.02
    t.set_learning_rate(lr)
    for s in range(3):
        c = t.coincidences(torch.from_numpy(X[s]).cuda(), torch.from_numpy(Dm[s]).cuda()).cpu().numpy()
        assert np.array_equal(c, O.coincidences_mean_count(X[s], Dm[s], lr, dp.dw_min, up))
    names = t.get_hidden_parameter_names()
    kinds = {"cs": O.DEV_CONSTANT_STEP, "sb": O.DEV_SOFT_BOUNDS}
    dev = O.DeviceArrays.from_hidden(kinds[kind], names, t.get_hidden_parameters().numpy(), 0.0, True)
    W_or = W.copy()
    O.update(W_or, X, Dm, lr, dp.dw_min, up, dev)
    t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
    W_new = t.get_weights().numpy()
    assert np.abs(W_new - W).max() > 1e-3
    assert np.abs(W_new - W_or).max() <= 1e-6


@pytest.mark.parametrize("pulse_type", ["long_trains", "separate_sign_trains"])
def test_stochastic_update_long_trains_and_separate_sign_trains(pulse_type):
    """Pulse trains longer than one 32-bit word (desired_BL 80, learning rate large enough that
    update management asks for about 50 slots) and the `Stochastic` pulse type (separate trains
    for positive and negative lines): mean and spread of the weight change per element agree with
    the oracle's loop over the pulse slots."""
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(23)
    x_size, d_size, m, reps = 24, 20, 6, 150
    p = H.training_params(noise=True, pulse_det=False)
    if pulse_type == "long_trains":
        p.update.desired_bl = 80
        lr = 0.5
    else:
        p.update.pulse_type = D.PulseType.Stochastic
        lr = 0.05
    dp = H.device("cs", True)
    t, cfg = _tile(p, dp, x_size, d_size)
    W0 = rng.uniform(-0.2, 0.2, (d_size, x_size)).astype(np.float32)
    X, Dm = _inputs(rng, m, x_size, d_size)
    up = O.Up.from_c(cfg.update)
    up.pulse_type = O.PULSE_STOCHASTIC_COMPRESSED  # the oracle's compressed trains: same law
    if pulse_type == "long_trains":
        xm, dmx = np.abs(X).max(axis=1), np.abs(Dm).max(axis=1)
        assert (np.ceil(lr * xm * dmx / dp.dw_min) > 31).mean() > 0.5  # trains of more than one word
    hp = t.get_hidden_parameters().numpy()
    dev = O.DeviceArrays.from_hidden(O.DEV_CONSTANT_STEP, t.get_hidden_parameter_names(), hp,
                                     dp.dw_min_std, True)
    t.set_learning_rate(lr)
    xg, dg = torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda()
    dws, dwo = [], []
    org = np.random.default_rng(7)
    for _ in range(reps):
        t.set_weights(torch.from_numpy(W0))
        Wc = t.get_weights().numpy()
        t.update(xg, dg)
        dws.append(t.get_weights().numpy() - Wc)
        Wo = Wc.copy()
        O.update(Wo, X, Dm, lr, dp.dw_min, up, dev, org)
        dwo.append(Wo - Wc)
    dws, dwo = np.stack(dws), np.stack(dwo)
    H.assert_moments_agree(dws, dwo)
    assert np.abs(dws).max() > 0


def test_none_with_device_clips_after_every_sample():
    """PulseType::NoneWithDevice (rpu_weight_updater.cpp:216-223): the floating-point rank-one
    update of every sample is followed by the clip to the element's bounds, so a weight that
    reaches its bound in the middle of a batch continues from there."""
    from aihwkit_b200.rpu_base import devices as D
    from oracle import ref

    rng = np.random.default_rng(77)
    x_size, d_size, m = 70, 40, 24
    p = H.training_params(noise=False, pulse_det=True)
    p.update.pulse_type = D.PulseType.NoneWithDevice
    dp = H.device("cs", False, w_max=0.3, w_min=-0.3)
    t, cfg = _tile(p, dp, x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.2, 0.2, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    names, hp = t.get_hidden_parameter_names(), t.get_hidden_parameters().numpy()
    hi, lo = hp[names.index("max_bound")], hp[names.index("min_bound")]
    X, Dm = _inputs(rng, m, x_size, d_size)
    Dm *= 5.0
    lr = 0.2
    t.set_learning_rate(lr)
    t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
    W_new = t.get_weights().numpy()
    want, summed = W.copy(), W.copy()
    for s in range(m):
        want = np.clip(want - np.float32(lr) * np.outer(Dm[s], X[s]).astype(np.float32), lo, hi)
    summed = np.clip(W - np.float32(lr) * (Dm.T @ X), lo, hi)
    assert np.abs(W_new - want).max() <= 2e-6
    assert np.abs(summed - want).max() > 0.01  # the order of clip and sum matters for this input
    if ref.available():
        rt = ref.RefTile(cfg)
        rt.set_hidden_parameters(hp)
        rt.set_weights(W)
        rt.set_learning_rate(lr)
        rt.update(X, Dm)
        assert np.abs(W_new - rt.get_weights()).max() <= 2e-6


@pytest.mark.parametrize("nm", [5, 6])  # AverageAbsMax, AverageAbsMaxSingleValue (C ABI only)
def test_running_average_noise_management(nm):
    """AverageAbsMax noise management (rpu_forward_backward_pass.cpp:139-150): the input scale of a
    sample is the running value s <- s (1 - nm_decay) + nm_decay max|x| after that sample; the
    value carries over from call to call and is shared by forward and backward."""
    from aihwkit_b200.rpu_base import devices as D
    from oracle import ref

    rng = np.random.default_rng(61)
    x_size, d_size, m = 48, 40, 37
    p = H.training_params(noise=False, pulse_det=True, bm=False)
    for io in (p.forward_io, p.backward_io):
        io.noise_management = nm
        io.nm_decay = 0.1
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    fio = O.IO.from_c(cfg.forward_io)
    state = -1.0
    rt = None
    if ref.available():
        rt = ref.RefTile(cfg)
        rt.set_weights(W)
    for call in range(3):
        X = (rng.uniform(-1, 1, (m, x_size)) * rng.uniform(0.2, 1.5)).astype(np.float32)
        backward = call == 1
        inp = rng.normal(0, 0.3, (m, d_size)).astype(np.float32) if backward else X
        y = (t.backward if backward else t.forward)(torch.from_numpy(inp).cuda()).cpu().numpy()
        # the running value after every sample, then the chain of the oracle with that scale
        s_val = np.empty(m, np.float32)
        for s in range(m):
            amax = np.abs(inp[s]).max()
            state = amax if state < 0 else np.float32(state * np.float32(0.9) + np.float32(0.1) * amax)
            s_val[s] = state
        io_c = O.IO.from_c(cfg.backward_io if backward else cfg.forward_io, backward=backward)
        Wop = W.T if backward else W
        v = np.clip(np.rint((inp / s_val[:, None]) / io_c.res_in) * io_c.res_in, -1, 1).astype(np.float32)
        pre = (v @ Wop.T).astype(np.float32)
        want = np.clip(np.rint(pre / io_c.res_out) * io_c.res_out, -io_c.out_bound, io_c.out_bound)
        want = (want * s_val[:, None]).astype(np.float32)
        lsb = (io_c.res_out * s_val)[:, None]
        frac, worst = H.lsb_report(y, want, lsb)
        assert frac <= 2e-3 and worst <= 1.001, (call, frac, worst)
        if rt is not None:
            yr = rt.backward(inp) if backward else rt.forward(inp)
            frac, worst = H.lsb_report(y, yr, lsb)
            assert frac <= 2e-3 and worst <= 1.001, (call, frac, worst)
    assert fio.noise_management in (5, 6)


def test_stochastic_rounding_of_pulse_probabilities():
    """update.sto_round (sparse_bit_line_maker.cpp:174, :224; utility_functions.h:186-193): the
    pulse probabilities are rounded to `res` up or down at random, so a coarse `res` leaves the mean
    update where the fine one has it, while rounding to nearest moves it; moments against the
    compiled reference with the same setting."""
    from oracle import ref

    rng = np.random.default_rng(91)
    x_size, d_size, m, reps = 24, 16, 6, 200
    W0 = np.zeros((d_size, x_size), np.float32)
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)

    def mean_update(res, sto, use_ref=False):
        p = H.training_params(noise=False, pulse_det=False)
        p.update.res = res
        p.update.sto_round = sto
        dp = H.device("cs", False, dw_min_dtod=0.0, up_down_dtod=0.0, w_max_dtod=0.0, w_min_dtod=0.0)
        cfg = p._config(x_size, d_size, dp, seed=5)
        if use_ref:
            t = ref.RefTile(cfg)
            t.set_learning_rate(0.05)
            out = []
            for _ in range(reps):
                t.set_weights(W0)
                t.update(X, Dm)
                out.append(t.get_weights())
            return np.stack(out)
        from aihwkit_b200.rpu_base import tiles as T

        t = T.AnalogTile(cfg, cuda_device=0)
        t.set_learning_rate(0.05)
        xg, dg = torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda()
        out = []
        for _ in range(reps):
            t.set_weights(torch.from_numpy(W0))
            t.update(xg, dg)
            out.append(t.get_weights().numpy())
        return np.stack(out)

    fine = mean_update(0.0, False)
    sto = mean_update(0.25, True)
    near = mean_update(0.25, False)
    se = np.sqrt(fine.var(axis=0) / reps + sto.var(axis=0) / reps) + 1e-9
    z = (fine.mean(axis=0) - sto.mean(axis=0)) / se
    assert np.abs(z).max() < 5.5 and abs(z.mean()) < 0.5, (np.abs(z).max(), z.mean())
    # rounding to nearest at this resolution changes the update as a whole
    assert np.abs(near.mean(axis=0) - fine.mean(axis=0)).sum() > 0.2 * np.abs(fine.mean(axis=0)).sum()
    if ref.available():
        H.assert_moments_agree(sto, mean_update(0.25, True, use_ref=True))


@pytest.mark.parametrize("pulse_det", [False, True])
@pytest.mark.parametrize("m,bl", [(7, 31), (70, 31), (40, 80)])
def test_pulse_counters_account_for_the_weight_change(pulse_det, m, bl):
    """count_pulses: with a noise-free ConstantStep device far from its bounds the weight change
    of every element is (pulses up) * step_up - (pulses down) * step_down, through the staged and
    the streaming update kernel, one and several train segments, stochastic and implicit pulses;
    the counters add up over calls and are empty for a device that does not count."""
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(m + bl)
    x_size, d_size = 45, 37
    p = H.training_params(noise=False, pulse_det=pulse_det)
    p.update.desired_bl = bl
    dp = H.device("cs", False, dw_min=0.001, dw_min_dtod=0.3, up_down=0.1, up_down_dtod=0.05, w_max=5.0, w_min=-5.0,
                  w_max_dtod=0.0, w_min_dtod=0.0)
    assert T.AnalogTile(p._config(x_size, d_size, dp, seed=5), cuda_device=0).get_pulse_counters().numel() == 0
    dp.count_pulses = True
    t = T.AnalogTile(p._config(x_size, d_size, dp, seed=5), cuda_device=0)
    assert int(t.get_pulse_counters().abs().sum()) == 0
    names = t.get_hidden_parameter_names()
    hp = t.get_hidden_parameters().numpy().astype(np.float64)
    step_up, step_down = hp[names.index("dwmin_up")], hp[names.index("dwmin_down")]
    w0 = t.get_weights().numpy().astype(np.float64)
    t.set_learning_rate(0.05)
    total = None
    for k in range(3):
        X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        Dm = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
        t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
        c = t.get_pulse_counters().numpy()
        assert c.shape == (2, d_size, x_size) and (c >= 0).all()
        if total is not None:
            assert (c >= total).all()  # counters only grow
        total = c
    w1 = t.get_weights().numpy().astype(np.float64)
    want = total[0] * step_up - total[1] * step_down
    assert total.sum() > 10 * x_size * d_size // 20
    assert np.abs((w1 - w0) - want).max() <= 2e-5 + 1e-6 * np.abs(want).max(), np.abs((w1 - w0) - want).max()
    assert np.abs(w1).max() < 4.9  # no bound was reached
