"""GPU parity at the sizes the benchmarks run, so that the kernel variants the timed
configurations select are the ones under test:

* the four-weights-per-thread update kernel (chosen once the grid fills the GPU three times over)
  and more than one 128-sample super-block: SoftBounds 256 x 2304 with 640 columns, and the
  Tiki-Taka tile 1024 x 1024 with 256 columns and a transfer every second update;
* the mapped inference layer 4096 x 4096 on 64 tiles with a batch of 8192 rows (grouped work-item
  order with more than one chunk group, eight in-splits per work item);
* the convolution tile 256 x 2304 through the indexed interface on whole 32 x 32 images.

Criteria are the ones of the small-size tests (the reference's own, src/rpucuda/cuda/
rpucuda_pulsed_test.cpp:437-480, 1050-1131): deterministic pulses and noise off - weights within
1e-6 of the compiled reference / the oracle after every update; ADC outputs at most one step off
per in-split on at most 0.1 % of the elements; noise on - moments and a KS test."""

import numpy as np
import pytest
import torch

from oracle import analog_tile_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _gpu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _ref_or_none(cfg, hidden, w):
    """The compiled reference tile with the GPU tile's per-element parameters and weights."""
    from oracle import ref

    if not ref.available():
        return None
    rt = ref.RefTile(cfg)
    rt.set_hidden_parameters(hidden)
    rt.set_weights(w)
    return rt


def test_softbounds_update_conv_tile_deterministic():
    """256 x 2304 SoftBounds, 640 columns in one call: five super-blocks, four weights per thread."""
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(31)
    x_size, d_size, m = 2304, 256, 640
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.device("sb", False, dw_min=0.001, w_max=0.6, w_min=-0.6, dw_min_dtod=0.3)
    cfg = p._config(x_size, d_size, dp, seed=5)
    t = T.AnalogTile(cfg, cuda_device=0)
    W = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().numpy()
    hp = t.get_hidden_parameters().numpy()
    X = np.maximum(rng.standard_normal((m, x_size)), 0).astype(np.float32)
    Dm = rng.normal(0, 0.01, (m, d_size)).astype(np.float32)
    X[5] = 0.0
    lr = 0.01
    t.set_learning_rate(lr)
    rt = _ref_or_none(cfg, hp, W)
    if rt is not None:
        rt.set_learning_rate(lr)
        W = rt.get_weights()
    W_or = W.copy()
    for step in range(2):
        t.update(_gpu(X), _gpu(Dm))
        if rt is not None:
            rt.update(X, Dm)
            W_or = rt.get_weights()
        else:
            dev = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS, t.get_hidden_parameter_names(), hp, 0.0, True)
            O.update(W_or, X, Dm, lr, dp.dw_min, O.Up.from_c(cfg.update), dev)
        W_new = t.get_weights().numpy()
        assert np.abs(W_new - W).max() > 0
        assert np.abs(W_new - W_or).max() <= 1e-6, f"update {step}"


def test_softbounds_update_conv_tile_stochastic_statistics():
    """Stochastic pulses with device noise at the same size: the elements of one large update are
    the ensemble. Mean weight change per gradient bin and the spread agree with the reference."""
    from scipy import stats
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(32)
    x_size, d_size, m = 2304, 256, 1536  # large enough for the streaming update kernel
    p = H.training_params(noise=True, pulse_det=False)
    dp = H.device("sb", True, dw_min=0.001, w_max=0.6, w_min=-0.6, dw_min_dtod=0.3)
    cfg = p._config(x_size, d_size, dp, seed=5)
    t = T.AnalogTile(cfg, cuda_device=0)
    W0 = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W0))
    W0 = t.get_weights().numpy()
    hp = t.get_hidden_parameters().numpy()
    X = np.maximum(rng.standard_normal((m, x_size)), 0).astype(np.float32)
    Dm = rng.normal(0, 0.01, (m, d_size)).astype(np.float32)
    lr = 0.01
    t.set_learning_rate(lr)
    t.update(_gpu(X), _gpu(Dm))
    dw = t.get_weights().numpy() - W0
    rt = _ref_or_none(cfg, hp, W0)
    if rt is not None:
        rt.set_learning_rate(lr)
        rt.update(X, Dm)
        dwo = rt.get_weights() - W0
    else:
        dev = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS, t.get_hidden_parameter_names(), hp,
                                         dp.dw_min_std, True)
        Wo = W0.copy()
        O.update(Wo, X, Dm, lr, dp.dw_min, O.Up.from_c(cfg.update), dev, np.random.default_rng(1))
        dwo = Wo - W0
    grad = -(Dm.T @ X)
    # both follow the gradient equally well
    c, co = np.corrcoef(dw.ravel(), grad.ravel())[0, 1], np.corrcoef(dwo.ravel(), grad.ravel())[0, 1]
    assert c > 0.1 and abs(c - co) < 0.02, (c, co)
    # mean change per gradient decile and overall spread
    edges = np.quantile(grad, np.linspace(0, 1, 11))
    which = np.clip(np.searchsorted(edges, grad.ravel(), side="right") - 1, 0, 9)
    for b in range(10):
        a, r = dw.ravel()[which == b], dwo.ravel()[which == b]
        se = np.sqrt(a.var() / a.size + r.var() / r.size)
        assert abs(a.mean() - r.mean()) < 6 * se, (b, a.mean(), r.mean(), se)
    assert abs(dw.std() / dwo.std() - 1.0) < 0.03
    # distribution of the changes on a random subset of the elements
    pick = rng.choice(dw.size, 4000, replace=False)
    ks = stats.ks_2samp(dw.ravel()[pick], dwo.ravel()[pick])
    assert ks.pvalue > 0.01, ks


def test_tiki_taka_benchmark_tile_deterministic():
    """TransferCompound of two SoftBoundsReference devices, 1024 x 1024, 256 columns per update,
    transfer every 2 updates, deterministic pulses: fast tile and visible weights follow the
    compiled reference update by update."""
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(33)
    x_size = d_size = 1024
    m = 256
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.transfer_device(noise=False, det=True, transfer_every=2.0, units_in_mbatch=True,
                           n_reads=1, transfer_lr=1.0)
    cfg = p._config(x_size, d_size, dp, seed=9)
    t = T.AnalogTile(cfg, cuda_device=0)
    names = t.get_hidden_parameter_names()
    hp = t.get_hidden_parameters().numpy()
    ia = names.index("hidden_weights_0")
    rt = _ref_or_none(cfg, hp, np.zeros((d_size, x_size), np.float32))
    orc = None
    if rt is None:
        fast = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS_REFERENCE, names, hp, 0.0, False, suffix="_0")
        slow = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS_REFERENCE, names, hp, 0.0, False, suffix="_1")
        orc = O.TransferOracle(t.get_weights().numpy().copy(), fast, slow, cfg.transfer,
                               O.Up.from_c(cfg.update), dp._vec_par[0].dw_min, dp._vec_par[1].dw_min,
                               x_size, d_size)
    lr = 0.05
    t.set_learning_rate(lr)
    if rt is not None:
        rt.set_learning_rate(lr)
    moved = False
    for step in range(4):
        X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        Dm = rng.normal(0, 0.05, (m, d_size)).astype(np.float32)
        t.update(_gpu(X), _gpu(Dm))
        if rt is not None:
            rt.update(X, Dm)
            a_or = rt.get_hidden_parameters()[rt.hidden_parameter_names().index("hidden_weights_0")]
            c_or = rt.get_weights()
        else:
            orc.update(X, Dm, lr)
            a_or, c_or = orc.w_fast, orc.w
        a = t.get_hidden_parameters().numpy()[ia]
        c = t.get_weights().numpy()
        assert np.abs(a - a_or).max() <= 1e-6, f"fast tile, update {step}"
        assert np.abs(c - c_or).max() <= 1e-6, f"visible weights, update {step}"
        moved = moved or np.abs(c).max() > 0
    assert np.abs(a).max() > 0 and moved


def _layer_oracle(W, X, cfg, max_tile, rng=None):
    from aihwkit_b200.sharded import split_sizes

    io = O.IO.from_c(cfg.forward_io)
    out_sizes, in_sizes = split_sizes(W.shape[0], max_tile), split_sizes(W.shape[1], max_tile)
    y = np.zeros((X.shape[0], W.shape[0]), np.float32)
    lsb = np.zeros_like(y)
    c0 = 0
    for isz in in_sizes:
        r0 = 0
        for osz in out_sizes:
            yt, _, scale, _ = O.forward(W[r0:r0 + osz, c0:c0 + isz], X[:, c0:c0 + isz], io, rng,
                                        return_pre_adc=True)
            y[:, r0:r0 + osz] += yt
            lsb[:, r0:r0 + osz] = np.maximum(lsb[:, r0:r0 + osz], (io.res_out / scale)[:, None])
            r0 += osz
        c0 += isz
    return y, lsb, len(in_sizes)


def test_inference_layer_full_size_noise_off():
    """Benchmark configuration 1 at its own size: 4096 x 4096 on 64 tiles, 8192 rows."""
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(41)
    size, max_tile, m = 4096, 512, 8192
    p = H.inference_params(noise=False)
    cfg = p._config(1, 1, D.IdealResistiveDeviceParameter(), seed=3)
    arr = T.TileArray(cfg, size, size, max_tile, max_tile, cuda_device=0)
    W = (rng.standard_normal((size, size)) / 64.0).astype(np.float32)
    arr.set_weights(torch.from_numpy(W))
    X = rng.standard_normal((m, size)).astype(np.float32)
    X[17] = 0.0
    y = arr.forward(_gpu(X)).cpu().numpy()
    y_or, lsb, n_in = _layer_oracle(W, X, cfg, max_tile)
    diff = np.abs(y - y_or)
    assert np.all(y[17] == 0)
    assert (diff > 1e-3 * lsb).mean() <= 1e-3 * n_in
    assert (diff <= 1.001 * lsb * n_in).all()


def test_inference_layer_full_size_noise_statistics():
    """The same layer with the inference noise: repeated full-batch calls, compared on a few rows
    from the first, a middle and the last work item with the oracle's moments and a KS test."""
    from scipy import stats
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(42)
    size, max_tile, m, reps = 4096, 512, 8192, 60
    p = H.inference_params(noise=True)
    cfg = p._config(1, 1, D.IdealResistiveDeviceParameter(), seed=3)
    arr = T.TileArray(cfg, size, size, max_tile, max_tile, cuda_device=0)
    W = (rng.standard_normal((size, size)) / 64.0).astype(np.float32)
    arr.set_weights(torch.from_numpy(W))
    X = rng.standard_normal((m, size)).astype(np.float32)
    rows = np.array([0, 1, 255, 256, 4099, 4100, 8190, 8191])
    cols = np.r_[0:64, 2040:2104, 4032:4096]
    xg = _gpu(X)
    ys = np.stack([arr.forward(xg)[rows][:, cols].cpu().numpy() for _ in range(reps)])
    org = np.random.default_rng(1)
    yo = np.stack([_layer_oracle(W, X[rows], cfg, max_tile, org)[0][:, cols] for _ in range(reps)])
    H.assert_moments_agree(ys, yo, std_tol=0.05)
    ks = stats.ks_2samp((ys - yo.mean(axis=0)).ravel(), (yo - yo.mean(axis=0)).ravel())
    assert ks.pvalue > 0.01, ks


def test_conv_tile_indexed_on_whole_images():
    """Benchmark configuration 3's tile (256 x 2304, 3 x 3 kernel, 256 channels, 32 x 32 maps)
    through forward_indexed / backward_indexed / update_indexed on four images (4096 columns)."""
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(43)
    n, c, h, w, c_out = 4, 256, 32, 32, 256
    idx = O.conv_indices((c, h, w), (3, 3), (1, 1), (1, 1))
    x_size = c * 9
    m_batch = idx.size // x_size
    p = H.training_params(noise=False, pulse_det=True, bm=True)
    dp = H.device("sb", False, dw_min=0.001, w_max=0.6, w_min=-0.6, dw_min_dtod=0.3)
    cfg = p._config(x_size, c_out, dp, seed=5)
    t = T.AnalogTile(cfg, cuda_device=0)
    w0 = (rng.standard_normal((c_out, x_size)) * 0.05).astype(np.float32)
    t.set_weights(torch.from_numpy(w0))
    w0 = t.get_weights().numpy()
    hp = t.get_hidden_parameters().numpy()
    t.set_matrix_indices(_gpu(idx))
    X = np.maximum(rng.standard_normal((n, c, h, w)), 0).astype(np.float32)
    Dm = rng.normal(0, 0.01, (n, c_out, h, w)).astype(np.float32)
    fio, bio = O.IO.from_c(cfg.forward_io), O.IO.from_c(cfg.backward_io, backward=True)

    cols = O.indexed_input(X, idx, x_size, m_batch, n, True)
    y_ref, _, scale, _ = O.forward(w0, cols, fio, return_pre_adc=True)
    y = t.forward_indexed(_gpu(X), torch.empty(n, c_out, h, w, device="cuda")).cpu().numpy()
    got = O.to_sample_major(y, c_out, m_batch, n, True)
    frac, worst = H.lsb_report(got, y_ref, (fio.res_out / scale)[:, None])
    assert frac <= 5e-3 and worst <= 1.001, (frac, worst)

    d_cols = O.to_sample_major(Dm, c_out, m_batch, n, True)
    xg_ref = O.indexed_output(O.backward(w0, d_cols, bio), idx, x_size, m_batch, n, True, X.size)
    xg = t.backward_indexed(_gpu(Dm), torch.full(X.shape, 7.0, device="cuda")).cpu().numpy()
    step = float((bio.res_out * np.abs(d_cols).max(axis=1)).max())
    diff = np.abs(xg.reshape(n, -1) - xg_ref)
    assert diff.max() <= 1.001 * step and np.mean(diff > 1e-6) <= 5e-3

    lr = 0.01
    t.set_learning_rate(lr)
    t.update_indexed(_gpu(X), _gpu(Dm))
    rt = _ref_or_none(cfg, hp, w0)
    if rt is not None:
        rt.set_learning_rate(lr)
        rt.update(cols, d_cols)
        w1 = rt.get_weights()
    else:
        dev = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS, t.get_hidden_parameter_names(), hp, 0.0, True)
        w1 = w0.copy()
        O.update(w1, cols, d_cols, lr, dp.dw_min, O.Up.from_c(cfg.update), dev)
    w_new = t.get_weights().numpy()
    assert np.abs(w_new - w0).max() > 0
    assert np.abs(w_new - w1).max() <= 1e-6


@pytest.mark.parametrize("kind,x_size,d_size,m", [("sb", 2304, 256, 1536), ("cs", 300, 100, 70),
                                                  ("sbr", 256, 256, 1100)])
def test_streaming_update_equals_staged_update(kind, x_size, d_size, m):
    """The two kernels of the stochastic pulsed update - blocks of samples staged per weight tile,
    and the stream over the samples of each x-line that large batches take - see the same pulse
    trains (same noise key and call counter) and apply the same pulses in the same per-weight
    order: without device noise their results are identical bit for bit."""
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import tiles as T

    lib = _cabi.lib()
    rng = np.random.default_rng(x_size)
    p = H.training_params(noise=True, pulse_det=False)
    dp = H.device(kind, False, dw_min=0.001, dw_min_dtod=0.3)  # per-element spread, no pulse noise
    cfg = p._config(x_size, d_size, dp, seed=5)
    W0 = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    X = np.maximum(rng.standard_normal((m, x_size)), 0).astype(np.float32)
    Dm = rng.normal(0, 0.05, (m, d_size)).astype(np.float32)
    results = []
    try:
        for mode in (1, 2):
            _cabi.check(lib.ab200_set_update_path(mode))
            t = T.AnalogTile(cfg, cuda_device=0)
            t.set_weights(torch.from_numpy(W0))
            t.set_learning_rate(0.02)
            for _ in range(2):
                t.update(_gpu(X), _gpu(Dm))
            results.append(t.get_weights().numpy())
    finally:
        _cabi.check(lib.ab200_set_update_path(0))
    assert np.abs(results[0] - W0).max() > 0
    assert np.array_equal(results[0], results[1])
