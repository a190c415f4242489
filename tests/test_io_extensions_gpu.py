"""GPU checks of two IO settings whose noise std-dev differs from element to element:

* ``w_noise_type = PCMRead``: the Gaussian added to output i has std-dev
  ``w_noise * sqrt(sum_j |w_ij| v_j^2)``, v the DAC output
  (src/rpucuda/rpu_forward_backward_pass.cpp:353-381);
* ``out_noise_std``: every output line keeps ``|out_noise * (1 + out_noise_std * N(0,1))|`` for the
  life of the tile (:306-313, :696), forward and backward lines drawn separately.

Both are random, so the criteria are moments: the empirical std-dev of every output element over
repeated calls against the closed form (PCMRead) and against the compiled reference tile run on
the same inputs; the spread, mean and persistence of the per-line values (out_noise_std)."""

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _params(out_noise, w_noise=0.0, pcm=False, out_noise_std=0.0):
    from aihwkit_b200.rpu_base import devices as D

    p = H.training_params(noise=False, pulse_det=True, bm=False, adc=False, out_bound=0.0)
    for io in (p.forward_io, p.backward_io):
        io.out_noise = out_noise
        io.out_noise_std = out_noise_std
        io.w_noise = w_noise
        io.w_noise_type = D.WeightNoiseType.PCMRead if pcm else D.WeightNoiseType.None_
    return p


def _repeat(fn, n):
    return np.stack([fn() for _ in range(n)])


@pytest.mark.parametrize("x_size,d_size,m", [(128, 96, 16), (300, 70, 40)])
def test_pcm_read_noise_std_per_element(x_size, d_size, m):
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    rng = np.random.default_rng(x_size)
    p = _params(out_noise=0.0, w_noise=0.1, pcm=True)
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=9)
    t = T.AnalogTile(cfg, cuda_device=0)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().cpu().numpy()  # clipped to the bounds of the devices
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    xg = torch.from_numpy(X).cuda()
    reps = 400
    ys = _repeat(lambda: t.forward(xg).cpu().numpy(), reps)
    # closed form: v = DAC(x / amax), output rescaled by amax
    amax = np.abs(X).max(axis=1, keepdims=True)
    res = np.float32(2.0 / 126.0)
    v = np.clip(np.rint(X / amax / res) * res, -1, 1)
    sig = 0.1 * np.sqrt((v.astype(np.float64) ** 2) @ np.abs(W.astype(np.float64)).T) * amax
    mean = (v.astype(np.float64) @ W.astype(np.float64).T) * amax
    est = ys.std(axis=0)
    # sampling error of a std-dev estimate from `reps` draws: 1 / sqrt(2 reps) = 3.5 %
    ratio = est / sig
    assert abs(ratio.mean() - 1.0) < 0.01, ratio.mean()
    assert np.abs(ratio - 1.0).max() < 5.5 / np.sqrt(2 * reps), np.abs(ratio - 1.0).max()
    zmean = (ys.mean(axis=0) - mean) / (sig / np.sqrt(reps))
    assert np.abs(zmean).max() < 5.5, np.abs(zmean).max()
    # backward: the transposed weights, std-dev per input line
    Dm = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
    dg = torch.from_numpy(Dm).cuda()
    gs = _repeat(lambda: t.backward(dg).cpu().numpy(), reps)
    dmax = np.abs(Dm).max(axis=1, keepdims=True)
    vd = np.clip(np.rint(Dm / dmax / res) * res, -1, 1)
    sig_b = 0.1 * np.sqrt((vd.astype(np.float64) ** 2) @ np.abs(W.astype(np.float64))) * dmax
    rb = gs.std(axis=0) / sig_b
    assert abs(rb.mean() - 1.0) < 0.01 and np.abs(rb - 1.0).max() < 5.5 / np.sqrt(2 * reps)
    if ref.available():
        rt = ref.RefTile(cfg)
        rt.set_weights(W)
        yr = _repeat(lambda: rt.forward(X), reps)
        rr = est / yr.std(axis=0)
        assert abs(rr.mean() - 1.0) < 0.015 and np.abs(rr - 1.0).max() < 0.3, (rr.mean(), rr.max())


def test_pcm_read_with_bound_management_rerun():
    """Rows that clip are re-run with a halved input: the re-run kernel draws with the std-dev of
    the halved input as well."""
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(3)
    x_size, d_size, m = 64, 32, 8
    p = H.training_params(noise=False, pulse_det=True, bm=True, adc=False, out_bound=1.0)
    p.forward_io.w_noise = 0.05
    p.forward_io.w_noise_type = D.WeightNoiseType.PCMRead
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=9)
    t = T.AnalogTile(cfg, cuda_device=0)
    W = np.full((d_size, x_size), 0.05, np.float32)  # every output = 0.05 * sum(v): clips at 1
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().cpu().numpy()  # clipped to the bounds of the devices
    X = rng.uniform(0.5, 1.0, (m, x_size)).astype(np.float32)
    xg = torch.from_numpy(X).cuda()
    ys = _repeat(lambda: t.forward(xg).cpu().numpy(), 300)
    n_rerun, max_red = t.last_bm_stats()
    assert n_rerun == m and max_red >= 2.0
    exact = X @ W.T
    # bound management recovers the unclipped value (up to the coarser DAC grid) plus noise
    assert np.abs(ys.mean(axis=0) - exact).max() < 0.05 * np.abs(exact).max()
    assert ys.std(axis=0).min() > 0.0


def test_out_noise_std_per_line_values_persist():
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    rng = np.random.default_rng(17)
    x_size, d_size, m = 96, 256, 32
    out_noise, spread = 0.1, 0.4
    p = _params(out_noise=out_noise, out_noise_std=spread)
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=21)
    t = T.AnalogTile(cfg, cuda_device=0)
    W = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().cpu().numpy()  # clipped to the bounds of the devices
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    X /= np.abs(X).max(axis=1, keepdims=True)  # abs-max 1: the output factor is 1 for every row
    xg = torch.from_numpy(X).cuda()
    reps = 100
    ys = _repeat(lambda: t.forward(xg).cpu().numpy(), reps)
    dev = ys - ys.mean(axis=0, keepdims=True)
    # per-line std-dev from the two halves of the repeats: the same lines are noisy in both
    a = dev[: reps // 2].reshape(-1, d_size).std(axis=0)
    b = dev[reps // 2:].reshape(-1, d_size).std(axis=0)
    assert np.corrcoef(a, b)[0, 1] > 0.98
    line = dev.reshape(-1, d_size).std(axis=0) * np.sqrt(reps / (reps - 1.0))
    # E|1 + s z| = 1 up to the 0.6 % of the mass below zero; spread of 256 lines: +-4.4 % (1 sigma)
    assert abs(line.mean() / out_noise - 1.0) < 0.1, line.mean()
    assert abs(line.std() / line.mean() / spread - 1.0) < 0.2, line.std() / line.mean()
    # the backward lines have their own values (x_size of them)
    Dm = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
    Dm /= np.abs(Dm).max(axis=1, keepdims=True)
    dg = torch.from_numpy(Dm).cuda()
    gs = _repeat(lambda: t.backward(dg).cpu().numpy(), reps)
    gdev = (gs - gs.mean(axis=0, keepdims=True)).reshape(-1, x_size)
    gline = gdev.std(axis=0) * np.sqrt(reps / (reps - 1.0))
    assert abs(gline.mean() / out_noise - 1.0) < 0.15
    assert abs(gline.std() / gline.mean() / spread - 1.0) < 0.35
    # a second tile with another seed has other lines
    cfg2 = p._config(x_size, d_size, H.device("cs", False), seed=22)
    t2 = T.AnalogTile(cfg2, cuda_device=0)
    t2.set_weights(torch.from_numpy(W))
    y2 = _repeat(lambda: t2.forward(xg).cpu().numpy(), reps)
    line2 = (y2 - y2.mean(axis=0, keepdims=True)).reshape(-1, d_size).std(axis=0)
    assert np.corrcoef(line, line2)[0, 1] < 0.5
    if ref.available():
        rt = ref.RefTile(cfg)
        rt.set_weights(W)
        yr = _repeat(lambda: rt.forward(X), reps)
        rline = (yr - yr.mean(axis=0, keepdims=True)).reshape(-1, d_size).std(axis=0)
        assert abs(rline.mean() / line.mean() - 1.0) < 0.15
        assert abs((rline.std() / rline.mean()) / (line.std() / line.mean()) - 1.0) < 0.3


def test_line_noise_settings_take_the_cuda_core_kernels_at_tensor_core_sizes():
    """A mapped-layer-sized forward with PCMRead noise is accepted (the tensor-core kernel is not
    eligible) and its noise follows the closed form on a sample of elements."""
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(5)
    x_size, d_size, m = 512, 512, 512
    p = _params(out_noise=0.02, w_noise=0.05, pcm=True)
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=9)
    t = T.AnalogTile(cfg, cuda_device=0)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().cpu().numpy()  # clipped to the bounds of the devices
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    xg = torch.from_numpy(X).cuda()
    reps = 60
    ys = _repeat(lambda: t.forward(xg)[:8].cpu().numpy(), reps)
    amax = np.abs(X[:8]).max(axis=1, keepdims=True)
    res = np.float32(2.0 / 126.0)
    v = np.clip(np.rint(X[:8] / amax / res) * res, -1, 1).astype(np.float64)
    sig = np.sqrt(0.02 ** 2 + 0.05 ** 2 * ((v ** 2) @ np.abs(W.astype(np.float64)).T)) * amax
    ratio = ys.std(axis=0) / sig
    assert abs(ratio.mean() - 1.0) < 0.02 and np.abs(ratio - 1.0).max() < 0.5


_LINE_SETTINGS = {
    "ir_drop": dict(ir_drop=1.5, ir_drop_g_ratio=3000.0),  # a wire ratio that makes the drop visible
    "v_offset": dict(v_offset_std=0.05),
    "r_series": dict(v_offset_std=0.03, r_series=0.02),
    "nonlinearity": dict(out_nonlinearity=0.15, out_nonlinearity_std=0.2),
    "all": dict(ir_drop=1.0, ir_drop_g_ratio=3000.0, v_offset_std=0.05, r_series=0.02, out_nonlinearity=0.1,
                out_nonlinearity_std=0.2),
}


@pytest.mark.parametrize("name", sorted(_LINE_SETTINGS))
@pytest.mark.parametrize("bm", [False, True])
def test_line_non_idealities_against_reference(name, bm):
    """IR drop, voltage offsets, series resistance and output non-linearity
    (src/rpucuda/rpu_forward_backward_pass.cpp:388-517, :673-719) with noise off: the GPU tile,
    given the per-line values the compiled reference drew, returns the reference's outputs up to
    single ADC steps; forward (with and without bound-management re-runs) and backward."""
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    if not ref.available():
        pytest.skip("compiled reference not built")
    rng = np.random.default_rng(len(name))
    x_size, d_size, m = 150, 70, 48
    p = H.training_params(noise=False, pulse_det=True, bm=bm, out_bound=2.0 if bm else 12.0)
    for io in (p.forward_io, p.backward_io):
        for k, v in _LINE_SETTINGS[name].items():
            setattr(io, k, v)
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=9)
    t = T.AnalogTile(cfg, cuda_device=0)
    rt = ref.RefTile(cfg)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().cpu().numpy()
    rt.set_weights(W)
    for backward, n in ((False, d_size), (True, x_size)):
        for which in (0, 1):
            v = rt.get_io_vector(backward, which, n)
            if v.size:
                assert t.get_io_vector(backward, which).numel() == n
                t.set_io_vector(backward, which, torch.from_numpy(v))
                assert np.array_equal(t.get_io_vector(backward, which).numpy(), v)
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
    y = t.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    yr = rt.forward(X)
    res_out = 2.0 * (2.0 if bm else 12.0) / 510.0
    # the unit of comparison: one ADC step of the row at its last bound-management round
    lsb = res_out * np.abs(X).max(axis=1, keepdims=True) * (t.last_bm_stats()[1] if bm else 1.0)
    frac, worst = H.lsb_report(y, yr, lsb)
    assert frac <= 5e-3 and worst <= 1.001, (frac, worst)
    if bm:
        assert t.last_bm_stats()[0] > 0
    # the setting changes the output (against the same tile without it)
    p0 = H.training_params(noise=False, pulse_det=True, bm=bm, out_bound=2.0 if bm else 12.0)
    t0 = T.AnalogTile(p0._config(x_size, d_size, H.device("cs", False), seed=9), cuda_device=0)
    t0.set_weights(torch.from_numpy(W))
    assert np.abs(t0.forward(torch.from_numpy(X).cuda()).cpu().numpy() - y).max() > 2 * res_out
    g = t.backward(torch.from_numpy(Dm).cuda()).cpu().numpy()
    gr = rt.backward(Dm)
    lsb_b = (2.0 * 12.0 / 510.0) * np.abs(Dm).max(axis=1, keepdims=True)
    frac, worst = H.lsb_report(g, gr, lsb_b)
    assert frac <= 5e-3 and worst <= 1.001, (frac, worst)


def test_weight_noise_enters_before_the_non_linearity():
    """With an output non-linearity the additive weight noise is compressed by it while the output
    noise is not: the std-dev of an output follows nlf / (1 + |nl y|)^2 * w_noise ||v|| (first
    order) instead of the merged sqrt(w^2 + o^2)."""
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(12)
    x_size, d_size, m = 64, 32, 8
    p = H.training_params(noise=False, pulse_det=True, bm=False, adc=False, out_bound=0.0)
    p.forward_io.w_noise = 0.02
    p.forward_io.w_noise_type = D.WeightNoiseType.AdditiveConstant
    p.forward_io.out_nonlinearity = 0.5
    p.forward_io.slope_calibration = 0.0
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=9)
    t = T.AnalogTile(cfg, cuda_device=0)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().cpu().numpy()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    X /= np.abs(X).max(axis=1, keepdims=True)
    xg = torch.from_numpy(X).cuda()
    ys = _repeat(lambda: t.forward(xg).cpu().numpy(), 300)
    res = np.float32(2.0 / 126.0)
    v = np.clip(np.rint(X / res) * res, -1, 1).astype(np.float64)
    y0 = v @ W.astype(np.float64).T
    nl = t.get_io_vector(False, 1).numpy().astype(np.float64)[None, :]
    sig = 0.02 * np.sqrt((v ** 2).sum(axis=1, keepdims=True)) / (1.0 + np.abs(nl * y0)) ** 2
    ratio = ys.std(axis=0) / sig
    assert abs(ratio.mean() - 1.0) < 0.02, ratio.mean()


@pytest.mark.parametrize("mv", ["PosNegSeparate", "PosNegSeparateDigitalSum"])
@pytest.mark.parametrize("bm", [False, True])
@pytest.mark.parametrize("lines", ["none", "all"])
def test_pos_neg_separate_against_reference(mv, bm, lines):
    """Negative and positive inputs in two passes through the array, summed before or after the
    output stage (computeAnalogMV, src/rpucuda/rpu_forward_backward_pass.cpp:820-876), noise
    off: outputs of the compiled reference up to single ADC steps (two for the digital sum, whose
    two conversions can each flip), forward with and without bound-management re-runs, and
    backward; alone and on top of the line non-idealities, which each pass sees on its own."""
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    if not ref.available():
        pytest.skip("compiled reference not built")
    rng = np.random.default_rng(31)
    x_size, d_size, m = 150, 70, 48
    out_bound = 2.0 if bm else 12.0
    p = H.training_params(noise=False, pulse_det=True, bm=bm, out_bound=out_bound)
    for io in (p.forward_io, p.backward_io):
        io.mv_type = getattr(D.AnalogMVType, mv)
        if lines == "all":
            for k, v in _LINE_SETTINGS["all"].items():
                setattr(io, k, v)
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=9)
    t = T.AnalogTile(cfg, cuda_device=0)
    rt = ref.RefTile(cfg)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().cpu().numpy()
    rt.set_weights(W)
    if lines == "all":
        for backward, n in ((False, d_size), (True, x_size)):
            for which in (0, 1):
                v = rt.get_io_vector(backward, which, n)
                if v.size:
                    t.set_io_vector(backward, which, torch.from_numpy(v))
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
    steps = 2.002 if mv.endswith("DigitalSum") else 1.001
    y = t.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    yr = rt.forward(X)
    res_out = 2.0 * out_bound / 510.0
    lsb = res_out * np.abs(X).max(axis=1, keepdims=True) * (t.last_bm_stats()[1] if bm else 1.0)
    frac, worst = H.lsb_report(y, yr, lsb)
    assert frac <= 1e-2 and worst <= steps, (frac, worst)
    if bm:
        assert t.last_bm_stats()[0] > 0
    g = t.backward(torch.from_numpy(Dm).cuda()).cpu().numpy()
    gr = rt.backward(Dm)
    lsb_b = (2.0 * 12.0 / 510.0) * np.abs(Dm).max(axis=1, keepdims=True)
    frac, worst = H.lsb_report(g, gr, lsb_b)
    assert frac <= 1e-2 and worst <= steps, (frac, worst)
    if mv.endswith("DigitalSum") and not bm and lines == "none":
        # two conversions: the result lies off the single-pass ADC grid for many elements
        p1 = H.training_params(noise=False, pulse_det=True, bm=False, out_bound=out_bound)
        t1 = T.AnalogTile(p1._config(x_size, d_size, H.device("cs", False), seed=9), cuda_device=0)
        t1.set_weights(torch.from_numpy(W))
        y1 = t1.forward(torch.from_numpy(X).cuda()).cpu().numpy()
        assert np.mean(np.abs(y1 - y) > 0.25 * lsb) > 0.1


@pytest.mark.parametrize("mv", ["PosNegSeparate", "PosNegSeparateDigitalSum"])
def test_pos_neg_separate_noise_moments(mv):
    """Output noise and additive weight noise under the two-pass types: the analog sum carries one
    output-noise draw and the weight noise of both halves (w^2 ||v||^2 in total), the digital sum
    two output-noise draws; std-dev per element against the closed form and the reference."""
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    rng = np.random.default_rng(37)
    x_size, d_size, m = 96, 48, 12
    p = H.training_params(noise=False, pulse_det=True, bm=False, adc=False, out_bound=0.0)
    io = p.forward_io
    io.mv_type = getattr(D.AnalogMVType, mv)
    io.out_noise, io.w_noise = 0.03, 0.02
    io.w_noise_type = D.WeightNoiseType.AdditiveConstant
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=9)
    t = T.AnalogTile(cfg, cuda_device=0)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().cpu().numpy()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    X /= np.abs(X).max(axis=1, keepdims=True)
    xg = torch.from_numpy(X).cuda()
    reps = 400
    ys = _repeat(lambda: t.forward(xg).cpu().numpy(), reps)
    res = np.float32(2.0 / 126.0)
    v = np.clip(np.rint(X / res) * res, -1, 1).astype(np.float64)
    n_out = 2.0 if mv.endswith("DigitalSum") else 1.0
    sig = np.sqrt(n_out * 0.03 ** 2 + 0.02 ** 2 * (v ** 2).sum(axis=1, keepdims=True)) * np.ones((1, d_size))
    ratio = ys.std(axis=0) / sig
    assert abs(ratio.mean() - 1.0) < 0.01, ratio.mean()
    assert np.abs(ratio - 1.0).max() < 5.5 / np.sqrt(2 * reps), np.abs(ratio - 1.0).max()
    zmean = (ys.mean(axis=0) - v @ W.astype(np.float64).T) / (sig / np.sqrt(reps))
    assert np.abs(zmean).max() < 5.5
    if ref.available():
        rt = ref.RefTile(cfg)
        rt.set_weights(W)
        yr = _repeat(lambda: rt.forward(X), reps)
        rr = ys.std(axis=0) / yr.std(axis=0)
        assert abs(rr.mean() - 1.0) < 0.02 and np.abs(rr - 1.0).max() < 0.35


@pytest.mark.parametrize("adc,w_noise", [(True, 0.0), (True, 0.03), (False, 0.0)])
def test_out_noise_std_on_the_tensor_core_path(adc, w_noise):
    """out_noise_std with the tensor-core kernels forced on (their LINE variants read the tile's
    table of per-line std-devs): the std-dev of every output line over repeats follows
    sqrt(line^2 + (w_noise ||v||)^2), forward and backward, and equals what the CUDA-core kernels
    give for the same tile."""
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(41)
    x_size, d_size, m = 128, 192, 256
    p = H.training_params(noise=False, pulse_det=True, bm=False, adc=adc, out_bound=12.0 if adc else 0.0)
    for io in (p.forward_io, p.backward_io):
        io.out_noise, io.out_noise_std = 0.1, 0.4
        io.w_noise = w_noise
        io.w_noise_type = D.WeightNoiseType.AdditiveConstant if w_noise > 0 else D.WeightNoiseType.None_
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=21)
    t = T.AnalogTile(cfg, cuda_device=0)
    W = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    X /= np.abs(X).max(axis=1, keepdims=True)
    Dm = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
    Dm /= np.abs(Dm).max(axis=1, keepdims=True)
    xg, dg = torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda()
    res = np.float32(2.0 / 126.0)
    vx = np.clip(np.rint(X / res) * res, -1, 1).astype(np.float64)
    vd = np.clip(np.rint(Dm / res) * res, -1, 1).astype(np.float64)
    lib = _cabi.lib()
    reps = 40
    lines = {}
    try:
        for mode in (2, 1):  # tensor cores wherever possible, then CUDA cores only
            assert lib.ab200_set_mvm_path(mode) == 0
            for backward, inp, v, n in ((False, xg, vx, d_size), (True, dg, vd, x_size)):
                fn = (lambda: t.backward(inp).cpu().numpy()) if backward else (lambda: t.forward(inp).cpu().numpy())
                ys = _repeat(fn, reps)
                table = t.get_io_vector(backward, 2).numpy().astype(np.float64)  # out-noise values
                assert table.shape == (n,)
                want = np.sqrt(table[None, :] ** 2 + (w_noise ** 2) * (v ** 2).sum(axis=1, keepdims=True))
                if adc:  # the ADC step adds its rounding noise
                    want = np.sqrt(want ** 2 + (2 * 12.0 / 510.0) ** 2 / 12.0)
                dev = ys - ys.mean(axis=0, keepdims=True)
                est = np.sqrt((dev ** 2).sum(axis=0) / (reps - 1.0))
                ratio = (est / want).mean(axis=0)  # per line, averaged over the rows
                # (a line far below the ADC step does not dither it: no closed form there)
                ok = table > (0.05 if adc else 0.0)
                assert ok.mean() > 0.8
                assert np.abs(ratio[ok] - 1.0).max() < 0.06, (mode, backward, np.abs(ratio[ok] - 1.0).max())
                lines[(mode, backward)] = est.mean(axis=0)
    finally:
        lib.ab200_set_mvm_path(0)
    for backward in (False, True):
        assert np.corrcoef(lines[(2, backward)], lines[(1, backward)])[0, 1] > 0.99
