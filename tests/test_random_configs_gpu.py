"""Seeded sweep over random tile configurations, noise off, against the compiled reference tile.

Every case draws its own shape (ragged sizes, single rows and columns included), memory layouts
(transposed inputs / outputs, bias column), noise and bound management types, DAC / ADC
resolutions, MV type, device kind and pulse type, then checks forward, backward and a few pulsed
updates on the GPU tile against the reference's CPU tile built from the same configuration:
outputs within one ADC step (the reference's own GPU-vs-CPU criterion is a relative tolerance on
unit-scale data, src/rpucuda/cuda/rpucuda_pulsed_test.cpp:437-480), weights to 1e-6. Each case runs
on the automatic kernel selection and with the tensor-core kernels forced on wherever they apply."""

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu

N_CASES = 48


def _draw_case(seed):
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(1000 + seed)
    pick = lambda seq: seq[int(rng.integers(len(seq)))]  # noqa: E731
    c = dict(seed=seed)
    c["x_size"] = int(pick([1, 2, 7, 31, 64, 100, 129, 256, 333, 515]))
    c["d_size"] = int(pick([1, 3, 8, 33, 64, 127, 200, 256]))
    c["m"] = int(pick([1, 2, 5, 17, 64, 130, 257]))
    c["bias"] = bool(rng.integers(2)) and c["x_size"] > 1
    c["x_trans"], c["d_trans"] = bool(rng.integers(2)), bool(rng.integers(2))
    c["nm"] = pick([D.NoiseManagementType.None_, D.NoiseManagementType.AbsMax, D.NoiseManagementType.Max,
                    D.NoiseManagementType.Constant, D.NoiseManagementType.AbsMaxNPSum])
    c["bm"] = pick([D.BoundManagementType.None_, D.BoundManagementType.Iterative,
                    D.BoundManagementType.IterativeWorstCase])
    c["inp_res"] = float(pick([1 / 126.0, 1 / 254.0, 1 / 30.0]))
    c["out_res"] = float(pick([1 / 510.0, 1 / 254.0, 1 / 62.0]))
    c["out_bound"] = float(pick([12.0, 3.0, 1.0]))
    c["mv"] = pick([D.AnalogMVType.OnePass, D.AnalogMVType.OnePass, D.AnalogMVType.PosNegSeparate,
                    D.AnalogMVType.PosNegSeparateDigitalSum])
    c["asym"] = float(pick([0.0, 0.0, 0.05]))
    c["kind"] = pick(["cs", "ls", "sb", "sbr", "es", "ps", "pw"])
    c["pulse"] = pick([D.PulseType.DeterministicImplicit, D.PulseType.MeanCount, D.PulseType.NoneWithDevice])
    c["bl"] = int(pick([31, 10, 63]))
    c["um"], c["ublm"] = bool(rng.integers(2)), bool(rng.integers(2))
    c["lr"] = float(pick([0.01, 0.1]))
    return c, rng


def _row_step(ref_rows, floor):
    """One ADC step per row, read off the reference's own outputs: the values of a row lie on
    the grid step * k, so the smallest gap between two of them is a (small) multiple of the step.
    Rows with a single distinct value fall back to `floor` or the value itself."""
    out = np.empty((ref_rows.shape[0], 1))
    for r, row in enumerate(ref_rows.astype(np.float64)):
        u = np.unique(row)
        gaps = np.diff(u)
        gaps = gaps[gaps > 1e-7 * max(np.abs(u).max(), 1e-30)]
        out[r, 0] = gaps.min() if gaps.size else max(np.abs(u).max(), float(floor[r, 0]))
    return np.maximum(out, floor)


def _build(c):
    from aihwkit_b200.rpu_base import devices as D

    p = D.AnalogTileParameter()
    for io in (p.forward_io, p.backward_io):
        io.inp_res, io.out_res = c["inp_res"], c["out_res"]
        io.out_noise = 0.0
        io.out_bound, io.inp_bound = c["out_bound"], 1.0
        io.noise_management = c["nm"]
        io.nm_thres = 1.5 if c["nm"] == D.NoiseManagementType.Constant else 0.0
        io.mv_type = c["mv"]
        io.inp_asymmetry = io.out_asymmetry = c["asym"]
    p.forward_io.bound_management = c["bm"]
    p.update.pulse_type = c["pulse"]
    p.update.desired_bl = c["bl"]
    p.update.update_management, p.update.update_bl_management = c["um"], c["ublm"]
    dp = H.piecewise_device(False) if c["kind"] == "pw" else H.device(c["kind"], False)
    return p._config(c["x_size"], c["d_size"], dp, seed=5)


@pytest.mark.parametrize("seed", range(N_CASES))
def test_random_configuration_against_reference(seed):
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    if not ref.available():
        pytest.skip("compiled reference not built")
    c, rng = _draw_case(seed)
    cfg = _build(c)
    x_size, d_size, m, bias = c["x_size"], c["d_size"], c["m"], c["bias"]
    x_in = x_size - (1 if bias else 0)
    rt = ref.RefTile(cfg)
    W = rng.uniform(-0.4, 0.4, (d_size, x_size)).astype(np.float32)
    rt.set_weights(W)
    W = rt.get_weights()
    # inputs with a wide spread of row maxima; one all-zero row
    X = (rng.uniform(-1, 1, (m, x_in)) * rng.uniform(0.05, 2.0, (m, 1))).astype(np.float32)
    Dm = (rng.normal(0, 0.3, (m, d_size)) * rng.uniform(0.05, 2.0, (m, 1))).astype(np.float32)
    if m > 2:
        X[1] = 0.0
        Dm[2] = 0.0
    Xa = np.ascontiguousarray(X.T) if c["x_trans"] else X
    Da = np.ascontiguousarray(Dm.T) if c["d_trans"] else Dm
    yr = rt.forward(Xa, bias=bias, x_trans=c["x_trans"], d_trans=c["d_trans"])
    gr = rt.backward(Da, bias=bias, d_trans=c["d_trans"], x_trans=c["x_trans"])
    steps = 2.002 if c["mv"].name.endswith("DigitalSum") else 1.001
    lib = _cabi.lib()
    try:
        for mode in (0, 2):
            assert lib.ab200_set_mvm_path(mode) == 0
            t = T.AnalogTile(cfg, cuda_device=0)
            t.set_weights(torch.from_numpy(W))
            assert np.array_equal(t.get_weights().numpy(), W)
            y = t.forward(torch.from_numpy(Xa).cuda(), bias, c["x_trans"], c["d_trans"]).cpu().numpy()
            assert y.shape == yr.shape
            # one ADC step of the row (at the scale of its last bound-management round); the
            # largest output magnitude bounds that scale from below
            ym = (yr.T if c["d_trans"] else yr)
            yg = (y.T if c["d_trans"] else y)
            floor = np.maximum(np.abs(ym).max(axis=1, keepdims=True) / c["out_bound"], 1e-30) * \
                (2.0 * c["out_bound"] * c["out_res"])
            frac, worst = H.lsb_report(yg, ym, _row_step(ym, floor))
            assert worst <= steps and frac <= 0.02, ("forward", mode, c, frac, worst)
            g = t.backward(torch.from_numpy(Da).cuda(), bias, c["d_trans"], c["x_trans"]).cpu().numpy()
            assert g.shape == gr.shape
            gm = (gr.T if c["x_trans"] else gr)
            gg = (g.T if c["x_trans"] else g)
            floor_b = np.maximum(np.abs(gm).max(axis=1, keepdims=True) / c["out_bound"], 1e-30) * \
                (2.0 * c["out_bound"] * c["out_res"])
            frac, worst = H.lsb_report(gg, gm, _row_step(gm, floor_b))
            assert worst <= steps and frac <= 0.02, ("backward", mode, c, frac, worst)
    finally:
        lib.ab200_set_mvm_path(0)
    # pulsed updates, weights after each call
    t = T.AnalogTile(cfg, cuda_device=0)
    t.set_weights(torch.from_numpy(W))
    t.set_learning_rate(c["lr"])
    rt.set_learning_rate(c["lr"])
    for k in range(3):
        Xu = (rng.uniform(-1, 1, (m, x_in))).astype(np.float32)
        Du = (rng.normal(0, 0.5, (m, d_size))).astype(np.float32)
        Xua = np.ascontiguousarray(Xu.T) if c["x_trans"] else Xu
        Dua = np.ascontiguousarray(Du.T) if c["d_trans"] else Du
        t.update(torch.from_numpy(Xua).cuda(), torch.from_numpy(Dua).cuda(), bias, c["x_trans"], c["d_trans"])
        rt.update(Xua, Dua, bias=bias, x_trans=c["x_trans"], d_trans=c["d_trans"])
        diff = np.abs(t.get_weights().numpy() - rt.get_weights()).max()
        tol = 2e-6 if c["pulse"].name == "NoneWithDevice" else 1e-6
        assert diff <= tol, ("update", k, c, diff)


N_COMPOUND_CASES = 40


def _draw_compound(seed):
    rng = np.random.default_rng(5000 + seed)
    pick = lambda seq: seq[int(rng.integers(len(seq)))]  # noqa: E731
    fam = pick(["transfer", "buffered", "chopped", "dynamic", "mixed"])
    x_size, d_size, m = int(pick([3, 8, 13, 40])), int(pick([2, 9, 16, 33])), int(pick([1, 4, 7, 20]))
    if fam == "transfer":
        dp = H.transfer_device(False, transfer_every=float(pick([1.0, 2.0, 3.0])),
                               units_in_mbatch=bool(rng.integers(2)), n_reads=int(pick([1, 2, 3])),
                               transfer_lr=float(pick([0.01, 0.1, 1.0])), det=True)
        dp.transfer_forward.out_noise = 0.0
    elif fam == "buffered":
        dp = H.buffered_transfer_device(transfer_every=float(pick([1.0, 2.0, 5.0])), n_reads=int(pick([1, 2, 3])),
                                        thres_scale=float(pick([0.5, 1.0, 2.0])),
                                        momentum=float(pick([0.0, 0.3])), forget_buffer=bool(rng.integers(2)),
                                        transfer_lr=float(pick([0.5, 1.0, 4.0])))
    elif fam == "chopped":
        dp = H.chopped_transfer_device(transfer_every=float(pick([1.0, 2.0, 3.0])),
                                       in_chop_prob=float(pick([0.0, 0.25, 0.5, 1.0])), in_chop_random=False,
                                       momentum=float(pick([0.0, 0.3])), forget_buffer=bool(rng.integers(2)),
                                       transfer_lr=float(pick([1.0, 4.0])),
                                       buffer_granularity=float(pick([0.5, 1.0, 2.0])),
                                       correct_gradient_magnitudes=bool(rng.integers(2)),
                                       auto_granularity=float(pick([0.0, 0.0, 20.0])))
        if float(dp.in_chop_prob) == 1.0:
            dp.in_chop_random = True  # probability one: every transfer flips, no draw decides anything
    elif fam == "dynamic":
        dp = H.dynamic_transfer_device(in_chop_prob=float(pick([0.2, 0.34, 0.5])),
                                       tail_weightening=float(pick([1.0, 2.5, 5.0])),
                                       buffer_cap=float(pick([0.0, 0.5, 10.0])),
                                       correct_accumulation=bool(rng.integers(2)),
                                       transfer_every=float(pick([1.0, 2.0])),
                                       momentum=float(pick([0.0, 0.2])), forget_buffer=bool(rng.integers(2)),
                                       transfer_lr=float(pick([1.0, 4.0])),
                                       buffer_granularity=float(pick([0.5, 1.0])))
    else:
        bins = pick([(9, 5), (5, 3), (21, 11)])
        dp = H.mixed_precision_device(kind=pick(["sb", "cs", "sbr"]), n_x_bins=bins[0], n_d_bins=bins[1],
                                      transfer_every=int(pick([1, 2])),
                                      n_rows_per_transfer=int(pick([-1, 1, 3, d_size])),
                                      granularity=float(pick([0.0, 0.004])), transfer_lr=float(pick([0.5, 1.0])))
    return fam, dp, x_size, d_size, m, float(pick([0.05, 0.1, 0.3])), rng


@pytest.mark.parametrize("seed", range(N_COMPOUND_CASES))
def test_random_compound_against_reference(seed):
    """Random parameters of the Tiki-Taka family (plain, buffered, chopped, dynamic) and of the
    mixed-precision compound, deterministic pulses and chopper schedules, noise off: visible
    weights and every hidden plane (fast tile, buffers, means, chi) follow the compiled reference
    through ten update calls."""
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    if not ref.available():
        pytest.skip("compiled reference not built")
    fam, dp, x_size, d_size, m, lr, rng = _draw_compound(seed)
    p = H.training_params(noise=False, pulse_det=True)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = T.AnalogTile(cfg, cuda_device=0)
    rt = ref.RefTile(cfg)
    names = t.get_hidden_parameter_names()
    assert names == rt.hidden_parameter_names()
    assert np.array_equal(t.get_hidden_parameters().numpy(), rt.get_hidden_parameters())
    state = [k for k, n in enumerate(names)
             if n.startswith(("hidden_weights", "buffered_FP", "running_mean", "past_mean"))]
    t.set_learning_rate(lr)
    rt.set_learning_rate(lr)
    for step in range(10):
        x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        d = rng.normal(0, 0.5, (m, d_size)).astype(np.float32)
        t.update(torch.from_numpy(x).cuda(), torch.from_numpy(d).cuda())
        rt.update(x, d)
        hp, hr = t.get_hidden_parameters().numpy(), rt.get_hidden_parameters()
        for k in state:
            tol = 1e-6 if names[k].startswith("hidden_weights") and not names[k].endswith("chi") else 1e-4
            assert np.abs(hp[k] - hr[k]).max() <= tol, (fam, names[k], step, np.abs(hp[k] - hr[k]).max())
        assert np.abs(t.get_weights().numpy() - rt.get_weights()).max() <= 1e-6, (fam, "weights", step)


@pytest.mark.parametrize("seed", range(20))
def test_random_stochastic_updates_agree_between_the_two_kernels(seed):
    """Stochastic pulse trains at random ragged sizes, train lengths (one to four 31-slot
    segments) and device kinds, also through a Tiki-Taka compound: the staged kernel and the
    streaming kernel see the same trains and apply the same pulses in the same per-weight order,
    so without device noise the weights (and the fast tile) agree bit for bit; and they move."""
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(11000 + seed)
    pick = lambda seq: seq[int(rng.integers(len(seq)))]  # noqa: E731
    x_size, d_size = int(pick([1, 5, 31, 33, 100, 257, 600])), int(pick([1, 7, 32, 65, 130, 300]))
    m = int(pick([1, 3, 31, 32, 33, 100, 257]))
    bl = int(pick([1, 7, 31, 40, 63, 100]))
    compound = bool(rng.integers(4) == 0)
    p = H.training_params(noise=True, pulse_det=False)
    p.update.desired_bl = bl
    p.update.update_management, p.update.update_bl_management = bool(rng.integers(2)), bool(rng.integers(2))
    if compound:
        dp = H.transfer_device(False, transfer_every=float(pick([1.0, 3.0])), units_in_mbatch=False,
                               n_reads=int(pick([1, 2])), transfer_lr=0.1, det=True)
        dp.transfer_forward.out_noise = 0.0
    else:
        dp = H.device(pick(["cs", "ls", "sb", "sbr", "es", "ps"]), False, dw_min=0.002, dw_min_dtod=0.3)
    cfg = p._config(x_size, d_size, dp, seed=5)
    W0 = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    X = (np.maximum(rng.standard_normal((m, x_size)), 0) if rng.integers(2)
         else rng.uniform(-1, 1, (m, x_size))).astype(np.float32)
    Dm = rng.normal(0, 0.2, (m, d_size)).astype(np.float32)
    lib = _cabi.lib()
    results = []
    try:
        for mode in (1, 2):
            _cabi.check(lib.ab200_set_update_path(mode))
            t = T.AnalogTile(cfg, cuda_device=0)
            t.set_weights(torch.from_numpy(W0))
            t.set_learning_rate(0.05)
            for _ in range(3):
                t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
            results.append((t.get_weights().numpy(), t.get_hidden_parameters().numpy()))
    finally:
        _cabi.check(lib.ab200_set_update_path(0))
    assert np.array_equal(results[0][0], results[1][0])
    assert np.array_equal(results[0][1], results[1][1])
    if np.abs(X).max() > 0 and m * x_size * d_size > 64:
        moved = np.abs(results[0][0] - np.clip(W0, -0.6, 0.6)).max() > 0 or \
            (compound and np.abs(results[0][1]).max() > 0)
        assert moved


@pytest.mark.parametrize("seed", range(10))
def test_random_noisy_forward_moments_against_reference(seed):
    """Random combinations of the stochastic IO settings (output noise, additive or PCMRead weight
    noise, input noise, stochastic DAC / ADC rounding, asymmetries, per-line output noise, MV
    type): mean and std-dev per output element over 300 repeats against the same number of repeats
    of the compiled reference (the reference's own criterion for noisy passes,
    src/rpucuda/cuda/rpucuda_pulsed_test.cpp:364-435)."""
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    if not ref.available():
        pytest.skip("compiled reference not built")
    rng = np.random.default_rng(13000 + seed)
    pick = lambda seq: seq[int(rng.integers(len(seq)))]  # noqa: E731
    x_size, d_size, m = int(pick([20, 48, 100])), int(pick([12, 30, 64])), int(pick([4, 9]))
    p = H.training_params(noise=False, pulse_det=True, bm=False, out_bound=12.0)
    io = p.forward_io
    io.out_noise = float(pick([0.02, 0.06, 0.2]))
    io.w_noise = float(pick([0.0, 0.02, 0.05]))
    io.w_noise_type = pick([D.WeightNoiseType.AdditiveConstant, D.WeightNoiseType.PCMRead])
    io.inp_noise = float(pick([0.0, 0.0, 0.02]))
    io.inp_sto_round, io.out_sto_round = bool(rng.integers(2)), bool(rng.integers(2))
    io.inp_asymmetry, io.out_asymmetry = float(pick([0.0, 0.03])), float(pick([0.0, 0.03]))
    io.mv_type = pick([D.AnalogMVType.OnePass, D.AnalogMVType.OnePass, D.AnalogMVType.PosNegSeparate,
                       D.AnalogMVType.PosNegSeparateDigitalSum])
    io.out_res = float(pick([1 / 510.0, -1.0]))
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=9)
    t = T.AnalogTile(cfg, cuda_device=0)
    rt = ref.RefTile(cfg)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(W))
    W = t.get_weights().numpy()
    rt.set_weights(W)
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    xg = torch.from_numpy(X).cuda()
    reps = 300
    ys = np.stack([t.forward(xg).cpu().numpy() for _ in range(reps)])
    yr = np.stack([rt.forward(X) for _ in range(reps)])
    H.assert_moments_agree(ys, yr, z_max=5.5, std_tol=0.06)
    # element by element: std-dev within the sampling error of two estimates from `reps` draws
    ratio = ys.std(axis=0) / np.maximum(yr.std(axis=0), 1e-12)
    assert np.abs(ratio - 1.0).max() < 6.0 / np.sqrt(reps), np.abs(ratio - 1.0).max()


@pytest.mark.parametrize("seed", range(16))
def test_random_floating_point_tiles(seed):
    """FloatingPointTile (perfect IO, floating-point update; RPUSimple) at random shapes, layouts
    and bias settings: forward, backward and the rank update against float64 numpy, on the
    automatic kernel selection and with the tensor-core path forced on (which perfect IO cannot
    take: the CUDA-core kernels must serve it either way), also through host buffers."""
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(15000 + seed)
    pick = lambda seq: seq[int(rng.integers(len(seq)))]  # noqa: E731
    x_size, d_size, m = int(pick([1, 3, 30, 129, 512, 700])), int(pick([1, 5, 64, 200, 513])), int(pick([1, 7, 130, 600]))
    bias = bool(rng.integers(2)) and x_size > 1
    x_trans, d_trans = bool(rng.integers(2)), bool(rng.integers(2))
    x_in = x_size - (1 if bias else 0)
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    X = rng.uniform(-1, 1, (m, x_in)).astype(np.float32)
    Dm = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
    Xb = np.concatenate([X, np.ones((m, 1), np.float32)], 1) if bias else X
    Xa = np.ascontiguousarray(X.T) if x_trans else X
    Da = np.ascontiguousarray(Dm.T) if d_trans else Dm
    y_want = Xb.astype(np.float64) @ W.astype(np.float64).T
    g_want = (Dm.astype(np.float64) @ W.astype(np.float64))[:, :x_in]
    tol = 2e-6 * max(x_size, d_size) ** 0.5 + 1e-6
    lib = _cabi.lib()
    try:
        for mode in (0, 2):
            assert lib.ab200_set_mvm_path(mode) == 0
            t = T.FloatingPointTile(x_size, d_size).cuda(0)
            t.set_weights(torch.from_numpy(W))
            y = t.forward(torch.from_numpy(Xa).cuda(), bias, x_trans, d_trans).cpu().numpy()
            y = y.T if d_trans else y
            assert np.abs(y - y_want).max() <= tol * max(np.abs(y_want).max(), 1.0), ("forward", mode)
            g = t.backward(torch.from_numpy(Da).cuda(), bias, d_trans, x_trans).cpu().numpy()
            g = g.T if x_trans else g
            assert g.shape == g_want.shape
            assert np.abs(g - g_want).max() <= tol * max(np.abs(g_want).max(), 1.0), ("backward", mode)
            if mode == 0:  # host buffers
                yh = t.forward(torch.from_numpy(Xa), bias, x_trans, d_trans).numpy()
                assert np.array_equal(yh.T if d_trans else yh, y)
            t.set_learning_rate(0.1)
            t.update(torch.from_numpy(Xa).cuda(), torch.from_numpy(Da).cuda(), bias, x_trans, d_trans)
            w_want = W.astype(np.float64) - 0.1 * Dm.astype(np.float64).T @ Xb.astype(np.float64)
            assert np.abs(t.get_weights().numpy() - w_want).max() <= 2e-6 * m ** 0.5 * max(np.abs(w_want).max(), 1.0) + 1e-6
    finally:
        lib.ab200_set_mvm_path(0)
