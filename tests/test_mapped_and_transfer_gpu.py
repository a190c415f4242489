"""GPU parity of the mapped-tile layer and of the Tiki-Taka (TransferCompound) tile."""

import numpy as np
import pytest
import torch

from oracle import analog_tile_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _array_oracle(W, X, cfg, max_out, max_in, rng=None):
    """TileModuleArray.forward restated with the single-tile oracle
    (src/aihwkit/simulator/tiles/array.py:155-182)."""
    from aihwkit_b200.sharded import split_sizes

    io = O.IO.from_c(cfg.forward_io)
    out_sizes, in_sizes = split_sizes(W.shape[0], max_out), split_sizes(W.shape[1], max_in)
    y = np.zeros((X.shape[0], W.shape[0]), np.float32)
    lsb = np.zeros_like(y)
    c0 = 0
    for isz in in_sizes:
        r0 = 0
        for osz in out_sizes:
            yt, _, scale, _ = O.forward(W[r0 : r0 + osz, c0 : c0 + isz], X[:, c0 : c0 + isz], io, rng,
                                        return_pre_adc=True)
            y[:, r0 : r0 + osz] += yt
            lsb[:, r0 : r0 + osz] = np.maximum(lsb[:, r0 : r0 + osz], (io.res_out / scale)[:, None])
            r0 += osz
        c0 += isz
    return y, lsb, len(in_sizes)


@pytest.mark.parametrize("out_size,in_size,max_tile,m", [(256, 384, 128, 40), (768, 2304, 512, 24),
                                                         (100, 1030, 512, 7)])
def test_mapped_forward_noise_off(out_size, in_size, max_tile, m):
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(out_size)
    p = H.inference_params(noise=False)
    cfg = p._config(1, 1, D.IdealResistiveDeviceParameter(), seed=3)
    arr = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
    W = rng.normal(0, 1 / np.sqrt(in_size), (out_size, in_size)).astype(np.float32)
    arr.set_weights(torch.from_numpy(W))
    assert np.array_equal(arr.get_weights().numpy(), W)
    X = rng.normal(0, 1, (m, in_size)).astype(np.float32)
    y = arr.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    y_or, lsb, n_in = _array_oracle(W, X, cfg, max_tile, max_tile)
    diff = np.abs(y - y_or)
    # each in-split contributes its own ADC step; allow one step per in-split at most
    assert (diff > 1e-3 * lsb).mean() <= 1e-3 * n_in
    assert (diff <= 1.001 * lsb * n_in).all()
    # host-buffer entry point gives the same numbers
    y_h = arr.forward(torch.from_numpy(X))
    assert np.array_equal(y_h.numpy(), y)


@pytest.mark.parametrize("m,out_size,in_size,max_out,max_in", [(40, 512, 640, 256, 320), (256, 512, 640, 256, 320),
                                                               (300, 200, 1000, 128, 400), (130, 700, 300, 512, 128),
                                                               (9, 64, 900, 64, 300)])
def test_mapped_forward_iterative_bound_management(m, out_size, in_size, max_out, max_in):
    """A 2 x 2 mapped layer with the training IO (iterative bound management) and an output bound
    small enough that many rows clip in the first round: every tile re-runs its clipped rows on its
    own before its result joins the sum over the in-splits. 256 rows take the tensor-core kernel
    per tile, 40 rows the CUDA-core one."""
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(m)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
    cfg = p._config(1, 1, H.device("cs", False), seed=3)
    arr = T.TileArray(cfg, out_size, in_size, max_out, max_in, cuda_device=0)
    W = rng.uniform(-0.5, 0.5, (out_size, in_size)).astype(np.float32)
    arr.set_weights(torch.from_numpy(W))
    W = arr.get_weights().numpy()  # clipped to the device bounds
    X = rng.uniform(-1, 1, (m, in_size)).astype(np.float32)
    y = arr.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    y_or, lsb, n_in = _array_oracle(W, X, cfg, max_out, max_in)
    # the test is only meaningful when the first round clips
    io = O.IO.from_c(cfg.forward_io)
    from aihwkit_b200.sharded import split_sizes

    o0, i0 = split_sizes(out_size, max_out)[0], split_sizes(in_size, max_in)[0]
    _, _, _, reductions = O.forward(W[:o0, :i0], X[:, :i0], io, return_pre_adc=True)
    assert (reductions > 1).mean() > 0.2
    diff = np.abs(y - y_or)
    assert (diff > 1e-3 * lsb).mean() <= 2e-3 * n_in
    assert (diff <= 1.001 * lsb * n_in).all()


def test_mapped_forward_sharded_partials_add_up():
    """The partial sums of disjoint in-split ranges add up to the full layer (noise off), which
    is what the multi-GPU reduce relies on; with noise on, the full layer and the sum of the
    shards are bit-identical because noise keys depend on global tile coordinates only."""
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(4)
    out_size, in_size, max_tile, m = 384, 1024, 256, 33
    for noise in (False, True):
        p = H.inference_params(noise=noise)
        cfg = p._config(1, 1, D.IdealResistiveDeviceParameter(), seed=77)
        W = rng.normal(0, 1 / 32.0, (out_size, in_size)).astype(np.float32)
        X = torch.from_numpy(rng.normal(0, 1, (m, in_size)).astype(np.float32)).cuda()
        full = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
        full.set_weights(torch.from_numpy(W))
        y_full = full.forward(X)
        parts = []
        for b, e in ((0, 1), (1, 3), (3, 4)):
            a = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0,
                            in_split_range=(b, e))
            a.set_weights(torch.from_numpy(W))
            parts.append(a.forward(X))
        y_sum = parts[0] + parts[1] + parts[2]
        assert torch.allclose(y_full, y_sum, atol=1e-5, rtol=1e-6)


@pytest.mark.parametrize("m", [33, 300])
def test_mapped_forward_blocks_of_tiles_add_up(m):
    """A 2-D map of the tiles (blocks over in-splits and out-splits, as a layer with two in-splits
    is spread over more than two ranks): every block writes its own output columns and zeros
    elsewhere, the bias enters with the blocks of in-split 0 only, the noise is that of the tile's
    place in the whole layer - so the blocks' outputs add up to the full layer's, noise included."""
    from aihwkit_b200.rpu_base import devices as D, tiles as T
    from aihwkit_b200.sharded import block_of_rank, split_sizes

    rng = np.random.default_rng(14)
    out_size, in_size, max_tile = 2304, 768, 512  # in-splits [384, 384], five out-splits of 460/461
    p = H.inference_params(noise=True)
    cfg = p._config(1, 1, D.IdealResistiveDeviceParameter(), seed=21)
    W = rng.normal(0, 0.02, (out_size, in_size)).astype(np.float32)
    bias = rng.normal(0, 0.1, out_size).astype(np.float32)
    X = torch.from_numpy(rng.normal(0, 1, (m, in_size)).astype(np.float32)).cuda()
    full = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
    full.set_weights(torch.from_numpy(W), weight_scaling_omega=1.0)
    full.set_bias(torch.from_numpy(bias))
    y_full = full.forward(X)
    n_in, n_out = len(split_sizes(in_size, max_tile)), len(split_sizes(out_size, max_tile))
    world = 8
    total = torch.zeros_like(y_full)
    for rank in range(world):
        (ib, ie), (ob, oe) = block_of_rank(n_in, n_out, rank, world)
        blk = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0,
                          in_split_range=(ib, ie), out_split_range=(ob, oe))
        blk.set_weights(torch.from_numpy(W), weight_scaling_omega=1.0)
        blk.set_bias(torch.from_numpy(bias))
        total += blk.forward(X)
    assert torch.allclose(total, y_full, atol=2e-5, rtol=1e-6)
    assert float(y_full.abs().max()) > 0


def test_mapped_forward_noise_statistics():
    from scipy import stats
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(9)
    out_size, in_size, max_tile, m, reps = 128, 512, 256, 16, 100
    p = H.inference_params(noise=True)
    cfg = p._config(1, 1, D.IdealResistiveDeviceParameter(), seed=5)
    arr = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
    W = rng.normal(0, 1 / np.sqrt(in_size), (out_size, in_size)).astype(np.float32)
    arr.set_weights(torch.from_numpy(W))
    X = rng.normal(0, 1, (m, in_size)).astype(np.float32)
    xg = torch.from_numpy(X).cuda()
    ys = np.stack([arr.forward(xg).cpu().numpy() for _ in range(reps)])
    org = np.random.default_rng(1)
    yo = np.stack([_array_oracle(W, X, cfg, max_tile, max_tile, org)[0] for _ in range(reps)])
    H.assert_moments_agree(ys, yo, std_tol=0.05)
    ks = stats.ks_2samp((ys - yo.mean(axis=0)).ravel(), (yo - yo.mean(axis=0)).ravel())
    assert ks.pvalue > 0.01, ks


def _transfer_setup(x_size, d_size, noise, det, **kw):
    from aihwkit_b200.rpu_base import tiles as T

    p = H.training_params(noise=noise, pulse_det=det)
    dp = H.transfer_device(noise=noise, det=det, **kw)
    cfg = p._config(x_size, d_size, dp, seed=9)
    return T.AnalogTile(cfg, cuda_device=0), cfg, dp


def _transfer_oracle(t, cfg, dp, x_size, d_size):
    names = t.get_hidden_parameter_names()
    hp = t.get_hidden_parameters().numpy()
    fast = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS_REFERENCE, names, hp,
                                      dp._vec_par[0].dw_min_std, False, suffix="_0")
    slow = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS_REFERENCE, names, hp,
                                      dp._vec_par[1].dw_min_std, False, suffix="_1")
    w = t.get_weights().numpy().copy()
    return O.TransferOracle(w, fast, slow, cfg.transfer, O.Up.from_c(cfg.update),
                            dp._vec_par[0].dw_min, dp._vec_par[1].dw_min, x_size, d_size)


@pytest.mark.parametrize("every,units,m", [(2.0, True, 12), (5.0, False, 12), (1.0, False, 7)])
def test_transfer_deterministic(every, units, m):
    """Noise off, deterministic pulses: fast tile A and visible weights C follow the oracle's
    sample-by-sample Tiki-Taka sequencing, including transfers in the middle of a batch."""
    x_size, d_size = 40, 24
    t, cfg, dp = _transfer_setup(x_size, d_size, noise=False, det=True, transfer_every=every,
                                 units_in_mbatch=units, n_reads=2, transfer_lr=1.0)
    rng = np.random.default_rng(3)
    orc = _transfer_oracle(t, cfg, dp, x_size, d_size)
    lr = 0.1
    t.set_learning_rate(lr)
    names = t.get_hidden_parameter_names()
    ia = names.index("hidden_weights_0")
    for _ in range(6):
        X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        Dm = rng.normal(0, 0.5, (m, d_size)).astype(np.float32)
        t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
        orc.update(X, Dm, lr)
    A = t.get_hidden_parameters().numpy()[ia]
    C = t.get_weights().numpy()
    assert np.abs(orc.a).max() > 0 and np.abs(orc.c).max() > 0
    assert np.abs(A - orc.a).max() <= 1e-6
    assert np.abs(C - orc.c).max() <= 1e-6


def test_transfer_noisy_statistics():
    """Noise on, stochastic pulses: moments of A and C over repeats agree with the oracle."""
    x_size, d_size, m, reps = 16, 12, 8, 60
    rng = np.random.default_rng(5)
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.5, (m, d_size)).astype(np.float32)
    t, cfg, dp = _transfer_setup(x_size, d_size, noise=True, det=False, transfer_every=1.0,
                                 units_in_mbatch=True, n_reads=4, transfer_lr=1.0)
    names = t.get_hidden_parameter_names()
    ia = names.index("hidden_weights_0")
    lr = 0.1
    t.set_learning_rate(lr)
    org = np.random.default_rng(11)
    As, Cs, Ao, Co = [], [], [], []
    xg, dg = torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda()
    for _ in range(reps):
        t.set_weights(torch.zeros(d_size, x_size))
        orc = _transfer_oracle(t, cfg, dp, x_size, d_size)
        for _ in range(4):
            t.update(xg, dg)
            orc.update(X, Dm, lr, org)
        As.append(t.get_hidden_parameters().numpy()[ia])
        Cs.append(t.get_weights().numpy())
        Ao.append(orc.a.copy())
        Co.append(orc.c.copy())
    As, Cs, Ao, Co = (np.stack(v) for v in (As, Cs, Ao, Co))
    for mine, ref in ((As, Ao), (Cs, Co)):
        H.assert_moments_agree(mine, ref, std_tol=0.15)


@pytest.mark.parametrize("pinned", [False, True])
def test_mapped_forward_host_pipeline(pinned):
    """Host-buffer entry point with several row chunks in flight (pageable and page-locked
    buffers) against the device path, noise off."""
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(12)
    out_size, in_size, max_tile, m = 192, 320, 128, 3 * 1024 + 77  # 4 chunks, ragged tail
    cfg = H.inference_params(noise=False)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=3)
    arr = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
    arr.set_weights(torch.from_numpy(rng.normal(0, 0.05, (out_size, in_size)).astype(np.float32)))
    x = torch.from_numpy(rng.normal(0, 1, (m, in_size)).astype(np.float32))
    y_dev = arr.forward(x.cuda()).cpu()
    if pinned:
        xp = x.pin_memory()
        out = torch.empty(m, out_size).pin_memory()
        y = arr.forward(xp, out=out)
        assert y.data_ptr() == out.data_ptr()
    else:
        y = arr.forward(x)
    # the short tail chunk may run on the CUDA-core kernel: allow rare one-step ADC differences
    lsb = 2 * 10.0 / 254.0 * float(x.abs().max()) * 3

    def close(a, b):
        d = (a - b).abs()
        return float((d > 1e-6).float().mean()) <= 2e-3 and float(d.max()) <= lsb

    assert close(y, y_dev)
    # twice in a row: buffers and events are reused
    assert close(arr.forward(x), y_dev)


def test_mapped_forward_local_input_equals_full_width_input():
    """A shard fed only its own input columns gives the same partial sum as the same shard fed
    the full-width input (same noise: keys depend on global tile coordinates)."""
    from aihwkit_b200.rpu_base import devices as D, tiles as T
    from aihwkit_b200.sharded import column_range

    rng = np.random.default_rng(21)
    out_size, in_size, max_tile, m = 256, 1000, 256, 150
    cfg = H.inference_params(noise=True)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=31)
    W = torch.from_numpy(rng.normal(0, 0.05, (out_size, in_size)).astype(np.float32))
    X = torch.from_numpy(rng.normal(0, 1, (m, in_size)).astype(np.float32)).cuda()
    for rank in range(2):
        c0, c1 = column_range(in_size, max_tile, rank, 2)
        from aihwkit_b200.sharded import in_split_range

        b, e = in_split_range(4, rank, 2)
        outs = []
        for local in (False, True):
            a = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0,
                            in_split_range=(b, e))
            a.set_weights(W)
            assert a.local_in_size == c1 - c0
            if local:
                outs.append(a.forward_local(X[:, c0:c1].contiguous()))
            else:
                outs.append(a.forward(X))
            torch.cuda.synchronize()
        assert torch.equal(outs[0], outs[1])


def test_resume_from_extra_state_continues_identically():
    """Checkpoint / resume: a Tiki-Taka tile rebuilt from weights, hidden parameters and
    dump_extra() continues exactly like the uninterrupted one (transfer counters and noise call
    counters are part of the extra state), also through a deep copy."""
    import copy

    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(3)
    x_size, d_size, m = 24, 16, 5
    p = H.training_params(noise=True, pulse_det=False)
    dp = H.transfer_device(noise=True, transfer_every=1.0, units_in_mbatch=False, n_reads=2)
    cfg = p._config(x_size, d_size, dp, seed=11)
    a = T.AnalogTile(cfg, cuda_device=0)
    a.set_learning_rate(0.1)
    batches = [(torch.from_numpy(rng.uniform(-1, 1, (m, x_size)).astype(np.float32)).cuda(),
                torch.from_numpy(rng.normal(0, 0.5, (m, d_size)).astype(np.float32)).cuda())
               for _ in range(6)]
    for x, d in batches[:3]:
        a.update(x, d)
    # rebuild from the saved pieces
    b = T.AnalogTile(cfg, cuda_device=0)
    # order as in the reference's __setstate__ (tiles/base.py): weights first - setting them
    # zeroes the hidden fast tile and its counters - then hidden parameters, then the extra state
    b.set_weights(a.get_weights())
    b.set_hidden_parameters(a.get_hidden_parameters())
    b.load_extra(a.dump_extra(), strict=True)
    c = copy.deepcopy(a)
    for x, d in batches[3:]:
        a.update(x, d)
        b.update(x, d)
        c.update(x, d)
    assert torch.equal(a.get_weights(), b.get_weights())
    assert torch.equal(a.get_hidden_parameters(), b.get_hidden_parameters())
    assert torch.equal(a.get_weights(), c.get_weights())
    ya = a.forward(batches[0][0])
    assert torch.equal(ya, b.forward(batches[0][0]))  # same noise stream after the resume


@pytest.mark.parametrize("which", ["chopped", "dynamic", "mixed"])
def test_resume_of_the_later_compounds(which):
    """Checkpoint / resume in the middle of a chopper period and of a row window: choppers,
    switch marks, the pass counter and the mixed-precision counters travel in the extra state
    (hidden planes in the hidden parameters), so a rebuilt tile and a deep copy continue bit for
    bit like the uninterrupted one (regular chopper schedules, stochastic pulses)."""
    import copy

    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(5)
    x_size, d_size, m = 12, 10, 5
    p = H.training_params(noise=True, pulse_det=False)
    if which == "chopped":
        dp = H.chopped_transfer_device(transfer_lr=4.0, in_chop_prob=0.3, in_chop_random=False, out_chop_prob=0.0)
    elif which == "dynamic":
        dp = H.dynamic_transfer_device(transfer_lr=4.0, in_chop_prob=0.3, tail_weightening=2.5)
    else:
        dp = H.mixed_precision_device(n_rows_per_transfer=3)
    cfg = p._config(x_size, d_size, dp, seed=11)
    a = T.AnalogTile(cfg, cuda_device=0)
    a.set_learning_rate(0.1)
    batches = [(torch.from_numpy(rng.uniform(-1, 1, (m, x_size)).astype(np.float32)).cuda(),
                torch.from_numpy(rng.normal(0, 0.5, (m, d_size)).astype(np.float32)).cuda())
               for _ in range(16)]
    for x, d in batches[:9]:
        a.update(x, d)
    extra = a.dump_extra()
    if which != "mixed":
        assert len(extra["rpu_device.in_chopper"]) == x_size and len(extra["rpu_device.out_chopper"]) == d_size
        assert extra["rpu_device.transfer_counter"][0] > 0 and sum(extra["rpu_device.in_chopper"]) > 0
        assert ("rpu_device.in_chopper_switched" in extra) == (which == "dynamic")
    else:
        assert extra["rpu_device.mixed.current_update_index"][0] == 9 * m
    b = T.AnalogTile(cfg, cuda_device=0)
    b.set_weights(a.get_weights())
    b.set_hidden_parameters(a.get_hidden_parameters())
    b.load_extra(extra, strict=True)
    c = copy.deepcopy(a)
    for x, d in batches[9:]:
        a.update(x, d)
        b.update(x, d)
        c.update(x, d)
    assert torch.equal(a.get_weights(), b.get_weights()) and torch.equal(a.get_weights(), c.get_weights())
    assert torch.equal(a.get_hidden_parameters(), b.get_hidden_parameters())
    assert torch.equal(a.get_hidden_parameters(), c.get_hidden_parameters())
    # without the extra state the continuation differs: the state is needed, not decoration
    e = T.AnalogTile(cfg, cuda_device=0)
    e.set_weights(batches[0][0].new_zeros(d_size, x_size).cpu())
    assert not torch.equal(a.get_hidden_parameters(), e.get_hidden_parameters())


def _scaled_array_oracle(W, X, bias, cfg, max_tile, omega):
    """Mapped forward with the layer-wise weight scaling and the digital bias: every tile holds
    w / alpha with alpha = max|w_tile| / omega and its ADC output is multiplied by alpha
    (tiles/periphery.py:437-500, 785-805); the bias is added once (tiles/array.py:178-181)."""
    from aihwkit_b200.sharded import split_sizes

    io = O.IO.from_c(cfg.forward_io)
    out_sizes, in_sizes = split_sizes(W.shape[0], max_tile), split_sizes(W.shape[1], max_tile)
    y = np.zeros((X.shape[0], W.shape[0]), np.float32)
    lsb = np.zeros_like(y)
    scales = np.ones((len(in_sizes), len(out_sizes)), np.float32)
    c0 = 0
    for ii, isz in enumerate(in_sizes):
        r0 = 0
        for oi, osz in enumerate(out_sizes):
            wt = W[r0 : r0 + osz, c0 : c0 + isz]
            alpha = np.float32(np.abs(wt).max() / np.float32(omega)) if omega > 0 else np.float32(1)
            alpha = np.float32(1) if alpha == 0 else alpha
            scales[ii, oi] = alpha
            yt, _, scale, _ = O.forward((wt / alpha).astype(np.float32), X[:, c0 : c0 + isz], io, None,
                                        return_pre_adc=True)
            y[:, r0 : r0 + osz] += yt * alpha
            lsb[:, r0 : r0 + osz] = np.maximum(lsb[:, r0 : r0 + osz], (alpha * io.res_out / scale)[:, None])
            r0 += osz
        c0 += isz
    return y + bias[None, :], lsb, scales


@pytest.mark.parametrize("out_size,in_size,max_tile,m,mode", [(256, 384, 128, 40, 1), (768, 2304, 512, 300, 2),
                                                              (100, 1030, 512, 7, 1), (300, 700, 256, 200, 3)])
def test_mapped_forward_weight_scaling_and_bias(out_size, in_size, max_tile, m, mode):
    """Per-tile output scales and the digital bias applied inside the layer's kernels, on the
    CUDA-core path (mode 1) and both tensor-core kernel variants (modes 2, 3)."""
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(out_size + mode)
    cfg = H.inference_params(noise=False)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=3)
    W = rng.normal(0, 0.02, (out_size, in_size)).astype(np.float32)
    bias = rng.normal(0, 0.1, out_size).astype(np.float32)
    X = rng.normal(0, 1, (m, in_size)).astype(np.float32)
    lib = _cabi.lib()
    assert lib.ab200_set_mvm_path(mode) == 0
    try:
        arr = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
        arr.set_weights(torch.from_numpy(W), weight_scaling_omega=0.8)
        arr.set_bias(torch.from_numpy(bias))
        y = arr.forward(torch.from_numpy(X).cuda()).cpu().numpy()
        y_or, lsb, scales = _scaled_array_oracle(W, X, bias, cfg, max_tile, 0.8)
        assert np.allclose(arr.get_tile_scales().numpy(), scales, rtol=1e-6)
        assert np.allclose(arr.get_weights().numpy(), W, rtol=1e-6, atol=1e-9)
        n_in = scales.shape[0]
        diff = np.abs(y - y_or)
        assert (diff > 1e-3 * lsb).mean() <= 2e-3 * n_in
        assert (diff <= 1.001 * lsb * n_in + 1e-6).all()
        # removing the bias and the scaling gives the plain layer again
        arr.set_bias(None)
        arr.set_weights(torch.from_numpy(W))
        y0 = arr.forward(torch.from_numpy(X).cuda()).cpu().numpy()
        y0_or, lsb0, _ = _array_oracle(W, X, cfg, max_tile, max_tile)
        assert (np.abs(y0 - y0_or) <= 1.001 * lsb0 * n_in).all()
    finally:
        lib.ab200_set_mvm_path(0)


@pytest.mark.parametrize("omega,out_size,in_size,max_tile,m", [(0.0, 96, 200, 64, 12), (0.5, 96, 200, 64, 12),
                                                             (0.7, 130, 520, 256, 150), (0.0, 300, 65, 128, 33),
                                                             (0.4, 512, 1024, 512, 260)])
def test_mapped_backward_and_update(omega, out_size, in_size, max_tile, m):
    """Training calls of the mapped layer: backward sums the tiles' IO-managed transposed MVMs over
    the out-splits, update pulses every tile with its block of activations and gradients; with
    weight scaling the gradient is multiplied (backward) / divided (update) by the tile's scale."""
    from aihwkit_b200.rpu_base import tiles as T
    from aihwkit_b200.sharded import split_sizes

    rng = np.random.default_rng(21)
    p = H.training_params(noise=False, pulse_det=True, bm=False)
    dp = H.device("sb", False)
    cfg = p._config(1, 1, dp, seed=3)
    arr = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
    W = rng.uniform(-0.3, 0.3, (out_size, in_size)).astype(np.float32)
    arr.set_weights(torch.from_numpy(W), weight_scaling_omega=omega)
    scales = arr.get_tile_scales().numpy()
    Wl = arr.get_weights().numpy()  # logical weights after the per-element clipping
    X = rng.uniform(-1, 1, (m, in_size)).astype(np.float32)
    Dm = rng.normal(0, 0.1, (m, out_size)).astype(np.float32)
    out_sizes, in_sizes = split_sizes(out_size, max_tile), split_sizes(in_size, max_tile)
    bio = O.IO.from_c(cfg.backward_io, backward=True)
    up = O.Up.from_c(cfg.update)
    lr = 0.02
    arr.set_learning_rate(lr)

    g = arr.backward(torch.from_numpy(Dm).cuda()).cpu().numpy()
    g_or = np.zeros_like(g)
    W_new = np.zeros_like(Wl)
    c0 = 0
    for ii, isz in enumerate(in_sizes):
        r0 = 0
        for oi, osz in enumerate(out_sizes):
            a = scales[ii, oi]
            wt = (Wl[r0 : r0 + osz, c0 : c0 + isz] / a).astype(np.float32)
            g_or[:, c0 : c0 + isz] += O.backward(wt, (Dm[:, r0 : r0 + osz] * a).astype(np.float32), bio)
            # tile (i, o) of the array draws its device parameters with construction seed
            # base + 4099 * i + o
            dpt = H.device("sb", False, seed=dp.construction_seed + 4099 * ii + oi)
            ref_tile = T.AnalogTile(p._config(isz, osz, dpt, seed=3))
            dev = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS, ref_tile.get_hidden_parameter_names(),
                                             ref_tile.get_hidden_parameters().numpy(), 0.0, True)
            wn = wt.copy()
            O.update(wn, X[:, c0 : c0 + isz], (Dm[:, r0 : r0 + osz] / a).astype(np.float32), lr,
                     dp.dw_min, up, dev)
            W_new[r0 : r0 + osz, c0 : c0 + isz] = wn * a
            r0 += osz
        c0 += isz
    step = bio.res_out * np.abs(Dm).max() * scales.max() * len(out_sizes)
    assert np.abs(g - g_or).max() <= 1.001 * step
    assert np.mean(np.abs(g - g_or) > 1e-6) <= 5e-3
    arr.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
    W_got = arr.get_weights().numpy()
    assert np.abs(W_got - Wl).max() > 1e-4
    assert np.abs(W_got - W_new).max() <= 2e-6


@pytest.mark.parametrize("forget,momentum,thres", [(True, 0.0, 2.0), (False, 0.3, 2.0), (True, 0.5, 0.5)])
def test_buffered_transfer_deterministic(forget, momentum, thres):
    """Tiki-Taka v2 on the GPU: fast tile, digital buffer and visible weights follow the oracle
    (pinned to the compiled reference in tests/test_oracle_vs_reference.py) update by update,
    with transfers falling inside the batches."""
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(13)
    x_size, d_size, m = 12, 10, 4
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.buffered_transfer_device(thres_scale=thres, momentum=momentum, forget_buffer=forget,
                                    transfer_lr=4.0)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = T.AnalogTile(cfg, cuda_device=0)
    lr = 0.1
    t.set_learning_rate(lr)
    names, hp = t.get_hidden_parameter_names(), t.get_hidden_parameters().numpy()
    assert names[-1] == "buffered_FP_weight_0"
    fast = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS_REFERENCE, names, hp, 0.0, False, "_0")
    slow = O.DeviceArrays.from_hidden(O.DEV_SOFT_BOUNDS_REFERENCE, names, hp, 0.0, False, "_1")
    orc = O.TransferOracle(np.zeros((d_size, x_size), np.float32), fast, slow, cfg.transfer,
                           O.Up.from_c(cfg.update), 0.002, 0.002, x_size, d_size)
    org = np.random.default_rng(0)
    for _ in range(10):
        x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        d = rng.normal(0, 0.5, (m, d_size)).astype(np.float32)
        t.update(torch.from_numpy(x).cuda(), torch.from_numpy(d).cuda())
        orc.update(x, d, lr, org)
        hp = t.get_hidden_parameters().numpy()
        assert np.abs(hp[names.index("hidden_weights_0")] - orc.a).max() <= 1e-6
        assert np.abs(hp[names.index("buffered_FP_weight_0")] - orc.h).max() <= 1e-5
        assert np.abs(t.get_weights().numpy() - orc.c).max() <= 1e-6
    assert np.abs(orc.c).max() > 0
    # the buffer travels with the hidden parameters
    t2 = T.AnalogTile(cfg, cuda_device=0)
    t2.set_weights(t.get_weights())
    t2.set_hidden_parameters(t.get_hidden_parameters())
    assert torch.equal(t2.get_hidden_parameters(), t.get_hidden_parameters())


@pytest.mark.parametrize("kw", [
    dict(),                                              # every transfer flips its in chopper
    dict(in_chop_prob=0.3, in_chop_random=False),        # regular: every fourth pass
    dict(in_chop_prob=0.0),                              # choppers never move: Tiki-Taka v2 in buffer units
    dict(momentum=0.3, forget_buffer=False, buffer_granularity=0.5, correct_gradient_magnitudes=True),
    dict(auto_granularity=30.0, transfer_every=2.0),
])
def test_chopped_transfer_deterministic_against_reference(kw):
    """Tiki-Taka with choppers (src/rpucuda/rpu_chopped_transfer_device.cpp:357-515) with
    deterministic pulses and chopper schedules that involve no random draw: fast tile, buffer and
    visible weights follow the compiled reference update by update, transfers falling inside the
    batches (so that a chopper flips between two samples of one update call)."""
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    if not ref.available():
        pytest.skip("compiled reference not built")
    rng = np.random.default_rng(17)
    x_size, d_size, m = 12, 10, 5
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.chopped_transfer_device(transfer_lr=4.0, **kw)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = T.AnalogTile(cfg, cuda_device=0)
    rt = ref.RefTile(cfg)
    names = t.get_hidden_parameter_names()
    assert names == rt.hidden_parameter_names()
    assert np.array_equal(t.get_hidden_parameters().numpy(), rt.get_hidden_parameters())
    ia, ih = names.index("hidden_weights_0"), names.index("buffered_FP_weight_0")
    lr = 0.1
    t.set_learning_rate(lr)
    rt.set_learning_rate(lr)
    moved = False
    for step in range(12):
        x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        d = rng.normal(0, 0.5, (m, d_size)).astype(np.float32)
        t.update(torch.from_numpy(x).cuda(), torch.from_numpy(d).cuda())
        rt.update(x, d)
        hp, hr = t.get_hidden_parameters().numpy(), rt.get_hidden_parameters()
        assert np.abs(hp[ia] - hr[ia]).max() <= 1e-6, f"fast tile, update {step}"
        assert np.abs(hp[ih] - hr[ih]).max() <= 1e-4, f"buffer, update {step}"
        assert np.abs(t.get_weights().numpy() - rt.get_weights()).max() <= 1e-6, f"weights, update {step}"
        moved = moved or np.abs(rt.get_weights()).max() > 0
    assert moved and np.abs(hr[ia]).max() > 0


@pytest.mark.parametrize("kw", [
    dict(),                                               # period of two passes
    dict(in_chop_prob=0.3, tail_weightening=2.5),         # period of four passes, heavier tail
    dict(momentum=0.2, forget_buffer=False, buffer_cap=0.5, buffer_granularity=0.5),
    dict(correct_accumulation=True, in_chop_prob=0.25, correct_gradient_magnitudes=True),
])
def test_dynamic_transfer_deterministic_against_reference(kw):
    """Tiki-Taka with choppers and a running-mean reference
    (src/rpucuda/rpu_dynamic_transfer_device.cpp:198-343) with deterministic pulses and the
    regular chopper schedule: fast tile, buffer, running mean, reference mean and visible weights
    follow the compiled reference update by update; writes start after the first chopper period."""
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    if not ref.available():
        pytest.skip("compiled reference not built")
    rng = np.random.default_rng(23)
    x_size, d_size, m = 6, 10, 5
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.dynamic_transfer_device(transfer_lr=4.0, **kw)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = T.AnalogTile(cfg, cuda_device=0)
    rt = ref.RefTile(cfg)
    names = t.get_hidden_parameter_names()
    assert names == rt.hidden_parameter_names()
    assert names[-3:] == ["buffered_FP_weight", "running_mean_weight", "past_mean_weight"]
    assert np.array_equal(t.get_hidden_parameters().numpy(), rt.get_hidden_parameters())
    ia = names.index("hidden_weights_0")
    lr = 0.1
    t.set_learning_rate(lr)
    rt.set_learning_rate(lr)
    moved = False
    for step in range(16):
        x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        d = rng.normal(0, 0.5, (m, d_size)).astype(np.float32)
        t.update(torch.from_numpy(x).cuda(), torch.from_numpy(d).cuda())
        rt.update(x, d)
        hp, hr = t.get_hidden_parameters().numpy(), rt.get_hidden_parameters()
        assert np.abs(hp[ia] - hr[ia]).max() <= 1e-6, f"fast tile, update {step}"
        for q, name in enumerate(names[-3:]):
            assert np.abs(hp[-3 + q] - hr[-3 + q]).max() <= 1e-4, f"{name}, update {step}"
        assert np.abs(t.get_weights().numpy() - rt.get_weights()).max() <= 1e-6, f"weights, update {step}"
        moved = moved or np.abs(rt.get_weights()).max() > 0
    assert moved and np.abs(hr[-1]).max() > 0 and np.abs(hr[-2]).max() > 0
    # the three digital planes travel with the hidden parameters
    t2 = T.AnalogTile(cfg, cuda_device=0)
    t2.set_weights(t.get_weights())
    t2.set_hidden_parameters(t.get_hidden_parameters())
    assert torch.equal(t2.get_hidden_parameters(), t.get_hidden_parameters())


def test_chopped_transfer_random_choppers_statistics():
    """Random in / out chopper flips: the slow tile still integrates the gradient (the de-chopped
    read has the sign of the accumulated gradient whatever the chopper history)."""
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(19)
    x_size, d_size, m = 16, 12, 8
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.chopped_transfer_device(transfer_lr=4.0, in_chop_prob=0.5, out_chop_prob=0.3)
    t = T.AnalogTile(p._config(x_size, d_size, dp, seed=3), cuda_device=0)
    t.set_learning_rate(0.1)
    X = rng.uniform(0.2, 1, (m, x_size)).astype(np.float32)
    Dm = np.abs(rng.normal(0, 0.5, (m, d_size))).astype(np.float32) + 0.1  # constant-sign gradient
    for _ in range(40):
        t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
    w = t.get_weights().numpy()
    assert (w < 0).mean() > 0.95 and np.abs(w).max() > 0.01  # w -= lr d x^T, all terms positive


@pytest.mark.parametrize("kw", [
    dict(),                                                   # all rows after every batch
    dict(n_rows_per_transfer=3),                              # a running window of three rows
    dict(transfer_every=2, n_rows_per_transfer=4, granularity=0.004, transfer_lr=0.5),
    dict(kind="cs", n_x_bins=5, n_d_bins=3),
])
def test_mixed_precision_deterministic_against_reference(kw):
    """Mixed-precision compound (src/rpucuda/rpu_mixedprec_device.cpp:148-345,
    rpu_mixedprec_device_base.cpp:282-352) with both inputs quantised and deterministic pulses:
    the digital accumulator chi and the weights follow the compiled reference update by update
    (the transfer falls after the first sample of a batch, so every call is cut in two)."""
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import ref

    if not ref.available():
        pytest.skip("compiled reference not built")
    rng = np.random.default_rng(29)
    x_size, d_size, m = 12, 10, 5
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.mixed_precision_device(**kw)
    cfg = p._config(x_size, d_size, dp, seed=3)
    t = T.AnalogTile(cfg, cuda_device=0)
    rt = ref.RefTile(cfg)
    names = t.get_hidden_parameter_names()
    assert names == rt.hidden_parameter_names() and names[-1] == "hidden_weights_chi"
    assert np.array_equal(t.get_hidden_parameters().numpy(), rt.get_hidden_parameters())
    lr = 0.1
    t.set_learning_rate(lr)
    rt.set_learning_rate(lr)
    for step in range(10):
        x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        d = rng.normal(0, 0.5, (m, d_size)).astype(np.float32)
        t.update(torch.from_numpy(x).cuda(), torch.from_numpy(d).cuda())
        rt.update(x, d)
        hp, hr = t.get_hidden_parameters().numpy(), rt.get_hidden_parameters()
        assert np.abs(hp[-1] - hr[-1]).max() <= 1e-6, f"chi, update {step}"
        assert np.abs(t.get_weights().numpy() - rt.get_weights()).max() <= 1e-6, f"weights, update {step}"
    assert np.abs(rt.get_weights()).max() > 0.01 and np.abs(hr[-1]).max() > 0
    # chi travels with the hidden parameters; set_weights clears it and the counters
    t2 = T.AnalogTile(cfg, cuda_device=0)
    t2.set_hidden_parameters(t.get_hidden_parameters())
    assert torch.equal(t2.get_hidden_parameters(), t.get_hidden_parameters())
    t.set_weights(t.get_weights())
    assert float(t.get_hidden_parameters()[-1].abs().max()) == 0.0


def test_mixed_precision_unquantised_stochastic_pulses():
    """No quantisation (a plain rank-one accumulation) and stochastic transfer pulses on a
    constant-step device far from its bounds: the weights follow -lr * sum d x^T on average, and
    what chi keeps is the last batch plus less than one granularity per element."""
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(31)
    x_size, d_size, m, lr, n_upd = 24, 16, 8, 0.002, 12
    p = H.training_params(noise=False, pulse_det=False)
    dp = H.mixed_precision_device(kind="cs", n_x_bins=0, n_d_bins=0)
    t = T.AnalogTile(p._config(x_size, d_size, dp, seed=3), cuda_device=0)
    t.set_learning_rate(lr)
    X = rng.uniform(0.2, 1, (m, x_size)).astype(np.float32)
    Dm = np.abs(rng.normal(0, 0.5, (m, d_size))).astype(np.float32) + 0.1
    for _ in range(n_upd):
        t.update(torch.from_numpy(X).cuda(), torch.from_numpy(Dm).cuda())
    w = t.get_weights().numpy()
    chi = t.get_hidden_parameters().numpy()[-1]
    per_batch = lr * Dm.T @ X
    # the transfer of a batch happens one sample into the next: n_upd - 1 batches have moved
    want = -(n_upd - 1) * per_batch
    assert np.abs(want).max() < 0.3  # far from the bounds
    assert (w <= 0).all() and abs(w.sum() / want.sum() - 1.0) < 0.1, w.sum() / want.sum()
    assert np.abs(chi).max() < per_batch.max() + 2 * 0.002 + 1e-6
    # chi + what reached the device is the digital sum up to the stochastic pulse counts
    total = -(w - chi)
    assert abs(total.sum() / (n_upd * per_batch).sum() - 1.0) < 0.1


@pytest.mark.parametrize("seed", range(16))
def test_random_mapped_layers_forward(seed):
    """Random layer shapes and tile sizes (ragged last tiles, single in- or out-splits), with and
    without weight scaling and digital bias, on the CUDA-core kernels and both tensor-core
    variants: one ADC step per in-split of the array oracle."""
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(9000 + seed)
    pick = lambda seq: seq[int(rng.integers(len(seq)))]  # noqa: E731
    out_size, in_size = int(pick([10, 100, 257, 512, 700])), int(pick([30, 129, 512, 640, 1100]))
    max_tile = int(pick([64, 100, 256, 512]))
    m = int(pick([1, 9, 130, 300]))
    omega = float(pick([0.0, 0.6]))
    with_bias = bool(rng.integers(2))
    mode = int(pick([1, 2, 3]))
    p = H.inference_params(noise=False)
    p.forward_io.inp_res = float(pick([1 / 254.0, 1 / 126.0]))
    p.forward_io.out_res = float(pick([1 / 254.0, 1 / 510.0]))
    cfg = p._config(1, 1, D.IdealResistiveDeviceParameter(), seed=3)
    W = rng.normal(0, 0.5 / np.sqrt(in_size), (out_size, in_size)).astype(np.float32)
    bias = rng.normal(0, 0.1, out_size).astype(np.float32) if with_bias else np.zeros(out_size, np.float32)
    X = (rng.normal(0, 1, (m, in_size)) * rng.uniform(0.1, 3.0, (m, 1))).astype(np.float32)
    lib = _cabi.lib()
    assert lib.ab200_set_mvm_path(mode) == 0
    try:
        arr = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
        arr.set_weights(torch.from_numpy(W), weight_scaling_omega=omega)
        if with_bias:
            arr.set_bias(torch.from_numpy(bias))
        y = arr.forward(torch.from_numpy(X).cuda()).cpu().numpy()
        y_or, lsb, scales = _scaled_array_oracle(W, X, bias, cfg, max_tile, omega)
        n_in = scales.shape[0]
        diff = np.abs(y - y_or)
        assert (diff > 1e-3 * lsb).mean() <= 3e-3 * n_in, (mode, (diff > 1e-3 * lsb).mean())
        assert (diff <= 1.001 * lsb * n_in + 1e-6).all(), (mode, (diff / lsb).max())
    finally:
        lib.ab200_set_mvm_path(0)
