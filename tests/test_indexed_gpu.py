"""Indexed (im2col-free) convolution interface on the GPU: against the vectors of the compiled
reference (tests/golden/indexed_conv.npz), against the numpy oracle on fresh inputs in both index
layouts, and on a case large enough for the tensor-core path."""

import ctypes as C
import os

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _gpu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _check_lsb(got, want, lsb, frac_max=2e-3):
    frac, worst = H.lsb_report(got, want, lsb)
    assert frac <= frac_max and worst <= 1.001, (frac, worst)


def test_golden_indexed_conv():
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import analog_tile_oracle as O

    g = np.load(os.path.join(GOLD, "indexed_conv.npz"))
    n = g["x"].shape[0]
    c_out, x_size = g["w0"].shape
    m_batch = g["indices"].size // x_size
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=float(g["out_bound"]))
    cfg = p._config(x_size, c_out, H.device("sb", False), seed=1)
    t = T.AnalogTile(cfg, cuda_device=0)
    t.set_hidden_parameters(torch.from_numpy(g["hidden"]))
    t.set_weights(torch.from_numpy(g["w0"]))
    assert not t.has_matrix_indices()
    with pytest.raises(RuntimeError, match="not set"):
        t.forward_indexed(_gpu(g["x"]), torch.empty(g["y"].shape, device="cuda"))
    t.set_matrix_indices(torch.from_numpy(g["indices"]))  # host tensor: the tile copies it
    assert t.has_matrix_indices()

    fio, bio = O.IO.from_c(cfg.forward_io), O.IO.from_c(cfg.backward_io, backward=True)
    cols = O.indexed_input(g["x"], g["indices"], x_size, m_batch, n, True)
    _, _, scale, _ = O.forward(g["w0"], cols, fio, return_pre_adc=True)
    y = t.forward_indexed(_gpu(g["x"]), torch.empty(g["y"].shape, device="cuda")).cpu().numpy()
    lsb = O.from_sample_major(np.repeat((fio.res_out / scale)[:, None], c_out, 1), c_out, m_batch, n, True)
    _check_lsb(y.reshape(n, c_out, m_batch), g["y"].reshape(n, c_out, m_batch), lsb)

    xg = t.backward_indexed(_gpu(g["d"]), torch.empty(g["x"].shape, device="cuda")).cpu().numpy()
    # every image element sums at most 9 ADC values; allow one ADC step of the largest row scale
    d_cols = O.to_sample_major(g["d"], c_out, m_batch, n, True)
    step = float((bio.res_out * np.abs(d_cols).max(axis=1)).max())
    assert np.abs(xg - g["g"]).max() <= 1.001 * step
    assert np.mean(np.abs(xg - g["g"]) > 1e-6) <= 5e-3

    t.set_learning_rate(float(g["lr"]))
    t.update_indexed(_gpu(g["x"]), _gpu(g["d"]))
    assert np.abs(t.get_weights().numpy() - g["w1"]).max() <= 1e-6


@pytest.fixture
def mvm_path(request):
    """Kernel selection of the MVM for one test: 0 automatic, 2 tensor cores wherever possible."""
    from aihwkit_b200 import _cabi

    lib = _cabi.lib()
    assert lib.ab200_set_mvm_path(request.param) == 0
    yield request.param
    lib.ab200_set_mvm_path(0)


@pytest.mark.parametrize("trans", [True, False])
@pytest.mark.parametrize("analog_bias", [False, True])
@pytest.mark.parametrize("mvm_path", [0, 2], indirect=True)
def test_layouts_against_oracle(trans, analog_bias, mvm_path):
    """Both index layouts through the C ABI (the Python binding only uses `trans`); on the
    tensor-core path the DAC kernel and the bound-management re-run gather the rows from the
    images themselves, on the CUDA-core path the unfolded matrix is written first."""
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import analog_tile_oracle as O

    rng = np.random.default_rng(11)
    n, c, h, w, c_out = 3, 6, 10, 7, 9
    idx_t = O.conv_indices((c, h, w), (3, 2), (1, 2), (1, 0), (1, 1), analog_bias)
    x_size = c * 6 + (1 if analog_bias else 0)
    m_batch = idx_t.size // x_size
    idx = idx_t if trans else np.ascontiguousarray(idx_t.reshape(x_size, m_batch).T).reshape(-1)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=3.0)
    dp = H.device("cs", False)
    cfg = p._config(x_size, c_out, dp, seed=5)
    t = T.AnalogTile(cfg, cuda_device=0)
    w0 = rng.uniform(-0.5, 0.5, (c_out, x_size)).astype(np.float32)
    t.set_weights(torch.from_numpy(w0))
    w0 = t.get_weights().numpy()
    lib = _cabi.lib()
    idx_dev = _gpu(idx.astype(np.int32))  # device tensor this time
    _cabi.check(lib.ab200_tile_set_matrix_indices(t._h, idx_dev.data_ptr(), idx_dev.numel(), None))
    del idx_dev  # the tile owns a copy

    X = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
    d_shape = (n, c_out, m_batch) if trans else (n, m_batch, c_out)
    Dm = rng.normal(0, 0.1, d_shape).astype(np.float32)
    xd, dd = _gpu(X), _gpu(Dm)
    fio, bio = O.IO.from_c(cfg.forward_io), O.IO.from_c(cfg.backward_io, backward=True)

    cols = O.indexed_input(X, idx, x_size, m_batch, n, trans)
    y_ref, _, scale, _ = O.forward(w0, cols, fio, return_pre_adc=True)
    y = torch.empty(d_shape, device="cuda")
    _cabi.check(lib.ab200_tile_forward_indexed(t._h, xd.data_ptr(), y.data_ptr(), X.size, m_batch, n,
                                               int(trans), 0, None))
    torch.cuda.synchronize()
    got = O.to_sample_major(y.cpu().numpy(), c_out, m_batch, n, trans)
    _check_lsb(got, y_ref, (fio.res_out / scale)[:, None])

    d_cols = O.to_sample_major(Dm, c_out, m_batch, n, trans)
    xg_ref = O.indexed_output(O.backward(w0, d_cols, bio), idx, x_size, m_batch, n, trans, X.size)
    xg = torch.full(X.shape, 7.0, device="cuda")  # must be overwritten, not accumulated into
    _cabi.check(lib.ab200_tile_backward_indexed(t._h, dd.data_ptr(), xg.data_ptr(), X.size, m_batch, n,
                                                int(trans), None))
    torch.cuda.synchronize()
    step = float((bio.res_out * np.abs(d_cols).max(axis=1)).max())
    diff = np.abs(xg.cpu().numpy().reshape(n, -1) - xg_ref)
    assert diff.max() <= 1.001 * step and np.mean(diff > 1e-6) <= 5e-3
    # the sum over the entries that name an element has a fixed order: same bits on every run
    xg2 = torch.full(X.shape, -3.0, device="cuda")
    _cabi.check(lib.ab200_tile_backward_indexed(t._h, dd.data_ptr(), xg2.data_ptr(), X.size, m_batch, n,
                                                int(trans), None))
    torch.cuda.synchronize()
    assert torch.equal(xg, xg2)

    lr = 0.01
    t.set_learning_rate(lr)
    names = [t._lib.ab200_tile_hidden_parameter_name(t._h, k).decode()
             for k in range(t._lib.ab200_tile_hidden_parameter_count(t._h))]
    dev = O.DeviceArrays.from_hidden(O.DEV_CONSTANT_STEP, names, t.get_hidden_parameters().numpy(),
                                     0.0, True)
    _cabi.check(lib.ab200_tile_update_indexed(t._h, xd.data_ptr(), dd.data_ptr(), X.size, m_batch, n,
                                              int(trans), None))
    torch.cuda.synchronize()
    w1 = w0.copy()
    O.update(w1, cols, d_cols, lr, dp.dw_min, O.Up.from_c(cfg.update), dev)
    assert np.abs(t.get_weights().numpy() - w1).max() <= 1e-6


def test_errors():
    from aihwkit_b200.rpu_base import tiles as T

    p = H.training_params(noise=False, pulse_det=True)
    t = T.AnalogTile(p._config(18, 4, H.device("cs", False), seed=5), cuda_device=0)
    with pytest.raises(RuntimeError, match="negative"):
        t.set_matrix_indices(torch.tensor([3, -1, 2], dtype=torch.int32))
    t.set_matrix_indices(torch.full((18 * 5,), 40, dtype=torch.int32))
    x = torch.zeros(2, 2, 3, 3, device="cuda")  # 18 elements per image, index 40 needs 39
    with pytest.raises(RuntimeError, match="outside an image"):
        t.forward_indexed(x, torch.empty(2, 4, 5, 1, device="cuda"))
    with pytest.raises(RuntimeError, match="entries"):
        t.forward_indexed(torch.zeros(2, 50, device="cuda").reshape(2, 50, 1, 1),
                          torch.empty(2, 4, 3, 1, device="cuda"))


def test_conv_sized_for_tensor_cores():
    """3x3 convolution, 32 channels, 8 images of 16x16: 2048 columns, the tensor-core path."""
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import analog_tile_oracle as O

    rng = np.random.default_rng(12)
    n, c, h, w, c_out = 8, 32, 16, 16, 64
    idx = O.conv_indices((c, h, w), (3, 3), (1, 1), (1, 1))
    x_size = c * 9
    m_batch = idx.size // x_size
    p = H.training_params(noise=False, pulse_det=True, bm=False)
    cfg = p._config(x_size, c_out, H.device("cs", False), seed=5)
    t = T.AnalogTile(cfg, cuda_device=0)
    w0 = (rng.standard_normal((c_out, x_size)) * 0.1).astype(np.float32)
    t.set_weights(torch.from_numpy(w0))
    w0 = t.get_weights().numpy()
    t.set_matrix_indices(_gpu(idx))
    X = np.maximum(rng.standard_normal((n, c, h, w)), 0).astype(np.float32)
    fio = O.IO.from_c(cfg.forward_io)
    cols = O.indexed_input(X, idx, x_size, m_batch, n, True)
    y_ref, _, scale, _ = O.forward(w0, cols, fio, return_pre_adc=True)
    y = t.forward_indexed(_gpu(X), torch.empty(n, c_out, h, w, device="cuda")).cpu().numpy()
    got = O.to_sample_major(y, c_out, m_batch, n, True)
    _check_lsb(got, y_ref, (fio.res_out / scale)[:, None], frac_max=5e-3)
    # and against torch's own convolution when the analog IO is switched off entirely
    p2 = H.training_params(noise=False, pulse_det=True, bm=False)
    p2.forward_io.is_perfect = True
    t2 = T.AnalogTile(p2._config(x_size, c_out, H.device("cs", False), seed=5), cuda_device=0)
    t2.set_weights(torch.from_numpy(w0))
    t2.set_matrix_indices(_gpu(idx))
    y2 = t2.forward_indexed(_gpu(X), torch.empty(n, c_out, h, w, device="cuda"))
    tf32 = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False  # the comparison needs a true fp32 convolution
    try:
        conv = torch.nn.functional.conv2d(
            _gpu(X), _gpu(t2.get_weights().numpy().reshape(c_out, c, 3, 3)), padding=1)
    finally:
        torch.backends.cudnn.allow_tf32 = tf32
    assert torch.allclose(y2, conv, rtol=1e-4, atol=1e-4)


N_GEOMETRIES = 24


@pytest.mark.parametrize("seed", range(N_GEOMETRIES))
def test_random_convolution_geometries(seed):
    """Random convolution geometries (kernel, stride, padding, dilation, channels, map size, analog
    bias, both index layouts) through the three indexed entry points, on the automatic kernel
    selection and with the tensor-core kernels forced on (where the DAC kernel and the
    bound-management re-run gather the rows and the MVM kernels store image-major outputs),
    against the numpy restatement of the reference's copyIndexedInput / copyIndexedOutput."""
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import analog_tile_oracle as O

    rng = np.random.default_rng(7000 + seed)
    pick = lambda seq: seq[int(rng.integers(len(seq)))]  # noqa: E731
    c, h, w = int(pick([1, 3, 6, 16])), int(pick([4, 7, 12])), int(pick([5, 8, 11]))
    kernel = (int(pick([1, 2, 3])), int(pick([1, 2, 3])))
    stride = (int(pick([1, 2])), int(pick([1, 2])))
    padding = (int(pick([0, 1, 2])), int(pick([0, 1])))
    dilation = (int(pick([1, 1, 2])), 1)
    analog_bias, trans = bool(rng.integers(2)), bool(rng.integers(2))
    n, c_out = int(pick([1, 2, 5])), int(pick([1, 9, 40]))
    if h + 2 * padding[0] < dilation[0] * (kernel[0] - 1) + 1 or w + 2 * padding[1] < kernel[1]:
        pytest.skip("kernel larger than the padded map")
    idx_t = O.conv_indices((c, h, w), kernel, stride, padding, dilation, analog_bias)
    x_size = c * kernel[0] * kernel[1] + (1 if analog_bias else 0)
    m_batch = idx_t.size // x_size
    idx = idx_t if trans else np.ascontiguousarray(idx_t.reshape(x_size, m_batch).T).reshape(-1)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=float(pick([12.0, 2.0])))
    dp = H.device("cs", False)
    cfg = p._config(x_size, c_out, dp, seed=5)
    fio, bio = O.IO.from_c(cfg.forward_io), O.IO.from_c(cfg.backward_io, backward=True)
    X = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
    d_shape = (n, c_out, m_batch) if trans else (n, m_batch, c_out)
    Dm = rng.normal(0, 0.1, d_shape).astype(np.float32)
    cols = O.indexed_input(X, idx, x_size, m_batch, n, trans)
    d_cols = O.to_sample_major(Dm, c_out, m_batch, n, trans)
    lib = _cabi.lib()
    try:
        for mode in (0, 2):
            assert lib.ab200_set_mvm_path(mode) == 0
            t = T.AnalogTile(cfg, cuda_device=0)
            w0 = rng.uniform(-0.5, 0.5, (c_out, x_size)).astype(np.float32)
            t.set_weights(torch.from_numpy(w0))
            w0 = t.get_weights().numpy()
            idx32 = np.ascontiguousarray(idx, np.int32)  # host array this time; kept alive over the call
            _cabi.check(lib.ab200_tile_set_matrix_indices(t._h, idx32.ctypes.data, idx32.size, None))
            xd, dd = _gpu(X), _gpu(Dm)
            y_ref, _, scale, _ = O.forward(w0, cols, fio, return_pre_adc=True)
            y = torch.full(d_shape, 5.0, device="cuda")
            _cabi.check(lib.ab200_tile_forward_indexed(t._h, xd.data_ptr(), y.data_ptr(), X.size, m_batch, n,
                                                       int(trans), 0, None))
            torch.cuda.synchronize()
            got = O.to_sample_major(y.cpu().numpy(), c_out, m_batch, n, trans)
            zero_rows = scale == 0  # rows without input: output 0, no step to compare in
            lsb = np.where(zero_rows, 1.0, fio.res_out / np.where(zero_rows, 1.0, scale))[:, None]
            _check_lsb(got, y_ref, lsb, frac_max=1e-2)
            xg_ref = O.indexed_output(O.backward(w0, d_cols, bio), idx, x_size, m_batch, n, trans, X.size)
            xg = torch.full(X.shape, 7.0, device="cuda")
            _cabi.check(lib.ab200_tile_backward_indexed(t._h, dd.data_ptr(), xg.data_ptr(), X.size, m_batch, n,
                                                        int(trans), None))
            torch.cuda.synchronize()
            step = float((bio.res_out * np.abs(d_cols).max(axis=1)).max())
            diff = np.abs(xg.cpu().numpy().reshape(n, -1) - xg_ref)
            assert diff.max() <= 1.001 * step and np.mean(diff > 1e-6) <= 1e-2, (mode, diff.max(), step)
            t.set_learning_rate(0.01)
            names = t.get_hidden_parameter_names()
            dev = O.DeviceArrays.from_hidden(O.DEV_CONSTANT_STEP, names, t.get_hidden_parameters().numpy(),
                                             0.0, True)
            _cabi.check(lib.ab200_tile_update_indexed(t._h, xd.data_ptr(), dd.data_ptr(), X.size, m_batch, n,
                                                      int(trans), None))
            torch.cuda.synchronize()
            w1 = w0.copy()
            O.update(w1, cols, d_cols, 0.01, dp.dw_min, O.Up.from_c(cfg.update), dev)
            assert np.abs(t.get_weights().numpy() - w1).max() <= 1e-6, mode
    finally:
        lib.ab200_set_mvm_path(0)


@pytest.mark.parametrize("which", ["sb", "transfer", "chopped", "mixed"])
@pytest.mark.parametrize("n_img", [1, 6])
def test_indexed_update_equals_update_on_the_unfolded_matrix(which, n_img):
    """update_indexed (the pulse preparation gathers its samples from the images; a compound cuts
    the batch at its transfers) against update on the unfolded matrix with the same seed and
    stochastic pulses: the same samples, the same trains, the same weights and hidden planes bit
    for bit - small batches (staged kernel) and large ones (streaming kernel)."""
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import analog_tile_oracle as O

    rng = np.random.default_rng(17)
    c, h, w, c_out = 5, 9, 8, 11
    idx = O.conv_indices((c, h, w), (3, 3), (1, 1), (1, 1), (1, 1), True)
    x_size = c * 9 + 1
    m_batch = idx.size // x_size
    p = H.training_params(noise=True, pulse_det=False)
    if which == "sb":
        dp = H.device("sb", True)
    elif which == "transfer":
        dp = H.transfer_device(True, transfer_every=7.0, units_in_mbatch=False, n_reads=2)
    elif which == "chopped":
        dp = H.chopped_transfer_device(transfer_lr=4.0, in_chop_prob=0.3, in_chop_random=False, transfer_every=5.0)
    else:
        dp = H.mixed_precision_device(n_rows_per_transfer=4)
    cfg = p._config(x_size, c_out, dp, seed=5)
    a, b = T.AnalogTile(cfg, cuda_device=0), T.AnalogTile(cfg, cuda_device=0)
    a.set_matrix_indices(_gpu(idx))
    W = rng.uniform(-0.3, 0.3, (c_out, x_size)).astype(np.float32)
    for t in (a, b):
        t.set_weights(torch.from_numpy(W))
        t.set_learning_rate(0.05)
    for _ in range(3):
        X = np.maximum(rng.standard_normal((n_img, c, h, w)), 0).astype(np.float32)
        Dm = rng.normal(0, 0.2, (n_img, c_out, m_batch)).astype(np.float32)
        a.update_indexed(_gpu(X), _gpu(Dm.reshape(n_img, c_out, h, w)))
        cols = O.indexed_input(X, idx, x_size, m_batch, n_img, True)
        d_cols = O.to_sample_major(Dm, c_out, m_batch, n_img, True)
        b.update(_gpu(cols), _gpu(d_cols))
    assert float((a.get_weights() - torch.from_numpy(np.clip(W, -1, 1))).abs().max()) > 0 or which != "sb"
    assert torch.equal(a.get_weights(), b.get_weights())
    assert torch.equal(a.get_hidden_parameters(), b.get_hidden_parameters())


@pytest.mark.parametrize("mvm_path", [0, 2], indirect=True)
def test_indexed_forward_equals_forward_on_the_unfolded_matrix_with_noise(mvm_path):
    """forward_indexed with all noise sources of the training IO on against forward on the
    unfolded matrix with the same seed: same DAC codes, same noise counters (keyed by the row of
    the batch), so the image-major result is the transpose of the row-major one bit for bit -
    whether the DAC kernel gathers the rows itself (tensor-core path) or the matrix is written
    first."""
    from aihwkit_b200.rpu_base import tiles as T
    from oracle import analog_tile_oracle as O

    rng = np.random.default_rng(19)
    n_img, c, h, w, c_out = 3, 12, 10, 9, 40
    idx = O.conv_indices((c, h, w), (3, 3), (1, 1), (1, 1), (1, 1), False)
    x_size = c * 9
    m_batch = idx.size // x_size
    p = H.training_params(noise=True, pulse_det=False, bm=True, out_bound=3.0)
    cfg = p._config(x_size, c_out, H.device("cs", True), seed=5)
    a, b = T.AnalogTile(cfg, cuda_device=0), T.AnalogTile(cfg, cuda_device=0)
    a.set_matrix_indices(_gpu(idx))
    W = rng.uniform(-0.5, 0.5, (c_out, x_size)).astype(np.float32)
    for t in (a, b):
        t.set_weights(torch.from_numpy(W))
    for _ in range(2):
        X = rng.uniform(-1, 1, (n_img, c, h, w)).astype(np.float32)
        ya = a.forward_indexed(_gpu(X), torch.empty(n_img, c_out, h, w, device="cuda")).cpu().numpy()
        cols = O.indexed_input(X, idx, x_size, m_batch, n_img, True)
        yb = b.forward(_gpu(cols)).cpu().numpy()
        assert np.array_equal(O.to_sample_major(ya.reshape(n_img, c_out, m_batch), c_out, m_batch, n_img, True), yb)
        assert a.last_bm_stats() == b.last_bm_stats() and a.last_bm_stats()[0] > 0
