"""The allocation-free forward entry point against the regular tile entry point.

`ab200_mvm_forward_noalloc` exists for hosts that reserve the GPU's memory up front and forbid
allocation afterwards (a serving loop's execute callback, a real-time loop): it keeps its
per-sample scratch in a fixed array inside the library instead of growing it with cudaMalloc.
It has to give the same numbers as `ab200_tile_forward`.  Two calls in a row are checked because
all calls share that one array and it keeps the previous call's contents.
"""

import ctypes as C

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _stream(t):
    return int(torch.cuda.current_stream(t.device).cuda_stream)


@pytest.mark.parametrize("noise", [False, True])
def test_noalloc_forward_matches_tile_forward_twice(noise):
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import tiles as T

    lib = _cabi.lib()
    x_size, d_size = 200, 136
    # out_bound 3 makes iterative bound management re-run some rows, so the flag and counter part
    # of the shared scratch is exercised as well
    p = H.training_params(noise=noise, pulse_det=True, bm=True, out_bound=3.0)
    seed = 4242
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=seed)
    tile = T.AnalogTile(cfg, cuda_device=0)
    rng = np.random.default_rng(0)
    tile.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
    w_xd = tile.get_weights_cuda()
    io = cfg.forward_io

    for call, m in enumerate((96, 40)):  # second call is smaller: stale rows stay in the array
        x = torch.from_numpy(rng.uniform(-1, 1, (m, x_size)).astype(np.float32)).cuda()
        y_tile = tile.forward(x)  # the tile's `call`-th forward: noise key (seed, call)
        y = torch.full((m, d_size), float("nan"), device="cuda")
        rc = lib.ab200_mvm_forward_noalloc(C.byref(io), w_xd.data_ptr(), x_size, d_size,
                                           x.data_ptr(), y.data_ptr(), m, seed, call, _stream(x))
        assert rc == 0, lib.ab200_last_error()
        torch.cuda.synchronize()
        n_rerun, _ = tile.last_bm_stats()
        assert n_rerun > 0
        # same kernels, same noise key: identical within the tolerance of the parity tests
        assert torch.allclose(y, y_tile, rtol=0.0, atol=1e-6), (y - y_tile).abs().max()


def test_noalloc_forward_against_the_oracle_and_without_allocating():
    """Noise off: the entry point against the numpy oracle directly; and the call leaves the
    device's free memory as it found it (batch near the limit, bound management active)."""
    from aihwkit_b200 import _cabi
    from oracle import analog_tile_oracle as O

    lib = _cabi.lib()
    x_size, d_size, m = 96, 72, 16000
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=3.0)
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=7)
    rng = np.random.default_rng(5)
    w = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    w_xd = torch.from_numpy(np.ascontiguousarray(w.T)).cuda()
    xg = torch.from_numpy(x).cuda()
    y = torch.empty(m, d_size, device="cuda")

    def call(k):
        rc = lib.ab200_mvm_forward_noalloc(C.byref(cfg.forward_io), w_xd.data_ptr(), x_size, d_size,
                                           xg.data_ptr(), y.data_ptr(), m, 7, k, _stream(xg))
        assert rc == 0, lib.ab200_last_error()
        torch.cuda.synchronize()

    call(0)  # the first call on a device resolves the scratch array's address
    free_before, _ = torch.cuda.mem_get_info()
    call(1)
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    io = O.IO.from_c(cfg.forward_io)
    y_or, _, scale, _ = O.forward(w, x, io, return_pre_adc=True)
    frac, worst = H.lsb_report(y.cpu().numpy(), y_or, (io.res_out / scale)[:, None])
    assert frac <= 2e-3 and worst <= 1.001, (frac, worst)


def test_noalloc_rejects_oversized_batch():
    from aihwkit_b200 import _cabi

    lib = _cabi.lib()
    p = H.training_params(noise=False, pulse_det=True)
    cfg = p._config(8, 8, H.device("cs", False), seed=1)
    w = torch.zeros(8, 8, device="cuda")
    x = torch.zeros(1, 8, device="cuda")
    y = torch.zeros(1, 8, device="cuda")
    too_many = 16384 + 1
    rc = lib.ab200_mvm_forward_noalloc(C.byref(cfg.forward_io), w.data_ptr(), 8, 8, x.data_ptr(),
                                       y.data_ptr(), too_many, 1, 0, _stream(x))
    assert rc != 0
    assert b"exceeds" in lib.ab200_last_error()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_noalloc_forward_on_a_second_device():
    """Every GPU has its own copy of the scratch array; its address is resolved per device on the
    first call there."""
    from aihwkit_b200 import _cabi
    from oracle import analog_tile_oracle as O

    lib = _cabi.lib()
    x_size, d_size, m = 64, 48, 300
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=3.0)
    cfg = p._config(x_size, d_size, H.device("cs", False), seed=7)
    rng = np.random.default_rng(9)
    w = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    io = O.IO.from_c(cfg.forward_io)
    y_or, _, scale, _ = O.forward(w, x, io, return_pre_adc=True)
    for dev in (1, 0, 1):
        with torch.cuda.device(dev):
            w_xd = torch.from_numpy(np.ascontiguousarray(w.T)).cuda()
            xg = torch.from_numpy(x).cuda()
            y = torch.empty(m, d_size, device="cuda")
            rc = lib.ab200_mvm_forward_noalloc(C.byref(cfg.forward_io), w_xd.data_ptr(), x_size, d_size,
                                               xg.data_ptr(), y.data_ptr(), m, 7, 0, _stream(xg))
            assert rc == 0, lib.ab200_last_error()
            torch.cuda.synchronize()
            frac, worst = H.lsb_report(y.cpu().numpy(), y_or, (io.res_out / scale)[:, None])
            assert frac <= 2e-3 and worst <= 1.001, (dev, frac, worst)
