"""The tensor-core (tcgen05 / TMEM / TMA) MVM kernel against the oracle and against the
CUDA-core kernels, forced on with ab200_set_mvm_path(2) so that small and ragged shapes are
covered too."""

import numpy as np
import pytest
import torch

from oracle import analog_tile_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture()
def path():
    from aihwkit_b200 import _cabi

    lib = _cabi.lib()

    def set_path(mode):
        assert lib.ab200_set_mvm_path(mode) == 0

    yield set_path
    lib.ab200_set_mvm_path(0)


def _tile(p, dp, x, d, seed=5):
    from aihwkit_b200.rpu_base import tiles as T

    cfg = p._config(x, d, dp, seed=seed)
    return T.AnalogTile(cfg, cuda_device=0), cfg


SHAPES = [(64, 128, 128), (512, 512, 256), (100, 36, 33), (461, 300, 130), (1024, 1024, 256)]


@pytest.mark.parametrize("x_size,d_size,m", SHAPES)
def test_tc_forward_backward_pre_adc(path, x_size, d_size, m):
    """ADC off, noise off: integer DAC codes x (bf16 hi + lo) weights with fp32 accumulation
    stay within 1e-5 of the output range of the fp32 oracle."""
    path(2)
    rng = np.random.default_rng(x_size + m)
    p = H.training_params(noise=False, pulse_det=True, bm=False, adc=False, out_bound=0.0)
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    X[1] = 0.0
    y = t.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    y_or = O.forward(W, X, O.IO.from_c(cfg.forward_io))
    assert np.abs(y - y_or).max() <= 1e-5 * np.abs(y_or).max()
    assert np.all(y[1] == 0)
    g = t.backward(torch.from_numpy(Dm).cuda()).cpu().numpy()
    g_or = O.backward(W, Dm, O.IO.from_c(cfg.backward_io, backward=True))
    assert np.abs(g - g_or).max() <= 1e-5 * np.abs(g_or).max()


@pytest.mark.parametrize("x_size,d_size,m", SHAPES)
@pytest.mark.parametrize("out_bound", [12.0, 2.0])
def test_tc_forward_backward_post_adc(path, x_size, d_size, m, out_bound):
    path(2)
    rng = np.random.default_rng(7 * x_size + m)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=out_bound)
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    t.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
    W = t.get_weights().numpy()
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    fio = O.IO.from_c(cfg.forward_io)
    y = t.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    y_or, _, scale, red = O.forward(W, X, fio, return_pre_adc=True)
    frac, worst = H.lsb_report(y, y_or, (fio.res_out / scale)[:, None])
    assert frac <= 1e-3 and worst <= 1.001, (frac, worst)
    n_rerun, max_red = t.last_bm_stats()
    assert n_rerun == int((red > 1).sum()) and max_red == float(red.max())
    bio = O.IO.from_c(cfg.backward_io, backward=True)
    g = t.backward(torch.from_numpy(Dm).cuda()).cpu().numpy()
    g_or = O.backward(W, Dm, bio)
    frac, worst = H.lsb_report(g, g_or, (bio.res_out * np.abs(Dm).max(axis=1))[:, None])
    assert frac <= 1e-3 and worst <= 1.001, (frac, worst)


def test_tc_and_cuda_core_paths_draw_the_same_noise(path):
    """Noise on: both kernels key the noise by (seed, call, element), so the same call gives the
    same output up to rare ADC flips caused by the different product rounding."""
    rng = np.random.default_rng(3)
    x_size, d_size, m = 256, 192, 160
    p = H.training_params(noise=True, pulse_det=False, bm=True)
    outs = []
    for mode in (1, 2):
        path(mode)
        t, cfg = _tile(p, H.device("cs", True), x_size, d_size, seed=99)
        t.set_weights(torch.from_numpy(np.random.default_rng(1).uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
        X = torch.from_numpy(np.random.default_rng(2).uniform(-1, 1, (m, x_size)).astype(np.float32)).cuda()
        outs.append(t.forward(X).cpu().numpy())
    lsb = O.IO.from_c(cfg.forward_io).res_out * 1.0  # scale <= 1 since |x| <= 1
    diff = np.abs(outs[0] - outs[1])
    assert (diff > 1e-4).mean() <= 1e-3
    assert diff.max() <= 1.01 * lsb * np.abs(X.cpu().numpy()).max()


@pytest.mark.parametrize("out_size,in_size,max_tile,m", [(256, 384, 128, 140), (768, 2304, 512, 130),
                                                         (100, 1030, 512, 7), (1024, 1024, 512, 512)])
def test_tc_mapped_forward(path, out_size, in_size, max_tile, m):
    from aihwkit_b200.rpu_base import devices as D, tiles as T
    from tests.test_mapped_and_transfer_gpu import _array_oracle

    rng = np.random.default_rng(out_size)
    W = rng.normal(0, 1 / np.sqrt(in_size), (out_size, in_size)).astype(np.float32)
    X = rng.normal(0, 1, (m, in_size)).astype(np.float32)
    # noise off against the oracle
    path(2)
    cfg = H.inference_params(noise=False)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=3)
    arr = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
    arr.set_weights(torch.from_numpy(W))
    y = arr.forward(torch.from_numpy(X).cuda()).cpu().numpy()
    y_or, lsb, n_in = _array_oracle(W, X, cfg, max_tile, max_tile)
    diff = np.abs(y - y_or)
    assert (diff > 1e-3 * lsb).mean() <= 1e-3 * n_in
    assert (diff <= 1.001 * lsb * n_in).all()
    # noise on: tensor-core and CUDA-core paths agree call by call
    cfgn = H.inference_params(noise=True)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=8)
    outs = []
    for mode in (1, 2):
        path(mode)
        a = T.TileArray(cfgn, out_size, in_size, max_tile, max_tile, cuda_device=0)
        a.set_weights(torch.from_numpy(W))
        outs.append(a.forward(torch.from_numpy(X).cuda()).cpu().numpy())
    d2 = np.abs(outs[0] - outs[1])
    assert (d2 > 1e-3 * lsb).mean() <= 2e-3 * n_in
    assert (d2 <= 1.001 * lsb * n_in).all()


def test_tc_operand_cache_follows_weight_changes(path):
    path(2)
    rng = np.random.default_rng(5)
    x_size, d_size, m = 128, 128, 128
    p = H.training_params(noise=False, pulse_det=True, bm=False)
    t, cfg = _tile(p, H.device("cs", False), x_size, d_size)
    X = torch.from_numpy(rng.uniform(-1, 1, (m, x_size)).astype(np.float32)).cuda()
    Dm = torch.from_numpy(rng.normal(0, 0.1, (m, d_size)).astype(np.float32)).cuda()
    fio = O.IO.from_c(cfg.forward_io)
    for step in range(3):
        if step == 0:
            t.set_weights(torch.from_numpy(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)))
        else:
            t.set_learning_rate(0.05)
            t.update(X, Dm)  # weights move; the bf16 operand must be rebuilt
        W = t.get_weights().numpy()
        y = t.forward(X).cpu().numpy()
        y_or, _, scale, _ = O.forward(W, X.cpu().numpy(), fio, return_pre_adc=True)
        frac, worst = H.lsb_report(y, y_or, (fio.res_out / scale)[:, None])
        assert frac <= 1e-3 and worst <= 1.001, (step, frac, worst)


@pytest.mark.parametrize("out_size,in_size,max_tile,m", [(768, 2304, 512, 300), (1024, 1024, 512, 1024),
                                                         (256, 384, 128, 129)])
def test_cta_pair_and_single_cta_kernels_agree(path, out_size, in_size, max_tile, m):
    """The kernel variant that pairs two CTAs on a 256-row tile (mode 2, used whenever there are
    more than 128 rows) and the single-CTA variant (mode 3) compute the same products and draw
    the same noise: results are equal bit for bit, ragged last row block included."""
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(m)
    W = rng.normal(0, 1 / np.sqrt(in_size), (out_size, in_size)).astype(np.float32)
    X = torch.from_numpy(rng.normal(0, 1, (m, in_size)).astype(np.float32)).cuda()
    cfg = H.inference_params(noise=True)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=8)
    outs = []
    for mode in (2, 3):
        path(mode)
        a = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
        a.set_weights(torch.from_numpy(W))
        outs.append([a.forward(X).cpu().numpy() for _ in range(2)])
    assert np.array_equal(outs[0][0], outs[1][0])
    assert np.array_equal(outs[0][1], outs[1][1])
    assert not np.array_equal(outs[0][0], outs[0][1])  # a new call draws new noise
    # single tile with bound management, forward and backward
    p = H.training_params(noise=True, pulse_det=True, bm=True, out_bound=2.0)
    res = []
    for mode in (2, 3):
        path(mode)
        t, _ = _tile(p, H.device("cs", False), 384, 200, seed=6)
        t.set_weights(torch.from_numpy(W[:200, :384] * 5))
        y = t.forward(X[:, :384].contiguous()).cpu().numpy()
        g = t.backward(X[:, :200].contiguous()).cpu().numpy()
        res.append((y, g))
    assert np.array_equal(res[0][0], res[1][0])
    assert np.array_equal(res[0][1], res[1][1])


def test_forward_scatter_to_row_block_owners(path):
    """The scatter form of the mapped forward on one GPU: two local buffers stand in for the
    owners of the row blocks; rows land at out_table[r // rows_per_owner], whatever row block the
    sweep starts at, and equal the plain forward (same call counter => same noise)."""
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(2)
    out_size, in_size, max_tile, m = 384, 1024, 512, 700
    W = rng.normal(0, 1 / np.sqrt(in_size), (out_size, in_size)).astype(np.float32)
    X = torch.from_numpy(rng.normal(0, 1, (m, in_size)).astype(np.float32)).cuda()
    cfg = H.inference_params(noise=True)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=8)
    rows = 512
    results = []
    for rotate in (None, 0, 512):
        a = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
        a.set_weights(torch.from_numpy(W))
        if rotate is None:
            results.append(a.forward_local(X).cpu().numpy())
            continue
        owners = [torch.full((rows, out_size), -7.0, device="cuda") for _ in range(2)]
        table = torch.tensor([o.data_ptr() for o in owners], dtype=torch.int64, device="cuda")
        a.forward_scatter(X, table, rows, rotate)
        torch.cuda.synchronize()
        got = torch.cat(owners)[:m].cpu().numpy()
        assert float(owners[1][m - rows:].max()) == -7.0  # rows past the batch are not written
        results.append(got)
    assert np.array_equal(results[0], results[1])
    assert np.array_equal(results[0], results[2])
    # the owners' sum of the slots
    slots = torch.from_numpy(rng.normal(0, 1, (3, 64, 20)).astype(np.float32)).cuda()
    out = torch.empty(64, 20, device="cuda")
    _cabi.check(_cabi.lib().ab200_sum_slots(slots.data_ptr(), 3, 64 * 20, out.data_ptr(), None))
    torch.cuda.synchronize()
    assert torch.allclose(out, slots.sum(0), atol=1e-6)


@pytest.mark.parametrize("m", [700, 130])
def test_forward_scatter_of_adc_codes(path, m):
    """The codes form of the scatter on one GPU: two local slots stand in for the owners; the
    kernel writes one signed byte per element and in-split plus the per-row factors, the owner's
    kernel multiplies and sums. Same call counter => same noise => the plain forward, up to the
    clip bound being a hair below the integer code at saturation."""
    import ctypes as C

    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    rng = np.random.default_rng(4)
    out_size, in_size, max_tile = 384, 1536, 512  # three in-splits, one out-split of 384
    W = rng.normal(0, 1 / np.sqrt(in_size), (out_size, in_size)).astype(np.float32)
    X = torch.from_numpy(rng.normal(0, 1, (m, in_size)).astype(np.float32)).cuda()
    X[5] = 0.0  # a row without input: factor 0
    cfg = H.inference_params(noise=True)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=8)
    rows, planes = 512, 3
    ref_out = None
    for rotate in (None, 0, 512):
        a = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
        a.set_weights(torch.from_numpy(W))
        if rotate is None:
            assert a.scatter_codes_supported()
            ref_out = a.forward_local(X).cpu().numpy()
            continue
        codes = [torch.zeros(planes * rows * out_size, dtype=torch.uint8, device="cuda") for _ in range(2)]
        facs = [torch.zeros(planes * rows, device="cuda") for _ in range(2)]
        ct = torch.tensor([c.data_ptr() for c in codes], dtype=torch.int64, device="cuda")
        ft = torch.tensor([f.data_ptr() for f in facs], dtype=torch.int64, device="cuda")
        a.forward_scatter_codes(X, ct, ft, rows, rotate)
        outs = []
        for o in range(2):
            valid = max(0, min(rows, m - o * rows))
            out = torch.full((rows, out_size), -7.0, device="cuda")
            n_planes = (C.c_int * 1)(planes)
            _cabi.check(_cabi.lib().ab200_sum_code_slots(
                codes[o].data_ptr(), 0, facs[o].data_ptr(), 0, 1, n_planes, rows, valid, out_size,
                out.data_ptr(), None))
            outs.append(out[:valid])
        torch.cuda.synchronize()
        got = torch.cat(outs).cpu().numpy()
        assert got.shape == ref_out.shape
        assert np.abs(got - ref_out).max() <= 1e-5 * np.abs(ref_out).max()
        assert (got[5] == 0).all() and np.abs(got).max() > 0
    # a layer with a ragged out-split is not eligible
    b = T.TileArray(cfg, 400, in_size, max_tile, max_tile, cuda_device=0)
    assert not b.scatter_codes_supported()


def test_scatter_plan_in_parts_with_blocks_dealt_in_turn_and_arrival_flags(path):
    """General scatter on one GPU, two local buffers as owners: the batch goes through in two
    launches (row_base), its 256-row blocks are dealt to the owners in turn, every launch raises
    the sender's flag at both owners when its stores are out, and the owners' sum kernels look at
    the flags first (they are up by then: the launches of one stream run one after the other).
    Whole-batch noise counters: the result equals the plain forward of the whole batch run with
    the call counter of each part."""
    from aihwkit_b200 import _cabi
    from aihwkit_b200.rpu_base import devices as D, tiles as T

    lib = _cabi.lib()
    rng = np.random.default_rng(6)
    out_size, in_size, max_tile, m = 256, 1024, 512, 1500
    W = rng.normal(0, 1 / np.sqrt(in_size), (out_size, in_size)).astype(np.float32)
    X = torch.from_numpy(rng.normal(0, 1, (m, in_size)).astype(np.float32)).cuda()
    cfg = H.inference_params(noise=True)._config(1, 1, D.IdealResistiveDeviceParameter(), seed=8)
    n_owners, blk = 2, 256
    rows_per_owner = 3 * blk  # six blocks of the batch, three per owner
    parts = [(0, 1024), (1024, m - 1024)]  # each part starts a round of the deal
    # reference: the whole batch once per part (call counters 0 and 1), rows of the part taken
    ref = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
    ref.set_weights(torch.from_numpy(W))
    want = torch.empty(m, out_size, device="cuda")
    for r0, rows in parts:
        want[r0:r0 + rows] = ref.forward_local(X)[r0:r0 + rows]
    a = T.TileArray(cfg, out_size, in_size, max_tile, max_tile, cuda_device=0)
    a.set_weights(torch.from_numpy(W))
    slots = [torch.full((rows_per_owner, out_size), -7.0, device="cuda") for _ in range(n_owners)]
    flags = torch.zeros(n_owners, 64, dtype=torch.int32, device="cuda")  # one sender, one line each
    table = torch.tensor([s.data_ptr() for s in slots], dtype=torch.int64, device="cuda")
    flag_table = torch.tensor([flags[q].data_ptr() for q in range(n_owners)], dtype=torch.int64, device="cuda")
    outs = [torch.full((rows_per_owner, out_size), -9.0, device="cuda") for _ in range(n_owners)]
    for epoch, (r0, rows) in enumerate(parts, start=1):
        plan = _cabi.ScatterPlan()
        plan.out_table_dev = table.data_ptr()
        plan.flag_table_dev = flag_table.data_ptr()
        plan.n_owners, plan.rows_per_owner, plan.rotate_rows = n_owners, rows_per_owner, 0
        plan.row_base, plan.owner_block_rows, plan.epoch = r0, blk, epoch
        a.forward_scatter_plan(X[r0:r0 + rows], plan)
        for q in range(n_owners):
            # the owner's rows of this part
            lr0 = r0 // n_owners
            n = sum(min(blk, r0 + rows - b * blk) for b in range(r0 // blk, (r0 + rows + blk - 1) // blk)
                    if b % n_owners == q)
            _cabi.check(lib.ab200_sum_slots_wait(slots[q].data_ptr(), 1, rows_per_owner * out_size, lr0, n,
                                                 out_size, outs[q].data_ptr(), flags[q].data_ptr(), 1,
                                                 epoch, 50.0, None))
    torch.cuda.synchronize()
    assert flags[:, 0].tolist() == [2, 2]
    got = torch.empty(m, out_size, device="cuda")
    for b in range((m + blk - 1) // blk):
        n = min(blk, m - b * blk)
        lrow = (b // n_owners) * blk
        got[b * blk:b * blk + n] = outs[b % n_owners][lrow:lrow + n]
    assert torch.equal(got, want)
    timed_out = C_int()
    _cabi.check(lib.ab200_wait_status(0, timed_out.ref()))
    assert timed_out.value == 0


class C_int:
    def __init__(self):
        import ctypes

        self._c = ctypes.c_int(0)

    def ref(self):
        import ctypes

        return ctypes.byref(self._c)

    @property
    def value(self):
        return self._c.value


def test_owner_sum_gives_up_when_a_sender_never_arrives():
    """A flag nobody raises: the owner's kernel waits its (short) limit, returns without summing
    and the status call reports the wait that ran out. The device stays usable."""
    from aihwkit_b200 import _cabi

    lib = _cabi.lib()
    slots = torch.ones(2, 32, 64, device="cuda")
    out = torch.full((32, 64), -3.0, device="cuda")
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    flags[0] = 5  # one sender arrived, the other never does
    n = C_int()
    _cabi.check(lib.ab200_wait_status(0, n.ref()))  # clear
    _cabi.check(lib.ab200_sum_slots_wait(slots.data_ptr(), 2, 32 * 64, 0, 32, 64, out.data_ptr(),
                                         flags.data_ptr(), 2, 5, 20.0, None))
    torch.cuda.synchronize()
    _cabi.check(lib.ab200_wait_status(0, n.ref()))
    assert n.value == 1
    assert float(out.max()) == -3.0  # nothing was summed
    # with both flags up the same call goes through
    flags[1] = 7  # a later epoch counts as arrived
    _cabi.check(lib.ab200_sum_slots_wait(slots.data_ptr(), 2, 32 * 64, 0, 32, 64, out.data_ptr(),
                                         flags.data_ptr(), 2, 5, 20.0, None))
    torch.cuda.synchronize()
    _cabi.check(lib.ab200_wait_status(0, n.ref()))
    assert n.value == 0 and torch.equal(out, torch.full((32, 64), 2.0, device="cuda"))
