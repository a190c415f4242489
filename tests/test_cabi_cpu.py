"""CPU checks of the boundary: the library loads and exports every symbol the header declares,
the host-side tile logic (configuration, parameter draw, weights, hidden parameters, errors)
behaves like the reference's.  No compute call is made: there is no CPU compute path."""

import ctypes as C
import os

import numpy as np
import pytest
import torch

from aihwkit_b200 import _cabi
from aihwkit_b200.rpu_base import devices as D, tiles as T, cuda as rpu_cuda
from tests import helpers as H

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_library_exports_every_declared_symbol():
    lib = _cabi.lib()
    names = _cabi.declared_symbols()
    assert len(names) >= 40
    for name in names:
        assert hasattr(lib, name), name
    assert rpu_cuda.is_compiled()
    assert b"sm_100a" in lib.ab200_version()


def test_struct_sizes_match_header():
    # the ctypes mirrors have the layout the library was compiled with
    lib = _cabi.lib()
    for which, cls in enumerate((_cabi.IOParams, _cabi.UpdateParams, _cabi.DeviceParams,
                                 _cabi.TransferParams, _cabi.TileConfig, _cabi.ScatterPlan,
                                 _cabi.MixedPrecParams)):
        assert C.sizeof(cls) == lib.ab200_sizeof(which), cls.__name__
    assert C.sizeof(_cabi.IOParams) == 32 * 4
    assert C.sizeof(_cabi.TileConfig) % 8 == 0


def test_defaults_follow_reference_member_initialisers():
    lib = _cabi.lib()
    io = _cabi.IOParams()
    lib.ab200_default_io_params(C.byref(io))
    ref = D.AnalogTileInputOutputParameter()._to_c()
    for name, _ in _cabi.IOParams._fields_:
        assert getattr(io, name) == pytest.approx(getattr(ref, name)), name
    up = _cabi.UpdateParams()
    lib.ab200_default_update_params(C.byref(up))
    refu = D.AnalogTileUpdateParameter()._to_c()
    for name, _ in _cabi.UpdateParams._fields_:
        assert getattr(up, name) == pytest.approx(getattr(refu, name)), name
    for kind, cls in ((D.DEVICE_CONSTANT_STEP, D.ConstantStepResistiveDeviceParameter),
                      (D.DEVICE_SOFT_BOUNDS, D.SoftBoundsResistiveDeviceParameter),
                      (D.DEVICE_LINEAR_STEP, D.LinearStepResistiveDeviceParameter),
                      (D.DEVICE_EXP_STEP, D.ExpStepResistiveDeviceParameter),
                      (D.DEVICE_POW_STEP, D.PowStepResistiveDeviceParameter),
                      (D.DEVICE_PIECEWISE_STEP, D.PiecewiseStepResistiveDeviceParameter)):
        dp = _cabi.DeviceParams()
        lib.ab200_default_device_params(C.byref(dp), kind)
        refd = cls()._to_c()
        for name, _ in _cabi.DeviceParams._fields_:
            if kind in (D.DEVICE_CONSTANT_STEP, D.DEVICE_EXP_STEP, D.DEVICE_POW_STEP,
                        D.DEVICE_PIECEWISE_STEP) and name.startswith("ls_"):
                continue  # LinearStep-only fields are not read for other kinds
            if kind != D.DEVICE_EXP_STEP and name.startswith("es_"):
                continue  # ExpStep-only fields
            if kind != D.DEVICE_POW_STEP and name.startswith("ps_"):
                continue  # PowStep-only fields
            if name.startswith("pw_"):
                if kind == D.DEVICE_PIECEWISE_STEP:
                    assert dp.pw_n == refd.pw_n == 1 and dp.pw_up[0] == refd.pw_up[0] == 1.0
                    assert dp.pw_down[0] == refd.pw_down[0] == 1.0
                continue
            if name == "drift":
                for f, _ in _cabi.DriftParams._fields_:
                    assert getattr(dp.drift, f) == pytest.approx(getattr(refd.drift, f)), (kind, f)
                continue
            assert getattr(dp, name) == pytest.approx(getattr(refd, name)), (kind, name)
    # compounds: the library's defaults equal what the Python mirrors send for a fresh object
    tp = _cabi.TransferParams()
    lib.ab200_default_transfer_params(C.byref(tp))
    dyn = D.DynamicTransferResistiveDeviceParameter()
    for _ in range(2):
        dyn.append_parameter(D.ConstantStepResistiveDeviceParameter())
    ref_t = dyn._to_c()
    for name in ("tail_weightening", "buffer_cap", "buffer_granularity", "thres_scale", "step", "forget_buffer"):
        assert getattr(tp, name) == pytest.approx(getattr(ref_t, name)), name
    assert tp.dynamic == 0 and tp.chopped == 0 and ref_t.dynamic == 1 and ref_t.chopped == 1
    mp = _cabi.MixedPrecParams()
    lib.ab200_default_mixedprec_params(C.byref(mp))
    mixed = D.MixedPrecResistiveDeviceParameter()
    assert mixed.set_device_parameter(D.ConstantStepResistiveDeviceParameter())
    assert not mixed.set_device_parameter(D.IdealResistiveDeviceParameter())
    ref_m = mixed._to_c_mixed()
    for name, _ in _cabi.MixedPrecParams._fields_:
        if name != "enabled":
            assert getattr(mp, name) == pytest.approx(getattr(ref_m, name)), name
    assert mp.enabled == 0 and ref_m.enabled == 1


@pytest.mark.parametrize("kind", ["cs", "ls", "sb", "sbr"])
def test_host_parameter_draw_equals_reference_golden(kind):
    """For a given construction_seed the host-side draw reproduces the reference's per-element
    parameters bit for bit (golden `hidden` arrays come from the compiled reference)."""
    g = np.load(os.path.join(GOLD, f"det_{kind}_40x24_ob12.npz"))
    p = H.training_params(noise=False, pulse_det=True)
    t = T.AnalogTile(p._config(40, 24, H.device(kind, False), seed=1))
    assert np.array_equal(t.get_hidden_parameters().numpy(), g["hidden"])
    t.set_weights(torch.from_numpy(np.full((24, 40), 10.0, np.float32)))
    assert np.array_equal(t.get_weights().numpy(), g["hidden"][0])  # clipped to max_bound


def test_transfer_hidden_parameters_equal_reference_golden():
    g = np.load(os.path.join(GOLD, "transfer_det.npz"))
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.transfer_device(noise=False, det=True, transfer_every=2.0, units_in_mbatch=True,
                           n_reads=2, transfer_lr=1.0)
    t = T.AnalogTile(p._config(20, 12, dp, seed=1))
    names = t.get_hidden_parameter_names()
    assert len(names) == 20 and names[9] == "hidden_weights_0" and names[-1] == "hidden_weights_1"
    assert np.array_equal(t.get_hidden_parameters().numpy(), g["hidden0"])


def test_hidden_parameter_round_trip_and_weight_reclip():
    p = H.training_params(noise=False, pulse_det=True)
    t = T.AnalogTile(p._config(12, 8, H.device("sb", False), seed=1))
    hp = t.get_hidden_parameters()
    assert tuple(hp.shape) == (10, 8, 12)
    t.set_weights(torch.full((8, 12), 0.2))
    hp2 = hp.clone()
    hp2[0] = 0.05  # max_bound
    t.set_hidden_parameters(hp2)
    assert torch.equal(t.get_hidden_parameters(), hp2)
    assert float(t.get_weights().max()) <= 0.05 + 1e-7
    with pytest.raises(RuntimeError):
        t.set_hidden_parameters(hp[:3])


def test_compute_without_device_fails_loudly():
    p = H.training_params(noise=False, pulse_det=True)
    t = T.AnalogTile(p._config(8, 4, H.device("cs", False), seed=1))
    for call in (lambda: t.forward(torch.zeros(2, 8)), lambda: t.backward(torch.zeros(2, 4)),
                 lambda: t.update(torch.zeros(2, 8), torch.zeros(2, 4))):
        with pytest.raises(RuntimeError, match="no CPU compute path"):
            call()
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU fallback|not available"):
            t.cuda(0)


def test_unsupported_settings_raise():
    p = D.AnalogTileParameter()
    p.forward_io.v_offset_w_min = -1.0  # only read with voltage offsets on
    p._config(4, 4, D.ConstantStepResistiveDeviceParameter())
    p.forward_io.v_offset_std = 0.1
    with pytest.raises(RuntimeError, match="v_offset_w_min"):
        p._config(4, 4, D.ConstantStepResistiveDeviceParameter())
    p = D.AnalogTileParameter()
    p.update.pulse_type = D.PulseType.Stochastic  # separate +- trains: same law as the compressed type
    T.AnalogTile(p._config(4, 4, D.ConstantStepResistiveDeviceParameter()))
    p = D.AnalogTileParameter()
    p.forward_io.inp_bound = 2.0  # noise management expects bound == 1
    with pytest.raises(RuntimeError, match="expects bound==1"):
        T.AnalogTile(p._config(4, 4, D.ConstantStepResistiveDeviceParameter()))
    dp = D.ConstantStepResistiveDeviceParameter()
    dp.w_min = 0.1
    with pytest.raises(RuntimeError, match="needs to contain 0"):
        T.AnalogTile(D.AnalogTileParameter()._config(4, 4, dp))
    with pytest.raises(RuntimeError):
        T.AnalogTile(D.AnalogTileParameter()._config(0, 4, D.ConstantStepResistiveDeviceParameter()))
    # compounds: what the library refuses, it refuses when the tile is made (no device needed)
    mixed = D.MixedPrecResistiveDeviceParameter()
    with pytest.raises(RuntimeError, match="not implemented"):
        D.AnalogTileParameter()._config(4, 4, mixed)  # no analog device set
    assert mixed.set_device_parameter(D.ConstantStepResistiveDeviceParameter())
    mixed.n_x_bins = 5
    with pytest.raises(RuntimeError, match="only one of x and d"):
        D.AnalogTileParameter()._config(4, 4, mixed)
    dyn = H.dynamic_transfer_device(in_chop_prob=0.0)
    with pytest.raises(RuntimeError, match="needs to be positive"):
        D.AnalogTileParameter()._config(4, 4, dyn)
    chop = H.chopped_transfer_device()
    chop.n_reads_per_transfer = 2
    with pytest.raises(RuntimeError, match="n_reads_per_transfer==1"):
        D.AnalogTileParameter()._config(4, 4, chop)
    cfg = D.AnalogTileParameter()._config(4, 4, H.chopped_transfer_device())
    cfg.transfer.dynamic, cfg.transfer.chopped = 1, 0  # a raw struct that skips the Python checks
    with pytest.raises(RuntimeError, match="chopped = 1"):
        T.AnalogTile(cfg)
    cfg = D.AnalogTileParameter()._config(4, 4, D.ConstantStepResistiveDeviceParameter())
    cfg.forward_io.mv_type = 7
    with pytest.raises(RuntimeError, match="AnalogMVType not implemented"):
        T.AnalogTile(cfg)


def test_learning_rate_and_sizes():
    t = T.AnalogTile(D.AnalogTileParameter()._config(7, 5, D.ConstantStepResistiveDeviceParameter()))
    assert (t.get_x_size(), t.get_d_size()) == (7, 5)
    assert t.get_learning_rate() == pytest.approx(0.1)  # createRPUArray default
    t.set_learning_rate(0.02)
    assert t.get_learning_rate() == pytest.approx(0.02)
    with pytest.raises(RuntimeError, match="Invalid weights dimensions"):
        t.set_weights(torch.zeros(7, 5))


def test_split_sizes_follow_reference_rule():
    from aihwkit_b200.sharded import split_sizes, in_split_range, column_range

    assert split_sizes(4096, 512) == [512] * 8
    assert split_sizes(768, 512) == [384, 384]
    assert split_sizes(2304, 512) == [461, 461, 461, 461, 460]
    assert split_sizes(100, 0) == [100]
    for world in (1, 2, 3, 4, 8, 16):
        ranges = [in_split_range(8, r, world) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == 8
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    assert column_range(2304, 512, 1, 2) == (461 * 3, 2304)


def test_extra_state_round_trip_and_copy():
    """dump_extra / load_extra / copy on a host-side tile (no compute involved)."""
    import copy

    p = H.training_params(noise=False, pulse_det=True)
    t = T.AnalogTile(p._config(6, 4, H.device("sb", False), seed=9))
    t.set_learning_rate(0.03)
    t.set_weights(torch.full((4, 6), 0.1))
    extra = t.dump_extra()
    assert extra["learning_rate"][0] == pytest.approx(0.03)
    assert set(extra) >= {"rpu_device.current_update_idx", "noise.key0", "noise.forward_calls"}
    t2 = copy.deepcopy(t)
    assert t2.dump_extra() == extra
    assert torch.equal(t2.get_weights(), t.get_weights())
    assert torch.equal(t2.get_hidden_parameters(), t.get_hidden_parameters())
    extra["learning_rate"] = [0.5]
    t2.load_extra(extra, strict=True)
    assert t2.get_learning_rate() == pytest.approx(0.5)
    with pytest.raises(RuntimeError, match="unexpected key"):
        t2.load_extra({"bogus": [1.0]}, strict=True)
    t2.load_extra({"bogus": [1.0], "learning_rate": [0.25]})  # not strict: ignored
    assert t2.get_learning_rate() == pytest.approx(0.25)
    with pytest.raises(RuntimeError, match="is missing"):
        t2.load_extra({"learning_rate": [0.25]}, strict=True)


def test_public_header_is_plain_c(tmp_path):
    """The drop-in boundary is a C ABI: include/aihwkit_b200.h compiles as C99 with warnings on
    (plain pointers and sizes, no C++ or torch types), and a C program links every struct."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "hdr.c"
    src.write_text('#include "aihwkit_b200.h"\n'
                   "int main(void) {\n"
                   "  ab200_tile_config c; ab200_mixedprec_params m; ab200_scatter_plan p;\n"
                   "  ab200_weight_modifier_params w; ab200_drift_params d;\n"
                   "  (void)c; (void)m; (void)p; (void)w; (void)d;\n"
                   "  return sizeof(ab200_io_params) == 0;\n"
                   "}\n")
    res = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I",
                          os.path.join(root, "include"), "-c", str(src), "-o", str(tmp_path / "hdr.o")],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def test_c_program_links_and_drives_the_library(tmp_path):
    """A C program (no Python, no C++ runtime of its own) links libaihwkit_b200.so, fills a
    configuration from the library's defaults, makes a host-side tile, sets and reads weights and
    gets the library's refusal for a compute call without a device."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    libdir = os.path.join(root, "aihwkit_b200", "csrc")
    _cabi.lib()  # makes sure the library is built
    src = tmp_path / "main.c"
    src.write_text(r'''
#include <stdio.h>
#include <string.h>
#include "aihwkit_b200.h"
int main(void) {
  ab200_tile_config cfg;
  memset(&cfg, 0, sizeof(cfg));
  if (ab200_sizeof(4) != sizeof(cfg)) return 2;
  cfg.x_size = 6; cfg.d_size = 4; cfg.seed = 7;
  ab200_default_io_params(&cfg.forward_io);
  ab200_default_io_params(&cfg.backward_io);
  ab200_default_update_params(&cfg.update);
  cfg.device_kind = AB200_DEVICE_CONSTANT_STEP;
  ab200_default_device_params(&cfg.device[0], AB200_DEVICE_CONSTANT_STEP);
  ab200_default_transfer_params(&cfg.transfer);
  ab200_default_mixedprec_params(&cfg.mixed);
  ab200_tile *t = 0;
  if (ab200_tile_create(&cfg, -1, &t)) { printf("create: %s\n", ab200_last_error()); return 3; }
  float w[24], r[24], x[6] = {0}, y[4];
  for (int k = 0; k < 24; k++) w[k] = 0.01f * (float)(k - 12);
  if (ab200_tile_set_weights(t, w) || ab200_tile_get_weights(t, r)) return 4;
  for (int k = 0; k < 24; k++) if (r[k] != w[k]) return 5;
  if (ab200_tile_get_x_size(t) != 6 || ab200_tile_hidden_parameter_count(t) <= 0) return 6;
  int rc = ab200_tile_forward(t, x, y, 0, 1, 0, 0, 0, 0);   /* no device: must refuse, not compute */
  printf("%s|%d|%s\n", ab200_version(), rc, ab200_last_error());
  ab200_tile_destroy(t);
  return rc != 0 ? 0 : 7;
}
''')
    exe = tmp_path / "main"
    res = subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(root, "include"), str(src),
                          "-o", str(exe), f"-L{libdir}", "-laihwkit_b200", f"-Wl,-rpath,{libdir}"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, (run.returncode, run.stdout, run.stderr)
    version, rc, msg = run.stdout.strip().split("|", 2)
    assert version.startswith("aihwkit_b200") and int(rc) != 0 and "no CPU compute path" in msg


def test_product_code_never_touches_the_checker():
    """The oracle is test infrastructure: nothing under aihwkit_b200/ (Python or CUDA sources)
    names the oracle package or the working folder, and bench.py reaches it only in its
    CPU-baseline / reference-arm functions."""
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pat = re.compile(r"\b(from|import)\s+oracle\b|oracle/|_work/|\b_work\b")
    for base, _, files in os.walk(os.path.join(root, "aihwkit_b200")):
        if "build" in os.path.basename(base):
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(base, f), encoding="utf-8").read()
                assert not pat.search(text), os.path.join(base, f)
    bench = open(os.path.join(root, "bench.py"), encoding="utf-8").read()
    lines = bench.split("\n")
    users = set()
    for n, line in enumerate(lines):
        if re.search(r"\b(from|import)\s+oracle\b", line):
            k = n
            while k >= 0 and not lines[k].lstrip().startswith("def "):
                k -= 1
            users.add(lines[k].strip().split("(")[0].replace("def ", ""))
    assert users and all(("cpu" in u or "ref" in u) for u in users), users
