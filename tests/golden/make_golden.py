"""Generate the golden vectors of tests/golden/*.npz from the COMPILED REFERENCE (oracle/_ref).

    make -C oracle && python tests/golden/make_golden.py            # everything
    make -C oracle && python tests/golden/make_golden.py indexed    # only indexed_conv.npz
    make -C oracle && python tests/golden/make_golden.py extensions # only extensions_det.npz
    make -C oracle && python tests/golden/make_golden.py compounds  # only compounds_det.npz

Every array is an input or an output of the unmodified reference CPU tile
(RPU::RPUPulsed<float>) for the configurations built by tests/helpers.py; nothing here comes from
the numpy restatement or from the CUDA code.  The noisy cases store the reference's output samples
so that distributions can be compared where the reference itself cannot run.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref  # noqa: E402
from tests import helpers as H  # noqa: E402


def deterministic_case(kind, x_size, d_size, m, out_bound, seed):
    rng = np.random.default_rng(seed)
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=out_bound)
    dp = H.device(kind, False)
    cfg = p._config(x_size, d_size, dp, seed=seed)
    t = ref.RefTile(cfg)
    w = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(w)
    w0 = t.get_weights()
    x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    d = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    x[1] = 0
    y = t.forward(x)
    g = t.backward(d)
    lr = 0.01
    t.set_learning_rate(lr)
    counts = np.stack([t.coincidences(x[s], d[s], lr, dp.dw_min) for s in range(min(m, 4))])
    hp = t.get_hidden_parameters()
    t.update(x, d)
    w1 = t.get_weights()
    return dict(w0=w0, x=x, d=d, y=y, g=g, counts=counts, hidden=hp, w1=w1,
                lr=np.float32(lr), out_bound=np.float32(out_bound))


def noisy_forward_case(seed, reps=300):
    rng = np.random.default_rng(seed)
    x_size, d_size, m = 64, 32, 4
    p = H.training_params(noise=True, pulse_det=False, bm=True)
    cfg = p._config(x_size, d_size, H.device("cs", True), seed=seed)
    t = ref.RefTile(cfg)
    t.set_seed(seed)
    w = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(w)
    w0 = t.get_weights()
    x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    ys = np.stack([t.forward(x) for _ in range(reps)])
    return dict(w0=w0, x=x, ys=ys)


def noisy_inference_case(seed, reps=300):
    rng = np.random.default_rng(seed)
    x_size, d_size, m = 128, 24, 4
    p = H.inference_params(noise=True)
    from aihwkit_b200.rpu_base import devices as D

    cfg = p._config(x_size, d_size, D.IdealResistiveDeviceParameter(), seed=seed)
    t = ref.RefTile(cfg)
    t.set_seed(seed)
    w = rng.normal(0, 1 / np.sqrt(x_size), (d_size, x_size)).astype(np.float32)
    t.set_weights(w)
    x = rng.normal(0, 1, (m, x_size)).astype(np.float32)
    ys = np.stack([t.forward(x, is_test=True) for _ in range(reps)])
    return dict(w0=w, x=x, ys=ys)


def noisy_update_case(kind, seed, reps=150):
    rng = np.random.default_rng(seed)
    x_size, d_size, m = 16, 12, 8
    p = H.training_params(noise=True, pulse_det=False)
    dp = H.device(kind, True)
    cfg = p._config(x_size, d_size, dp, seed=seed)
    t = ref.RefTile(cfg)
    t.set_seed(seed)
    w = rng.uniform(-0.3, 0.3, (d_size, x_size)).astype(np.float32)
    x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    d = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    lr = 0.05
    t.set_learning_rate(lr)
    hp = t.get_hidden_parameters()
    dws = []
    for _ in range(reps):
        t.set_weights(w)
        w0 = t.get_weights()
        t.update(x, d)
        dws.append(t.get_weights() - w0)
    return dict(w=w, w0=w0, x=x, d=d, hidden=hp, dws=np.stack(dws).astype(np.float32),
                lr=np.float32(lr))


def transfer_case(seed):
    rng = np.random.default_rng(seed)
    x_size, d_size, m = 20, 12, 6
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.transfer_device(noise=False, det=True, transfer_every=2.0, units_in_mbatch=True,
                           n_reads=2, transfer_lr=1.0)
    cfg = p._config(x_size, d_size, dp, seed=seed)
    t = ref.RefTile(cfg)
    lr = 0.1
    t.set_learning_rate(lr)
    hp0 = t.get_hidden_parameters()
    xs, ds, ws, hs = [], [], [], []
    for _ in range(6):
        x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
        d = rng.normal(0, 0.5, (m, d_size)).astype(np.float32)
        t.update(x, d)
        xs.append(x)
        ds.append(d)
        ws.append(t.get_weights())
        names = t.hidden_parameter_names()
        hs.append(t.get_hidden_parameters()[names.index("hidden_weights_0")])
    return dict(hidden0=hp0, xs=np.stack(xs), ds=np.stack(ds), ws=np.stack(ws), a=np.stack(hs),
                lr=np.float32(lr))


def indexed_conv_case(seed):
    """Indexed convolution interface in the layout the Python binding uses (trans): a padded,
    strided 3x3 convolution with an analog bias row.  The index array is built here with plain
    loops (0 = padding, 1 = bias constant, j >= 2 = element j - 2 of the image)."""
    rng = np.random.default_rng(seed)
    n, c, h, w, c_out = 4, 5, 9, 8, 12
    kh = kw = 3
    stride, pad = (2, 1), (1, 1)
    ho = (h + 2 * pad[0] - kh) // stride[0] + 1
    wo = (w + 2 * pad[1] - kw) // stride[1] + 1
    x_size = c * kh * kw + 1
    idx = np.zeros((x_size, ho * wo), np.int32)
    for ci in range(c):
        for ki in range(kh):
            for kj in range(kw):
                for oy in range(ho):
                    for ox in range(wo):
                        y, xx = oy * stride[0] - pad[0] + ki, ox * stride[1] - pad[1] + kj
                        if 0 <= y < h and 0 <= xx < w:
                            idx[(ci * kh + ki) * kw + kj, oy * wo + ox] = 2 + (ci * h + y) * w + xx
    idx[-1] = 1
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
    dp = H.device("sb", False)
    cfg = p._config(x_size, c_out, dp, seed=seed)
    t = ref.RefTile(cfg)
    t.set_weights(rng.uniform(-0.5, 0.5, (c_out, x_size)).astype(np.float32))
    t.set_matrix_indices(idx)
    w0 = t.get_weights()
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
    d = rng.normal(0, 0.1, (n, c_out, ho, wo)).astype(np.float32)
    y = t.forward_indexed(x, d.shape)
    g = t.backward_indexed(d, x.shape)
    lr = 0.01
    t.set_learning_rate(lr)
    hp = t.get_hidden_parameters()
    t.update_indexed(x, d)
    return dict(w0=w0, indices=idx.reshape(-1), x=x, d=d, y=y, g=g, hidden=hp, w1=t.get_weights(),
                lr=np.float32(lr), out_bound=np.float32(2.0))


LINE_ALL = dict(ir_drop=1.0, ir_drop_g_ratio=3000.0, v_offset_std=0.05, r_series=0.02,
                out_nonlinearity=0.1, out_nonlinearity_std=0.2)


def extensions_case(seed):
    """Deterministic cases of the rows beyond the first tile: PiecewiseStep device, the
    non-idealities of the output lines (with the per-line values the reference drew), power-law
    drift, weight modifiers (read through a perfect-IO forward of the identity), the running-average
    noise management and the NoneWithDevice update."""
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(seed)
    out = {}
    # PiecewiseStep
    x_size, d_size, m = 40, 24, 9
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.piecewise_device(False)
    t = ref.RefTile(p._config(x_size, d_size, dp, seed=seed))
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    d = rng.normal(0, 0.1, (m, d_size)).astype(np.float32)
    out.update(pw_w0=t.get_weights(), pw_x=x, pw_d=d, pw_hidden=t.get_hidden_parameters())
    t.set_learning_rate(0.01)
    t.update(x, d)
    out["pw_w1"] = t.get_weights()
    # non-idealities of the output lines
    x_size, d_size, m = 60, 36, 12
    p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
    for io in (p.forward_io, p.backward_io):
        for k, v in LINE_ALL.items():
            setattr(io, k, v)
    t = ref.RefTile(p._config(x_size, d_size, H.device("cs", False), seed=seed))
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    d = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
    out.update(line_w0=t.get_weights(), line_x=x, line_d=d, line_y=t.forward(x), line_g=t.backward(d),
               line_voff_f=t.get_io_vector(False, 0, d_size), line_nl_f=t.get_io_vector(False, 1, d_size),
               line_voff_b=t.get_io_vector(True, 0, x_size), line_nl_b=t.get_io_vector(True, 1, x_size))
    # drift
    x_size, d_size = 30, 20
    p = H.training_params(noise=False, pulse_det=True)
    dp = H.device("cs", False)
    dp.drift.nu, dp.drift.nu_dtod, dp.drift.nu_k, dp.drift.g_offset, dp.drift.wg_ratio = 0.1, 0.3, 0.05, 0.2, 0.6
    t = ref.RefTile(p._config(x_size, d_size, dp, seed=seed))
    w = rng.uniform(0.05, 0.5, (d_size, x_size)).astype(np.float32)
    t.set_weights(w)
    out.update(drift_w0=t.get_weights(), drift_hidden=t.get_hidden_parameters())
    t.drift_weights(5.0)
    out["drift_w1"] = t.get_weights()
    w2 = t.get_weights().copy()
    w2[:5, :7] = 0.25
    t.set_weights(w2)
    out["drift_w2"] = t.get_weights()
    t.drift_weights(40.0)
    out["drift_w3"] = t.get_weights()
    # weight modifiers on a perfect-IO tile
    x_size, d_size = 24, 16
    pp = D.AnalogTileParameter()
    pp.forward_io.is_perfect = True
    pp.backward_io.is_perfect = True
    pp.update.pulse_type = D.PulseType.None_
    t = ref.RefTile(pp._config(x_size, d_size, D.IdealResistiveDeviceParameter(), seed=seed))
    w = rng.normal(0, 0.3, (d_size, x_size)).astype(np.float32)
    t.set_weights(w)
    eye = np.eye(x_size, dtype=np.float32)
    out["mod_w0"] = w
    for name, kw in (("disc", dict(type=T.WeightModifierType.Discretize, res=0.1)),
                     ("dorefa", dict(type=T.WeightModifierType.DoReFa, res=0.08, dorefa_clip=0.6))):
        wm = T.WeightModifierParameter()
        for k, v in kw.items():
            setattr(wm, k, v)
        t.modify_weights(wm)
        out["mod_" + name] = t.forward(eye).T.copy()
    # running-average noise management, two calls
    x_size, d_size, m = 32, 20, 15
    p = H.training_params(noise=False, pulse_det=True, bm=False)
    p.forward_io.noise_management = D.NoiseManagementType.AverageAbsMax
    p.forward_io.nm_decay = 0.1
    t = ref.RefTile(p._config(x_size, d_size, H.device("cs", False), seed=seed))
    t.set_weights(rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32))
    xs = np.stack([(rng.uniform(-1, 1, (m, x_size)) * s).astype(np.float32) for s in (1.0, 0.4)])
    out.update(nm_w0=t.get_weights(), nm_xs=xs, nm_ys=np.stack([t.forward(xs[0]), t.forward(xs[1])]))
    # NoneWithDevice
    x_size, d_size, m = 30, 20, 16
    p = H.training_params(noise=False, pulse_det=True)
    p.update.pulse_type = D.PulseType.NoneWithDevice
    t = ref.RefTile(p._config(x_size, d_size, H.device("cs", False, w_max=0.3, w_min=-0.3), seed=seed))
    t.set_weights(rng.uniform(-0.2, 0.2, (d_size, x_size)).astype(np.float32))
    x = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    d = (rng.normal(0, 0.5, (m, d_size))).astype(np.float32)
    out.update(nwd_w0=t.get_weights(), nwd_x=x, nwd_d=d, nwd_hidden=t.get_hidden_parameters())
    t.set_learning_rate(0.2)
    t.update(x, d)
    out["nwd_w1"] = t.get_weights()
    return out


COMPOUND_CASES = {
    # name -> (helper in tests/helpers.py, keyword arguments)
    "chopped": ("chopped_transfer_device", dict(transfer_lr=4.0, in_chop_prob=0.3, in_chop_random=False,
                                                momentum=0.3, forget_buffer=False, buffer_granularity=0.5)),
    "dynamic": ("dynamic_transfer_device", dict(transfer_lr=4.0, in_chop_prob=0.5, tail_weightening=2.5,
                                                momentum=0.2, forget_buffer=False, buffer_cap=0.5)),
    "mixed": ("mixed_precision_device", dict(n_rows_per_transfer=3)),
}


def compounds_case(seed):
    """The two-pass MV types (forward and backward outputs, alone and on top of the line
    non-idealities) and the weight / hidden-plane trajectories of the chopped and dynamic transfer
    compounds and of the mixed-precision compound over eight deterministic updates."""
    from aihwkit_b200.rpu_base import devices as D

    rng = np.random.default_rng(seed)
    out = {}
    x_size, d_size, m = 60, 36, 12
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    X = rng.uniform(-1, 1, (m, x_size)).astype(np.float32)
    Dm = rng.normal(0, 0.3, (m, d_size)).astype(np.float32)
    out.update(pn_w0=W, pn_x=X, pn_d=Dm)
    for mv in ("PosNegSeparate", "PosNegSeparateDigitalSum"):
        for lines in (False, True):
            p = H.training_params(noise=False, pulse_det=True, bm=True, out_bound=2.0)
            for io in (p.forward_io, p.backward_io):
                io.mv_type = getattr(D.AnalogMVType, mv)
                if lines:
                    for k, v in LINE_ALL.items():
                        setattr(io, k, v)
            t = ref.RefTile(p._config(x_size, d_size, H.device("cs", False), seed=seed))
            t.set_weights(W)
            key = f"pn_{mv}_{int(lines)}"
            out[key + "_w"] = t.get_weights()
            if lines:
                for backward, n, tag in ((False, d_size, "f"), (True, x_size, "b")):
                    out[f"{key}_voff_{tag}"] = t.get_io_vector(backward, 0, n)
                    out[f"{key}_nl_{tag}"] = t.get_io_vector(backward, 1, n)
            out[key + "_y"] = t.forward(X)
            out[key + "_g"] = t.backward(Dm)
    x_size, d_size, m = 12, 10, 5
    xs = rng.uniform(-1, 1, (8, m, x_size)).astype(np.float32)
    ds = rng.normal(0, 0.5, (8, m, d_size)).astype(np.float32)
    out.update(cp_x=xs, cp_d=ds)
    for name, (helper, kw) in COMPOUND_CASES.items():
        p = H.training_params(noise=False, pulse_det=True)
        t = ref.RefTile(p._config(x_size, d_size, getattr(H, helper)(**kw), seed=3))
        t.set_learning_rate(0.1)
        out[f"cp_{name}_hidden0"] = t.get_hidden_parameters()
        ws, hs = [], []
        for k in range(8):
            t.update(xs[k], ds[k])
            ws.append(t.get_weights())
            hs.append(t.get_hidden_parameters())
        out[f"cp_{name}_w"] = np.stack(ws)
        out[f"cp_{name}_hidden"] = np.stack(hs)
    return out


def main():
    if sys.argv[1:] == ["compounds"]:
        np.savez_compressed(os.path.join(HERE, "compounds_det.npz"), **compounds_case(14))
        print("wrote compounds_det.npz")
        return
    if sys.argv[1:] == ["extensions"]:
        np.savez_compressed(os.path.join(HERE, "extensions_det.npz"), **extensions_case(12))
        print("wrote extensions_det.npz")
        return
    if sys.argv[1:] == ["indexed"]:
        np.savez_compressed(os.path.join(HERE, "indexed_conv.npz"), **indexed_conv_case(9))
        print("wrote indexed_conv.npz")
        return
    out = {}
    for kind in ("cs", "ls", "sb", "sbr"):
        for (x, d, m, ob) in ((40, 24, 9, 12.0), (70, 33, 6, 2.0)):
            out[f"det_{kind}_{x}x{d}_ob{int(ob)}"] = deterministic_case(kind, x, d, m, ob, 100 + x)
    for name, case in out.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **case)
    np.savez_compressed(os.path.join(HERE, "noisy_forward.npz"), **noisy_forward_case(5))
    np.savez_compressed(os.path.join(HERE, "noisy_inference.npz"), **noisy_inference_case(6))
    for kind in ("cs", "sbr"):
        np.savez_compressed(os.path.join(HERE, f"noisy_update_{kind}.npz"), **noisy_update_case(kind, 7))
    np.savez_compressed(os.path.join(HERE, "transfer_det.npz"), **transfer_case(8))
    np.savez_compressed(os.path.join(HERE, "indexed_conv.npz"), **indexed_conv_case(9))
    np.savez_compressed(os.path.join(HERE, "extensions_det.npz"), **extensions_case(12))
    np.savez_compressed(os.path.join(HERE, "compounds_det.npz"), **compounds_case(14))
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
