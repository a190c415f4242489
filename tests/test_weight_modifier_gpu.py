"""modify_weights on the GPU (RPUSimple::modifyFBWeights, src/rpucuda/rpu.cpp:1749-1758;
WeightModifier::apply, weight_modifier.cpp:31-215): forward and backward read a modified copy of
the weights, updates go to the weights themselves.

The modified copy is observed through a forward pass with perfect IO on the identity matrix. The
deterministic modifiers are compared element by element with the compiled reference tile, the
random ones by moments against the closed form and against the reference."""

import numpy as np
import pytest
import torch

from oracle import ref
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _tiles(x_size, d_size, W):
    from aihwkit_b200.rpu_base import devices as D
    from aihwkit_b200.rpu_base import tiles as T

    p = D.AnalogTileParameter()
    p.forward_io.is_perfect = True
    p.backward_io.is_perfect = True
    p.update.pulse_type = D.PulseType.None_
    ideal = D.IdealResistiveDeviceParameter()
    cfg = p._config(x_size, d_size, ideal, seed=4)
    t = T.AnalogTile(cfg, cuda_device=0)
    t.set_weights(torch.from_numpy(W))
    rt = None
    if ref.available():
        rt = ref.RefTile(cfg)
        rt.set_weights(W)
    return t, rt


def _fb(t, x_size, is_test=False):
    eye = torch.eye(x_size, device="cuda")
    return t.forward(eye, is_test=is_test).cpu().numpy().T  # [d, x]


def _fb_ref(rt, x_size, is_test=False):
    return rt.forward(np.eye(x_size, dtype=np.float32), is_test=is_test).T


def _par(**kw):
    from aihwkit_b200.rpu_base import tiles as T

    wm = T.WeightModifierParameter()
    for k, v in kw.items():
        setattr(wm, k, v)
    return wm


@pytest.mark.parametrize("copy_last", [False, True])
def test_discretize_and_dorefa_against_reference(copy_last):
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(3)
    x_size, d_size = 48, 20
    W = rng.normal(0, 0.3, (d_size, x_size)).astype(np.float32)
    W[:, -1] = 5.0  # a bias column far above the rest: must not set the scale when it is copied
    t, rt = _tiles(x_size, d_size, W)
    for wm in (_par(type=T.WeightModifierType.Discretize, res=0.1, copy_last_column=copy_last),
               _par(type=T.WeightModifierType.Discretize, res=0.05, rel_to_actual_wmax=False,
                    assumed_wmax=0.8, copy_last_column=copy_last),
               _par(type=T.WeightModifierType.DoReFa, res=0.08, dorefa_clip=0.6,
                    copy_last_column=copy_last)):
        t.modify_weights(wm)
        fb = _fb(t, x_size)
        amax = np.abs(W[:, :-1] if copy_last else W).max() if wm.rel_to_actual_wmax else wm.assumed_wmax
        if int(wm.type) == int(T.WeightModifierType.Discretize):
            want = np.float32(amax) * np.round(W / np.float32(amax) / np.float32(wm.res)) * np.float32(wm.res)
        else:
            scale = abs(wm.dorefa_clip / np.tanh(np.float32(amax)))
            want = np.round(np.tanh(W) * np.float32(scale) / np.float32(wm.res)) * np.float32(wm.res)
        if copy_last:
            want[:, -1] = W[:, -1]
        off = np.abs(fb - want) > 1e-6
        assert off.mean() <= 0.005, off.mean()  # a value on a rounding tie may fall either way
        assert np.abs(fb - want).max() <= 1.001 * wm.res * max(float(amax), 1.0)
        # the weights themselves are untouched, and a test-mode forward reads them
        assert np.array_equal(t.get_weights().numpy(), W)
        assert np.abs(_fb(t, x_size, is_test=True) - W).max() <= 1e-6
        if rt is not None:
            rt.modify_weights(wm)
            fr = _fb_ref(rt, x_size)
            assert (np.abs(fb - fr) > 1e-6).mean() <= 0.005
    # enable_during_test: the test-mode forward reads the copy as well
    wm = _par(type=T.WeightModifierType.Discretize, res=0.1, enable_during_test=True)
    t.modify_weights(wm)
    assert np.array_equal(_fb(t, x_size, is_test=True), _fb(t, x_size))
    assert np.abs(_fb(t, x_size, is_test=True) - W).max() > 0.01


def test_backward_reads_the_copy_and_update_writes_the_weights():
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(5)
    x_size, d_size = 32, 24
    W = rng.normal(0, 0.3, (d_size, x_size)).astype(np.float32)
    t, _ = _tiles(x_size, d_size, W)
    t.modify_weights(_par(type=T.WeightModifierType.Discretize, res=0.2))
    fb = _fb(t, x_size)
    g = t.backward(torch.eye(d_size, device="cuda")).cpu().numpy()  # [d, x]
    assert np.abs(g - fb).max() <= 1e-6
    t.set_learning_rate(0.1)
    x = torch.from_numpy(rng.normal(0, 1, (4, x_size)).astype(np.float32)).cuda()
    d = torch.from_numpy(rng.normal(0, 1, (4, d_size)).astype(np.float32)).cuda()
    t.update(x, d)
    W1 = t.get_weights().numpy()
    assert np.abs(W1 - (W - 0.1 * d.cpu().numpy().T @ x.cpu().numpy())).max() <= 1e-5
    assert np.array_equal(_fb(t, x_size), fb)  # the copy stays until the next modify_weights
    t.modify_weights(_par(type=T.WeightModifierType.Copy))
    assert np.abs(_fb(t, x_size) - W1).max() <= 1e-6


@pytest.mark.parametrize("kind", ["AddNormal", "MultNormal", "Poly", "ProgNoise", "DiscretizeAddNormal",
                                  "DropConnect"])
def test_random_modifiers_moments(kind):
    from aihwkit_b200.rpu_base import tiles as T

    rng = np.random.default_rng(7)
    x_size, d_size = 128, 96
    W = rng.uniform(-0.5, 0.5, (d_size, x_size)).astype(np.float32)
    t, rt = _tiles(x_size, d_size, W)
    amax = float(np.abs(W).max())
    wm = _par(type=getattr(T.WeightModifierType, kind), std_dev=0.1, res=0.1, pdrop=0.0)
    if kind == "DropConnect":
        wm.pdrop = 0.3
    if kind in ("Poly", "ProgNoise"):
        wm.coeffs = [0.2, 0.5, -0.3]
        wm.g_max = 25.0
    reps = 40
    fbs = np.stack([(t.modify_weights(wm), _fb(t, x_size))[1] for _ in range(reps)])
    assert np.abs(fbs[0] - fbs[1]).max() > 0  # a fresh draw per call
    dev = fbs - W
    aw = np.abs(W) / amax
    if kind == "AddNormal":
        sig = np.full_like(W, 0.1 * amax)
    elif kind == "MultNormal":
        sig = np.abs(W) * 0.1 * amax
    elif kind == "Poly":
        sig = amax * 0.1 * (0.2 + 0.5 * aw - 0.3 * aw ** 2)
    elif kind == "ProgNoise":
        sig = amax * 0.1 / 25.0 * (0.2 + 0.5 * aw - 0.3 * aw ** 2)
    elif kind == "DiscretizeAddNormal":
        q = np.float32(amax) * np.round(W / np.float32(amax) / np.float32(0.1)) * np.float32(0.1)
        dev = fbs - q
        sig = np.full_like(W, 0.1 * amax)
    if kind == "DropConnect":
        dropped = fbs == 0
        assert abs(dropped.mean() - 0.3) < 0.005
        assert np.array_equal(np.where(dropped, 0, fbs), np.where(dropped, 0, np.broadcast_to(W, fbs.shape)))
    else:
        ratio = dev.std(axis=0)[sig > 1e-4] / sig[sig > 1e-4]
        assert abs(ratio.mean() * np.sqrt(reps / (reps - 1.0)) - 1.0) < 0.02, ratio.mean()
        assert abs(dev.mean()) < 5 * sig.mean() / np.sqrt(dev.size)
        if kind == "ProgNoise":
            assert np.all(np.sign(fbs) * np.sign(W) >= 0)  # the sign of a weight is kept
    if rt is not None:
        fr = np.stack([(rt.modify_weights(wm), _fb_ref(rt, x_size))[1] for _ in range(reps)])
        a, b = (fbs - W).ravel(), (fr - W).ravel()
        assert abs(a.std() / b.std() - 1.0) < 0.03
        assert abs(a.mean() - b.mean()) < 6 * b.std() / np.sqrt(b.size)


def test_modifiers_that_are_not_built_raise():
    from aihwkit_b200.rpu_base import tiles as T

    t, _ = _tiles(8, 8, np.zeros((8, 8), np.float32))
    with pytest.raises(RuntimeError, match="not implemented"):
        t.modify_weights(_par(type=T.WeightModifierType.PCMNoise, std_dev=0.1))
    with pytest.raises(RuntimeError, match="Per batch sample"):
        t.modify_weights(_par(type=T.WeightModifierType.AddNormal, std_dev=0.1, per_batch_sample=True))
