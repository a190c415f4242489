"""Run the reference's own Python package on top of the B200 analog tile.

``aihwkit`` (the pure-Python part of the reference: ``aihwkit.nn``, ``aihwkit.optim``,
``aihwkit.simulator.tiles`` ...) reaches its compiled simulator through one module,
``aihwkit.simulator.rpu_base`` (src/aihwkit/simulator/rpu_base_src/rpu_base.cpp:13-85: submodules
``devices``, ``tiles``, ``cuda``).  :func:`install` registers ``aihwkit_b200.rpu_base`` under that
name before ``aihwkit.simulator`` is imported, so that ``AnalogLinear``, ``AnalogConv2d``,
``AnalogSGD`` and the tile wrappers drive the sm_100a kernels unchanged::

    import aihwkit_b200.dropin
    aihwkit_b200.dropin.install()            # before the first ``import aihwkit.simulator``
    from aihwkit.nn import AnalogLinear      # the reference's Python, this package's tiles

There is no CPU compute path: modules must be moved to a CUDA device (``model.cuda()``) before the
first forward; host tiles only carry configuration, weights and per-element device parameters.
"""

from __future__ import annotations

import sys


def install() -> None:
    """Make ``aihwkit.simulator.rpu_base`` resolve to ``aihwkit_b200.rpu_base``."""
    from . import rpu_base
    from .rpu_base import cuda, devices, tiles

    if "aihwkit.simulator" in sys.modules:
        existing = getattr(sys.modules["aihwkit.simulator"], "rpu_base", None)
        if existing is not None and existing is not rpu_base:
            raise RuntimeError("aihwkit.simulator is already imported with another rpu_base; call "
                               "aihwkit_b200.dropin.install() before importing aihwkit.simulator")
    sys.modules["aihwkit.simulator.rpu_base"] = rpu_base
    sys.modules["aihwkit.simulator.rpu_base.devices"] = devices
    sys.modules["aihwkit.simulator.rpu_base.tiles"] = tiles
    sys.modules["aihwkit.simulator.rpu_base.cuda"] = cuda
