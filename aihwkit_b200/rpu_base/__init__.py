"""Mirror of ``aihwkit.simulator.rpu_base`` (src/aihwkit/simulator/rpu_base_src/rpu_base.cpp:13-85)."""

from . import cuda, devices, tiles  # noqa: F401
