"""Mirror of ``aihwkit.simulator.rpu_base.cuda`` (rpu_base.cpp:69-84)."""

import os

from .. import _cabi


def is_compiled() -> bool:
    """Whether the CUDA library has been built (the reference reports its USE_CUDA build flag)."""
    return os.path.exists(_cabi.LIB_PATH)
