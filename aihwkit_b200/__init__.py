"""B200-native implementation of aihwkit's analog-tile hot path.

``aihwkit_b200.rpu_base`` mirrors ``aihwkit.simulator.rpu_base`` (``devices``, ``tiles``,
``cuda``) for the analog tile: IO-managed forward / backward MVM and pulsed update, running as
hand-written sm_100a CUDA kernels behind the C ABI of ``include/aihwkit_b200.h``.
"""

__version__ = "0.1.0"
