"""B200-native execution backend for tt-lang tile programs.

Use it the way the reference's simulator is used (python/sim/ttlang_sim.py:22-34):
shadow the `ttl` and `ttnn` modules, then run the program unchanged::

    import ttl_b200; ttl_b200.install()
    import ttl, ttnn            # now the B200 backend

or run a program file with `python -m ttl_b200.launcher program.py`.
"""

from __future__ import annotations

import sys

from . import profile, ttl, ttnn  # noqa: F401
from .capi import BackendError  # noqa: F401
from .math import set_hardware_broadcast  # noqa: F401
from .recognize import Unsupported, set_row_fusion  # noqa: F401
from .stream import run_streamed  # noqa: F401

__version__ = "0.1"


def synchronize(device=None) -> None:
    """Wait for the work queued on `device` (default: the current CUDA device) on the current stream and raise
    `BackendError` (TTLB_ERR_TIMEOUT) if a bounded device-side wait of one of this backend's kernels ran out
    since the last check.  `ttnn.to_torch` and `run_streamed` make the same check."""
    import torch

    from . import capi

    dev = torch.cuda.current_device() if device is None else (device if isinstance(device, int) else torch.device(device).index)
    capi.context(dev).check_status(int(torch.cuda.current_stream(dev).cuda_stream))


def install() -> None:
    """Make `import ttl` / `import ttnn` resolve to this backend, and give programs that
    import the simulator's helper modules (`sim.testing`, `sim.typedefs`) working
    stand-ins so that they run unchanged."""
    import types

    from . import testing, trace

    sys.modules["ttl"] = ttl
    sys.modules["ttl.math"] = ttl.math
    sys.modules["ttnn"] = ttnn
    sim = types.ModuleType("sim")
    sim.ttl, sim.ttnn = ttl, ttnn
    typedefs = types.ModuleType("sim.typedefs")
    typedefs.Pipe = trace.Pipe
    typedefs.CoreCoord, typedefs.CoreRange = ttnn.CoreCoord, ttnn.CoreRange
    typedefs.Shape, typedefs.Size = tuple, int
    sim.testing, sim.typedefs = testing, typedefs
    sys.modules["sim"] = sim
    sys.modules["sim.testing"] = testing
    sys.modules["sim.typedefs"] = typedefs
