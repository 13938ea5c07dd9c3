"""`ttl` surface of the B200 backend: the names tt-lang programs import
(python/ttl/__init__.py:10-50, python/sim/__init__.py:32-66)."""

from __future__ import annotations

from . import math  # noqa: F401  (ttl.math.*)
from .kernel import compute, core, datamovement, grid_size, kernel  # noqa: F401
from .trace import (  # noqa: F401
    MAX_CBS,
    TILE_SHAPE,
    CircularBuffer,
    CopyTransaction,
    DstPipeIdentity,
    Pipe,
    PipeNet,
    SrcPipeIdentity,
    copy,
    make_circular_buffer_like,
)
from .ttnn import CoreCoord, CoreRange  # noqa: F401

Size = int
Shape = tuple
CopyTransferHandler = CopyTransaction

# the compiler package also exports the element-wise functions at top level
# (python/ttl/__init__.py:22-24) and itself as `ttl.ttl` (`from ttl import ttl`, python/ttl/ttl.py)
from .math import abs, exp, log, max, min, neg, relu, rsqrt, sigmoid, sqrt, tanh  # noqa: E402,F401,A004
import sys as _sys  # noqa: E402

ttl = _sys.modules[__name__]


def signpost(name: str) -> None:
    """Profiling marker (python/ttl/__init__.py); a no-op on this backend."""
    return None


def Program(*threads, grid):  # noqa: N802 - reference spelling
    """Explicit program object (python/sim/program.py:100): `Program(compute, dm0, dm1, grid=g)(*tensors)`."""
    from . import recognize as _rec
    from . import trace as _trace
    from . import ttnn as _ttnn

    def run(*args, **kwargs):
        fns = [(t.thread_type, t.__wrapped__) for t in threads]
        tr = _trace.run_program(fns, tuple(grid))
        tensors = [a for a in args if isinstance(a, _ttnn.Tensor)]
        _rec.build_plan(tr, tensors).run(tensors)

    return run
