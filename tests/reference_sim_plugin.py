"""pytest plugin used by test_reference_sim_tests.py: runs those of the reference simulator's own test files
(test/sim/*.py of the reference checkout) that exercise the PUBLIC surface - `ttl.kernel`, `ttl.core`,
`ttl.grid_size`, core-index flattening, and the `ttnn` tensor API - against this backend's shadow modules.

The files import the simulator as `python.sim` / `sim`; those names are made to resolve to the shadow modules.
A kernel call is traced and recognised as usual and its launch plan evaluated on the host by the plan oracle."""

import sys
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "tt-lang_b200"))
sys.path.insert(0, str(ROOT))

import ttl_b200  # noqa: E402

ttl_b200.install()

from oracle import plan_oracle  # noqa: E402
from ttl_b200 import recognize, trace, ttnn  # noqa: E402


def _run_on_host(self, tensors):
    plan_oracle.run_plan(self, [t._tensor for t in list(tensors) + self.extras])


recognize.Plan.run = _run_on_host

_sim = sys.modules["sim"]
_sim.TTNN_AVAILABLE = False          # the golden-comparison tests need a real ttnn installation and skip themselves
_sim.TILE_SHAPE = trace.TILE_SHAPE
_sim.copy = trace.copy
_python = types.ModuleType("python")
_python.sim = _sim
_kernel = types.ModuleType("python.sim.kernel")
_kernel.flatten_core_index = trace.flatten_core_index
sys.modules.update({"python": _python, "python.sim": _sim, "python.sim.kernel": _kernel, "sim.kernel": _kernel,
                    "python.sim.typedefs": sys.modules["sim.typedefs"], "python.sim.ttnn": ttnn})
