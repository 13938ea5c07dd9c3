"""pytest plugin used by test_reference_hw_tests.py: runs the reference's hardware-path test files
(test/python/*.py of the reference checkout) against this backend's front half on the CPU.

`import ttl` / `import ttnn` resolve to the shadow package; a kernel call is traced and recognised
as usual, and the resulting launch plan is evaluated on the host by the plan oracle instead of being
launched on a GPU, so the reference test's own assertions judge the recognised plan."""

import importlib.machinery
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "tt-lang_b200"))
sys.path.insert(0, str(ROOT))
os.environ["TTLANG_HAS_DEVICE"] = "1"   # the reference's helper module decides on this (test/ttlang_test_utils.py:29-32)

import ttl_b200  # noqa: E402

ttl_b200.install()
ttl_b200.set_hardware_broadcast(True)   # these tests are written against the compiler's broadcast (full source tiles)
for _name in ("ttl", "ttnn"):
    if getattr(sys.modules[_name], "__spec__", None) is None:
        sys.modules[_name].__spec__ = importlib.machinery.ModuleSpec(_name, None)

from oracle import plan_oracle  # noqa: E402
from ttl_b200 import recognize  # noqa: E402


def _run_on_host(self, tensors):
    allt = list(tensors) + self.extras
    plan_oracle.run_plan(self, [t._tensor for t in allt])


recognize.Plan.run = _run_on_host
