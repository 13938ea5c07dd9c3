"""The reference's script-style hardware tests (test/python/*.py driven by lit: `%python %s` + FileCheck on the
generated MLIR / C++), unchanged, run through the backend's front end on the CPU.

FileCheck's subject - the compiler's IR - does not exist here; what is checked is that every script traces, is
recognised as one fused element-wise launch per kernel call, and that the script's OWN result check (assert /
PASS / FAIL print) passes when the launch plan is evaluated by the plan oracle.  The scripts gate themselves on
TTLANG_HAS_DEVICE (test/ttlang_test_utils.py:29-30) and use the hardware broadcast convention.  Needs the
reference checkout; each script runs in its own interpreter."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

from conftest import reference_root  # noqa: E402

REFERENCE = reference_root() or Path("reference-checkout-not-found")
ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.skipif(not (REFERENCE / "test" / "python").exists(), reason="reference checkout not present")

SCRIPTS = [
    "simple_add.py", "simple_add_dram.py", "simple_add_f32.py", "simple_add_loop.py", "simple_add_multitile.py",
    "simple_add_with_stmt.py", "simple_bcast.py", "simple_fused.py", "simple_multicore.py", "many_fused_ops.py",
    "mixed_l1_dram.py", "test_dram_interleaved_add.py", "test_large_dram_streaming.py", "program_cache_lit.py",
    "debug_locations.py", "auto_profile_signposts.py",
]
# not run: simple_tensor_slice.py (compile-only: it addresses tile [0, 3] of a 2x2-tile tensor, which only an IR
# check can accept), smoketest.py (imports the MLIR bindings), test_ttnn_interop_add.py / test_block_allocation.py
# (real ttnn device tensors / Tensix L1 heuristics)

RUNNER = r"""
import contextlib, io, runpy, sys
root, ref, rel = sys.argv[1], sys.argv[2], sys.argv[3]
sys.path[:0] = [root + "/tt-lang_b200", root, ref + "/test"]
import ttl_b200
ttl_b200.install()
ttl_b200.set_hardware_broadcast(True)
from oracle import plan_oracle
from ttl_b200 import recognize
plans = []
def run(self, tensors):
    plans.append([l["kind"] for l in self.describe()])
    plan_oracle.run_plan(self, [t._tensor for t in list(tensors) + self.extras])
recognize.Plan.run = run
sys.argv = [rel]
out = io.StringIO()
try:
    with contextlib.redirect_stdout(out):
        runpy.run_path(ref + "/test/python/" + rel, run_name="__main__")
except SystemExit as e:
    if e.code not in (None, 0):
        raise
text = out.getvalue()
assert plans and all(p == ["eltwise"] for p in plans), plans
assert "FAIL" not in text and "Skipping" not in text, text[-400:]
print("RAN", len(plans))
"""


@pytest.mark.parametrize("rel", SCRIPTS)
def test_reference_lit_script_runs_and_passes_its_own_check(rel):
    env = {**os.environ, "TTLANG_HAS_DEVICE": "1"}
    r = subprocess.run([sys.executable, "-c", RUNNER, str(ROOT), str(REFERENCE), rel], capture_output=True, text=True,
                       env=env, timeout=300)
    assert r.returncode == 0 and "RAN" in r.stdout, (r.stdout[-300:], r.stderr[-1500:])
