"""The reference's own hardware-path tests (test/python/*.py of the reference checkout), unchanged,
run against this backend's front half: `import ttl` / `import ttnn` resolve to the shadow package,
every kernel call is traced and recognised, and the launch plan is evaluated on the host by the plan
oracle (tests/reference_hw_plugin.py), so the reference tests' own assertions judge what the
recogniser understood.  Needs the reference checkout (skipped elsewhere); CPU only - the kernels
these plans launch are covered by the GPU parity tests."""

import re
import subprocess
import sys
from pathlib import Path

import pytest

from conftest import reference_root  # noqa: E402

REFERENCE = reference_root() or Path("reference-checkout-not-found")
TESTS = Path(__file__).resolve().parent
pytestmark = pytest.mark.skipif(not (REFERENCE / "test" / "python").exists(), reason="reference checkout not present")

# file -> number of its tests that must pass (all of them, for these files)
EXPECTED = {
    "test_adversarial_multicore.py": 1,
    "test_axby.py": 1,
    "test_bcast_multicore.py": 1,
    "test_bcast_ops.py": 15,
    "test_bcast_shape_expansion.py": 6,
    "test_comprehensive_multicore.py": 1,
    "test_dst_multi_consumer.py": 5,
    "test_elementwise_ops.py": 13,
    "test_elementwise_shapes.py": 208,
    "test_grid_auto.py": 1,
    "test_intermediate_cb.py": 1,
    "test_multicore.py": 49,
    "test_sanity.py": 3,
    "test_tensor_slice.py": 241,
    "test_uneven_grids.py": 14,
}


@pytest.mark.parametrize("name", sorted(EXPECTED))
def test_reference_hardware_test_file_passes(name, tmp_path):
    ini = tmp_path / "empty.ini"
    ini.write_text("[pytest]\n")   # the reference's own ini asks for a plugin that is not installed
    cmd = [sys.executable, "-m", "pytest", str(REFERENCE / "test" / "python" / name), "-c", str(ini),
           "-p", "reference_hw_plugin", "-q", "--no-header", "-p", "no:cacheprovider"]
    env = {"PYTHONPATH": str(TESTS), "PATH": "/usr/bin:/bin", "HOME": str(tmp_path)}
    r = subprocess.run(cmd, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=900)
    tail = r.stdout.strip().splitlines()[-1] if r.stdout.strip() else r.stderr[-400:]
    m = re.search(r"(\d+) passed", tail)
    assert r.returncode == 0 and m and int(m.group(1)) == EXPECTED[name], tail
