"""The reference simulator's own tests of its public surface (test/sim/test_kernel.py: kernel decorator, core
coordinates, grid sizes, core-index flattening; test/sim/test_ttnnsim.py: the ttnn tensor API), unchanged, against
this backend's shadow modules (tests/reference_sim_plugin.py).  The other files of test/sim test the simulator's
internals (block state machines, generator transforms) and have no counterpart here.  Needs the reference
checkout (skipped elsewhere); CPU only."""

import re
import subprocess
import sys
from pathlib import Path

import pytest

from conftest import reference_root  # noqa: E402

REFERENCE = reference_root() or Path("reference-checkout-not-found")
TESTS = Path(__file__).resolve().parent
pytestmark = pytest.mark.skipif(not (REFERENCE / "test" / "sim").exists(), reason="reference checkout not present")

# file -> (tests that must pass, tests that skip themselves because no real ttnn is installed)
EXPECTED = {"test_kernel.py": (32, 0), "test_ttnnsim.py": (43, 17)}


@pytest.mark.parametrize("name", sorted(EXPECTED))
def test_reference_simulator_test_file_passes(name, tmp_path):
    ini = tmp_path / "empty.ini"
    ini.write_text("[pytest]\n")
    cmd = [sys.executable, "-m", "pytest", str(REFERENCE / "test" / "sim" / name), "-c", str(ini),
           "-p", "reference_sim_plugin", "-q", "--no-header", "-p", "no:cacheprovider"]
    env = {"PYTHONPATH": f"{TESTS}:{REFERENCE / 'test' / 'sim'}", "PATH": "/usr/bin:/bin", "HOME": str(tmp_path)}
    r = subprocess.run(cmd, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=600)
    tail = r.stdout.strip().splitlines()[-1] if r.stdout.strip() else r.stderr[-400:]
    passed = re.search(r"(\d+) passed", tail)
    skipped = re.search(r"(\d+) skipped", tail)
    want_pass, want_skip = EXPECTED[name]
    assert r.returncode == 0 and passed and int(passed.group(1)) == want_pass, tail
    assert (int(skipped.group(1)) if skipped else 0) == want_skip, tail
