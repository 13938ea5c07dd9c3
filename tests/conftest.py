import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "tt-lang_b200", ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def reference_root():
    """The tt-lang checkout the reference-driven tests read: $TTLANG_REFERENCE, else a directory named `reference`
    next to this repository; None when neither holds the simulator (those tests then skip)."""
    import os

    for cand in (os.environ.get("TTLANG_REFERENCE"), ROOT.parent / "reference"):
        if cand and (Path(cand) / "python" / "sim").is_dir():
            return Path(cand)
    return None


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")
    # the native library is built in-tree and is not under version control: build it when it is missing
    lib = ROOT / "tt-lang_b200" / "ttl_b200" / "libttlb200.so"
    runner = ROOT / "tt-lang_b200" / "ttl_b200" / "ttlang-b200-run"
    if not lib.exists() or not runner.exists():
        import importlib.util

        spec = importlib.util.spec_from_file_location("ttlb200_build", ROOT / "tt-lang_b200" / "build.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()


@pytest.fixture(scope="session")
def backend():
    """The B200 backend installed as `ttl` / `ttnn`, plus the tile programs loaded against it."""
    import importlib.util

    import ttl_b200

    ttl_b200.install()
    mods = {}
    for name in ("eltwise", "matmul", "reduce", "attention"):
        spec = importlib.util.spec_from_file_location(f"programs_b200_{name}", ROOT / "tests" / "programs" / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods[name] = mod
    return ttl_b200, mods


def load_golden(name):
    import numpy as np

    return np.load(ROOT / "tests" / "golden" / f"{name}.npz")


def golden_tensor(arr, dtype):
    """Fixture array -> torch tensor of `dtype` (bf16 is stored as uint16 bit patterns)."""
    import numpy as np
    import torch

    if dtype == torch.bfloat16:
        return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(arr.copy())


def digest(tensors):
    import hashlib

    import torch

    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()
