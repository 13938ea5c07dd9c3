"""The reference's own example programs, unchanged, traced and recognised by the backend.

Needs the reference checkout (skipped elsewhere).  The launch itself is stubbed out - this is a
CPU test of the front half (shadow modules, tracer, recogniser) on programs this repository did
not write; the GPU half is covered by the parity tests on tests/programs/."""

import contextlib
import io
import runpy
import sys
from pathlib import Path

import pytest

from conftest import reference_root  # noqa: E402

REFERENCE = reference_root() or Path("reference-checkout-not-found")
pytestmark = pytest.mark.skipif(not (REFERENCE / "examples").exists(), reason="reference checkout not present")

EXPECTED = {
    "examples/eltwise_add.py": {"eltwise"},
    "examples/eltwise_pipe.py": {"eltwise"},
    "examples/eltwise_pipe_core3.py": {"eltwise"},
    "examples/broadcast.py": {"eltwise"},
    "examples/broadcast_demo.py": {"eltwise"},
    "examples/general_broadcast.py": {"eltwise"},
    "examples/singlecore_matmul.py": {"matmul_f32"},
    "examples/multicore_matmul.py": {"matmul_f32"},
    "examples/metal_examples/singlecore_matmul/ttlang/singlecore_matmul.py": {"matmul_bf16"},
    "examples/metal_examples/multicore_matmul/ttlang/multicore_matmul.py": {"matmul_bf16"},
    "examples/tutorial/multicore.py": {"eltwise"},
    "examples/tutorial/multicore_grid_auto.py": {"eltwise"},
    "examples/tutorial/single_core_broadcast_multitile_blocks.py": {"eltwise"},
    "examples/tutorial/single_core_broadcast_single_tile_block.py": {"eltwise"},
    "examples/tutorial/single_core_multitile_block.py": {"eltwise"},
    "examples/tutorial/single_core_single_tile_block.py": {"eltwise"},
}


@pytest.mark.parametrize("rel", sorted(EXPECTED))
def test_reference_example_is_traced_and_recognised(rel, backend, monkeypatch):
    from ttl_b200 import recognize
    plans = []
    monkeypatch.setattr(recognize.Plan, "run", lambda self, tensors: plans.append(self.describe()))
    monkeypatch.setattr(sys, "argv", [rel])
    path = REFERENCE / rel
    monkeypatch.syspath_prepend(str(path.parent))
    monkeypatch.syspath_prepend(str(REFERENCE / "python"))   # the metal examples import utils.correctness from there
    try:
        with contextlib.redirect_stdout(io.StringIO()):
            runpy.run_path(str(path), run_name="__main__")
    except (AssertionError, SystemExit):
        pass   # the example's own result check fails because the stubbed launch computes nothing
    assert plans, "the program never reached a kernel launch"
    kinds = {l["kind"] for p in plans for l in p}
    assert kinds == EXPECTED[rel]


@pytest.mark.parametrize("rel,exc,text", [
    ("examples/copy_lock_error.py", RuntimeError, "copy lock error"),
    ("examples/eltwise_add_error.py", ValueError, "does not match Block shape"),
])
def test_reference_error_examples_fail_the_same_way(rel, exc, text, backend, monkeypatch):
    """The reference's intentionally wrong programs are refused while tracing, with the simulator's
    diagnosis (python/sim/block.py:839-843, python/sim/copyhandlers.py:299-310)."""
    monkeypatch.setattr(sys, "argv", [rel])
    path = REFERENCE / rel
    monkeypatch.syspath_prepend(str(path.parent))
    monkeypatch.syspath_prepend(str(REFERENCE / "python"))
    with pytest.raises(exc, match=text):
        with contextlib.redirect_stdout(io.StringIO()):
            runpy.run_path(str(path), run_name="__main__")


def test_reuse_matmul_example_runs_as_one_gemm(backend, monkeypatch):
    """examples/metal_examples/multicore_reuse_matmul: blocks of (per_core_M, 2) @ (2, per_core_N) tiles, the
    specification's general block dot product.  The reference simulator cannot run it, and the file as checked
    in does not import `ttl`, `get_large_matmul_params` or its `metal_examples.utils` helper: the test supplies
    those three names and nothing else.  The launch is evaluated by the plan oracle and the example's own
    `assert_with_ulp` check against torch.matmul judges the result."""
    import importlib.util
    import types

    from oracle import plan_oracle
    from ttl_b200 import recognize
    monkeypatch.syspath_prepend(str(REFERENCE / "python"))
    monkeypatch.syspath_prepend(str(REFERENCE / "examples"))
    from utils.block_allocation import get_large_matmul_params
    from utils.correctness import assert_with_ulp
    stub = types.ModuleType("metal_examples.utils")
    stub.assert_with_ulp = assert_with_ulp
    monkeypatch.setitem(sys.modules, "metal_examples.utils", stub)
    plans = []

    def run(self, tensors):
        plans.append(self.describe())
        plan_oracle.run_plan(self, [t._tensor for t in list(tensors) + self.extras])

    monkeypatch.setattr(recognize.Plan, "run", run)
    path = REFERENCE / "examples/metal_examples/multicore_reuse_matmul/ttlang/multicore_reuse_matmul.py"
    spec = importlib.util.spec_from_file_location("reference_reuse_matmul", path)
    mod = importlib.util.module_from_spec(spec)
    import ttl
    mod.ttl, mod.get_large_matmul_params = ttl, get_large_matmul_params
    with contextlib.redirect_stdout(io.StringIO()):
        spec.loader.exec_module(mod)
        mod.test_multicore_reuse_matmul_tt_lang(640, 640, 640)
    assert len(plans) == 1 and [l["kind"] for l in plans[0]] == ["matmul_bf16"]
    assert plans[0][0]["rect_tiles"] == (0, 20, 0, 20) and plans[0][0]["k_tiles"] == 20
