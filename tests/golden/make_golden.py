"""Generate tests/golden/*.npz by running the tile programs in tests/programs/ on the
UNMODIFIED reference simulator (python/sim under the reference checkout).

    python tests/golden/make_golden.py /path/to/tt-lang-checkout [fixture names...]

Run where the reference tree exists; the fixtures are committed so that the tests need no
reference at run time.  Each fixture holds the simulator's output (bf16 as uint16 bit
patterns), or for the large case a SHA-256 of the output bytes plus one corner, and a SHA-256
of the seeded inputs so that a drift of the input generator is detected.
"""

from __future__ import annotations

import hashlib
import importlib.util
import sys
import time
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
TESTS = HERE.parent
ROOT = TESTS.parent
sys.path.insert(0, str(TESTS))
sys.path.insert(0, str(ROOT))


def load_sim(reference: Path):
    sys.path.insert(0, str(reference / "python"))
    import sim  # type: ignore
    from sim.ttlang_sim import setup_simulator_imports  # type: ignore

    setup_simulator_imports()
    from oracle import sim_addons

    sim_addons.install(sim)
    return sim


def load_programs(tag: str):
    mods = {}
    for name in ("eltwise", "matmul", "reduce", "attention"):
        spec = importlib.util.spec_from_file_location(f"programs_{tag}_{name}", TESTS / "programs" / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods


def digest(tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def run_case_on_sim(case, mods, ttnn) -> torch.Tensor:
    """Simulator output for a case, in the case's dtype."""
    ins = case.make_inputs()
    work = [t.to(torch.float32) for t in ins] if case.mode == "f32" else ins
    tensors = [ttnn.from_torch(t.clone()) for t in work]
    out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=work[0].dtype))
    case.get_program(mods)(*tensors, out)
    return ttnn.to_torch(out).to(case.dtype)


def main() -> None:
    import os

    reference = Path(sys.argv[1]) if len(sys.argv) > 1 and sys.argv[1] != "-" else Path(os.environ.get("TTLANG_REFERENCE", ""))
    if not (reference / "python" / "sim").is_dir():
        raise SystemExit("usage: make_golden.py /path/to/tt-lang-checkout [fixture names...]  (or set TTLANG_REFERENCE and pass -)")
    sim = load_sim(reference)
    import ttnn  # the simulator's, after shadowing

    import cases

    mods = load_programs("sim")
    only = set(sys.argv[2:])   # optional: names of the fixtures to (re)generate
    for case in cases.CASES + cases.MATMUL_CASES + cases.REDUCE_CASES + cases.COMPOSITE_CASES + cases.MATH_CASES + cases.EPILOGUE_CASES + cases.OPERATOR_CASES + cases.ATTENTION_CASES + cases.ATTENTION_PIPELINE_CASES:
        if only and case.name not in only:
            continue
        t0 = time.time()
        out = run_case_on_sim(case, mods, ttnn)
        rec = {"input_digest": np.array(digest(case.make_inputs())), "mode": np.array(case.mode),
               "dtype": np.array(str(case.dtype))}
        if case.store == "digest":
            rec["out_digest"] = np.array(digest([out]))
            rec["corner"] = bits(out[:64, :64])
        else:
            rec["out"] = bits(out)
        np.savez_compressed(HERE / f"{case.name}.npz", **rec)
        print(f"{case.name}: {time.time() - t0:.2f}s")


if __name__ == "__main__":
    main()
