"""ttlang-b200-translate: show what a tt-lang program turns into on the B200 backend.

Counterpart of the reference's `ttlang-translate --ttkernel-to-cpp` (tools/ttlang-translate,
python/ttl/ttl_api.py:425-440 writes the generated C++ per kernel): runs the program file with the
launch stubbed out and prints, for every kernel call, the recognised launches and - for fused
element-wise programs - the CUDA source of the kernel specialised for it.  Works without a GPU.

    python -m ttl_b200.translate program.py [--no-source]
"""

from __future__ import annotations

import argparse
import contextlib
import io
import json
import runpy
import sys
from pathlib import Path
from typing import Any, List


def translate_file(path: str, with_source: bool = True) -> List[dict]:
    """Run `path` as __main__ with launches stubbed; return one record per kernel call."""
    import ttl_b200
    from ttl_b200 import capi, recognize

    ttl_b200.install()
    records: List[dict] = []

    def fake_run(self: Any, tensors: Any) -> None:
        rec = {"launches": self.describe()}
        if with_source:
            allt = list(tensors) + self.extras
            srcs = []
            ix = self.indexed(tensors)     # arguments, tensors derived in the body, temporaries of the plan
            for launch in self.launches:
                try:
                    if isinstance(launch, recognize.EltwiseLaunch):
                        srcs.append(capi.eltwise_source(_fake_pointers(launch.desc_cpu(allt))))
                    elif isinstance(launch, recognize.ReduceLaunch):
                        srcs.append(capi.reduce_source(launch.desc(ix, with_pointers=False)))
                    elif isinstance(launch, recognize.RowFusedLaunch):
                        srcs.append(capi.rowfused_source(launch.desc(ix, with_pointers=False)))
                    else:
                        srcs.append(None)      # hand-written kernels (GEMM, attention): nothing is generated
                except Exception as e:  # noqa: BLE001
                    srcs.append(f"// source unavailable: {e}")
            rec["cuda"] = srcs
        records.append(rec)

    orig = recognize.Plan.run
    recognize.Plan.run = fake_run  # type: ignore[assignment]
    p = Path(path)
    sys.path.insert(0, str(p.parent))
    old_argv = sys.argv
    sys.argv = [str(p)]
    try:
        with contextlib.redirect_stdout(io.StringIO()):
            try:
                runpy.run_path(str(p), run_name="__main__")
            except (AssertionError, SystemExit):
                pass  # the program's own result check fails: nothing was computed
    finally:
        recognize.Plan.run = orig  # type: ignore[assignment]
        sys.argv = old_argv
        sys.path.remove(str(p.parent))
    return records


def _fake_pointers(desc: Any) -> Any:
    # the generator only needs valid-looking, aligned addresses
    for k in range(desc.n_in):
        desc.inp[k].ptr = 0x10000 * (k + 1)
    desc.out = 0x1000000
    return desc


def main() -> None:
    ap = argparse.ArgumentParser(prog="ttlang-b200-translate")
    ap.add_argument("program")
    ap.add_argument("--no-source", action="store_true", help="print the launch plan only")
    a = ap.parse_args()
    for i, rec in enumerate(translate_file(a.program, with_source=not a.no_source)):
        print(f"// ---- kernel call {i}: {json.dumps(rec['launches'])}")
        for src in rec.get("cuda", []):
            if src:
                print(src)


if __name__ == "__main__":
    main()
