"""ttlang-b200-translate: show what a tt-lang program turns into on the B200 backend.

Counterpart of the reference's `ttlang-translate --ttkernel-to-cpp` (tools/ttlang-translate,
python/ttl/ttl_api.py:425-440 writes the generated C++ per kernel): runs the program file with the
launch stubbed out and prints, for every kernel call, the recognised launches and - for fused
element-wise programs - the CUDA source of the kernel specialised for it.  Works without a GPU.

    python -m ttl_b200.translate program.py [--no-source] [--emit DIR]

`--emit DIR` also writes, per kernel call, `DIR/call<i>/plan.json` (the launches with their operand addressing,
numeric opcodes and the tensor table) and the raw bytes of every argument tensor (`t<k>.bin`): the input of the
native runner `ttlang-b200-run` (cli/ttlang_b200_run.cpp), which executes the plan through the C ABI without Python.
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


def _tensor_entry(t: Any, directory: Path, name: str) -> dict:
    """Tensor table entry; the tensor's bytes go to `directory/name` (row-major, packed rows)."""
    import torch

    if t._packed is not None:
        if t._packed_bits != 8:
            raise ValueError("only bfloat8_b block-float tensors can be emitted")
        data, dtype = t._packed.cpu().contiguous(), "bfp8_b"
    else:
        data = t._tensor.cpu().contiguous()
        dtype = {torch.bfloat16: "bf16", torch.float32: "f32"}[data.dtype]
    (directory / name).write_bytes(data.view(torch.uint8).numpy().tobytes())
    return {"shape": list(t.shape), "dtype": dtype, "file": name}


def emit_plan(plan: Any, tensors: Any, directory: Path) -> None:
    """plan.json + tensor files for ttlang-b200-run."""
    import torch

    from ttl_b200 import capi

    directory.mkdir(parents=True, exist_ok=True)
    allt = list(tensors) + plan.extras
    table = [_tensor_entry(t, directory, f"t{k}.bin") for k, t in enumerate(allt)]
    temps = [{"shape": list(t._tensor.shape) if t._tensor.numel() else [0, 0],
              "dtype": {torch.bfloat16: "bf16", torch.float32: "f32"}[t._tensor.dtype]} for t in plan.temps]
    def numeric(d: dict) -> dict:
        d = dict(d)
        if "ops" in d:
            d["opcodes"] = [[capi.OPCODES[op], arg] for op, arg in d["ops"]]
        if d.get("act"):
            d["act_code"] = capi.ACTIVATIONS[d["act"]]
        if "phases" in d:
            d["phases"] = [numeric(ph) for ph in d["phases"]]
            d["final"] = numeric(d["final"])
        return d

    launches = [numeric(d) for d in plan.describe()]
    (directory / "plan.json").write_text(json.dumps({"tensors": table, "temps": temps, "launches": launches}, indent=1))


def translate_file(path: str, with_source: bool = True, emit: Any = None) -> List[dict]:
    """Run `path` as __main__ with launches stubbed; return one record per kernel call."""
    import ttl_b200
    from ttl_b200 import capi, recognize

    ttl_b200.install()
    records: List[dict] = []

    def fake_run(self: Any, tensors: Any) -> None:
        rec = {"launches": self.describe()}
        if emit is not None:
            emit_plan(self, tensors, Path(emit) / f"call{len(records)}")
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
    ap.add_argument("--emit", metavar="DIR", help="write plan.json and the tensors of every kernel call for ttlang-b200-run")
    a = ap.parse_args()
    for i, rec in enumerate(translate_file(a.program, with_source=not a.no_source, emit=a.emit)):
        print(f"// ---- kernel call {i}: {json.dumps(rec['launches'])}")
        for src in rec.get("cuda", []):
            if src:
                print(src)


if __name__ == "__main__":
    main()
