"""Build libttlb200.so (CUDA kernels + C ABI) in-tree for sm_100a with nvcc.

Usage: python tt-lang_b200/build.py [--force] [--verbose]

The library is written next to the Python package (ttl_b200/libttlb200.so) so that it
travels with the source tree.  cudart is linked statically and the CUDA driver API is
resolved at run time, so the library loads on a machine without a GPU (its entry
points then return TTLB_ERR_CUDA).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
INCLUDE = ROOT.parent / "include"
OUT = ROOT / "ttl_b200" / "libttlb200.so"
CLI_SRC = ROOT / "cli" / "ttlang_b200_run.cpp"
CLI_OUT = ROOT / "ttl_b200" / "ttlang-b200-run"    # the native runner, next to the library it loads
OBJ_DIR = ROOT / "build"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC,-fvisibility=hidden",
    f"-I{INCLUDE}",
    f"-I{CSRC}",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _newer(src: Path, dst: Path, deps: list[Path]) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *deps])


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))
    objs = []
    procs = []
    for src in sources:
        obj = OBJ_DIR / (src.name + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
                print(" ".join(cmd), flush=True)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            print(f"--- nvcc failed on {src.name}:\n{out}", file=sys.stderr)
        elif verbose and out:
            print(f"--- {src.name}:\n{out}")
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or not OUT.exists():
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static",
               "-o", str(OUT), *map(str, objs), "-ldl"]
        subprocess.run(cmd, check=True)
    if force or _newer(CLI_SRC, CLI_OUT, [OUT, *sorted(INCLUDE.glob("*.h"))]):
        # host-only program over the C ABI; finds libttlb200.so in its own directory
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", f"-I{INCLUDE}", str(CLI_SRC), "-o", str(CLI_OUT), f"-L{OUT.parent}", "-lttlb200",
               "-Xlinker", "-rpath=$ORIGIN", "-cudart", "static"]
        subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
