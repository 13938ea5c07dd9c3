"""Install the reference simulator, unmodified, next to the oracle so that it can be TIMED on the GPU box.

    python oracle/make_ref.py /path/to/tt-lang-checkout      (or set TTLANG_REFERENCE)

TEST / MEASUREMENT INFRASTRUCTURE ONLY (see oracle/__init__.py).  Copies the reference's `python/sim`
package byte for byte into `oracle/_ref/sim/` (kept out of version control; it travels with the working
tree like the built shared library) and records where it came from.  `bench.py --impl reference` and the
`cpu_baseline` figure run `ttlang-sim`'s own scheduler, circular buffers and block arithmetic from this copy
(python/sim/ttlang_sim.py:95-146, python/sim/program.py:363-647) on the same tile program the GPU arm
runs; when the copy is absent they fall back to the torch restatement in `oracle/tile_oracle.py`.
Nothing in the product path imports this folder.
"""

from __future__ import annotations

import hashlib
import json
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"


def install(reference: Path) -> Path:
    src = reference / "python" / "sim"
    if not src.is_dir():
        raise FileNotFoundError(f"{src} not found: pass the path of a tt-lang checkout")
    dst = DEST / "sim"
    if dst.exists():
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    digest = hashlib.sha256()
    files = sorted(p for p in dst.rglob("*.py"))
    for p in files:
        digest.update(p.read_bytes())
    commit = ""
    head = reference / ".git" / "HEAD"
    if head.exists():
        commit = head.read_text().strip()
    (DEST / "MANIFEST.json").write_text(json.dumps({
        "source": "python/sim of the tt-lang reference checkout, copied without modification",
        "files": len(files), "sha256": digest.hexdigest(), "git_head": commit}, indent=1))
    return dst


def load():
    """Import the installed simulator (with the `ttl` / `ttnn` shadow modules it sets up and the math add-ons
    of oracle/sim_addons.py) and return its `sim` package; None when it is not installed."""
    if not (DEST / "sim" / "__init__.py").exists():
        return None
    if str(DEST) not in sys.path:
        sys.path.insert(0, str(DEST))
    import sim  # type: ignore
    from sim.ttlang_sim import setup_simulator_imports  # type: ignore

    setup_simulator_imports()
    from oracle import sim_addons

    sim_addons.install(sim)
    return sim


if __name__ == "__main__":
    import os

    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TTLANG_REFERENCE")
    if not where:
        raise SystemExit("usage: make_ref.py /path/to/tt-lang-checkout  (or set TTLANG_REFERENCE)")
    print(install(Path(where)))
