"""Per-source-line timing report for tile programs on the B200 backend.

The reference's auto-profiler (python/ttl/_src/auto_profile.py, switched on with TTLANG_AUTO_PROFILE=1)
brackets every operation of the three Tensix threads with Tracy signposts and prints, per thread, the
cycles spent on each source line (docs/auto-profiler-examples/demo-one.txt).  On this backend a tile program
does not run line by line: the tracer turns it into a few GPU launches.  The report therefore has two views:
per LAUNCH - which kernel, how often, how long (CUDA events on the launching stream), and which program lines
it implements with how many block operations each - and per SOURCE LINE - the time of every launch the line
takes part in.

Switch it on before the first kernel call (plans built earlier carry no line information):
`TTLANG_AUTO_PROFILE=1` in the environment (report printed at exit), `ttl_b200.profile.enable()` from
code, or `python -m ttl_b200.launcher --profile program.py`.
"""

from __future__ import annotations

import atexit
import linecache
import os
from typing import Any, Dict, List, Tuple

from .trace import PROFILE

_records: List[Tuple[Any, Any, Any]] = []      # (launch, start event, end event)
_calls = 0
_at_exit = False


def enable(report_at_exit: bool = False) -> None:
    global _at_exit
    PROFILE.enabled = True
    if report_at_exit and not _at_exit:
        _at_exit = True
        atexit.register(lambda: print(report()))


def disable() -> None:
    PROFILE.enabled = False


def reset() -> None:
    global _calls
    _records.clear()
    _calls = 0


def run_timed(plan: Any, ctx: Any, tensors: Any, stream: int) -> None:
    """Plan.run with a pair of CUDA events around every launch."""
    import torch

    global _calls
    _calls += 1
    for l in plan.launches:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        l.run(ctx, tensors, stream)
        e1.record()
        _records.append((l, e0, e1))


def _kernel_name(kind: str) -> str:
    if kind == "eltwise":
        return "ttlb_eltwise_jit"
    if kind.startswith("reduce"):
        return "ttlb_reduce_jit"
    if kind == "row_fused":
        return "ttlb_rowfused_jit"
    return {"matmul_bf16": "ttlb_gemm_bf16", "matmul_f32": "ttlb_gemm_f32", "matmul_bfp8w": "ttlb_unpack_bfp8 + ttlb_gemm_bf16"}.get(kind, kind)


def summarize(records: List[Tuple[Any, float]], calls: int) -> str:
    """The report for (launch, microseconds) records; separated from the event handling so that the format
    can be produced without a GPU."""
    W = 100
    by_launch: Dict[int, Dict[str, Any]] = {}
    order: List[int] = []
    for l, us in records:
        rec = by_launch.get(id(l))
        if rec is None:
            rec = by_launch[id(l)] = {"launch": l, "n": 0, "us": 0.0, "min": us, "max": us}
            order.append(id(l))
        rec["n"] += 1
        rec["us"] += us
        rec["min"], rec["max"] = min(rec["min"], us), max(rec["max"], us)
    total = sum(r["us"] for r in by_launch.values()) or 1e-9
    out = ["=" * W, "TTLANG-B200 PROFILE REPORT", "=" * W, "",
           f"Kernel calls: {calls}", f"GPU launches: {len(records)}", f"GPU time: {total:,.1f} us", ""]
    per_line: Dict[Tuple[str, int], Dict[str, Any]] = {}
    for idx, key in enumerate(order, 1):
        r = by_launch[key]
        l = r["launch"]
        d = l.describe()
        what = d["kind"] + (f" dims={d['dims']}" if "dims" in d else "")
        if "phases" in d:
            what += " (" + " + ".join([ph["kind"] for ph in d["phases"]] + [d["final"]["kind"]]) + ")"
        out += ["=" * W,
                f"LAUNCH {idx}: {what} -> {_kernel_name(d['kind'])}   (x{r['n']}, avg={r['us'] / r['n']:,.1f} us, "
                f"{r['min']:,.1f}-{r['max']:,.1f}, total={r['us']:,.1f} us, {100 * r['us'] / total:.1f}% of total)",
                f"  output tensor {d['out']}, tiles {d['rect_tiles']}" + (f", ops {[o for o, _ in d['ops']]}" if "ops" in d else ""),
                "=" * W, "", f"{'LINE':<6} {'BLOCKS':<8} SOURCE", f"{'-' * 6} {'-' * 8} {'-' * 70}"]
        lines = getattr(l, "lines", {}) or {}
        for (fn, ln), n in sorted(lines.items()):
            src = linecache.getline(fn, ln).rstrip()
            out.append(f"{ln:<6} x{n:<7} {src}")
            pl = per_line.setdefault((fn, ln), {"us": 0.0, "launches": []})
            pl["us"] += r["us"]
            pl["launches"].append(idx)
        if not lines:
            out.append("(no line information: the plan was built before profiling was switched on)")
        out.append("")
    out += ["=" * W, "BY SOURCE LINE  (a line is charged the time of every launch it takes part in)", "=" * W, ""]
    files = sorted({fn for fn, _ in per_line})
    for fn in files:
        out += [f"FILE: {os.path.basename(fn)}", "", f"{'LINE':<6} {'%TIME':>7} {'US':>10}  SOURCE", f"{'-' * 6} {'-' * 7} {'-' * 10}  {'-' * 70}"]
        for (f2, ln), pl in sorted(per_line.items()):
            if f2 != fn:
                continue
            src = linecache.getline(fn, ln).rstrip()
            tags = ",".join(f"L{i}" for i in pl["launches"])
            out.append(f"{ln:<6} {100 * pl['us'] / total:6.1f}% {pl['us']:>10,.1f}  {src}  [{tags}]")
        out.append("")
    return "\n".join(out)


def report() -> str:
    """Synchronise, turn the recorded events into times, and format the report."""
    import torch

    if _records and torch.cuda.is_available():
        torch.cuda.synchronize()
    return summarize([(l, e0.elapsed_time(e1) * 1000.0) for l, e0, e1 in _records], _calls)


if os.environ.get("TTLANG_AUTO_PROFILE", "0") == "1":   # the reference's switch (python/ttl/_src/auto_profile.py)
    enable(report_at_exit=True)
