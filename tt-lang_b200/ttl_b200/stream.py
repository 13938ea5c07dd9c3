"""Running a row-parallel tile program on HOST tensors with the transfers overlapped.

A kernel call on tensors that live in host memory costs a host-to-device copy of every input, the
kernel, and a device-to-host copy of the result, one after the other; for an HBM-bound element-wise
program the PCIe copies are two orders of magnitude slower than the kernel.  When every output row
depends only on the same row of the full-size inputs (element-wise and broadcast programs), the rows can
be processed in chunks: the copy-in of chunk i+1, the kernel of chunk i and the copy-out of chunk i-1 run
at the same time on three streams, so a call takes about as long as its larger transfer direction.

The reference has no counterpart (ttnn.from_torch / to_torch are synchronous one-shot transfers,
python/sim/ttnnsim.py:554-580); the kernel itself is called exactly as a user would call it.
"""

from __future__ import annotations

from typing import Any, Callable, List, Sequence

import torch

from . import capi
from . import ttnn as _ttnn
from .recognize import TEMP_BASE, Unsupported

TILE = 32


def _check_row_parallel(plan: Any, split: Sequence[bool], chunk_rows: int) -> None:
    for l in plan.launches:
        d = l.describe()
        if d["kind"] == "row_fused":     # reductions over columns + element-wise: every row on its own
            inputs = [inp for ph in d["phases"] for inp in ph["inputs"]] + list(d["final"]["inputs"])
            inputs = [inp for inp in inputs if inp[0] < TEMP_BASE]    # the others are results kept on chip
        elif d["kind"] == "eltwise":
            inputs = d["inputs"]
        else:
            raise Unsupported(f"run_streamed needs a program whose output rows are independent; found a {d['kind']} launch")
        for (ti, rm, ro, _cm, _co) in inputs:
            whole = ti >= len(split) or not split[ti]
            # a split operand is read row for row (a chunk of one tile row shows up as "one tile repeated")
            row_for_row = ro == 0 and (rm == capi.IDX_SAME or (rm == capi.IDX_TILE and chunk_rows == TILE))
            if (not whole and not row_for_row) or (whole and rm == capi.IDX_SAME):
                raise Unsupported("run_streamed: an operand is read across rows (shifted or partially broadcast)")


def run_streamed(kernel: Callable[..., Any], host_inputs: Sequence[torch.Tensor], host_out: torch.Tensor,
                 chunks: int = 8) -> torch.Tensor:
    """`kernel(*inputs, out)` for tensors in (preferably pinned) host memory, in `chunks` row chunks with
    copy-in, kernel and copy-out overlapped.  Inputs with as many rows as the output are split by rows;
    the others (row vectors, scalars, single tiles) are copied once and passed whole.  The program must be
    row-parallel (checked on its launch plan; otherwise `Unsupported`).  Returns `host_out`, filled."""
    if not torch.cuda.is_available():
        raise capi.BackendError(capi.TTLB_ERR_CUDA, "no CUDA device: the B200 backend has no CPU fallback")
    rows, cols = host_out.shape
    if rows % TILE:
        raise ValueError("run_streamed: the output's rows must be a multiple of 32")
    split = [t.dim() == 2 and t.shape[0] == rows and rows > 1 for t in host_inputs]
    step = max(TILE, -(-rows // max(1, chunks) // TILE) * TILE)
    cur = torch.cuda.current_stream()
    dev = torch.device("cuda", torch.cuda.current_device())
    # device buffers are allocated whole, up front, on the calling stream: inside the loop only copies and
    # kernels are issued (no allocation, which could serialise the streams)
    dev_in = [torch.empty(t.shape, dtype=t.dtype, device=dev) if sp else _ttnn.from_torch(t)
              for t, sp in zip(host_inputs, split)]
    dev_out = torch.empty((rows, cols), dtype=host_out.dtype, device=dev)
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    s_in.wait_stream(cur)
    checked = set()
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        with torch.cuda.stream(s_in):
            for t, sp, d in zip(host_inputs, split, dev_in):
                if sp:
                    d[r0:r1].copy_(t[r0:r1], non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(s_in)
        parts = [_ttnn.Tensor(d[r0:r1]) if sp else d for sp, d in zip(split, dev_in)]
        y = _ttnn.Tensor(dev_out[r0:r1])
        if (r1 - r0) not in checked:
            _check_row_parallel(kernel.plan(*parts, y), split, r1 - r0)
            checked.add(r1 - r0)
        cur.wait_event(ready)
        kernel(*parts, y)
        done = torch.cuda.Event()
        done.record(cur)
        s_out.wait_event(done)
        with torch.cuda.stream(s_out):
            host_out[r0:r1].copy_(dev_out[r0:r1], non_blocking=True)
    # join: the buffers go back to the allocator in the calling stream's order only after every copy
    cur.wait_stream(s_in)
    cur.wait_stream(s_out)
    s_out.synchronize()
    capi.context(dev.index).check_status(int(cur.cuda_stream))   # a device-side wait that ran out must not pass silently
    return host_out
