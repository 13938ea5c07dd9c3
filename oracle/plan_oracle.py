"""CPU evaluation of a launch plan (test infrastructure only - never on the product path).

A plan is what the recogniser turns a tt-lang kernel call into: element-wise launches (operand
index modes + a small stack program, include/ttlb200.h) and matmul launches.  Evaluating the plan
on the host with torch shows that the front half (tracer + recogniser) preserved the program's
meaning, without a GPU: the reference's own hardware tests (test/python/*.py) are run this way.
Numerics follow the reference simulator: ops on bf16 tensors round after every op unless the
kernel asked for fp32 intermediates (python/sim/block.py:856-864)."""

from typing import Any, List, Sequence

import torch

from . import tile_oracle

TILE = 32
_SAME, _ZERO, _TILE, _FIRST = 0, 1, 2, 3

_IN_TENSOR_TYPE = {"floordiv", "rfloordiv", "mod", "rmod"}
_UNARY = dict(tile_oracle.UNARY)
_PARAM_UNARY = tile_oracle.PARAM_UNARY
_N_PARAMS = {"rsub_imm": 1, "relu_max": 1, "relu_min": 1, "leaky_relu": 1, "elu": 1, "celu": 2, "softplus": 3,
             "hardtanh": 2, "selu": 2, "pow_imm": 1}
_BINARY = {
    "add": lambda a, b: a + b, "sub": lambda a, b: a - b, "rsub": lambda a, b: b - a, "mul": lambda a, b: a * b,
    "div": lambda a, b: a / b, "rdiv": lambda a, b: b / a, "max": torch.maximum, "min": torch.minimum,
    "floordiv": torch.floor_divide, "rfloordiv": lambda a, b: torch.floor_divide(b, a),
    "mod": torch.remainder, "rmod": lambda a, b: torch.remainder(b, a),
    "pow": torch.pow, "rpow": lambda a, b: torch.pow(b, a),
}


def _index(mode: int, off: int, idx: torch.Tensor) -> torch.Tensor:
    if mode == _SAME:
        return idx + off
    if mode == _ZERO:
        return torch.full_like(idx, off)
    if mode == _FIRST:
        return off + idx - idx % TILE
    return off + idx % TILE


def _evaluate(inputs: Any, ops: Any, tensors: Sequence[torch.Tensor], rows: torch.Tensor, cols: torch.Tensor,
              rnd: bool, imms: Sequence[float] = ()) -> torch.Tensor:
    """The stack program of a launch on the index ranges `rows` x `cols`, as an fp32 matrix."""

    def operand(k: int) -> torch.Tensor:
        ti, rm, ro, cm, co = inputs[k]
        x = tensors[ti]
        if x.dim() == 1:
            x = x.reshape(1, -1)
        return x[_index(rm, ro, rows)][:, _index(cm, co, cols)].to(torch.float32)

    acc = torch.zeros(len(rows), len(cols))
    stack: List[torch.Tensor] = []
    for op, arg in ops:
        if op == "push":
            stack.insert(0, acc)
            continue
        if op == "load" or op in _BINARY:
            x = operand(arg) if arg >= 0 else stack.pop(0)
            if rnd and op in _IN_TENSOR_TYPE:
                # torch evaluates floor division and remainder step by step in the tensor's own type
                acc = _BINARY[op](acc.to(torch.bfloat16), x.to(torch.bfloat16)).to(torch.float32)
            else:
                acc = x if op == "load" else _BINARY[op](acc, x)
        elif op in _PARAM_UNARY:
            if rnd and op == "pow_imm":     # in the tensor's own type, see tile_oracle.PARAM_UNARY
                acc = _PARAM_UNARY[op](acc.to(torch.bfloat16), *imms[arg:arg + 1]).to(torch.float32)
            else:
                acc = _PARAM_UNARY[op](acc, *imms[arg:arg + _N_PARAMS[op]])
        else:
            acc = _UNARY[op](acc)
        if rnd and op != "load":
            acc = acc.to(torch.bfloat16).to(torch.float32)
    return acc


def run_eltwise(launch: Any, tensors: Sequence[torch.Tensor]) -> None:
    """Evaluate one element-wise launch into tensors[launch.out_index] (host tensors)."""
    out = tensors[launch.out_index]
    r0, r1, c0, c1 = launch.rect
    rows = torch.arange(0, 1) if launch.out_degenerate[0] else torch.arange(r0 * TILE, r1 * TILE)
    cols = torch.arange(0, 1) if launch.out_degenerate[1] else torch.arange(c0 * TILE, c1 * TILE)
    rnd = out.dtype == torch.bfloat16 and launch.round_each_op
    acc = _evaluate(launch.inputs, launch.ops, tensors, rows, cols, rnd, getattr(launch, "imms", ()))
    view = out if out.dim() == 2 else out.reshape(1, -1)
    view[rows[0]:rows[-1] + 1, cols[0]:cols[-1] + 1] = acc.to(out.dtype)


def run_reduce(launch: Any, tensors: Sequence[torch.Tensor]) -> None:
    """Evaluate one reduction launch (include/ttlb200.h, ttlb_reduce): values in fp32, combined along the
    reduced dims, times the scaler, one rounding; the result sits at index 0 of a reduced dim and the rest
    of a full result tile is zero."""
    out = tensors[launch.out_index]
    row0, nrows, col0, ncols = launch.region()
    rnd = out.dtype == torch.bfloat16 and launch.round_each_op
    vals = _evaluate(launch.inputs, launch.ops, tensors, torch.arange(row0, row0 + nrows),
                     torch.arange(col0, col0 + ncols), rnd, getattr(launch, "imms", ()))
    dims = list(launch.dims)
    res = vals.sum(dim=dims, keepdim=True) if launch.op == "sum" else vals.amax(dim=dims, keepdim=True)
    if launch.scaler is not None:
        si, srow, scol = launch.scaler
        res = res * tensors[si][srow, scol].to(torch.float32)
    orow = 0 if out.shape[0] == 1 else launch.rect[0] * TILE
    ocol = 0 if out.shape[1] == 1 else launch.rect[2] * TILE
    fill_r = (1 if out.shape[0] == 1 else TILE) if 0 in dims else nrows
    fill_c = (1 if out.shape[1] == 1 else TILE) if 1 in dims else ncols
    block = torch.zeros(fill_r, fill_c)
    block[:res.shape[0], :res.shape[1]] = res
    out[orow:orow + fill_r, ocol:ocol + fill_c] = block.to(out.dtype)


def run_gemm(launch: Any, tensors: Sequence[torch.Tensor]) -> None:
    a, b, out = tensors[launch.a_index], tensors[launch.b_index], tensors[launch.out_index]
    r0, r1, c0, c1 = (x * TILE for x in launch.rect)
    bias = None
    if launch.bias_index is not None:
        bt = tensors[launch.bias_index]
        bias = bt[:, c0:c1] if (bt.shape[0] == 1 and out.shape[0] != 1) else bt[r0:r1, c0:c1]   # one row, or a matrix
    act = getattr(launch, "act", None)
    if act is None:
        mode = "native" if out.dtype == torch.float32 else "f32"
        out[r0:r1, c0:c1] = tile_oracle.matmul_tiles(a[r0:r1], b[:, c0:c1], mode, bias=bias).to(out.dtype)
        return
    # bias and activation in the GEMM epilogue: on the fp32 accumulators, one rounding
    acc = tile_oracle.matmul_tiles(a[r0:r1].float(), b[:, c0:c1].float(), "native", bias=None if bias is None else bias.float())
    out[r0:r1, c0:c1] = _UNARY[act](acc).to(out.dtype)


class _WithTemps:
    """The call's tensors plus the plan's temporaries (indices from 1000 on name temporaries)."""

    def __init__(self, tensors: Sequence[torch.Tensor], temps: Sequence[torch.Tensor]):
        self.tensors, self.temps = list(tensors), list(temps)

    def __getitem__(self, i: int) -> torch.Tensor:
        return self.temps[i - 1000] if i >= 1000 else self.tensors[i]


def run_plan(plan: Any, tensors: Sequence[torch.Tensor]) -> None:
    """Evaluate the launches in order.  `tensors`: the call's arguments followed by the plan's extras, as
    host torch tensors; temporaries of the plan are replaced by host tensors of the same shape."""
    temps = getattr(plan, "temps", None)
    if temps:
        tensors = _WithTemps(tensors, [torch.zeros(t._tensor.shape, dtype=t._tensor.dtype) for t in temps])  # type: ignore[assignment]
    for launch in plan.launches:
        if hasattr(launch, "parts"):      # row-fused: the same stages, one after the other
            for part in launch.parts:
                run_reduce(part, tensors)
            run_eltwise(launch.final, tensors)
        elif hasattr(launch, "extent"):
            run_reduce(launch, tensors)
        else:
            (run_eltwise if hasattr(launch, "ops") else run_gemm)(launch, tensors)
