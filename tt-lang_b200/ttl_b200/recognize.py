"""From the trace of a tile program to GPU launches.

The reference decides what can be fused into one compute kernel by walking the IR:
a chain is fusable when every leaf comes straight from a circular buffer and every
interior node is an element-wise op or a broadcast of such a leaf
(lib/Dialect/TTL/IR/TTLOpsUtils.cpp:9-63, lib/Dialect/TTL/Transforms/ConvertTTLToCompute.cpp:113-229).
The trace already has that shape: every write is `output region <- expression over
input regions`.  Two families are recognised:

  * element-wise / broadcast expressions -> one `ttlb_eltwise` launch per maximal
    output rectangle sharing the same expression and operand addressing;
  * `out <- sum_k A[rows, k] @ B[k, cols]` over all K tiles -> a GEMM launch
    (block forms (1,1)@(1,1) and (M,1)@(1,N) only: those are the ones that mean a block
    matmul in the simulator, python/sim/block.py:870-920, 1012-1013).

Anything else raises Unsupported: there is no CPU fallback.
"""

from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import capi
from . import ttnn as _ttnn
from .trace import PROFILE, Acc, BatchedWrite, Bin, Expr, Leaf, Red, Rep, Trace, Un, Write, Zero

TILE = 32


class Unsupported(NotImplementedError):
    """The tile program is valid tt-lang but not (yet) runnable on the B200 backend."""


_REVERSE = {"add": "add", "mul": "mul", "max": "max", "min": "min", "sub": "rsub", "div": "rdiv",
            "floordiv": "rfloordiv", "mod": "rmod", "pow": "rpow"}
_UNARY = {"exp", "log", "sqrt", "rsqrt", "tanh", "sigmoid", "neg", "abs", "relu",
          "exp2", "expm1", "logp1", "square", "recip", "tan", "atan", "atanh", "sin", "asin", "asinh", "cos", "acos",
          "acosh", "gelu", "silu", "softsign", "hardsigmoid"} | set(capi.IMM_PARAMS)
_BINARY = {"add", "sub", "mul", "div", "max", "min", "floordiv", "mod", "pow"}


# --------------------------------------------------------------------------- #
# helpers
# --------------------------------------------------------------------------- #
def merge_rects(rects: Sequence[Tuple[int, int, int, int]]) -> List[Tuple[int, int, int, int]]:
    """Merge tile rectangles (r0, r1, c0, c1) that touch along a full edge."""
    cur = list(rects)
    while True:
        n = len(cur)
        cur.sort(key=lambda r: (r[0], r[1], r[2]))
        out: List[Tuple[int, int, int, int]] = []
        for r in cur:
            if out and out[-1][0] == r[0] and out[-1][1] == r[1] and out[-1][3] == r[2]:
                out[-1] = (r[0], r[1], out[-1][2], r[3])
            else:
                out.append(r)
        out.sort(key=lambda r: (r[2], r[3], r[0]))
        cur = []
        for r in out:
            if cur and cur[-1][2] == r[2] and cur[-1][3] == r[3] and cur[-1][1] == r[0]:
                cur[-1] = (cur[-1][0], r[1], r[2], r[3])
            else:
                cur.append(r)
        if len(cur) == n:
            return sorted(cur)


def _lines_of(w: Write) -> List[Tuple[str, int]]:
    """Program lines (file, line) that made write `w`: the copy to the output tensor and every op, reduction,
    accumulating store and copy-in of its expression (recorded while profiling is on)."""
    seen: Dict[int, None] = {}
    lines: Dict[Tuple[str, int], None] = {}
    if w.line is not None:
        lines[w.line] = None
    stack = [w.expr]
    while stack:
        x = stack.pop()
        if id(x) in seen:
            continue
        seen[id(x)] = None
        ln = getattr(x, "line", None)
        if ln is not None:
            lines[ln] = None
        if isinstance(x, Bin):
            stack += [x.a, x.b]
        elif isinstance(x, Un):
            stack.append(x.x)
        elif isinstance(x, Acc):
            stack.extend(x.terms)
        elif isinstance(x, Rep):
            stack.append(x.x)
        elif isinstance(x, Red):
            stack.append(x.x)
            if x.scaler is not None:
                stack.append(x.scaler)
    return list(lines)


def _contains_matmul(e: Expr) -> bool:
    stack = [e]
    while stack:
        x = stack.pop()
        if isinstance(x, Bin):
            if x.op == "matmul":
                return True
            stack.append(x.a)
            stack.append(x.b)
        elif isinstance(x, (Un, Rep)):
            stack.append(x.x)
        elif isinstance(x, Acc):
            stack.extend(x.terms)
    return False


def _expand_runs(e: Expr) -> Expr:
    """`e` with every run of accumulated terms (trace.Rep, made by batched loops) written out term by term."""
    if isinstance(e, Acc):
        terms: List[Expr] = []
        changed = False
        for t in e.terms:
            if isinstance(t, Rep):
                terms.extend(_expand_runs(x) for x in t.terms())
                changed = True
            else:
                n = _expand_runs(t)
                changed = changed or n is not t
                terms.append(n)
        if not changed:
            return e
        r: Expr = Acc(terms, e.shape)
    elif isinstance(e, Un):
        x = _expand_runs(e.x)
        if x is e.x:
            return e
        r = Un(e.op, x, e.params)
    elif isinstance(e, Bin):
        a, b = _expand_runs(e.a), _expand_runs(e.b)
        if a is e.a and b is e.b:
            return e
        r = Bin(e.op, a, b, e.shape)
    elif isinstance(e, Red):
        x = _expand_runs(e.x)
        sc = _expand_runs(e.scaler) if e.scaler is not None else None
        if x is e.x and sc is e.scaler:
            return e
        r = Red(e.op, x, sc, e.dims)
    elif isinstance(e, Rep):   # a run outside an accumulation cannot be made; keep the first term's meaning explicit
        r = Acc([_expand_runs(x) for x in e.terms()], e.shape)
    else:
        return e
    if getattr(e, "line", None) is not None:
        r.line = e.line
    return r


def _has_run(e: Expr) -> bool:
    stack = [e]
    while stack:
        x = stack.pop()
        if isinstance(x, Rep):
            return True
        if isinstance(x, Bin):
            stack += [x.a, x.b]
        elif isinstance(x, Un):
            stack.append(x.x)
        elif isinstance(x, Acc):
            stack.extend(x.terms)
        elif isinstance(x, Red):
            stack.append(x.x)
    return False


def _plain_matmul(t: Expr) -> bool:
    """`a_blk @ b_blk` with both operands straight from circular buffers, or a run of such terms."""
    if isinstance(t, Rep):
        t = t.x
    return isinstance(t, Bin) and t.op == "matmul" and isinstance(_unwrap(t.a), Leaf) and isinstance(_unwrap(t.b), Leaf)


TEMP_BASE = 1000   # tensor indices from here on name temporaries owned by the plan


class _Indexed:
    """Kernel arguments (+ tensors derived in the kernel body) and the plan's temporaries under one index space."""

    def __init__(self, tensors: Sequence[Any], temps: Sequence[Any]):
        self.tensors, self.temps = list(tensors), list(temps)

    def __getitem__(self, i: int) -> Any:
        return self.temps[i - TEMP_BASE] if i >= TEMP_BASE else self.tensors[i]

    def __len__(self) -> int:
        return len(self.tensors)


class _TensorTable:
    """Maps tensor objects of a trace to kernel-argument positions."""

    def __init__(self, args: Sequence[_ttnn.Tensor]):
        self.args = list(args)
        self.extras: List[_ttnn.Tensor] = []
        self.temps: List[_ttnn.Tensor] = []

    def tensor(self, i: int) -> _ttnn.Tensor:
        if i >= TEMP_BASE:
            return self.temps[i - TEMP_BASE]
        return self.args[i] if i < len(self.args) else self.extras[i - len(self.args)]

    def new_temp(self, shape: Tuple[int, int], like: _ttnn.Tensor) -> _ttnn.Tensor:
        t = _ttnn.Tensor(torch.zeros(shape, dtype=like._tensor.dtype, device=like._tensor.device))
        self.temps.append(t)
        return t

    def index(self, t: _ttnn.Tensor) -> int:
        for i, a in enumerate(self.temps):
            if a is t:
                return TEMP_BASE + i
        for i, a in enumerate(self.args):
            if a is t:
                return i
        for i, a in enumerate(self.extras):
            if a is t:
                return len(self.args) + i
        self.extras.append(t)
        return len(self.args) + len(self.extras) - 1


# --------------------------------------------------------------------------- #
# element-wise linearisation
# --------------------------------------------------------------------------- #
def _classify(leaf: Leaf, w: Write) -> Tuple[int, int, int, int]:
    """Index modes and element offsets of `leaf` relative to the write region `w`."""
    t = leaf.tensor
    trows, tcols = t.shape
    tt = t.tile_shape()
    res = []
    for (lo, hi, wlo, whi, n_elem, n_tiles, first) in (
            (leaf.r0, leaf.r1, w.r0, w.r1, trows, tt[0], leaf.first[0]),
            (leaf.c0, leaf.c1, w.c0, w.c1, tcols, tt[1], leaf.first[1])):
        if n_elem == 1:
            res += [capi.IDX_ZERO, 0]
        elif n_tiles == 1 or (hi - lo == 1 and whi - wlo > 1):
            # one tile repeated over the region; with `first`, its row / column 0 only
            res += [capi.IDX_ZERO if first else capi.IDX_TILE, lo * TILE]
        elif hi - lo == whi - wlo:
            res += [capi.IDX_FIRST if first else capi.IDX_SAME, (lo - wlo) * TILE]
        else:
            raise Unsupported(f"operand region {hi - lo} tiles does not line up with output region {whi - wlo} tiles")
    return res[0], res[1], res[2], res[3]


def _need(e: Expr) -> int:
    if isinstance(e, Leaf):
        return 0
    if isinstance(e, Un):
        return _need(e.x)
    if isinstance(e, Bin):
        if isinstance(e.b, Leaf):
            return _need(e.a)
        if isinstance(e.a, Leaf):
            return _need(e.b)
        na, nb = _need(e.a), _need(e.b)
        return min(max(na, nb + 1), max(nb, na + 1))
    raise Unsupported(f"cannot lower {type(e).__name__}")


class _Lin:
    def __init__(self, w: Write, table: _TensorTable):
        self.w, self.table = w, table
        self.inputs: List[Tuple[int, int, int, int, int]] = []
        self.ops: List[Tuple[str, int]] = []
        self.imms: List[float] = []    # scalar parameters of functions such as leaky_relu, in op order

    def slot(self, leaf: Leaf) -> int:
        rm, ro, cm, co = _classify(leaf, self.w)
        key = (self.table.index(leaf.tensor), rm, ro, cm, co)
        if key in self.inputs:
            return self.inputs.index(key)
        self.inputs.append(key)
        return len(self.inputs) - 1

    def emit(self, e: Expr) -> None:
        if isinstance(e, Acc):
            # sequential sum, each partial held in the block dtype
            self.emit(e.terms[0])
            for t in e.terms[1:]:
                self._bin_rhs("add", t)
            return
        if isinstance(e, Leaf):
            self.ops.append(("load", self.slot(e)))
        elif isinstance(e, Un):
            if e.op not in _UNARY:
                raise Unsupported(f"unary op {e.op}")
            self.emit(e.x)
            if e.op in capi.IMM_PARAMS:
                if len(e.params) != capi.IMM_PARAMS[e.op]:
                    raise Unsupported(f"{e.op} takes {capi.IMM_PARAMS[e.op]} scalar parameter(s)")
                if len(self.imms) + len(e.params) > capi.TTLB_MAX_IMM:
                    raise Unsupported(f"expression has more than {capi.TTLB_MAX_IMM} scalar parameters")
                self.ops.append((e.op, len(self.imms)))
                self.imms.extend(e.params)
            else:
                self.ops.append((e.op, 0))
        elif isinstance(e, Bin):
            if e.op not in _BINARY:
                raise Unsupported(f"binary op {e.op} inside an element-wise expression")
            a, b = _unwrap(e.a), _unwrap(e.b)
            if isinstance(b, Leaf):
                self.emit(a)
                self.ops.append((e.op, self.slot(b)))
            elif isinstance(a, Leaf):
                self.emit(b)
                self.ops.append((_REVERSE[e.op], self.slot(a)))
            elif _need(b) > _need(a):
                self.emit(b)
                self.ops.append(("push", 0))
                self.emit(a)
                self.ops.append((e.op, capi.TTLB_ARG_STACK))          # acc = a, popped = b
            else:
                self.emit(a)
                self.ops.append(("push", 0))
                self.emit(b)
                self.ops.append((_REVERSE[e.op], capi.TTLB_ARG_STACK))  # acc = b, popped = a
        elif isinstance(e, Zero):
            raise Unsupported("reading a reserved block that was never written")
        else:
            raise Unsupported(f"cannot lower {type(e).__name__}")

    def _bin_rhs(self, op: str, rhs: Expr) -> None:
        rhs = _unwrap(rhs)
        if isinstance(rhs, Leaf):
            self.ops.append((op, self.slot(rhs)))
        else:
            self.ops.append(("push", 0))
            self.emit(rhs)
            self.ops.append((_REVERSE[op], capi.TTLB_ARG_STACK))


def _unwrap(e: Expr) -> Expr:
    if isinstance(e, Acc) and len(e.terms) == 1:
        return _unwrap(e.terms[0])
    return e


def _stack_depth(ops: Sequence[Tuple[str, int]]) -> int:
    d = m = 0
    for op, arg in ops:
        if op == "push":
            d += 1
            m = max(m, d)
        elif arg == capi.TTLB_ARG_STACK:
            d -= 1
    return m


# --------------------------------------------------------------------------- #
# launches
# --------------------------------------------------------------------------- #
def _torch_of(t: _ttnn.Tensor) -> torch.Tensor:
    x = t._tensor
    if not x.is_cuda:
        raise capi.BackendError(capi.TTLB_ERR_CUDA,
                                "tensor is not in GPU memory: the B200 backend has no CPU fallback")
    if x.dim() != 2 or (x.shape[1] > 1 and x.stride(1) != 1):
        raise Unsupported("tensors must be 2-D with unit column stride")
    return x


def _dtype_code(dt: Any) -> int:
    if dt == torch.bfloat16:
        return capi.TTLB_BF16
    if dt == torch.float32:
        return capi.TTLB_F32
    raise Unsupported(f"element type {dt} (bfloat16 and float32 only)")


class EltwiseLaunch:
    def __init__(self, out_index: int, rect: Tuple[int, int, int, int], inputs: List[Tuple[int, int, int, int, int]],
                 ops: List[Tuple[str, int]], dtype: Any, round_each_op: bool, out_degenerate: Tuple[bool, bool],
                 imms: Sequence[float] = ()):
        self.imms = tuple(imms)
        self.out_index, self.rect, self.inputs, self.ops = out_index, rect, inputs, ops
        self.dtype, self.round_each_op, self.out_degenerate = dtype, round_each_op, out_degenerate

    def describe(self) -> Dict[str, Any]:
        d = {"kind": "eltwise", "out": self.out_index, "rect_tiles": self.rect, "inputs": self.inputs,
             "ops": self.ops, "round_each_op": self.round_each_op}
        if self.imms:
            d["imm"] = list(self.imms)
        return d

    def desc(self, tensors: Sequence[_ttnn.Tensor]) -> capi.EltwiseDesc:
        d = capi.EltwiseDesc()
        d.dtype = _dtype_code(self.dtype)
        d.round_each_op = 1 if self.round_each_op else 0
        d.n_in, d.n_ops = len(self.inputs), len(self.ops)
        for k, (ti, rm, ro, cm, co) in enumerate(self.inputs):
            x = _torch_of(tensors[ti])
            d.inp[k].ptr = x.data_ptr()
            d.inp[k].ld = x.stride(0) if x.shape[0] > 1 else x.shape[1]
            d.inp[k].row_mode, d.inp[k].row_off = rm, ro
            d.inp[k].col_mode, d.inp[k].col_off = cm, co
        for k, (op, arg) in enumerate(self.ops):
            d.ops[k].opcode, d.ops[k].arg = capi.OPCODES[op], arg
        for k, v in enumerate(self.imms):
            d.imm[k] = v
        o = _torch_of(tensors[self.out_index])
        d.out = o.data_ptr()
        d.out_ld = o.stride(0) if o.shape[0] > 1 else o.shape[1]
        r0, r1, c0, c1 = self.rect
        d.row0, d.rows = (0, 1) if self.out_degenerate[0] else (r0 * TILE, (r1 - r0) * TILE)
        d.col0, d.cols = (0, 1) if self.out_degenerate[1] else (c0 * TILE, (c1 - c0) * TILE)
        return d

    def desc_cpu(self, tensors: Sequence[_ttnn.Tensor]) -> capi.EltwiseDesc:
        """The descriptor with pitches and modes filled in but no device pointers (for translation)."""
        d = capi.EltwiseDesc()
        d.dtype = _dtype_code(self.dtype)
        d.round_each_op = 1 if self.round_each_op else 0
        d.n_in, d.n_ops = len(self.inputs), len(self.ops)
        for k, (ti, rm, ro, cm, co) in enumerate(self.inputs):
            x = tensors[ti]._tensor
            d.inp[k].ld = x.stride(0) if x.shape[0] > 1 else x.shape[1]
            d.inp[k].row_mode, d.inp[k].row_off = rm, ro
            d.inp[k].col_mode, d.inp[k].col_off = cm, co
        for k, (op, arg) in enumerate(self.ops):
            d.ops[k].opcode, d.ops[k].arg = capi.OPCODES[op], arg
        for k, v in enumerate(self.imms):
            d.imm[k] = v
        o = tensors[self.out_index]._tensor
        d.out_ld = o.stride(0) if o.shape[0] > 1 else o.shape[1]
        r0, r1, c0, c1 = self.rect
        d.row0, d.rows = (0, 1) if self.out_degenerate[0] else (r0 * TILE, (r1 - r0) * TILE)
        d.col0, d.cols = (0, 1) if self.out_degenerate[1] else (c0 * TILE, (c1 - c0) * TILE)
        return d

    def run(self, ctx: capi.Context, tensors: Sequence[_ttnn.Tensor], stream: int) -> None:
        ctx.eltwise(self.desc(tensors), stream)


class ReduceLaunch:
    """One `ttlb_reduce` launch: `inputs`/`ops` produce the values (offsets along a reduced dim are absolute,
    along a kept dim relative to the output rectangle), `extent` is the number of tiles reduced per dim."""

    def __init__(self, out_index: int, rect: Tuple[int, int, int, int], op: str, dims: Tuple[int, ...],
                 extent: Tuple[int, int], inputs: List[Tuple[int, int, int, int, int]], ops: List[Tuple[str, int]],
                 scaler: Optional[Tuple[int, int, int]], dtype: Any, round_each_op: bool, imms: Sequence[float] = ()):
        self.imms = tuple(imms)
        self.out_index, self.rect, self.op, self.dims, self.extent = out_index, rect, op, dims, extent
        self.inputs, self.ops, self.scaler, self.dtype, self.round_each_op = inputs, ops, scaler, dtype, round_each_op

    def describe(self) -> Dict[str, Any]:
        return {"kind": "reduce_" + self.op, "dims": list(self.dims), "out": self.out_index, "rect_tiles": self.rect,
                "reduced_tiles": self.extent, "inputs": self.inputs, "ops": self.ops, "scaler": self.scaler,
                "round_each_op": self.round_each_op, "imm": list(self.imms)}

    def region(self) -> Tuple[int, int, int, int]:
        """(row0, rows, col0, cols) of the values reduced, in elements of the program's index space."""
        r0, r1, c0, c1 = self.rect
        rows = (0, self.extent[0] * TILE) if 0 in self.dims else (r0 * TILE, (r1 - r0) * TILE)
        cols = (0, self.extent[1] * TILE) if 1 in self.dims else (c0 * TILE, (c1 - c0) * TILE)
        return rows[0], rows[1], cols[0], cols[1]

    def desc(self, tensors: Sequence[_ttnn.Tensor], with_pointers: bool = True) -> capi.ReduceDesc:
        r = capi.ReduceDesc()
        d = r.src
        d.dtype = _dtype_code(self.dtype)
        d.round_each_op = 1 if self.round_each_op else 0
        d.n_in, d.n_ops = len(self.inputs), len(self.ops)
        for k, (ti, rm, ro, cm, co) in enumerate(self.inputs):
            x = _torch_of(tensors[ti]) if with_pointers else tensors[ti]._tensor
            if with_pointers:
                d.inp[k].ptr = x.data_ptr()
            d.inp[k].ld = x.stride(0) if x.shape[0] > 1 else x.shape[1]
            d.inp[k].row_mode, d.inp[k].row_off = rm, ro
            d.inp[k].col_mode, d.inp[k].col_off = cm, co
        for k, (op, arg) in enumerate(self.ops):
            d.ops[k].opcode, d.ops[k].arg = capi.OPCODES[op], arg
        for k, v in enumerate(self.imms):
            d.imm[k] = v
        d.row0, d.rows, d.col0, d.cols = self.region()
        r.op = capi.REDUCE_SUM if self.op == "sum" else capi.REDUCE_MAX
        r.dims = (capi.REDUCE_ROWS if 0 in self.dims else 0) | (capi.REDUCE_COLS if 1 in self.dims else 0)
        o = _torch_of(tensors[self.out_index]) if with_pointers else tensors[self.out_index]._tensor
        esz = o.element_size()
        r.out_ld = o.stride(0) if o.shape[0] > 1 else o.shape[1]
        orow = 0 if o.shape[0] == 1 else self.rect[0] * TILE
        ocol = 0 if o.shape[1] == 1 else self.rect[2] * TILE
        r.fill_rows = 1 if o.shape[0] == 1 else TILE
        r.fill_cols = 1 if o.shape[1] == 1 else TILE
        if with_pointers:
            r.out = o.data_ptr() + (orow * r.out_ld + ocol) * esz
            if self.scaler is not None:
                si, srow, scol = self.scaler
                st = _torch_of(tensors[si])
                r.scaler = st.data_ptr() + (srow * (st.stride(0) if st.shape[0] > 1 else 0) + scol) * esz
        return r

    def run(self, ctx: capi.Context, tensors: Sequence[_ttnn.Tensor], stream: int) -> None:
        ctx.reduce(self.desc(tensors), stream)


ROW_FUSION = os.environ.get("TTLB200_ROW_FUSION", "1") != "0"
MAX_FUSED_VECTORS_PER_ROW = 2048


def set_row_fusion(enabled: bool) -> None:
    """Whether reductions over columns and the element-wise launch that consumes them are merged into one
    row-resident kernel (default on).  Affects plans built afterwards."""
    global ROW_FUSION
    ROW_FUSION = bool(enabled)


class RowFusedLaunch:
    """Reductions over columns (`parts`) and the element-wise launch (`final`) that reads their results,
    all over the same rows, as ONE `ttlb_rowfused` launch: every operand row is read once and held on chip;
    the reduction results never reach memory."""

    lines: Dict[Any, int] = {}

    def __init__(self, parts: List[ReduceLaunch], final: EltwiseLaunch):
        self.parts, self.final = parts, final
        self.out_index, self.rect = final.out_index, final.rect
        self._unfused = False

    def describe(self) -> Dict[str, Any]:
        return {"kind": "row_fused", "out": self.out_index, "rect_tiles": self.rect,
                "phases": [p.describe() for p in self.parts], "final": self.final.describe()}

    def _patch(self, d: capi.EltwiseDesc, inputs: Sequence[Tuple[int, int, int, int, int]]) -> None:
        produced = {p.out_index: i for i, p in enumerate(self.parts)}
        for k, (ti, *_rest) in enumerate(inputs):
            if ti in produced:
                d.inp[k].ptr = None
                d.inp[k].row_mode, d.inp[k].row_off = capi.IDX_PHASE, produced[ti]
                d.inp[k].col_mode, d.inp[k].col_off = capi.IDX_ZERO, 0

    def desc(self, tensors: Sequence[_ttnn.Tensor], with_pointers: bool = True) -> capi.RowFusedDesc:
        f = capi.RowFusedDesc()
        f.n_phases = len(self.parts)
        for i, p in enumerate(self.parts):
            rd = p.desc(tensors, with_pointers)
            rd.out = None          # the result is consumed on chip; the temporary is not written
            self._patch(rd.src, p.inputs)
            f.phase[i] = rd
        fd = self.final.desc(tensors) if with_pointers else self.final.desc_cpu(tensors)
        self._patch(fd, self.final.inputs)
        f.final = fd
        return f

    def run(self, ctx: capi.Context, tensors: Sequence[_ttnn.Tensor], stream: int) -> None:
        if not self._unfused:
            try:
                ctx.rowfused(self.desc(tensors), stream)
                return
            except capi.BackendError as e:
                if e.code != capi.TTLB_ERR_UNSUPPORTED:
                    raise
                self._unfused = True   # e.g. the operand rows do not fit in registers: launch by launch
        for p in self.parts:
            p.run(ctx, tensors, stream)
        self.final.run(ctx, tensors, stream)


def _fuse_epilogues(launches: List[Any]) -> List[Any]:
    """With fp32 intermediates: [bf16 GEMM into a temporary] + [element-wise launch over the same rectangle that
    only adds a bias (full matrix or one row) and/or applies an activation the GEMM epilogue knows] becomes the GEMM
    alone, with bias and activation applied to its fp32 accumulators before the one rounding."""
    readers: Dict[int, int] = {}
    for l in launches:
        for (ti, *_r) in getattr(l, "inputs", []):
            readers[ti] = readers.get(ti, 0) + 1
    out: List[Any] = []
    gone: Dict[int, None] = {}
    gemm_of = {l.out_index: l for l in launches if isinstance(l, GemmLaunch) and l.out_index >= TEMP_BASE}
    for l in launches:
        g = None
        if isinstance(l, EltwiseLaunch) and not l.round_each_op and l.dtype == torch.bfloat16 and 1 <= len(l.inputs) <= 2:
            temps_read = [k for k, inp in enumerate(l.inputs) if inp[0] in gemm_of]
            if len(temps_read) == 1:
                g = gemm_of[l.inputs[temps_read[0]][0]]
        ok = (g is not None and g.kind == "matmul_bf16" and g.bias_index is None and g.act is None
              and g.rect == l.rect and readers.get(g.out_index, 0) == 1 and not l.imms)
        bias = act = None
        if ok:
            t = temps_read[0]
            ok = l.inputs[t][1:] == (capi.IDX_SAME, 0, capi.IDX_SAME, 0)
            ops = list(l.ops)
            if ok and len(l.inputs) == 2:
                v = 1 - t
                ti, rm, ro, cm, co = l.inputs[v]
                # p + v or v + p, v a full matrix of the output's shape or one row
                ok = (ops[:2] in ([("load", t), ("add", v)], [("load", v), ("add", t)]) and (cm, co) == (capi.IDX_SAME, 0)
                      and ((rm, ro) == (capi.IDX_SAME, 0) or rm == capi.IDX_ZERO and ro == 0) and ti < TEMP_BASE)
                bias, ops = ti, ops[2:]
            elif ok:
                ok = ops[:1] == [("load", t)]
                ops = ops[1:]
            if ok and ops:
                ok = len(ops) == 1 and ops[0][0] in capi.ACTIVATIONS
                act = ops[0][0] if ok else None
            ok = ok and (bias is not None or act is not None)
        if not ok:
            out.append(l)
            continue
        fused = GemmLaunch(g.a_index, g.b_index, l.out_index, g.rect, g.k_tiles, g.b_is_bfp8, bias, act)
        fused.lines = {**(getattr(g, "lines", None) or {}), **(getattr(l, "lines", None) or {})}
        gone[id(g)] = None
        out.append(fused)
    return [l for l in out if id(l) not in gone]


def _fuse_rows(launches: List[Any]) -> List[Any]:
    """Merge [reductions over columns into temporaries] + [the element-wise launch that reads them] into
    RowFusedLaunch where every launch covers the same rows and full row length, and the temporaries have no
    other reader."""
    readers: Dict[int, int] = {}
    for l in launches:
        for (ti, *_r) in getattr(l, "inputs", []):
            if ti >= TEMP_BASE:
                readers[ti] = readers.get(ti, 0) + 1
        for attr in ("a_index", "b_index", "bias_index"):
            ti = getattr(l, attr, None)
            if ti is not None and ti >= TEMP_BASE:
                readers[ti] = readers.get(ti, 0) + 100   # read by a matmul: never fused away
    producer = {l.out_index: l for l in launches if isinstance(l, ReduceLaunch) and l.out_index >= TEMP_BASE}
    gone: Dict[int, None] = {}
    out: List[Any] = []
    for l in launches:
        if not isinstance(l, EltwiseLaunch) or l.out_degenerate != (False, False):
            out.append(l)
            continue
        r0, r1, c0, c1 = l.rect
        group: List[ReduceLaunch] = []
        inside: Dict[int, int] = {}
        ok = True

        def visit(inputs: Sequence[Tuple[int, int, int, int, int]]) -> None:
            nonlocal ok
            for (ti, rm, ro, cm, co) in inputs:
                if ti < TEMP_BASE or not ok:
                    continue
                p = producer.get(ti)
                if p is None:
                    continue     # a temporary filled by another kind of launch (a matmul): an ordinary operand here
                inside[ti] = inside.get(ti, 0) + 1
                if (p.dims != (1,) or p.rect != (r0, r1, 0, 1) or c0 != 0 or p.extent[1] != c1
                        or (rm, ro, cm, co) != (capi.IDX_SAME, 0, capi.IDX_ZERO, 0) or p.dtype != l.dtype
                        or p.round_each_op != l.round_each_op):
                    ok = False
                    return
                if p not in group:
                    visit(p.inputs)
                    group.append(p)

        visit(l.inputs)
        vec = 8 if l.dtype == torch.bfloat16 else 4
        if (not ok or not group or len(group) > capi.TTLB_MAX_PHASES or (c1 - c0) * TILE // vec > MAX_FUSED_VECTORS_PER_ROW
                or any(readers.get(ti, 0) != n for ti, n in inside.items())):
            out.append(l)
            continue
        for p in group:
            gone[id(p)] = None
        fused = RowFusedLaunch(group, l)
        lines: Dict[Any, int] = {}
        for part in group + [l]:
            for ln, n in (getattr(part, "lines", None) or {}).items():
                lines[ln] = lines.get(ln, 0) + n
        fused.lines = lines
        out.append(fused)
    return [l for l in out if id(l) not in gone]


class GemmLaunch:
    lines: Dict[Any, int] = {}

    def __init__(self, a_index: int, b_index: int, out_index: int, rect: Tuple[int, int, int, int], k_tiles: int,
                 b_is_bfp8: bool, bias_index: Optional[int] = None, act: Optional[str] = None):
        self.a_index, self.b_index, self.out_index, self.rect = a_index, b_index, out_index, rect
        # b_is_bfp8: 0 for plain weights, else the bits per value of the block-float tiles (8: bfloat8_b, 4: bfloat4_b)
        self.k_tiles, self.b_is_bfp8, self.bias_index = k_tiles, b_is_bfp8, bias_index
        self.act = act    # activation applied in the GEMM epilogue (fused from a following element-wise launch)
        self.kind = "matmul_bf16"   # set to "matmul_f32" by the recogniser for float32 programs

    def describe(self) -> Dict[str, Any]:
        d = {"kind": ("matmul_bfp4w" if self.b_is_bfp8 == 4 else "matmul_bfp8w") if self.b_is_bfp8 else self.kind, "a": self.a_index, "b": self.b_index,
             "out": self.out_index, "rect_tiles": self.rect, "k_tiles": self.k_tiles}
        if self.bias_index is not None:
            d["bias"] = self.bias_index
        if self.act is not None:
            d["act"] = self.act
        return d

    def run(self, ctx: capi.Context, tensors: Sequence[_ttnn.Tensor], stream: int) -> None:
        from . import ops

        r0, r1, c0, c1 = self.rect
        ops.launch_gemm(ctx, tensors[self.a_index], tensors[self.b_index], tensors[self.out_index],
                        (r0 * TILE, r1 * TILE, c0 * TILE, c1 * TILE), stream,
                        bias=None if self.bias_index is None else tensors[self.bias_index],
                        act=capi.ACTIVATIONS[self.act] if self.act else 0)


def _read_span(mode: int, off: int, lo: int, hi: int) -> Tuple[int, int]:
    """Elements [a, b) an operand reads along one dim for an output range of tiles [lo, hi)."""
    if mode in (capi.IDX_SAME, capi.IDX_FIRST):
        return lo * TILE + off, hi * TILE + off
    if mode == capi.IDX_TILE:
        return off, off + TILE
    return off, off + 1      # IDX_ZERO: one fixed row / column


def _check_hazards(launches: Sequence[Any]) -> None:
    """A plan's launches run as parallel kernels, ordered only where one reads a temporary another fills.  A
    program that reads tiles of a tensor it also writes (a shifted copy `t[i+1] = t[i] + b`, a read-back of a tile it
    stored, A or B of a matmul aliasing its output) would depend on an order the plan does not keep: refused.
    The one exception is an element-wise launch that reads exactly the elements it writes (in-place update)."""
    written: Dict[int, List[Tuple[int, int, int, int]]] = {}
    for l in launches:
        if l.out_index < TEMP_BASE:
            written.setdefault(l.out_index, []).append(l.rect)
    if not written:
        return

    def clash(what: str) -> Unsupported:
        return Unsupported(f"the program {what} a tensor it also writes; the launches of a plan run in parallel, so "
                           "the result would depend on their order")

    for l in launches:
        if isinstance(l, EltwiseLaunch):
            r0, r1, c0, c1 = l.rect
            for (ti, rm, ro, cm, co) in l.inputs:
                if ti not in written:
                    continue
                def same_place(mode: int, off: int, lo: int, hi: int) -> bool:
                    # element for element: SAME without a shift, or "one tile repeated" over a range of one tile
                    return (mode == capi.IDX_SAME and off == 0) or (mode == capi.IDX_TILE and hi - lo == 1 and off == lo * TILE)

                in_place = same_place(rm, ro, r0, r1) and same_place(cm, co, c0, c1)
                ra, rb = _read_span(rm, ro, r0, r1)
                ca, cb = _read_span(cm, co, c0, c1)
                for other in launches:
                    if other.out_index != ti:
                        continue
                    if other is l and in_place:
                        continue
                    o0, o1, p0, p1 = other.rect
                    if ra < o1 * TILE and o0 * TILE < rb and ca < p1 * TILE and p0 * TILE < cb:
                        raise clash("reads, at other positions, tiles of")
        else:
            parts = list(getattr(l, "parts", [])) + [getattr(l, "final", None)]
            reads = [inp[0] for part in parts if part is not None for inp in getattr(part, "inputs", [])]
            reads += [inp[0] for inp in getattr(l, "inputs", [])]
            reads += [getattr(l, a, None) for a in ("a_index", "b_index", "bias_index")]
            sc = getattr(l, "scaler", None)
            if sc is not None:
                reads.append(sc[0])
            for part in parts:
                sc = getattr(part, "scaler", None) if part is not None else None
                if sc is not None:
                    reads.append(sc[0])
            if any(ti is not None and ti in written for ti in reads):
                raise clash("reduces, or multiplies, tiles of")


def _extent(x: torch.Tensor) -> Tuple[int, int]:
    """[first byte, one past the last byte) a 2-D tensor can touch."""
    if x.numel() == 0:
        return 0, 0
    last = sum((n - 1) * st for n, st in zip(x.shape, x.stride()))
    return x.data_ptr(), x.data_ptr() + (last + 1) * x.element_size()


class Plan:
    """The launches one kernel call turns into."""

    def __init__(self, launches: List[Any], extras: List[_ttnn.Tensor], n_args: int,
                 temps: Optional[List[_ttnn.Tensor]] = None):
        self.launches, self.extras, self.n_args = launches, extras, n_args
        # results of reductions used inside larger expressions: small tensors owned by the plan
        self.temps: List[_ttnn.Tensor] = temps or []

    def indexed(self, tensors: Sequence[_ttnn.Tensor]) -> _Indexed:
        """The tensors a launch may name by index: the call's arguments, tensors derived in the kernel
        body, and the plan's temporaries."""
        return _Indexed(list(tensors) + self.extras, self.temps)

    @property
    def cacheable(self) -> bool:
        return not self.extras

    def describe(self) -> List[Dict[str, Any]]:
        return [l.describe() for l in self.launches]

    def _check_overlap(self, tensors: Sequence[_ttnn.Tensor]) -> None:
        """Two different argument tensors over the same memory (views of one storage), one of them written: the
        plan was built as if they were independent, so the call is refused."""
        outs = {l.out_index for l in self.launches if l.out_index < TEMP_BASE}
        if not outs:
            return
        spans = []
        for i, t in enumerate(tensors):
            x = t._packed if t._packed is not None else t._tensor
            spans.append(_extent(x) if x.is_cuda else (0, 0))
        for w in outs:
            if w >= len(spans):
                continue
            w0, w1 = spans[w]
            for i, (a0, a1) in enumerate(spans):
                if i != w and a0 < w1 and w0 < a1 and tensors[i] is not tensors[w]:
                    raise Unsupported(f"kernel arguments {i} and {w} share memory and argument {w} is written: the launches "
                                      "of a plan treat different arguments as independent tensors")

    def run(self, tensors: Sequence[_ttnn.Tensor]) -> None:
        allt = list(tensors) + self.extras
        dev = None
        for t in allt:
            if t._packed is not None:
                x = t._packed
            else:
                x = t._tensor
            if x.is_cuda:
                dev = x.device.index
                break
        ctx = capi.context(dev)
        stream = capi.current_stream(dev)     # of the tensors' device, which need not be the current one
        self._check_overlap(allt)
        for t in self.temps:
            if not t._tensor.is_cuda or t._tensor.device.index != dev:
                t._tensor = torch.zeros(t._tensor.shape, dtype=t._tensor.dtype, device=torch.device("cuda", dev))
        ix = _Indexed(allt, self.temps)
        if PROFILE.enabled:
            from . import profile
            profile.run_timed(self, ctx, ix, stream)
            return
        for l in self.launches:
            l.run(ctx, ix, stream)


# --------------------------------------------------------------------------- #
# plan construction
# --------------------------------------------------------------------------- #
def _matmul_terms(w: Write) -> Optional[Tuple[List[Bin], Optional[Leaf]]]:
    """The write as a block matmul: its `a @ b` terms and, for the specification's matmul with bias
    (`y.store(c, acc=True)` before the K loop, docs/sphinx/specs/TTLangSpecification.md:290-312), the
    block the accumulation starts from."""
    e = w.expr
    terms = list(e.terms) if isinstance(e, Acc) else [e]
    bias = None
    if len(terms) > 1 and isinstance(terms[0], Leaf):
        bias, terms = terms[0], terms[1:]
    if terms and all(isinstance(t.x if isinstance(t, Rep) else t, Bin) and (t.x if isinstance(t, Rep) else t).op == "matmul"
                     for t in terms):
        return terms, bias  # type: ignore[return-value]
    return None


def _reduce_terms(w: Write) -> Optional[List[Red]]:
    e = _unwrap(w.expr)
    terms = list(e.terms) if isinstance(e, Acc) else [e]
    terms = [_unwrap(t) for t in terms]
    if terms and all(isinstance(t, Red) for t in terms):
        return terms  # type: ignore[return-value]
    return None


class _Region:
    """Stand-in for a Write when operands are classified against a region that is not an output region."""

    def __init__(self, r0: int, r1: int, c0: int, c1: int):
        self.r0, self.r1, self.c0, self.c1 = r0, r1, c0, c1


def _recognise_reduce(w: Write, terms: List[Red], table: _TensorTable, oi: int, fp32_intermediates: bool) -> Any:
    """Key of a write `out_blk <- reduce(x)` or `out_blk <- sum_k reduce_sum(x_k)` (accumulating stores over
    blocks that tile the reduced extent).  Offsets along a reduced dim are absolute (the region starts at tile
    0), along a kept dim relative to the write region, so that neighbouring writes share a key and merge."""
    t0 = terms[0]
    op, dims = t0.op, t0.dims
    odt = w.tensor.dtype
    if (w.r1 - w.r0, w.c1 - w.c0) != t0.shape:
        raise Unsupported(f"reduction result of {t0.shape} tiles stored into a block of {(w.r1 - w.r0, w.c1 - w.c0)} tiles")
    for d in (0, 1):
        if d not in dims and w.tensor.shape[d] == 1:
            raise Unsupported("a reduction keeps a dimension in which the output tensor is degenerate")
    if len(terms) > 1:
        if op != "sum":
            raise Unsupported("store(acc=True) adds: only reduce_sum results can be accumulated over blocks")
        if odt != torch.float32 and not fp32_intermediates:
            raise Unsupported("accumulating reduce_sum over blocks of a bfloat16 tensor rounds every partial sum in "
                              "the simulator; run the kernel with fp32_dest_acc_en=True (fp32 partial sums, one rounding)")
    sc_key = None
    per_term = []
    for t in terms:
        if t.op != op or t.dims != dims or t.x.shape != t0.x.shape:
            raise Unsupported("accumulated reductions must be the same reduction of equal-shape blocks")
        if _contains_matmul(t.x) or _contains_red(t.x):
            raise Unsupported("a reduction of a matmul, or accumulated reductions of reductions, are not supported yet")
        k = None
        if t.scaler is not None:
            sl = _unwrap(t.scaler)
            if not isinstance(sl, Leaf):
                raise Unsupported("the scaler of a reduction must come straight from a circular buffer")
            st = sl.tensor
            if st.dtype != odt:
                raise Unsupported(f"mixed element types ({st.dtype} scaler, {odt} output)")
            k = (table.index(st), 0 if st.shape[0] == 1 else sl.r0 * TILE, 0 if st.shape[1] == 1 else sl.c0 * TILE)
        if t is t0:
            sc_key = k
        elif k != sc_key:
            raise Unsupported("accumulated reductions must use the same scaler")
        rr = (0, t.x.shape[0]) if 0 in dims else (w.r0, w.r1)
        cc = (0, t.x.shape[1]) if 1 in dims else (w.c0, w.c1)
        lin = _Lin(_Region(rr[0], rr[1], cc[0], cc[1]), table)  # type: ignore[arg-type]
        lin.emit(t.x)
        per_term.append(lin)
    base = per_term[0]
    if len(base.inputs) > capi.TTLB_MAX_IN or len(base.ops) > capi.TTLB_MAX_OPS or _stack_depth(base.ops) > 2:
        raise Unsupported("the reduced expression is too large (operands, ops or temporaries)")
    for (ti, rm, _ro, cm, _co) in base.inputs:
        t = table.tensor(ti)
        if t.dtype != odt:
            raise Unsupported(f"mixed element types ({t.dtype} operand, {odt} output)")
    for d, name in ((0, "row"), (1, "column")):
        if d in dims and not any((inp[1] if d == 0 else inp[3]) in (capi.IDX_SAME, capi.IDX_TILE) for inp in base.inputs):
            raise Unsupported(f"a reduction over {name}s needs an operand that varies along them")
    # the blocks of the terms must tile a rectangle of the reduced dims
    deltas = []
    for lin in per_term:
        if lin.ops != base.ops or lin.imms != base.imms or len(lin.inputs) != len(base.inputs):
            raise Unsupported("accumulated reductions must reduce the same expression")
        dr = dc = None
        for a, b in zip(lin.inputs, base.inputs):
            if (a[0], a[1], a[3]) != (b[0], b[1], b[3]):
                raise Unsupported("accumulated reductions must reduce the same expression")
            for mode, oa, ob, which in ((a[1], a[2], b[2], 0), (a[3], a[4], b[4], 1)):
                if mode == capi.IDX_SAME:
                    cur = dr if which == 0 else dc
                    if cur is not None and cur != oa - ob:
                        raise Unsupported("operands of an accumulated reduction move by different steps")
                    if which == 0:
                        dr = oa - ob
                    else:
                        dc = oa - ob
                elif oa != ob:
                    raise Unsupported("a broadcast operand of an accumulated reduction changes between blocks")
        deltas.append((dr or 0, dc or 0))
    hr, hc = t0.x.shape[0] * TILE, t0.x.shape[1] * TILE
    mr, mc = min(d[0] for d in deltas), min(d[1] for d in deltas)
    cells = sorted(((d[0] - mr) // hr, (d[1] - mc) // hc) for d in deltas)
    nr, nc = cells[-1][0] + 1, cells[-1][1] + 1
    ok = all((d[0] - mr) % hr == 0 and (d[1] - mc) % hc == 0 for d in deltas)
    if not ok or cells != [(i, j) for i in range(nr) for j in range(nc)] or (nr > 1 and 0 not in dims) or (nc > 1 and 1 not in dims):
        raise Unsupported("the blocks of an accumulated reduction do not tile a rectangle exactly once")
    inputs = tuple((ti, rm, ro + (mr if rm == capi.IDX_SAME else 0), cm, co + (mc if cm == capi.IDX_SAME else 0))
                   for (ti, rm, ro, cm, co) in base.inputs)
    extent = (t0.x.shape[0] * nr if 0 in dims else 0, t0.x.shape[1] * nc if 1 in dims else 0)
    anchor = (w.r0 if 0 in dims else -1, w.c0 if 1 in dims else -1)
    return (oi, op, dims, extent, inputs, tuple(base.ops), sc_key, anchor, tuple(base.imms))


def _contains_red(e: Expr) -> bool:
    stack = [e]
    while stack:
        x = stack.pop()
        if isinstance(x, Red):
            return True
        if isinstance(x, Bin):
            stack += [x.a, x.b]
        elif isinstance(x, (Un, Rep)):
            stack.append(x.x)
        elif isinstance(x, Acc):
            stack.extend(x.terms)
    return False


def _lower_reductions(w: Write, table: _TensorTable, temps: Dict[Any, _ttnn.Tensor],
                      out: List[Tuple[Write, int]]) -> Tuple[Expr, int]:
    """Replace every reduction inside the expression of write `w` by a read of a temporary and append the
    write that fills the temporary to `out`, innermost first.  A reduction over columns of a block that
    spans the write's rows leaves one value per row: it goes to a [rows, 1] temporary indexed like the
    output's rows (and likewise [1, cols] for a reduction over rows), so the writes of neighbouring blocks
    fill neighbouring parts of one temporary and merge into one launch.  This is what a tile program does
    when it passes a reduction result on through a circular buffer: the value is held in a tile of the
    tensor's element type.  Returns the rewritten expression and its level (1 + the deepest temporary read)."""
    memo: Dict[int, Tuple[Expr, int]] = {}
    slot = [0]
    oi = table.index(w.tensor)

    def like(new: Expr, old: Expr) -> Expr:   # a rebuilt node keeps the program line of the node it replaces
        ln = getattr(old, "line", None)
        if ln is not None:
            new.line = ln
        return new

    def go(e: Expr) -> Tuple[Expr, int]:
        if isinstance(e, (Leaf, Zero)):
            return e, 0
        hit = memo.get(id(e))
        if hit is not None:
            return hit
        mm_terms = list(e.terms) if isinstance(e, Acc) else [e]
        if len(mm_terms) > 1 and isinstance(mm_terms[0], Leaf):
            mm_terms = mm_terms[1:]     # accumulation that starts from a bias block
        if mm_terms and all(isinstance(t, Bin) and t.op == "matmul" for t in mm_terms):
            # a block matmul whose result is used further (bias / activation epilogues): the product goes to a
            # temporary of the output's shape, in the output's element type like a block in a circular buffer
            if e.shape != (w.r1 - w.r0, w.c1 - w.c0) or 1 in w.tensor.shape:
                raise Unsupported("a matmul inside an expression must produce the block it is stored into")
            key = (oi, slot[0], "mm", ())
            slot[0] += 1
            t = temps.get(key)
            if t is None:
                t = temps[key] = table.new_temp(tuple(w.tensor.shape), w.tensor)
            lvl = _expand_write(Write(t, w.r0, w.r1, w.c0, w.c1, e, w.core, getattr(e, "line", None)), table, temps, out)
            res0: Tuple[Expr, int] = (Leaf(t, w.r0, w.r1, w.c0, w.c1), lvl + 1)
            memo[id(e)] = res0
            return res0
        if isinstance(e, Un):
            x, l = go(e.x)
            res: Tuple[Expr, int] = (e if x is e.x else like(Un(e.op, x, e.params), e), l)
        elif isinstance(e, Bin):
            a, la = go(e.a)
            b, lb = go(e.b)
            res = (e if (a is e.a and b is e.b) else like(Bin(e.op, a, b, e.shape), e), max(la, lb))
        elif isinstance(e, Acc):
            parts = [go(t) for t in e.terms]
            res = (like(Acc([p[0] for p in parts], e.shape), e), max(p[1] for p in parts))
        elif isinstance(e, Red):
            if len(e.dims) != 1:
                raise Unsupported("a reduction over both dimensions inside a larger expression is not supported: "
                                  "store it into its own output tensor")
            x, l = go(e.x)
            kept = 1 - e.dims[0]
            span = (w.r1 - w.r0, w.c1 - w.c0)[kept]
            if e.shape[kept] != span or w.tensor.shape[kept] == 1:
                raise Unsupported("a reduction inside an expression must keep the extent of the block it is stored into")
            key = (oi, slot[0], e.op, e.dims)
            slot[0] += 1
            t = temps.get(key)
            if t is None:
                shape = (w.tensor.shape[0], 1) if kept == 0 else (1, w.tensor.shape[1])
                t = temps[key] = table.new_temp(shape, w.tensor)
            region = (w.r0, w.r1, 0, 1) if kept == 0 else (0, 1, w.c0, w.c1)
            out.append((Write(t, region[0], region[1], region[2], region[3], like(Red(e.op, x, e.scaler, e.dims), e),
                              w.core), l))
            res = (Leaf(t, *region), l + 1)
        else:
            raise Unsupported(f"cannot lower {type(e).__name__}")
        memo[id(e)] = res
        return res

    return go(w.expr)


def _first_leaf_like(e: Expr, shape: Tuple[int, int]) -> Optional[Leaf]:
    stack = [e]
    while stack:
        x = stack.pop()
        if isinstance(x, Leaf):
            if x.shape == shape and not any(x.first):
                return x
        elif isinstance(x, Bin):
            stack += [x.b, x.a]
        elif isinstance(x, Un):
            stack.append(x.x)
        elif isinstance(x, Acc):
            stack.extend(reversed(x.terms))
        elif isinstance(x, Red):
            stack.append(x.x)
    return None


def _lower_matmul_operands(w: Write, table: _TensorTable, temps: Dict[Any, _ttnn.Tensor],
                           out: List[Tuple[Write, int]]) -> Tuple[Expr, int]:
    """A block matmul write whose operands are expressions rather than blocks straight from a circular buffer
    (`relu(a_blk) @ b_blk`, `softmax(s_blk) @ v_blk`): every such operand is first written to a temporary laid out
    like a matrix operand - [output rows, K] for the left one, [K, output columns] for the right one - by writes of
    their own, and the matmul reads the temporaries.  The K range of an operand block comes from the other operand
    when that is a plain block, else from a block of equal shape inside the expression."""
    e = w.expr
    terms = list(e.terms) if isinstance(e, Acc) else [e]
    bias = None
    if len(terms) > 1 and isinstance(terms[0], Leaf):
        bias, terms = terms[0], terms[1:]
    oi = table.index(w.tensor)
    level = 0
    new_terms: List[Expr] = []
    for t in terms:
        a, b = _unwrap(t.a), _unwrap(t.b)
        ops = {"a": a, "b": b}
        for side in ("a", "b"):
            x = ops[side]
            if isinstance(x, Leaf):
                continue
            other = ops["b" if side == "a" else "a"]
            if isinstance(other, Leaf):
                k0, k1, k_total = ((other.r0, other.r1, other.tensor.shape[0]) if side == "a"
                                   else (other.c0, other.c1, other.tensor.shape[1]))
            else:
                inner = _first_leaf_like(x, x.shape)
                if inner is None:
                    raise Unsupported("cannot tell which K tiles a computed matmul operand covers")
                k0, k1, k_total = ((inner.c0, inner.c1, inner.tensor.shape[1]) if side == "a"
                                   else (inner.r0, inner.r1, inner.tensor.shape[0]))
            if x.shape != ((w.r1 - w.r0, k1 - k0) if side == "a" else (k1 - k0, w.c1 - w.c0)) or 1 in w.tensor.shape:
                raise Unsupported("a computed matmul operand must have the shape of the operand block")
            key = (oi, "mm_" + side)
            tmp = temps.get(key)
            if tmp is None:
                shape = (w.tensor.shape[0], k_total) if side == "a" else (k_total, w.tensor.shape[1])
                tmp = temps[key] = table.new_temp(shape, w.tensor)
            region = (w.r0, w.r1, k0, k1) if side == "a" else (k0, k1, w.c0, w.c1)
            lvl = _expand_write(Write(tmp, region[0], region[1], region[2], region[3], x, w.core, getattr(x, "line", None)),
                                table, temps, out)
            level = max(level, lvl + 1)
            ops[side] = Leaf(tmp, *region)
        nt = Bin("matmul", ops["a"], ops["b"], t.shape)
        if getattr(t, "line", None) is not None:
            nt.line = t.line
        new_terms.append(nt)
    if not isinstance(e, Acc):
        return new_terms[0], level
    acc = Acc(([bias] if bias is not None else []) + new_terms, e.shape)
    if getattr(e, "line", None) is not None:
        acc.line = e.line
    return acc, level


def _expand_write(w: Write, table: _TensorTable, temps: Dict[Any, _ttnn.Tensor], out: List[Tuple[Write, int]]) -> int:
    """Append write `w` to `out`, preceded by the writes that fill the temporaries it needs (reductions and matmuls
    inside its expression, computed matmul operands).  Returns the level of `w` (0: reads inputs only)."""
    if _has_run(w.expr):
        # runs of accumulated terms stay compact only where the matmul recogniser reads them directly
        e = w.expr
        terms = list(e.terms) if isinstance(e, Acc) else [e]
        if len(terms) > 1 and isinstance(terms[0], Leaf):
            terms = terms[1:]
        if not all(_plain_matmul(t) for t in terms):
            w = Write(w.tensor, w.r0, w.r1, w.c0, w.c1, _expand_runs(w.expr), w.core, w.line)
    mm = _matmul_terms(w)
    if mm is not None:
        if all(_plain_matmul(t) for t in mm[0]):
            out.append((w, 0))
            return 0
        expr, level = _lower_matmul_operands(w, table, temps, out)
    elif _reduce_terms(w) is None and (_contains_matmul(w.expr) or _contains_red(w.expr)):
        expr, level = _lower_reductions(w, table, temps, out)
    else:
        out.append((w, 0))
        return 0
    out.append((Write(w.tensor, w.r0, w.r1, w.c0, w.c1, expr, w.core, w.line), level))
    return level


def build_plan(trace: Trace, arg_tensors: Sequence[_ttnn.Tensor], fp32_intermediates: bool = False) -> Plan:
    table = _TensorTable(arg_tensors)
    # 1. every write gets a key (what is computed, from where); 2. writes must not overlap, except that
    # several cores writing the very same region with the very same expression (programs that do not
    # partition their loops over the grid) are one write.
    cover: Dict[int, np.ndarray] = {}
    seen: Dict[Any, Any] = {}
    out_tensors: Dict[int, _ttnn.Tensor] = {}
    elt_groups: Dict[Any, List[Tuple[int, int, int, int]]] = {}
    elt_meta: Dict[Any, Any] = {}
    mm_groups: Dict[Any, List[Tuple[int, int, int, int]]] = {}
    red_groups: Dict[Any, List[Tuple[int, int, int, int]]] = {}
    # reductions inside larger expressions first become writes of their own into temporaries
    temps: Dict[Any, _ttnn.Tensor] = {}
    writes: List[Tuple[Write, int]] = []
    for w in trace.writes:
        if isinstance(w, BatchedWrite):
            writes.append((w, 0))     # a matmul written by batched loops: all its iterations are recognised at once
        else:
            _expand_write(w, table, temps, writes)
    level_of: Dict[Any, int] = {}
    lines_of: Dict[Any, Dict[Tuple[str, int], int]] = {}   # per launch key: program line -> writes it took part in
    for w, level in writes:
        oi = table.index(w.tensor)
        out_tensors[oi] = w.tensor
        tr, tc = w.tensor.tile_shape()
        if isinstance(w, BatchedWrite):
            key = _recognise_matmul_batched(w, table, oi)
            if key is None:
                # its iterations differ in more than the output block: one write per iteration, the ordinary way
                for x in w.expand():
                    _expand_write(x, table, temps, writes)
                continue
            grid = cover.setdefault(oi, np.zeros((tr, tc), dtype=bool))
            regions = w.regions()
            for region in regions:
                r0, r1, c0, c1 = region
                if not (0 <= r0 < r1 <= tr and 0 <= c0 < c1 <= tc):
                    raise ValueError(f"write region [{r0}:{r1}, {c0}:{c1}] is outside the {tr}x{tc}-tile tensor")
                covered = grid[r0:r1, c0:c1]
                if covered.any():
                    if seen.get((oi, region)) == key:
                        continue
                    raise Unsupported(f"output tiles [{r0}:{r1}, {c0}:{c1}] are written more than once")
                covered[...] = True
                seen[(oi, region)] = key
                mm_groups.setdefault(key, []).append(region)
            level_of[key] = max(level_of.get(key, 0), level)
            if PROFILE.enabled:
                per_key = lines_of.setdefault(key, {})
                for ln in _lines_of(w):
                    per_key[ln] = per_key.get(ln, 0) + len(regions)
            continue
        if not (0 <= w.r0 < w.r1 <= tr and 0 <= w.c0 < w.c1 <= tc):
            raise ValueError(f"write region [{w.r0}:{w.r1}, {w.c0}:{w.c1}] is outside the {tr}x{tc}-tile tensor")
        region = (w.r0, w.r1, w.c0, w.c1)
        mm = _matmul_terms(w)
        red = _reduce_terms(w)
        if red is not None:
            key = ("red",) + _recognise_reduce(w, red, table, oi, fp32_intermediates)
        elif mm is not None:
            terms, bias = mm
            key = ("mm",) + tuple(_recognise_matmul(w, terms, table, oi)) + (_recognise_bias(w, bias, table),)
        else:
            if _contains_matmul(w.expr):
                raise Unsupported("matmul mixed with element-wise ops in one store is not supported yet")
            lin = _Lin(w, table)
            lin.emit(w.expr)
            if len(lin.inputs) > capi.TTLB_MAX_IN:
                raise Unsupported(f"expression reads {len(lin.inputs)} distinct operands (max {capi.TTLB_MAX_IN})")
            if len(lin.ops) > capi.TTLB_MAX_OPS:
                raise Unsupported(f"expression needs {len(lin.ops)} ops (max {capi.TTLB_MAX_OPS})")
            if _stack_depth(lin.ops) > 2:
                raise Unsupported("expression needs more than two temporaries")
            odt = w.tensor.dtype
            for (ti, *_rest) in lin.inputs:
                t = table.tensor(ti)
                if t.dtype != odt:
                    raise Unsupported(f"mixed element types ({t.dtype} operand, {odt} output)")
                for dim in (0, 1):
                    if w.tensor.shape[dim] == 1 and t.shape[dim] != 1:
                        raise Unsupported("a degenerate output dimension needs degenerate operands")
            key = ("elt", oi, tuple(lin.inputs), tuple(lin.ops), tuple(lin.imms))
            elt_meta[key] = (odt, (w.tensor.shape[0] == 1, w.tensor.shape[1] == 1))
        grid = cover.setdefault(oi, np.zeros((tr, tc), dtype=bool))
        covered = grid[w.r0:w.r1, w.c0:w.c1]
        if covered.any():
            if seen.get((oi, region)) == key:
                continue   # the same write again, from another core
            raise Unsupported(f"output tiles [{w.r0}:{w.r1}, {w.c0}:{w.c1}] are written more than once")
        covered[...] = True
        seen[(oi, region)] = key
        {"mm": mm_groups, "elt": elt_groups, "red": red_groups}[key[0]].setdefault(key, []).append(region)
        level_of[key] = max(level_of.get(key, 0), level)
        if PROFILE.enabled:
            per_key = lines_of.setdefault(key, {})
            for ln in _lines_of(w):
                per_key[ln] = per_key.get(ln, 0) + 1

    class _Launches(list):   # appending a launch also hands it the program lines of its key
        def add(self, key: Any, launch: Any) -> None:
            launch.lines = lines_of.get(key, {})
            self.append((level_of[key], launch))

    launches = _Launches()
    for key, rects in elt_groups.items():
        _, oi, inputs, ops, imms = key
        odt, degen = elt_meta[key]
        for rect in merge_rects(rects):
            launches.add(key, EltwiseLaunch(oi, rect, list(inputs), list(ops), odt,
                                            round_each_op=not fp32_intermediates, out_degenerate=degen, imms=imms))
    for key, rects in red_groups.items():
        _, oi, op, dims, extent, inputs, ops, sc_key, _anchor, imms = key
        for rect in merge_rects(rects):
            launches.add(key, ReduceLaunch(oi, rect, op, dims, extent, list(inputs), list(ops), sc_key,
                                           out_tensors[oi].dtype, round_each_op=not fp32_intermediates, imms=imms))
    for key, rects in mm_groups.items():
        _, ai, bi, oi, kt, b8, ci = key
        f32 = out_tensors[oi].dtype == torch.float32
        if ci is not None and f32:
            raise Unsupported("matmul with bias: bfloat16 A, bias and output only")
        for rect in merge_rects(rects):
            gl = GemmLaunch(ai, bi, oi, rect, kt, b8, ci)
            if f32:
                gl.kind = "matmul_f32"
            launches.add(key, gl)
    # a launch that reads a temporary runs after the launch that fills it
    ordered = [l for _, l in sorted(launches, key=lambda p: p[0])]
    if fp32_intermediates:
        ordered = _fuse_epilogues(ordered)
    if ROW_FUSION:
        ordered = _fuse_rows(ordered)
    _check_hazards(ordered)
    # temporaries that the fusions made unnecessary keep their index but give their memory back
    used: Dict[int, None] = {}
    for l in ordered:
        for part in list(getattr(l, "parts", [])) + [getattr(l, "final", l), l]:
            for (ti, *_r) in getattr(part, "inputs", []):
                used[ti] = None
            for attr in ("out_index", "a_index", "b_index", "bias_index"):
                used[getattr(part, attr, None)] = None  # type: ignore[index]
    for i, t in enumerate(table.temps):
        if TEMP_BASE + i not in used:
            t._tensor = torch.empty((0, 0), dtype=t._tensor.dtype, device=t._tensor.device)
    return Plan(ordered, table.extras, len(table.args), table.temps)


def _recognise_matmul_batched(w: BatchedWrite, table: _TensorTable, oi: int) -> Any:
    """Key of a matmul written by batched loops, all iterations checked at once with array comparisons (the same
    conditions as _recognise_matmul / _recognise_bias); None when the K tiles differ between iterations, in which
    case the caller goes through the iterations one by one."""
    mm = _matmul_terms(w)
    assert mm is not None
    terms, bias = mm
    na = 4   # loop axes of the tile-coordinate arrays (symloop.NEST_AXES)
    for t in terms:
        x = t.x if isinstance(t, Rep) else t
        for v in (x.a.c0, x.a.c1, x.b.r0, x.b.r1):
            if isinstance(v, np.ndarray) and any(sz > 1 for sz in v.shape[:na]):
                return None

    def same(p: Any, q: Any) -> bool:
        return bool(np.all(np.equal(p, q)))

    for t in terms:
        x = t.x if isinstance(t, Rep) else t
        if not (same(x.a.r0, w.r0) and same(x.a.r1, w.r1) and same(x.b.c0, w.c0) and same(x.b.c1, w.c1)):
            raise Unsupported("matmul operand rows/columns do not line up with the output block")
    # the K side does not depend on the iteration: judged on the first one
    first = w.expand(1)[0]
    mm1 = _matmul_terms(first)
    assert mm1 is not None
    key = tuple(_recognise_matmul(first, mm1[0], table, oi))
    ci = None
    if bias is not None:
        if not (same(bias.r0, w.r0) and same(bias.r1, w.r1) and same(bias.c0, w.c0) and same(bias.c1, w.c1)):
            raise Unsupported("matmul with bias: the bias block is not the block of the output tile being computed")
        ci = _recognise_bias(first, mm1[1], table)
    return ("mm",) + key + (ci,)


def _recognise_bias(w: Write, bias: Optional[Leaf], table: _TensorTable) -> Optional[int]:
    if bias is None:
        return None
    t = bias.tensor
    if tuple(t.shape) != tuple(w.tensor.shape) or t.dtype != w.tensor.dtype:
        raise Unsupported("matmul with bias: the bias tensor must have the output's shape and element type")
    if (bias.r0, bias.r1, bias.c0, bias.c1) != (w.r0, w.r1, w.c0, w.c1):
        raise Unsupported("matmul with bias: the bias block is not the block of the output tile being computed")
    return table.index(t)


def _recognise_matmul(w: Write, terms: List[Any], table: _TensorTable, oi: int) -> Any:
    first = terms[0].x if isinstance(terms[0], Rep) else terms[0]
    a0, b0 = _unwrap(first.a), _unwrap(first.b)
    if not (isinstance(a0, Leaf) and isinstance(b0, Leaf)):
        raise Unsupported("matmul operands must come straight from circular buffers")
    ta, tb = a0.tensor, b0.tensor
    kt = ta.tile_shape()[1]
    if tb.tile_shape()[0] != kt:
        raise ValueError(f"Incompatible matrix shapes for multiplication: {ta.shape} @ {tb.shape}")
    ks: List[Any] = []
    for t in terms:
        run = isinstance(t, Rep)
        x = t.x if run else t
        a, b = _unwrap(x.a), _unwrap(x.b)
        if not (isinstance(a, Leaf) and isinstance(b, Leaf)) or a.tensor is not ta or b.tensor is not tb:
            raise Unsupported("matmul accumulation must read the same A and B tensors in every step")
        if a.shape[1] != b.shape[0] or (a.shape[1] > 1 and a.shape == b.shape):
            # equal-shape multi-tile blocks mean a tile-wise product in the simulator (python/sim/block.py:885-905),
            # a block dot product in the specification: refused rather than guessed
            raise Unsupported(f"matmul of blocks {a.shape} @ {b.shape}: (M,K) @ (K,N) blocks only "
                              "(equal-shape multi-tile blocks are ambiguous)")
        if not run:
            if (a.r0, a.r1) != (w.r0, w.r1) or (b.c0, b.c1) != (w.c0, w.c1):
                raise Unsupported("matmul operand rows/columns do not line up with the output block")
            if (a.c0, a.c1) != (b.r0, b.r1):
                raise Unsupported("matmul step multiplies different K tiles of A and B")
            ks.append(np.arange(a.c0, a.c1))
            continue
        # a run of steps (a batched K loop): the same checks on whole arrays of tile coordinates
        n = 1
        for sz in t.sizes:
            n *= sz

        def col(v: Any) -> "np.ndarray":
            """The coordinate for every step of the run, in the order the steps accumulate."""
            if isinstance(v, np.ndarray):
                if v.size == n and len(t.axes) == 1:
                    return v.reshape(-1)
                full = [1] * v.ndim
                for ax, sz in zip(t.axes, t.sizes):
                    full[ax] = sz
                return np.broadcast_to(v, full).reshape(-1)
            return np.full(n, v, dtype=np.int64)

        ar0, ar1, ac0, ac1 = (col(v) for v in (a.r0, a.r1, a.c0, a.c1))
        br0, br1, bc0, bc1 = (col(v) for v in (b.r0, b.r1, b.c0, b.c1))
        if ((ar0 != w.r0).any() or (ar1 != w.r1).any() or (bc0 != w.c0).any() or (bc1 != w.c1).any()):
            raise Unsupported("matmul operand rows/columns do not line up with the output block")
        if (ac0 != br0).any() or (ac1 != br1).any():
            raise Unsupported("matmul step multiplies different K tiles of A and B")
        width = a.shape[1]
        ks.append((ac0[:, None] + np.arange(width)[None, :]).reshape(-1))
    allk = np.sort(np.concatenate(ks)) if ks else np.zeros(0, dtype=np.int64)
    if allk.size != kt or (allk != np.arange(kt)).any():
        raise Unsupported(f"matmul accumulates K tiles {sorted(set(allk.tolist()))[:4]}... instead of all {kt} exactly once")
    b8 = 0 if tb._packed is None else tb._packed_bits    # 0: plain weights; 8 / 4: block-float tiles
    all_bf16 = ta.dtype == torch.bfloat16 and (b8 or tb.dtype == torch.bfloat16) and w.tensor.dtype == torch.bfloat16
    all_f32 = ta.dtype == torch.float32 and not b8 and tb.dtype == torch.float32 and w.tensor.dtype == torch.float32
    if not (all_bf16 or all_f32):
        raise Unsupported(f"matmul element types A={ta.dtype} B={tb.dtype} out={w.tensor.dtype}: all bfloat16 "
                          "(optionally bfloat8_b weights) or all float32")
    return (table.index(ta), table.index(tb), oi, kt, b8)
