"""Symbolic execution of a tt-lang tile program.

The reference runs a `@ttl.kernel` either by compiling its three threads to MLIR
(python/ttl/ttl_api.py:818-1122) or by stepping them on real data in the simulator
(python/sim/program.py:100-682).  This module runs the very same thread functions,
on every core of the grid, with circular buffers and blocks that carry *expressions
over tile regions* instead of data.  The outcome is the list of writes the program
performs, `output region <- expression over input regions`, which the recogniser
turns into GPU launches.

Semantics kept from the simulator:
  * per-core fresh circular buffers, thread closures rebound per core
    (python/sim/program.py:69-97, 152-194); cores numbered 0..prod(grid)-1
    (python/sim/program.py:213-223);
  * reserve/push/wait/pop FIFO discipline, one pending reserve and one pending wait
    per buffer (python/sim/cb.py:249-408), `with` sugar pushes/pops on exit
    (python/sim/cb.py:24-71);
  * `store(acc=True)`: first store assigns, later ones add (python/sim/block.py:805-868);
  * block shapes broadcast NumPy-style over the tile grid (python/sim/block.py:783-803),
    copy shape rule with size-1 dims kept as one tile (python/sim/copyhandlers.py:103-131,
    295-380);
  * pipes deliver a sent block to each destination core (python/sim/copyhandlers.py:228-292,
    383-470); a program where every thread is blocked is reported as a deadlock
    (python/sim/program.py:603-647).
"""

from __future__ import annotations

import copy as _copy
import os
import sys
import threading
import types
from collections import deque
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import symloop as _sl
from . import ttnn as _ttnn
from .symloop import NeedsConcrete

TILE_SHAPE = (32, 32)
MAX_CBS = 32


# --------------------------------------------------------------------------- #
# Expression IR (block level: every node stands for a grid of tiles)
# --------------------------------------------------------------------------- #
class Expr:
    __slots__ = ("shape", "line")
    shape: Tuple[int, int]


class _ProfileSwitch:
    """While `enabled`, expression nodes and writes remember the program line that created them, so that a
    launch can be reported against the source lines it implements (profile.py)."""
    enabled = False


PROFILE = _ProfileSwitch()
_PKG_DIR = os.path.dirname(os.path.abspath(__file__))


def _site() -> Optional[Tuple[str, int]]:
    """(file, line) of the tile-program statement being executed: the innermost frame outside this package."""
    if not PROFILE.enabled:
        return None
    f = sys._getframe(1)
    while f is not None and os.path.abspath(f.f_code.co_filename).startswith(_PKG_DIR):
        f = f.f_back
    return (f.f_code.co_filename, f.f_lineno) if f is not None else None


def _tag(e: "Expr") -> "Expr":
    if PROFILE.enabled:
        e.line = _site()
    return e


class Leaf(Expr):
    """Tile region [r0:r1, c0:c1] (tile coordinates) of input tensor `tensor`.  `first[d]` set: along
    dim d every element reads element 0 of its tile (the hardware broadcast of a full tile whose first
    row / column carries the data, `ttl.math.broadcast` on non-degenerate tiles)."""

    __slots__ = ("tensor", "r0", "r1", "c0", "c1", "first")

    def __init__(self, tensor: "_ttnn.Tensor", r0: int, r1: int, c0: int, c1: int,
                 first: Tuple[bool, bool] = (False, False)):
        self.tensor, self.r0, self.r1, self.c0, self.c1, self.first = tensor, r0, r1, c0, c1, first
        # tile coordinates are ints, or (traced with batched loops, symloop.py) int64 arrays with one axis per loop;
        # the extent is the same for every iteration and is then set by the creator
        self.shape = (r1 - r0, c1 - c0) if type(r0) is int and type(r1) is int and type(c0) is int and type(c1) is int \
            else (0, 0)


class Zero(Expr):
    """A freshly reserved block: all zeros (python/sim/cb.py:343-346)."""

    __slots__ = ()

    def __init__(self, shape: Tuple[int, int]):
        self.shape = shape


class Un(Expr):
    """Element-wise function of one block; `params` are the scalar parameters of functions such as
    leaky_relu(x, slope)."""

    __slots__ = ("op", "x", "params")

    def __init__(self, op: str, x: Expr, params: Tuple[float, ...] = ()):
        self.op, self.x, self.params, self.shape = op, x, params, x.shape


class Bin(Expr):
    __slots__ = ("op", "a", "b")

    def __init__(self, op: str, a: Expr, b: Expr, shape: Tuple[int, int]):
        self.op, self.a, self.b, self.shape = op, a, b, shape


class Acc(Expr):
    """Running sum built by repeated `store(..., acc=True)`: terms are added in order,
    each partial sum held in the block's dtype."""

    __slots__ = ("terms",)

    def __init__(self, terms: List[Expr], shape: Tuple[int, int]):
        self.terms, self.shape = terms, shape


class Red(Expr):
    """`ttl.math.reduce_sum / reduce_max(x, scaler, dims)`: the elements of block `x` combined along the
    block dims in `dims` (0: rows, 1: columns), times the scaler.  The reduced dims of the result are one
    tile long; the value sits in the tile's first row / column / element."""

    __slots__ = ("op", "x", "scaler", "dims")

    def __init__(self, op: str, x: Expr, scaler: Optional[Expr], dims: Tuple[int, ...]):
        self.op, self.x, self.scaler, self.dims = op, x, scaler, dims
        self.shape = (1 if 0 in dims else x.shape[0], 1 if 1 in dims else x.shape[1])


class Rep(Expr):
    """A run of accumulated terms: `x` once for every index of the sequence axes `axes` (array axes of the tile
    coordinates inside `x`, sizes `sizes`, first axis slowest).  Made when `store(..., acc=True)` runs in a
    batched loop nested deeper than the block it accumulates into (the K loop of a matmul)."""

    __slots__ = ("x", "axes", "sizes")

    def __init__(self, x: Expr, axes: Tuple[int, ...], sizes: Tuple[int, ...]):
        self.x, self.axes, self.sizes, self.shape = x, axes, sizes, x.shape

    def terms(self) -> List[Expr]:
        """The terms the run stands for, in order."""
        out = []
        for idx in np.ndindex(*self.sizes):
            sel = dict(zip(self.axes, idx))
            out.append(map_coords(self.x, lambda a: _pick(a, sel)))
        return out


def _pick(a: "np.ndarray", sel: Dict[int, int]) -> Any:
    """Array `a` at index sel[axis] along the given axes (kept with size 1); an int when nothing is left."""
    ix = tuple(slice(sel[ax], sel[ax] + 1) if ax in sel and a.shape[ax] > 1 else slice(None) for ax in range(a.ndim))
    b = a[ix]
    return int(b.reshape(-1)[0]) if b.size == 1 else b


def map_coords(e: Expr, fn: Callable[["np.ndarray"], Any], memo: Optional[Dict[int, Expr]] = None) -> Expr:
    """`e` with every array-valued tile coordinate replaced by fn(array); shared subtrees stay shared."""
    if memo is None:
        memo = {}
    hit = memo.get(id(e))
    if hit is not None:
        return hit
    r: Expr
    if isinstance(e, Leaf):
        cs = [fn(c) if isinstance(c, np.ndarray) else c for c in (e.r0, e.r1, e.c0, e.c1)]
        if all(a is b for a, b in zip(cs, (e.r0, e.r1, e.c0, e.c1))):
            r = e
        else:
            r = Leaf(e.tensor, cs[0], cs[1], cs[2], cs[3], e.first)
            r.shape = e.shape
    elif isinstance(e, Un):
        x = map_coords(e.x, fn, memo)
        r = e if x is e.x else Un(e.op, x, e.params)
    elif isinstance(e, Bin):
        a, b = map_coords(e.a, fn, memo), map_coords(e.b, fn, memo)
        r = e if (a is e.a and b is e.b) else Bin(e.op, a, b, e.shape)
    elif isinstance(e, Acc):
        ts = [map_coords(t, fn, memo) for t in e.terms]
        r = e if all(a is b for a, b in zip(ts, e.terms)) else Acc(ts, e.shape)
    elif isinstance(e, Red):
        x = map_coords(e.x, fn, memo)
        sc = map_coords(e.scaler, fn, memo) if e.scaler is not None else None
        r = e if (x is e.x and sc is e.scaler) else Red(e.op, x, sc, e.dims)
    elif isinstance(e, Rep):
        x = map_coords(e.x, fn, memo)
        r = e if x is e.x else Rep(x, e.axes, e.sizes)
    else:
        r = e
    if r is not e and getattr(e, "line", None) is not None:
        r.line = e.line
    memo[id(e)] = r
    return r


def _rep_axes_used(e: Expr) -> int:
    """Number of sequence axes the runs inside `e` already occupy."""
    top = 0
    stack, seen = [e], set()
    while stack:
        x = stack.pop()
        if id(x) in seen:
            continue
        seen.add(id(x))
        if isinstance(x, Rep):
            top = max(top, max(x.axes) - _sl.NEST_AXES + 1)
            stack.append(x.x)
        elif isinstance(x, Bin):
            stack += [x.a, x.b]
        elif isinstance(x, Un):
            stack.append(x.x)
        elif isinstance(x, Acc):
            stack.extend(x.terms)
        elif isinstance(x, Red):
            stack.append(x.x)
            if x.scaler is not None:
                stack.append(x.scaler)
    return top


class Write:
    """`tensor[r0:r1, c0:c1] <- expr` (tile coordinates)."""

    __slots__ = ("tensor", "r0", "r1", "c0", "c1", "expr", "core", "line")

    def __init__(self, tensor: "_ttnn.Tensor", r0: int, r1: int, c0: int, c1: int, expr: Expr, core: int,
                 line: Optional[Tuple[str, int]] = None):
        self.tensor, self.r0, self.r1, self.c0, self.c1, self.expr, self.core = tensor, r0, r1, c0, c1, expr, core
        self.line = line


class BatchedWrite(Write):
    """The writes of all iterations of the batched loops live at the copy (`sizes`: their trip counts): the tile
    coordinates and those inside `expr` are arrays over the loop axes.  Trace.finish() turns it into one Write per
    iteration."""

    __slots__ = ("sizes",)

    def __init__(self, tensor: "_ttnn.Tensor", r0: Any, r1: Any, c0: Any, c1: Any, expr: Expr, core: int,
                 line: Optional[Tuple[str, int]], sizes: Tuple[int, ...]):
        super().__init__(tensor, r0, r1, c0, c1, expr, core, line)
        self.sizes = sizes

    def count(self) -> int:
        count = 1
        for n in self.sizes:
            count *= n
        return count

    def regions(self) -> List[Tuple[int, int, int, int]]:
        """(r0, r1, c0, c1) of every iteration, in order."""
        n = self.count()
        cols = [np.broadcast_to(c, tuple(self.sizes) + c.shape[len(self.sizes):]).reshape(n).tolist()
                if isinstance(c, np.ndarray) else [c] * n for c in (self.r0, self.r1, self.c0, self.c1)]
        return list(zip(*cols))

    def plain_matmul(self) -> bool:
        """`sum_k a_blk @ b_blk` (optionally starting from a bias block) with every operand straight from a
        circular buffer: the form the recogniser reads for all iterations at once."""
        e = self.expr
        terms = list(e.terms) if isinstance(e, Acc) else [e]
        if len(terms) > 1 and isinstance(terms[0], Leaf):
            terms = terms[1:]
        for t in terms:
            x = t.x if isinstance(t, Rep) else t
            if not (isinstance(x, Bin) and x.op == "matmul" and isinstance(x.a, Leaf) and isinstance(x.b, Leaf)):
                return False
        return bool(terms)

    def expand(self, limit: Optional[int] = None) -> List[Write]:
        count = self.count()
        d = len(self.sizes)
        columns: Dict[int, Any] = {}     # id(array) -> per-iteration values (list of ints, or of arrays over the sequence axes)

        def column(a: "np.ndarray") -> Any:
            col = columns.get(id(a))
            if col is None:
                rest = a.shape[_sl.NEST_AXES:]
                full = np.broadcast_to(a, tuple(self.sizes) + a.shape[d:])
                if all(s == 1 for s in rest):
                    col = full.reshape(count).tolist()
                else:
                    flat = full.reshape((count,) + (1,) * _sl.NEST_AXES + rest)
                    col = [flat[i] for i in range(count)]
                columns[id(a)] = (a, col)
                return col
            return col[1]

        def coord(c: Any, i: int) -> Any:
            return column(c)[i] if isinstance(c, np.ndarray) else c

        out = []
        for i in range(count if limit is None else min(count, limit)):
            expr = map_coords(self.expr, lambda a, i=i: column(a)[i])
            out.append(Write(self.tensor, coord(self.r0, i), coord(self.r1, i), coord(self.c0, i), coord(self.c1, i), expr,
                             self.core, self.line))
        return out


def infer_broadcast_shape(left: Tuple[int, ...], right: Tuple[int, ...]) -> Tuple[int, int]:
    if len(left) != len(right):
        raise ValueError(f"Shape dimension mismatch: {left} vs {right}")
    out = []
    for i, (l, r) in enumerate(zip(left, right)):
        if l != r and l != 1 and r != 1:
            raise ValueError(
                f"Cannot broadcast: incompatible shapes {left} and {right}. "
                f"Dimension {i} has sizes {l} and {r} which are incompatible "
                f"(must be equal or one must be 1).")
        out.append(max(l, r))
    return tuple(out)  # type: ignore[return-value]


# --------------------------------------------------------------------------- #
# Cooperative scheduler: one OS thread per tile-program thread, one runs at a time
# --------------------------------------------------------------------------- #
_tls = threading.local()


def current_core() -> int:
    c = getattr(_tls, "core", None)
    if c is None:
        raise RuntimeError("core not available - function must be called within Program context")
    return c


# The compiler front end keeps the grid of the last kernel in a module global (python/ttl/operators.py:36), which
# programs written against it read back with ttl.grid_size() after the kernel has returned; the simulator raises
# outside a kernel (python/sim/kernel.py:116-118).  The simulator's behaviour is the default.
GRID_OUTLIVES_KERNEL = False


def set_grid_outlives_kernel(enabled: bool) -> None:
    global GRID_OUTLIVES_KERNEL
    GRID_OUTLIVES_KERNEL = bool(enabled)


def current_grid() -> Tuple[int, ...]:
    g = getattr(_tls, "grid", None)
    if g is None and GRID_OUTLIVES_KERNEL:
        g = getattr(_tls, "last_grid", None)
    if g is None:
        raise RuntimeError("grid not available - function must be called within a kernel context")
    return g


def set_grid(grid: Optional[Tuple[int, ...]]) -> None:
    _tls.grid = grid
    if grid is not None:
        _tls.last_grid = grid


class DeadlockError(RuntimeError):
    pass


class _Worker:
    def __init__(self, sched: "Scheduler", name: str, fn: Callable[[], Any], core: int, kind: str):
        self.sched, self.name, self.fn, self.core, self.kind = sched, name, fn, core, kind
        self.go = threading.Event()
        self.done = False
        self.error: Optional[BaseException] = None
        self.blocked_on: Optional[Callable[[], bool]] = None
        self.blocked_desc = ""
        self.thread = threading.Thread(target=self._run, name=name, daemon=True)

    def _run(self) -> None:
        self.go.wait()
        self.go.clear()
        _tls.core = self.core
        _tls.grid = self.sched.grid
        _tls.kind = self.kind
        _tls.worker = self
        _tls.trace = self.sched.trace
        st = _sl.STATE
        st.nest, st.enabled, st.nobatch, st.batched_loops = [], self.sched.batching, self.sched.nobatch, 0
        self.nest = st.nest
        self.budget = self.sched.trace.budget or 0
        try:
            if not self.sched.aborting:
                self.fn()
        except (_Abort, _BudgetSpent):   # a verification probe stops a thread that has done its share
            pass
        except BaseException as e:  # noqa: BLE001 - reported to the caller of the kernel
            self.error = e
        finally:
            self.sched.trace.batched_loops += st.batched_loops
            st.nest = None
            self.done = True
            self.sched.back.set()

    def block(self, ready: Callable[[], bool], desc: str) -> None:
        """Park this worker until `ready()` holds."""
        while not ready():
            self.blocked_on, self.blocked_desc = ready, desc
            self.sched.back.set()
            self.go.wait()
            self.go.clear()
            if self.sched.aborting:
                raise _Abort()
        self.blocked_on = None


class _Abort(BaseException):
    pass


class _BudgetSpent(BaseException):
    pass


class Scheduler:
    def __init__(self, grid: Tuple[int, ...], trace: "Trace"):
        self.grid = grid
        self.trace = trace
        self.workers: List[_Worker] = []
        self.back = threading.Event()
        self.aborting = False
        self.batching = False                 # run batchable loops once for all their iterations (symloop.py)
        self.nobatch: Any = frozenset()       # loop sites that must run iteration by iteration

    def add(self, name: str, fn: Callable[[], Any], core: int, kind: str) -> None:
        self.workers.append(_Worker(self, name, fn, core, kind))

    def _resume(self, w: _Worker) -> None:
        self.back.clear()
        w.go.set()
        self.back.wait()

    def run(self) -> None:
        for w in self.workers:
            w.thread.start()
        pending = deque(self.workers)
        error: Optional[BaseException] = None
        failed: Optional[_Worker] = None
        while pending and error is None:
            progressed = False
            for _ in range(len(pending)):
                w = pending.popleft()
                if w.blocked_on is not None and not w.blocked_on():
                    pending.append(w)
                    continue
                self._resume(w)
                progressed = True
                if w.error is not None:
                    error, failed = w.error, w
                    break
                if not w.done:
                    pending.append(w)
            if not progressed and error is None:
                lines = [f"  {w.name}: blocked on {w.blocked_desc}" for w in pending]
                error = DeadlockError("Deadlock detected: all threads are blocked\n" + "\n".join(lines))
                # a loop that feeds itself through a circular buffer starves when it runs once for all its
                # iterations: run the loops the blocked threads are in iteration by iteration and look again
                sites = set()
                for w in pending:
                    sites |= _sl.sites_of(getattr(w, "nest", None) or ())
                if sites:
                    error = NeedsConcrete(sites, "threads starve while their loops are batched")
        if error is not None:
            self.aborting = True
            for w in self.workers:
                if not w.done:
                    self._resume(w)
        for w in self.workers:
            w.thread.join()
        if error is not None:
            if failed is not None and not isinstance(error, DeadlockError):
                try:
                    error.add_note(f"(raised in tile-program thread {failed.name})")
                except Exception:  # pragma: no cover
                    pass
            raise error


def _worker() -> _Worker:
    w = getattr(_tls, "worker", None)
    if w is None:
        raise RuntimeError("Thread context not set. Must be called within a kernel thread.")
    return w


# --------------------------------------------------------------------------- #
# Blocks and circular buffers
# --------------------------------------------------------------------------- #
def _make_rep(v: Expr, extra: Sequence[Any]) -> Expr:
    """`v`, whose tile coordinates vary along the axes of the batched loops `extra`, as the run of terms those
    loops store one after the other: their axes are moved to free sequence axes."""
    used = _rep_axes_used(v)
    if used + len(extra) > _sl.REP_AXES:
        raise NeedsConcrete(_sl.sites_of(extra), "accumulation nested too deeply")
    axes = tuple(_sl.NEST_AXES + used + i for i in range(len(extra)))
    moves = [(f.axis, ax) for f, ax in zip(extra, axes)]

    def move(a: "np.ndarray") -> "np.ndarray":
        for src, dst in moves:
            if a.shape[src] > 1:
                a = np.swapaxes(a, src, dst)
        return a

    return Rep(map_coords(v, move), axes, tuple(f.n for f in extra))


class _Seg:
    """A run of pushed blocks in a circular buffer's queue: what a reserve / push pair inside batched loops with
    trip counts `sizes` pushed, first loop slowest.  `off` entries have been popped already."""

    __slots__ = ("shape", "dtype", "expr", "sizes", "count", "off")

    def __init__(self, shape: Tuple[int, int], dtype: Any, expr: Expr, sizes: Tuple[int, ...]):
        self.shape, self.dtype, self.expr, self.sizes, self.off = shape, dtype, expr, sizes, 0
        self.count = 1
        for n in sizes:
            self.count *= n

    def left(self) -> int:
        return self.count - self.off

    def element(self) -> "Block":
        """The next entry as an ordinary block."""
        idx = np.unravel_index(self.off, self.sizes)
        sel = {ax: int(i) for ax, i in enumerate(idx)}
        return Block(self.shape, self.dtype, map_coords(self.expr, lambda a: _pick(a, sel)), "FULL", "wait")

    def take(self, m: int, frames: Sequence[Any]) -> Optional["Block"]:
        """The next `m` entries as one block batched over the loops `frames` (m = product of their trip counts);
        None when the run cannot be cut that way."""
        want = tuple(f.n for f in frames)
        if m > self.left():
            return None
        d, e = len(self.sizes), len(want)
        if self.off == 0 and m == self.count and want == self.sizes:
            return Block(self.shape, self.dtype, self.expr, "FULL", "wait", nest=tuple(frames))
        # the run's trailing loops as a unit: `m` entries = all of sizes[j:], starting at a multiple of m
        j, tail = d, 1
        while j > 0 and tail < m:
            j -= 1
            tail *= self.sizes[j]
        if tail != m or self.off % m:
            return None
        lead = np.unravel_index(self.off // m, self.sizes[:j]) if j else ()
        sel = {ax: int(i) for ax, i in enumerate(lead)}
        na = _sl.NEST_AXES

        def cut(a: "np.ndarray") -> Any:
            b = _pick(a, sel)
            if not isinstance(b, np.ndarray):
                return b
            rest = b.shape[na:]
            if want == self.sizes[j:]:
                # same loop structure: the run's axes j.. become axes 0..
                return b.reshape(b.shape[j:na] + (1,) * j + rest)
            full = np.broadcast_to(b, (1,) * j + tuple(self.sizes[j:]) + b.shape[d:])
            return full.reshape(want + (1,) * (na - e) + rest)

        return Block(self.shape, self.dtype, map_coords(self.expr, cut), "FULL", "wait", nest=tuple(frames))


class Block:
    """A reserved or waited window of a circular buffer, or a temporary (the value of
    an expression).  Holds the symbolic value of its tiles."""

    __slots__ = ("_shape", "expr", "dtype", "state", "kind", "temporary", "nest", "_acc_frames")

    # states: "MW" must-write (reserved), "NAW" copy in flight into it, "FULL" holds a value,
    #         "ACC" accumulating, "OS" out of scope (pushed / popped)
    def __init__(self, shape: Tuple[int, int], dtype: Any, expr: Optional[Expr], state: str, kind: str,
                 temporary: bool = False, nest: Tuple[Any, ...] = ()):
        self._shape, self.dtype, self.expr, self.state, self.kind, self.temporary = (
            tuple(shape), dtype, expr, state, kind, temporary)
        # the batched loops (symloop.Frame) live when the block was made: its tile coordinates vary along their axes
        self.nest = nest
        self._acc_frames: Optional[set] = None   # loops nested deeper under which terms were accumulated into it

    @property
    def shape(self) -> Tuple[int, int]:
        return self._shape  # type: ignore[return-value]

    def __len__(self) -> int:
        return self._shape[0] * self._shape[1]

    def block(self) -> "Block":
        return self

    def __getitem__(self, idx: Any) -> Any:
        raise RuntimeError(
            "Block indexing (block[index]) is not allowed. "
            "Blocks must be used as whole units in operations like store() or arithmetic. "
            "Use block directly without indexing.")

    def __setitem__(self, idx: Any, value: Any) -> None:
        raise RuntimeError("Direct assignment to Block is not allowed. Use block.store() or copy() instead.")

    # -- reading ---------------------------------------------------------
    def value(self) -> Expr:
        if self.state == "MW":
            raise RuntimeError(
                "Cannot read from Block: Block is in must-write (MW) state. "
                "Current state: MW, Expected operations: [STORE, STORE_ACC]")
        if self.state in ("NAW", "OS"):
            raise RuntimeError(
                f"Cannot read from Block: Block has no access ({self.state} state). Current state: {self.state}")
        assert self.expr is not None
        if self.nest:
            _sl.require_live(self.nest, "a block")
        if self._acc_frames is not None:
            live = [f for f in _sl.nest() if f in self._acc_frames]
            if live:
                raise NeedsConcrete(_sl.sites_of(live), "a block is read while a loop is still accumulating into it")
        return self.expr

    # -- writing ---------------------------------------------------------
    def store(self, items: Any, acc: bool = False) -> None:
        src = _as_block(items)
        # the simulator also takes a sequence of tile tensors and checks length, then write access
        # (python/sim/block.py:839-843); the same order here, so that programs get the same error
        if not isinstance(src, (Block, list, tuple)):
            raise TypeError("store() takes a block or a block expression")
        if len(src) != len(self):
            raise ValueError("Length mismatch in store()")
        if self.state == "NAW":
            raise RuntimeError(
                "Cannot write to Block: Block is locked as copy destination until tx.wait() completes "
                "(copy lock error). Current state: NAW, Expected operations: [TX_WAIT]")
        if self.state == "OS":
            raise RuntimeError("Cannot write to Block: Block has no access (OS state). Current state: OS")
        if not self.temporary and self.kind == "wait":
            raise RuntimeError("Cannot write to Block: a waited block is read-only in a compute thread")
        if not isinstance(src, Block):
            raise TypeError("store() of a sequence of tile tensors is not supported on the GPU: store a block or a block expression")
        v = src.value()
        cur = _sl.nest()
        if cur or self.nest:
            _sl.require_live(self.nest, "a block")
            extra = tuple(cur[len(self.nest):])
            if extra:
                # the store runs in loops nested deeper than the block: it stands for a sequence of stores
                if not acc:
                    raise NeedsConcrete(_sl.sites_of(extra), "a block of an outer loop is overwritten inside the loop")
                if self._acc_frames is not None and any(f in self._acc_frames for f in extra):
                    raise NeedsConcrete(_sl.sites_of(extra), "two accumulating stores into one block in one loop body")
                v = _make_rep(v, extra)
                self._acc_frames = (self._acc_frames or set()) | set(extra)
        if acc:
            if self.state == "MW":  # first accumulating store assigns
                self.expr = _tag(Acc([v], self._shape))
            elif isinstance(self.expr, Acc):
                self.expr.terms.append(v)
            else:
                assert self.expr is not None
                self.expr = _tag(Acc([self.expr, v], self._shape))
            self.state = "ACC"
        else:
            self.expr = v
            self.state = "FULL"

    # -- arithmetic ------------------------------------------------------
    def _binary(self, other: Any, op: str) -> "Block":
        o = _as_block(other)
        if not isinstance(o, Block):
            raise TypeError(f"unsupported operand type(s) for {op}: 'Block' and '{type(other).__name__}'")
        a, b = self.value(), o.value()
        if op == "matmul" and self._shape != o._shape:
            # block dot product (docs/sphinx/specs/TTLangSpecification.md:694): (M, K) @ (K, N) -> (M, N)
            if self._shape[1] != o._shape[0]:
                raise ValueError(f"Incompatible block shapes for matmul: {self._shape} @ {o._shape}")
            shape = (self._shape[0], o._shape[1])
        elif self._shape == o._shape:
            shape = self._shape
        else:
            shape = infer_broadcast_shape(self._shape, o._shape)
        return Block(shape, self.dtype, _tag(Bin(op, a, b, shape)), "FULL", "temp", temporary=True,
                     nest=tuple(_sl.nest()) if (self.nest or o.nest) else ())

    def __add__(self, o: Any) -> "Block": return self._binary(o, "add")
    def __sub__(self, o: Any) -> "Block": return self._binary(o, "sub")
    def __mul__(self, o: Any) -> "Block": return self._binary(o, "mul")
    def __truediv__(self, o: Any) -> "Block": return self._binary(o, "div")
    def __matmul__(self, o: Any) -> "Block": return self._binary(o, "matmul")

    def __floordiv__(self, o: Any) -> "Block": return self._binary(o, "floordiv")
    def __mod__(self, o: Any) -> "Block": return self._binary(o, "mod")

    def __pow__(self, o: Any) -> "Block":
        """block ** block, or block ** integer: ONE op on every tile as in the simulator, which hands both to
        torch (python/sim/block.py:981-1010)."""
        if isinstance(o, int) and not isinstance(o, bool):
            return self._unary("pow_imm", (float(o),))
        return self._binary(o, "pow")

    def _unary(self, op: str, params: Tuple[float, ...] = ()) -> "Block":
        return Block(self._shape, self.dtype, _tag(Un(op, self.value(), params)), "FULL", "temp", temporary=True,
                     nest=self.nest)


class _BlockContext:
    """`with cb.reserve() as blk` / `with cb.wait() as blk` wrapper; also usable without
    `with`, in which case it stands for the block (python/sim/cb.py:24-156)."""

    def __init__(self, cb: "CircularBuffer", block: Block, on_exit: Callable[[], None]):
        self._cb, self._block, self._on_exit = cb, block, on_exit

    def block(self) -> Block:
        return self._block

    @property
    def shape(self) -> Tuple[int, int]:
        return self._block.shape

    @property
    def _shape(self) -> Tuple[int, int]:
        return self._block.shape

    def __enter__(self) -> Block:
        return self._block

    def __exit__(self, exc_type: Any, exc: Any, tb: Any) -> None:
        if exc_type is not None and issubclass(exc_type, (_Abort, _BudgetSpent, NeedsConcrete)):
            return    # the trace is being abandoned: a half-written block must not travel on
        try:
            self._on_exit()
        except Exception:
            if exc_type is None:
                raise

    def __len__(self) -> int:
        return len(self._block)

    def __getitem__(self, idx: Any) -> Any:
        return self._block[idx]

    def __setitem__(self, idx: Any, v: Any) -> None:
        self._block[idx] = v

    def store(self, items: Any, acc: bool = False) -> None:
        self._block.store(items, acc=acc)

    def __add__(self, o: Any) -> Block: return self._block + o
    def __sub__(self, o: Any) -> Block: return self._block - o
    def __mul__(self, o: Any) -> Block: return self._block * o
    def __truediv__(self, o: Any) -> Block: return self._block / o
    def __matmul__(self, o: Any) -> Block: return self._block @ o
    def __pow__(self, o: Any) -> Block: return self._block ** o


class ReserveContext(_BlockContext):
    pass


class WaitContext(_BlockContext):
    pass


def _as_block(obj: Any) -> Any:
    if isinstance(obj, _BlockContext):
        return obj.block()
    return obj


class CircularBuffer:
    """Symbolic circular buffer.  `shape` is the block shape in tiles handed out by
    reserve()/wait(); capacity is shape[0]*shape[1]*buffer_factor tiles
    (python/sim/cb.py:184-225, python/ttl/circular_buffer.py:45-164)."""

    def __init__(self, element: Any, shape: Sequence[int], buffer_factor: int = 2, _live: bool = False):
        if len(shape) != 2:
            raise ValueError(f"Shape must be a 2-tuple, got {tuple(shape)}")
        if any((not isinstance(s, int)) or s <= 0 for s in shape):
            raise ValueError(f"Shape entries must be positive integers, got {tuple(shape)}")
        if not isinstance(buffer_factor, int) or not (1 <= buffer_factor <= 32):
            raise ValueError(f"buffer_factor must be in range [1, 32], got {buffer_factor}")
        self.element = element
        self._shape = (int(shape[0]), int(shape[1]))
        self._buffer_factor = buffer_factor
        self._live = _live
        self._name = "cb"
        self._queue: Deque[Any] = deque()      # Block, or _Seg (a run pushed by batched loops)
        self._pending_reserved: Optional[Block] = None
        self._pending_waited: Optional[Block] = None
        self._pending_n = 1                    # queue entries the waited block stands for
        self._strict = False
        self._pushed_in: set = set()           # live batched loops in whose body a push / a wait has happened
        self._waited_in: set = set()

    @property
    def shape(self) -> Tuple[int, int]:
        return self._shape

    @property
    def buffer_factor(self) -> int:
        return self._buffer_factor

    @property
    def capacity_tiles(self) -> int:
        return self._shape[0] * self._shape[1] * self._buffer_factor

    def _check_live(self) -> None:
        if not self._live:
            raise RuntimeError(
                "CircularBuffer was not properly initialized with a CBAPI instance. "
                "This likely means it was created outside of a kernel context. "
                "CircularBuffers must be created within @ttl.kernel decorated functions.")

    def _dtype(self) -> Any:
        return getattr(self.element, "dtype", None)

    def can_reserve(self) -> bool:
        if not self._strict:
            return True
        used = len(self._queue) + (1 if self._pending_waited is not None else 0)
        return used < self._buffer_factor

    def can_wait(self) -> bool:
        return len(self._queue) > 0

    def _available(self) -> int:
        return sum(q.left() if type(q) is _Seg else 1 for q in self._queue)

    @staticmethod
    def _once_per_body(seen: set, cur: Sequence[Any], what: str) -> set:
        """A batched loop body may touch one end of a circular buffer once: a second push (wait) would have to be
        interleaved with the first, iteration by iteration."""
        again = [f for f in cur if f in seen]
        if again:
            raise NeedsConcrete(_sl.sites_of(again), f"a loop body {what} the same circular buffer twice")
        return {f for f in seen if f in cur} | set(cur)

    def reserve(self) -> ReserveContext:
        self._check_live()
        tr = getattr(_tls, "trace", None)
        if tr is not None and tr.budget is not None:
            _spend()
        if self._pending_reserved is not None:
            raise RuntimeError(
                "Cannot call reserve() again before push(): "
                "CircularBuffer already has a pending reserved block. "
                "You must call push() before calling reserve() again.")
        if not self.can_reserve():
            _worker().block(self.can_reserve, f"{self._name}.reserve()")
        blk = Block(self._shape, self._dtype(), Zero(self._shape), "MW", "reserve", nest=tuple(_sl.nest()))
        self._pending_reserved = blk
        return ReserveContext(self, blk, self.push)

    def push(self) -> None:
        self._check_live()
        blk = self._pending_reserved
        if blk is None:
            raise RuntimeError("push() without a pending reserve()")
        if blk.state == "MW":
            raise RuntimeError(
                "Cannot push Block: it was reserved but never written "
                "(expected copy(..., blk) or blk.store(...))")
        if blk.state == "NAW":
            raise RuntimeError("Cannot push Block: copy into it has not been waited on (expected tx.wait())")
        cur = _sl.nest()
        if cur or blk.nest:
            if tuple(cur) != blk.nest:
                raise NeedsConcrete(_sl.sites_of(cur) | _sl.sites_of(blk.nest), "a block is pushed outside the loop that reserved it")
            self._pushed_in = self._once_per_body(self._pushed_in, cur, "pushes into")
            self._pending_reserved = None
            assert blk.expr is not None
            self._queue.append(_Seg(blk.shape, blk.dtype, blk.expr, tuple(f.n for f in cur)))
            blk.state = "OS"
            return
        self._pending_reserved = None
        self._queue.append(Block(blk.shape, blk.dtype, blk.expr, "FULL", "wait"))
        blk.state = "OS"

    def wait(self) -> WaitContext:
        self._check_live()
        tr = getattr(_tls, "trace", None)
        if tr is not None and tr.budget is not None:
            _spend()
        if self._pending_waited is not None:
            raise RuntimeError(
                "Cannot call wait() again before pop(): "
                "CircularBuffer already has a pending waited block. "
                "You must call pop() before calling wait() again.")
        cur = _sl.nest()
        if cur:
            # inside batched loops: one wait per iteration = the next m entries, which must be one pushed run
            self._waited_in = self._once_per_body(self._waited_in, cur, "waits on")
            m = 1
            for f in cur:
                m *= f.n
            if self._available() < m:
                _worker().block(lambda: self._available() >= m, f"{self._name}.wait()")
            head = self._queue[0]
            blk = head.take(m, cur) if type(head) is _Seg else None
            if blk is None:
                raise NeedsConcrete({cur[-1].site}, "the blocks a loop waits for were not pushed by a loop of the same shape")
            self._pending_waited, self._pending_n = blk, m
            return WaitContext(self, blk, self.pop)
        if not self._queue:
            _worker().block(self.can_wait, f"{self._name}.wait()")
        blk = self._queue[0]
        if type(blk) is _Seg:
            blk = blk.element()
        self._pending_waited, self._pending_n = blk, 1
        return WaitContext(self, blk, self.pop)

    def pop(self) -> None:
        self._check_live()
        blk = self._pending_waited
        if blk is None:
            raise RuntimeError("pop() without a pending wait()")
        self._pending_waited = None
        head = self._queue[0]
        if type(head) is _Seg:
            head.off += self._pending_n
            if head.off >= head.count:
                self._queue.popleft()
        else:
            self._queue.popleft()
        blk.state = "OS"

    def validate_no_pending_blocks(self) -> None:
        errs = []
        if self._pending_reserved is not None:
            errs.append("Pending reserved block. Did you forget to call push()?")
        if self._pending_waited is not None:
            errs.append("Pending waited block. Did you forget to call pop()?")
        if self._queue:
            errs.append(f"{self._available()} pushed block(s) were never consumed")
        if errs:
            raise RuntimeError(f"CircularBuffer {self._name} has incomplete blocks at end of execution:\n"
                               + "\n".join(f"  - {e}" for e in errs))

    def __repr__(self) -> str:
        return (f"CircularBuffer(shape={self._shape}, capacity_tiles={self.capacity_tiles}, "
                f"buffer_factor={self._buffer_factor})")


def make_circular_buffer_like(element: Any, shape: Sequence[int], buffer_factor: int = 2) -> CircularBuffer:
    return CircularBuffer(element, shape, buffer_factor)


# --------------------------------------------------------------------------- #
# Pipes
# --------------------------------------------------------------------------- #
def core_coords(cid: int, grid: Tuple[int, ...], dims: int) -> Any:
    """Coordinates of linear core id `cid` (last grid dim fastest), flattened or padded
    to `dims` entries exactly as python/sim/kernel.py:158-199 does."""
    coords: List[int] = []
    for s in reversed(grid):
        coords.append(cid % s)
        cid //= s
    coords.reverse()
    if dims < len(coords):
        flat = coords[0]
        for i in range(1, len(coords) - dims + 1):
            flat = flat * grid[i] + coords[i]
        coords = [flat] + coords[len(coords) - dims + 1:]
    while len(coords) < dims:
        coords.append(0)
    return coords[0] if dims == 1 else tuple(coords)


def grid_size_of(grid: Tuple[int, ...], dims: int) -> Any:
    """python/sim/kernel.py:89-155."""
    if dims <= 0:
        raise ValueError(f"dims must be positive, got {dims}")
    n = len(grid)
    if dims == n:
        res = tuple(grid)
    elif dims < n:
        flat = 1
        for d in grid[dims - 1:]:
            flat *= d
        res = tuple(grid[:dims - 1]) + (flat,)
    else:
        res = tuple(grid) + (1,) * (dims - n)
    return res[0] if dims == 1 else res


def flatten_core_index(core_coord: Any, grid: Optional[Tuple[int, ...]] = None) -> int:
    """python/sim/kernel.py:52-87 (there the grid always comes from the kernel context)."""
    if isinstance(core_coord, int):
        return core_coord
    if grid is None:
        grid = current_grid()
    coords = list(core_coord)
    lin = coords[0]
    for i in range(1, len(coords)):
        lin = lin * grid[i] + coords[i]
    return int(lin)


def _dst_cores(dst: Any, grid: Tuple[int, ...]) -> List[int]:
    """Linear ids of the destination cores of a pipe (python/sim/pipe.py:73-203)."""
    total = 1
    for g in grid:
        total *= g
    if isinstance(dst, int):
        return [dst]
    if isinstance(dst, tuple) and any(isinstance(i, slice) for i in dst):
        dims = len(dst)
        gs = grid_size_of(grid, dims)
        gs = gs if isinstance(gs, tuple) else (gs,)
        out = []
        for cid in range(total):
            cc = core_coords(cid, grid, dims)
            cc = cc if isinstance(cc, tuple) else (cc,)
            ok = True
            for i, item in enumerate(dst):
                if isinstance(item, slice):
                    start = item.start if item.start is not None else 0
                    stop = item.stop if item.stop is not None else gs[i]
                    step = item.step if item.step is not None else 1
                    if not (start <= cc[i] < stop and (cc[i] - start) % step == 0):
                        ok = False
                        break
                elif cc[i] != item:
                    ok = False
                    break
            if ok:
                out.append(cid)
        return out
    if isinstance(dst, tuple) and len(dst) == 2 and all(isinstance(i, tuple) for i in dst):
        first, second = dst
        dims = len(first)
        out = []
        for cid in range(total):
            cc = core_coords(cid, grid, dims)
            cc = cc if isinstance(cc, tuple) else (cc,)
            if all(min(first[i], second[i]) <= cc[i] <= max(first[i], second[i]) for i in range(dims)):
                out.append(cid)
        return out
    if isinstance(dst, tuple):
        dims = len(dst)
        return [cid for cid in range(total) if core_coords(cid, grid, dims) == dst]
    return []


class Pipe:
    """Description of a core-to-core(s) transfer (python/sim/typedefs.py:41-101)."""

    def __init__(self, src_core: Any, dst_core_range: Any):
        self.src_core = src_core
        self.dst_core_range = dst_core_range

    def _key(self) -> Any:
        def h(o: Any) -> Any:
            if isinstance(o, slice):
                return ("slice", o.start, o.stop, o.step)
            if isinstance(o, (tuple, list)):
                return tuple(h(i) for i in o)
            return o
        return (h(self.src_core), h(self.dst_core_range))

    def __hash__(self) -> int:
        return hash(self._key())

    def __eq__(self, other: object) -> bool:
        return isinstance(other, Pipe) and self._key() == other._key()

    def __repr__(self) -> str:
        return f"Pipe(src_core={self.src_core}, dst_core_range={self.dst_core_range})"

    def has_current_core(self) -> bool:
        grid = current_grid()
        cid = current_core()
        return cid == flatten_core_index(self.src_core, grid) or cid in _dst_cores(self.dst_core_range, grid)


class SrcPipeIdentity:
    def __init__(self, pipe: Pipe):
        self.pipe = pipe

    @property
    def dst(self) -> Any:
        return self.pipe.dst_core_range


class DstPipeIdentity:
    def __init__(self, pipe: Pipe):
        self.pipe = pipe

    @property
    def src(self) -> Any:
        return self.pipe.src_core


class PipeNet:
    """python/sim/pipe.py:203-270."""

    def __init__(self, pipes: List[Pipe]):
        self._pipes = list(pipes)

    def if_src(self, cond_fun: Callable[[SrcPipeIdentity], Any]) -> None:
        grid, cid = current_grid(), current_core()
        for p in self._pipes:
            if cid == flatten_core_index(p.src_core, grid):
                cond_fun(SrcPipeIdentity(p))

    def if_dst(self, cond_fun: Callable[[DstPipeIdentity], Any]) -> None:
        grid, cid = current_grid(), current_core()
        for p in self._pipes:
            if cid in _dst_cores(p.dst_core_range, grid):
                cond_fun(DstPipeIdentity(p))


# --------------------------------------------------------------------------- #
# copy
# --------------------------------------------------------------------------- #
def _shape_in_tiles_with_skip(shape: Tuple[int, ...]) -> Tuple[int, ...]:
    return tuple(1 if d == 1 else d // t for d, t in zip(shape, TILE_SHAPE))


class CopyTransaction:
    """Handle returned by ttl.copy; the transfer takes effect at wait()
    (python/sim/copy.py:37-153)."""

    def __init__(self, src: Any, dst: Any):
        self._src, self._dst = src, dst
        self._completed = False
        self._line = _site()
        s, d = _as_block(src), _as_block(dst)
        s = s.pipe if isinstance(s, (SrcPipeIdentity, DstPipeIdentity)) else s
        d = d.pipe if isinstance(d, (SrcPipeIdentity, DstPipeIdentity)) else d
        self._s, self._d = s, d
        if isinstance(s, _ttnn.Tensor) and isinstance(d, Block):
            self._mode = "t2b"
            if len(s.shape) != 2:
                raise ValueError(f"Tensor must be 2-dimensional, got shape {s.shape}")
            self._check_dst_block(d)
            st = _shape_in_tiles_with_skip(s.shape)
            if st != d.shape:
                raise ValueError(
                    f"Tensor shape {s.shape} (={st} tiles) does not match "
                    f"Block shape {d.shape} tiles (={tuple(a * b for a, b in zip(d.shape, TILE_SHAPE))} elements)")
            d.state = "NAW"
        elif isinstance(s, Block) and isinstance(d, _ttnn.Tensor):
            self._mode = "b2t"
            if len(d.shape) != 2:
                raise ValueError(f"Tensor must be 2-dimensional, got shape {d.shape}")
            dt = _shape_in_tiles_with_skip(d.shape)
            if dt != s.shape:
                raise ValueError(
                    f"Tensor shape {d.shape} (={dt} tiles) does not match "
                    f"Block shape {s.shape} tiles (={tuple(a * b for a, b in zip(s.shape, TILE_SHAPE))} elements)")
            s.value()
        elif isinstance(s, Block) and isinstance(d, Pipe):
            if _sl.nest():
                raise NeedsConcrete(_sl.live_sites(), "a pipe is used inside the loop")
            self._mode = "b2p"
            s.value()
        elif isinstance(s, Pipe) and isinstance(d, Block):
            if _sl.nest():
                raise NeedsConcrete(_sl.live_sites(), "a pipe is used inside the loop")
            self._mode = "p2b"
            self._check_dst_block(d)
            d.state = "NAW"
        else:
            raise ValueError(f"No copy handler registered for ({type(src).__name__}, {type(dst).__name__})")

    @staticmethod
    def _check_dst_block(d: Block) -> None:
        if d.state == "OS":
            raise RuntimeError("Cannot write to Block: Block has no access (OS state). Current state: OS")
        if d.kind == "wait":
            raise RuntimeError("Cannot copy into a waited block")
        if d.state == "NAW":
            raise RuntimeError(
                "Cannot write to Block: Block is locked as copy destination until tx.wait() completes "
                "(copy lock error). Current state: NAW, Expected operations: [TX_WAIT]")

    def can_wait(self) -> bool:
        if self._mode == "p2b":
            return _trace().pipe_ready(self._s, current_core())
        return True

    @property
    def is_completed(self) -> bool:
        return self._completed

    def wait(self) -> None:
        if self._completed:
            return
        tr = _trace()
        s, d = self._s, self._d
        if self._mode == "t2b":
            base, r0, r1, c0, c1 = s._origin if s._origin is not None else (s, 0, s.tile_shape()[0], 0, s.tile_shape()[1])
            tr.note_input(base)
            cur = _sl.nest()
            if cur or d.nest:
                if tuple(cur) != d.nest:
                    raise NeedsConcrete(_sl.sites_of(cur) | _sl.sites_of(d.nest), "a copy fills a block of another loop")
                r0, r1, c0, c1 = (_sl.as_coord(x) for x in (r0, r1, c0, c1))
            d.expr = Leaf(base, r0, r1, c0, c1)
            d.expr.shape = d.shape
            d.expr.line = self._line
            d.state = "FULL"
        elif self._mode == "b2t":
            base, r0, r1, c0, c1 = d._origin if d._origin is not None else (d, 0, d.tile_shape()[0], 0, d.tile_shape()[1])
            v = s.value()
            cur = _sl.nest()
            if cur:
                r0, r1, c0, c1 = (_sl.as_coord(x) for x in (r0, r1, c0, c1))
                tr.writes.append(BatchedWrite(base, r0, r1, c0, c1, v, current_core(), self._line, tuple(f.n for f in cur)))
            else:
                tr.writes.append(Write(base, r0, r1, c0, c1, v, current_core(), self._line))
        elif self._mode == "b2p":
            tr.pipe_send(d, s.value(), len(_dst_cores(d.dst_core_range, current_grid())))
        else:  # p2b
            cid = current_core()
            if not tr.pipe_ready(s, cid):
                _worker().block(lambda: tr.pipe_ready(s, cid), f"copy({s!r}, block).wait()")
            v = tr.pipe_recv(s)
            if v.shape[0] * v.shape[1] != len(d):
                raise ValueError(
                    f"Destination Block length ({len(d)}) does not match pipe data length ({v.shape[0] * v.shape[1]})")
            d.expr = v
            d.state = "FULL"
        self._completed = True


def copy(src: Any, dst: Any) -> CopyTransaction:
    return CopyTransaction(src, dst)


# --------------------------------------------------------------------------- #
# Trace of one kernel call
# --------------------------------------------------------------------------- #
class Trace:
    def __init__(self, grid: Tuple[int, ...]):
        self.grid = grid
        self.writes: List[Write] = []
        self.inputs: List[_ttnn.Tensor] = []
        self._pipes: Dict[Pipe, Deque[List[Any]]] = {}
        self.batched_loops = 0          # batched loop instances that ran (symloop.py)
        self.budget: Optional[int] = None    # circular-buffer operations each thread may make (verification runs only)

    def finish(self) -> None:
        """One Write per iteration in place of every BatchedWrite, in program order; batched matmul writes stay
        as they are (the recogniser checks all their iterations at once)."""
        if any(isinstance(w, BatchedWrite) for w in self.writes):
            out: List[Write] = []
            for w in self.writes:
                if isinstance(w, BatchedWrite) and not w.plain_matmul():
                    out.extend(w.expand())
                else:
                    out.append(w)
            self.writes = out

    def note_input(self, t: "_ttnn.Tensor") -> None:
        for x in self.inputs:
            if x is t:
                return
        self.inputs.append(t)

    def pipe_send(self, pipe: Pipe, value: Expr, receivers: int) -> None:
        self._pipes.setdefault(pipe, deque()).append([value, max(1, receivers)])

    def pipe_ready(self, pipe: Pipe, core: int) -> bool:
        q = self._pipes.get(pipe)
        return bool(q)

    def pipe_recv(self, pipe: Pipe) -> Expr:
        q = self._pipes[pipe]
        head = q[0]
        head[1] -= 1
        if head[1] == 0:
            q.popleft()
        return head[0]


def _trace() -> Trace:
    t = getattr(_tls, "trace", None)
    if t is None:
        raise RuntimeError("ttl.copy must be called within a kernel thread")
    return t


def thread_kind() -> str:
    return getattr(_tls, "kind", "")


# --------------------------------------------------------------------------- #
# Running a program on every core
# --------------------------------------------------------------------------- #
def _make_cell(value: Any) -> Any:
    def inner() -> Any:
        return value
    assert inner.__closure__ is not None
    return inner.__closure__[0]


def _rebind(func: types.FunctionType, per_core: Dict[int, Any]) -> types.FunctionType:
    """New function object whose closure cells holding circular buffers (or containers
    of per-core state) point at this core's private copies (python/sim/program.py:69-97)."""
    free = func.__code__.co_freevars
    cells = []
    for name, cell in zip(free, func.__closure__ or ()):
        try:
            v = cell.cell_contents
        except ValueError:
            cells.append(cell)
            continue
        cells.append(_make_cell(per_core[id(v)]) if id(v) in per_core else cell)
    return types.FunctionType(func.__code__, func.__globals__, func.__name__, func.__defaults__, tuple(cells))


BATCH_LOOPS = os.environ.get("TTLB200_BATCH_LOOPS", "1") != "0"
VERIFY_BATCHED = os.environ.get("TTLB200_TRACE_VERIFY", "1") != "0"
VERIFY_BUDGET = 6000      # circular-buffer operations traced iteration by iteration per sampled core
_NOBATCH: Dict[Any, set] = {}      # per program (code objects of its threads): loop sites that must stay concrete


def _spend() -> None:
    w = _tls.worker
    w.budget -= 1
    if w.budget < 0:
        raise _BudgetSpent()


def run_program(threads: List[Tuple[str, types.FunctionType]], grid: Tuple[int, ...], strict_cb: bool = False) -> Trace:
    """Execute the thread functions of one kernel call on every core and return the trace.

    `threads` is [(kind, function)] with kind "compute" or "dm".  Counted loops that pass the checks of
    symloop.py run once for all their iterations; when a loop body turns out to need its iterations one by one
    the trace starts again with that loop run conventionally.  A batched trace is checked against a conventional
    trace of the first writes of a few sampled cores before it is used.
    """
    batching = BATCH_LOOPS and not strict_cb
    if not batching:
        return _run_once(threads, grid, strict_cb, False, frozenset())
    key = tuple(fn.__code__ for _, fn in threads)
    nobatch = _NOBATCH.setdefault(key, set())
    fast = [(kind, _sl.transform(fn)) for kind, fn in threads]
    if all(a[1] is b[1] for a, b in zip(fast, threads)):
        return _run_once(threads, grid, strict_cb, False, frozenset())
    for _ in range(64):
        try:
            trace = _run_once(fast, grid, strict_cb, True, frozenset(nobatch))
        except NeedsConcrete as e:
            if not e.sites or e.sites <= nobatch:
                break         # no loop left to blame: trace conventionally
            nobatch |= e.sites
            continue
        if trace.batched_loops and VERIFY_BATCHED and not _verify(threads, grid, trace):
            import warnings

            warnings.warn("ttl_b200: the batched trace of a tile program disagrees with its iteration-by-iteration trace "
                          "on a sampled core; tracing every iteration instead (TTLB200_BATCH_LOOPS=0 skips the attempt)",
                          RuntimeWarning, stacklevel=2)
            break
        return trace
    return _run_once(threads, grid, strict_cb, False, frozenset())


def same_expr(a: Expr, b: Expr) -> bool:
    """Structural equality of two expressions; runs of accumulated terms are compared term by term."""
    if isinstance(a, Acc) or isinstance(b, Acc):
        ta = _flat_terms(a)
        tb = _flat_terms(b)
        return len(ta) == len(tb) and all(same_expr(x, y) for x, y in zip(ta, tb))
    if type(a) is not type(b) or tuple(a.shape) != tuple(b.shape):
        return False
    if isinstance(a, Leaf):
        return (a.tensor is b.tensor and a.first == b.first
                and all(int(np.asarray(x).reshape(-1)[0]) == int(np.asarray(y).reshape(-1)[0])
                        for x, y in zip((a.r0, a.r1, a.c0, a.c1), (b.r0, b.r1, b.c0, b.c1))))
    if isinstance(a, Un):
        return a.op == b.op and a.params == b.params and same_expr(a.x, b.x)
    if isinstance(a, Bin):
        return a.op == b.op and same_expr(a.a, b.a) and same_expr(a.b, b.b)
    if isinstance(a, Red):
        return (a.op == b.op and a.dims == b.dims and same_expr(a.x, b.x) and (a.scaler is None) == (b.scaler is None)
                and (a.scaler is None or same_expr(a.scaler, b.scaler)))
    if isinstance(a, Rep):
        ta, tb = a.terms(), b.terms()
        return len(ta) == len(tb) and all(same_expr(x, y) for x, y in zip(ta, tb))
    return isinstance(a, Zero)


def _flat_terms(e: Expr) -> List[Expr]:
    out: List[Expr] = []
    for t in (e.terms if isinstance(e, Acc) else [e]):
        if isinstance(t, Rep):
            out.extend(t.terms())
        else:
            out.append(t)
    return out


def _verify(threads: List[Tuple[str, types.FunctionType]], grid: Tuple[int, ...], trace: Trace) -> bool:
    """Trace the first, the middle and the last core that wrote anything iteration by iteration (each thread up
    to VERIFY_BUDGET circular-buffer operations) and compare the writes they get that far with the batched trace's."""
    cores = sorted({w.core for w in trace.writes})
    if not cores:
        return True
    for core in sorted({cores[0], cores[len(cores) // 2], cores[-1]}):
        probe = Trace(grid)
        probe.budget = VERIFY_BUDGET
        try:
            _run_once(threads, grid, False, False, frozenset(), only_core=core, trace=probe)
        except BaseException:   # noqa: BLE001 - a probe that stops early (budget, starvation) still gives a prefix
            pass
        want = probe.writes
        got: List[Write] = []
        for w in trace.writes:
            if w.core != core:
                continue
            if len(got) >= len(want):
                break
            got.extend(w.expand(len(want) - len(got)) if isinstance(w, BatchedWrite) else [w])
        if len(want) > len(got) or not want:
            return False
        for a, b in zip(want, got):
            if (a.tensor is not b.tensor or (a.r0, a.r1, a.c0, a.c1) != (b.r0, b.r1, b.c0, b.c1)
                    or not same_expr(a.expr, b.expr)):
                return False
    return True


def _run_once(threads: List[Tuple[str, types.FunctionType]], grid: Tuple[int, ...], strict_cb: bool, batching: bool,
              nobatch: Any, only_core: Optional[int] = None, trace: Optional[Trace] = None) -> Trace:
    total = 1
    for g in grid:
        total *= g
    if trace is None:
        trace = Trace(grid)
    sched = Scheduler(grid, trace)
    sched.batching, sched.nobatch = batching, nobatch
    all_cbs: List[Tuple[int, CircularBuffer]] = []
    # closure values shared by the thread functions
    shared: Dict[int, Any] = {}
    for _, fn in threads:
        for cell in fn.__closure__ or ():
            try:
                v = cell.cell_contents
            except ValueError:
                continue
            shared[id(v)] = v
    n_cbs = sum(1 for v in shared.values() if isinstance(v, CircularBuffer)) + sum(
        sum(1 for x in v if isinstance(x, CircularBuffer)) for v in shared.values() if isinstance(v, (list, tuple)))
    if n_cbs > MAX_CBS:
        raise RuntimeError(f"A kernel may use at most {MAX_CBS} circular buffers, got {n_cbs}")
    for core in range(total) if only_core is None else [only_core]:
        per_core: Dict[int, Any] = {}

        def fresh_cb(v: CircularBuffer) -> CircularBuffer:
            if id(v) not in per_core:
                cb = CircularBuffer(v.element, v.shape, v.buffer_factor, _live=True)
                cb._strict = strict_cb
                per_core[id(v)] = cb
                all_cbs.append((core, cb))
            return per_core[id(v)]

        def clone(v: Any) -> Any:
            """Per-core copy of a container; circular buffers inside it become this core's."""
            if isinstance(v, CircularBuffer):
                return fresh_cb(v)
            if isinstance(v, list):
                return [clone(x) for x in v]
            if isinstance(v, tuple) and any(isinstance(x, (CircularBuffer, list, tuple, dict)) for x in v):
                return tuple(clone(x) for x in v)
            if isinstance(v, dict):
                return {k: clone(x) for k, x in v.items()}
            if isinstance(v, set):
                return _copy.deepcopy(v)
            return v

        for key, v in shared.items():
            if isinstance(v, CircularBuffer):
                fresh_cb(v)
            elif isinstance(v, (list, dict, set, tuple)):
                c = clone(v)
                if c is not v:
                    per_core[key] = c
        # name buffers after the variables that hold them (for deadlock reports)
        for _, fn in threads:
            for name, cell in zip(fn.__code__.co_freevars, fn.__closure__ or ()):
                try:
                    v = cell.cell_contents
                except ValueError:
                    continue
                if isinstance(v, CircularBuffer) and id(v) in per_core:
                    per_core[id(v)]._name = name
        order = sorted(range(len(threads)), key=lambda i: 0 if threads[i][0] == "dm" else 1)
        for i in order:
            kind, fn = threads[i]
            sched.add(f"core{core}-{fn.__name__}", _rebind(fn, per_core), core, kind)
    sched.run()
    errs = []
    for core, cb in all_cbs:
        try:
            cb.validate_no_pending_blocks()
        except RuntimeError as e:
            errs.append(f"core{core}.{cb._name}: {e}")
    if errs:
        raise RuntimeError("Kernel execution completed with incomplete CircularBuffer operations:\n" + "\n".join(errs))
    trace.finish()
    return trace
