"""Batched execution of counted loops in tile-program threads.

A tile program written the way the reference's examples are (examples/multicore_matmul.py:92-139,
examples/singlecore_matmul.py:36-45) steps through its tiles one at a time: `for k in range(Kt)` around a
reserve / copy / push, a wait / matmul / pop.  Tracing such a loop iteration by iteration costs time in
proportion to the number of tile operations (16.7 million for an 8192-cubed matmul in 1x1-tile blocks).  The
reference meets the same loops with an AST transform of the thread functions (python/sim/xformyield.py:295-337
rewrites them into generators); this module transforms them too, for a different purpose: a counted loop whose
body passes a static check runs ONCE with its loop variable standing for all of its values at the same time
(`SymInt`, a NumPy array with one axis per live loop), so the cost of tracing follows the program text.

What may be batched is decided conservatively, first on the syntax tree (no break / return / yield, no store
to a name that is carried from one iteration to the next or read after the loop, no mutation of containers) and
then while running: anything that needs a concrete value of the loop variable (`if k == 0`, `range(k)`,
`blocks[k]`, a second push into the same circular buffer in one iteration, ...) raises `NeedsConcrete`, which
names the loops involved; the trace is then started again with those loops run iteration by iteration.
"""

from __future__ import annotations

import ast
import inspect
import itertools
import textwrap
import threading
import types
from typing import Any, Dict, Iterable, List, Optional, Sequence, Set, Tuple

import numpy as np

NEST_AXES = 4      # array axes 0..3: one per live batched loop, outermost first
REP_AXES = 4       # array axes 4..7: sequence axes of accumulated terms (trace.Rep)
NDIM = NEST_AXES + REP_AXES
MIN_TRIP = 4       # shorter loops are not worth batching

Site = Tuple[str, int, int]    # (file, line, column) of a `for` statement


class NeedsConcrete(Exception):
    """Raised while a batched loop body runs when it cannot stand for all iterations at once."""

    def __init__(self, sites: Iterable[Site], why: str):
        super().__init__(why)
        self.sites = frozenset(sites)
        self.why = why


class Frame:
    """One live batched loop: `n` iterations along array axis `axis`."""

    __slots__ = ("fid", "site", "n", "axis")
    _ids = itertools.count(1)

    def __init__(self, site: Site, n: int, axis: int):
        self.fid, self.site, self.n, self.axis = next(Frame._ids), site, n, axis


class _State(threading.local):
    nest: Optional[List[Frame]] = None     # None: not inside a traced tile-program thread
    enabled = False
    nobatch: Set[Site] = frozenset()       # type: ignore[assignment]
    batched_loops = 0                      # batched loop instances entered by this thread


STATE = _State()


def nest() -> Sequence[Frame]:
    n = STATE.nest
    return n if n is not None else ()


def sites_of(frames: Iterable[Frame]) -> Set[Site]:
    return {f.site for f in frames}


def live_sites() -> Set[Site]:
    return sites_of(nest())


def require_live(frames: Sequence[Frame], what: str) -> None:
    """`frames` (the loops a value was made under) must be the outermost live loops, in order."""
    cur = nest()
    if len(frames) > len(cur) or any(a is not b for a, b in zip(frames, cur)):
        raise NeedsConcrete(sites_of(frames) | sites_of(cur), f"{what} is used outside the loop iteration that made it")


# --------------------------------------------------------------------------- #
# the loop variable
# --------------------------------------------------------------------------- #
class SymInt:
    """An integer that stands for the values a loop variable (or arithmetic on it) takes over all iterations
    of the live batched loops: `v` has NDIM axes, axis i varying with the loop at nest depth i."""

    __slots__ = ("v", "frames")

    def __init__(self, v: np.ndarray, frames: Tuple[Frame, ...]):
        self.v, self.frames = v, frames

    # -- helpers -----------------------------------------------------------
    def _varying(self) -> Set[Site]:
        s = {f.site for f in self.frames if self.v.shape[f.axis] > 1}
        return s or sites_of(self.frames)

    def _fail(self, why: str) -> "NeedsConcrete":
        return NeedsConcrete(self._varying(), f"the loop variable {why}")

    def const(self) -> Optional[int]:
        """The value when it is the same for every iteration, else None."""
        lo = int(self.v.min())
        return lo if lo == int(self.v.max()) else None

    def array(self) -> np.ndarray:
        require_live(self.frames, "a value derived from a loop variable")
        return self.v

    def _pair(self, o: Any) -> Any:
        if isinstance(o, SymInt):
            a, b = self.frames, o.frames
            short, long_ = (a, b) if len(a) <= len(b) else (b, a)
            if any(x is not y for x, y in zip(short, long_)):
                raise NeedsConcrete(sites_of(a) | sites_of(b), "values of different loop iterations are combined")
            return o.v, long_
        if isinstance(o, (bool, np.bool_)):
            return NotImplemented, None
        if isinstance(o, (int, np.integer)):
            return int(o), self.frames
        return NotImplemented, None

    def _bin(self, o: Any, fn: Any, swap: bool = False) -> Any:
        ov, frames = self._pair(o)
        if ov is NotImplemented:
            return NotImplemented
        return SymInt(fn(ov, self.v) if swap else fn(self.v, ov), frames)

    # -- arithmetic ----------------------------------------------------------
    def __add__(self, o: Any) -> Any: return self._bin(o, np.add)
    def __radd__(self, o: Any) -> Any: return self._bin(o, np.add, True)
    def __sub__(self, o: Any) -> Any: return self._bin(o, np.subtract)
    def __rsub__(self, o: Any) -> Any: return self._bin(o, np.subtract, True)
    def __mul__(self, o: Any) -> Any: return self._bin(o, np.multiply)
    def __rmul__(self, o: Any) -> Any: return self._bin(o, np.multiply, True)
    def __floordiv__(self, o: Any) -> Any: return self._bin(o, np.floor_divide)
    def __rfloordiv__(self, o: Any) -> Any: return self._bin(o, np.floor_divide, True)
    def __mod__(self, o: Any) -> Any: return self._bin(o, np.mod)
    def __rmod__(self, o: Any) -> Any: return self._bin(o, np.mod, True)
    def __neg__(self) -> "SymInt": return SymInt(-self.v, self.frames)
    def __pos__(self) -> "SymInt": return self

    def __divmod__(self, o: Any) -> Any:
        q = self.__floordiv__(o)
        return NotImplemented if q is NotImplemented else (q, self.__mod__(o))

    def __truediv__(self, o: Any) -> Any: raise self._fail("is divided with /")
    def __rtruediv__(self, o: Any) -> Any: raise self._fail("is divided with /")
    def __pow__(self, o: Any) -> Any: raise self._fail("is raised to a power")

    # -- anything that needs ONE value ---------------------------------------
    def _cmp(self, o: Any, fn: Any) -> bool:
        d = self.__sub__(o)
        if d is NotImplemented:
            raise self._fail("is compared with a non-integer")
        r = fn(d.v, 0)
        if r.all():
            return True
        if not r.any():
            return False
        raise self._fail("is compared (the result differs between iterations)")

    def __eq__(self, o: Any) -> bool: return self._cmp(o, lambda a, b: a == b)  # type: ignore[override]
    def __ne__(self, o: Any) -> bool: return self._cmp(o, lambda a, b: a != b)  # type: ignore[override]
    def __lt__(self, o: Any) -> bool: return self._cmp(o, lambda a, b: a < b)
    def __le__(self, o: Any) -> bool: return self._cmp(o, lambda a, b: a <= b)
    def __gt__(self, o: Any) -> bool: return self._cmp(o, lambda a, b: a > b)
    def __ge__(self, o: Any) -> bool: return self._cmp(o, lambda a, b: a >= b)

    def _one(self, why: str) -> int:
        c = self.const()
        if c is None:
            raise self._fail(why)
        return c

    def __index__(self) -> int: return self._one("is used as an index or a count")
    def __int__(self) -> int: return self._one("is converted to int")
    def __bool__(self) -> bool: return bool(self._one("is used as a condition"))
    def __hash__(self) -> int: return hash(self._one("is used as a key"))
    def __float__(self) -> float: return float(self._one("is converted to float"))

    def __repr__(self) -> str:
        return f"SymInt(shape={tuple(s for s in self.v.shape if s > 1)})"


def as_coord(x: Any) -> Any:
    """A tile coordinate as it is kept in expressions: a Python int, or (batched) an int64 array with NDIM axes."""
    if isinstance(x, SymInt):
        c = x.const() if x.v.size <= 64 else None
        return c if c is not None else x.array()
    return x


def const_extent(lo: Any, hi: Any, what: str) -> int:
    """hi - lo, which must be the same for every iteration (block shapes are fixed)."""
    d = hi - lo
    if isinstance(d, SymInt):
        c = d.const()
        if c is None:
            raise d._fail(f"changes the size of {what}")
        return c
    return int(d)


# --------------------------------------------------------------------------- #
# run time of a transformed loop
# --------------------------------------------------------------------------- #
def _columns(it: Any) -> Optional[Tuple[List[np.ndarray], int, bool]]:
    """The values `it` yields, as one array per unpacked element: (columns, count, scalar?)."""
    if isinstance(it, range):
        n = len(it)
        return ([np.arange(it.start, it.stop, it.step, dtype=np.int64)], n, True) if n else None
    if isinstance(it, (list, tuple)) and len(it) >= MIN_TRIP:
        first = it[0]
        if type(first) is int:
            if all(type(x) is int for x in it):
                return [np.asarray(it, dtype=np.int64)], len(it), True
            return None
        if type(first) is tuple and first and all(
                type(x) is tuple and len(x) == len(first) and all(type(y) is int for y in x) for x in it):
            arr = np.asarray(it, dtype=np.int64)
            return [arr[:, j] for j in range(arr.shape[1])], len(it), False
    return None


def loop(it: Any, site: Site) -> Any:
    """Iterator for `for ... in it` at `site`: all values at once when the loop can be batched, else `it`."""
    st = STATE
    cur = st.nest
    if cur is None or not st.enabled or site in st.nobatch or len(cur) >= NEST_AXES:
        yield from it
        return
    cols = _columns(it)
    if cols is None or cols[1] < MIN_TRIP:
        yield from it
        return
    arrays, n, scalar = cols
    f = Frame(site, n, len(cur))
    cur.append(f)
    st.batched_loops += 1
    try:
        shape = [1] * NDIM
        shape[f.axis] = n
        frames = tuple(cur)
        vals = [SymInt(a.reshape(shape), frames) for a in arrays]
        yield vals[0] if scalar else tuple(vals)
    finally:
        if cur and cur[-1] is f:
            cur.pop()


def pop_call(obj: Any) -> Any:
    """`obj.pop()` inside a loop body that may be batched: a circular buffer pops its waited block; anything
    else (a list used as a work queue) changes from iteration to iteration."""
    if not hasattr(obj, "_pending_waited") and nest():
        raise NeedsConcrete(live_sites(), "a container is popped inside the loop")
    return obj.pop()


# --------------------------------------------------------------------------- #
# static check and transform
# --------------------------------------------------------------------------- #
_MUTATORS = {"append", "extend", "insert", "add", "update", "remove", "clear", "setdefault", "popleft", "appendleft",
             "discard", "sort", "reverse", "popitem", "send", "throw"}


def _names(node: ast.AST, ctx: type) -> Set[str]:
    return {n.id for n in ast.walk(node) if isinstance(n, ast.Name) and isinstance(n.ctx, ctx)}


def _target_names(t: ast.AST) -> Optional[Set[str]]:
    """Names bound by an assignment target; None when it stores into a container or an attribute."""
    if isinstance(t, ast.Name):
        return {t.id}
    if isinstance(t, (ast.Tuple, ast.List)):
        out: Set[str] = set()
        for e in t.elts:
            s = _target_names(e.value if isinstance(e, ast.Starred) else e)
            if s is None:
                return None
            out |= s
        return out
    return None


def _reads_before_write(stmts: Sequence[ast.stmt], names: Set[str], written: Set[str]) -> Tuple[Set[str], Set[str]]:
    """Names of `names` that may be read before this statement list has definitely written them, and the names
    it definitely writes (`written`: already written on entry)."""
    reads: Set[str] = set()
    w = set(written)

    def loads(node: Optional[ast.AST]) -> None:
        if node is not None:
            reads.update(n for n in _names(node, ast.Load) if n in names and n not in w)

    for s in stmts:
        if isinstance(s, ast.Assign):
            loads(s.value)
            for t in s.targets:
                tn = _target_names(t)
                if tn is None:
                    loads(t)
                else:
                    w |= tn
        elif isinstance(s, ast.AugAssign):
            loads(s.value)
            loads(s.target)
            if isinstance(s.target, ast.Name):
                if s.target.id in names and s.target.id not in w:
                    reads.add(s.target.id)
                w.add(s.target.id)
        elif isinstance(s, ast.AnnAssign):
            loads(s.value)
            if s.value is not None and isinstance(s.target, ast.Name):
                w.add(s.target.id)
        elif isinstance(s, ast.If):
            loads(s.test)
            r1, w1 = _reads_before_write(s.body, names, w)
            r2, w2 = _reads_before_write(s.orelse, names, w)
            reads |= r1 | r2
            w = w1 & w2
        elif isinstance(s, (ast.For, ast.AsyncFor)):
            loads(s.iter)
            tn = _target_names(s.target) or set()
            r1, _ = _reads_before_write(s.body, names, w | tn)
            r2, _ = _reads_before_write(s.orelse, names, w)
            reads |= r1 | r2
        elif isinstance(s, ast.While):
            loads(s.test)
            r1, _ = _reads_before_write(list(s.body) + list(s.orelse), names, w)
            reads |= r1
        elif isinstance(s, (ast.With, ast.AsyncWith)):
            for item in s.items:
                loads(item.context_expr)
                if item.optional_vars is not None:
                    tn = _target_names(item.optional_vars)
                    if tn is None:
                        loads(item.optional_vars)
                    else:
                        w |= tn
            r1, w1 = _reads_before_write(s.body, names, w)
            reads |= r1
            w = w1
        elif isinstance(s, (ast.Return, ast.Raise)):
            loads(s)
            break
        else:   # expressions, try blocks, nested definitions, ...: every load counts, no write is certain
            loads(s)
    return reads, w


class _Transformer(ast.NodeTransformer):
    """Rewrites `for T in IT:` into `for T in __ttl_loop__(IT, site):` where the static check passes."""

    def __init__(self, filename: str):
        self.filename = filename
        self.changed = 0
        self._after: List[List[ast.stmt]] = []    # statement lists that run after the node being visited

    # statement lists are walked by hand so that each loop knows what follows it
    def _block(self, stmts: List[ast.stmt], after: List[ast.stmt]) -> List[ast.stmt]:
        out: List[ast.stmt] = []
        for i, s in enumerate(stmts):
            self._after.append(list(stmts[i + 1:]) + after)
            out.append(self.visit(s))
            self._after.pop()
        return out

    def _following(self) -> List[ast.stmt]:
        return self._after[-1] if self._after else []

    def visit_FunctionDef(self, node: ast.FunctionDef) -> Any:
        if self._after:        # a nested definition: left alone
            return node
        node.body = self._block(node.body, [])
        return node

    def visit_If(self, node: ast.If) -> Any:
        after = self._following()
        node.body = self._block(node.body, after)
        node.orelse = self._block(node.orelse, after)
        return node

    def visit_With(self, node: ast.With) -> Any:
        node.body = self._block(node.body, self._following())
        return node

    def visit_While(self, node: ast.While) -> Any:
        after = self._following()
        node.body = self._block(node.body, list(node.body) + after)
        return node

    def visit_Try(self, node: ast.Try) -> Any:
        return node            # loops inside try blocks stay as they are

    def visit_Match(self, node: ast.Match) -> Any:
        return node

    def visit_For(self, node: ast.For) -> Any:
        after = self._following()
        ok = self._batchable(node, after)
        # the body of this loop is followed by itself (the next iteration) and then by what follows the loop
        node.body = self._block(node.body, list(node.body) + after)
        if ok:
            site = ast.Tuple(elts=[ast.Constant(self.filename), ast.Constant(node.lineno), ast.Constant(node.col_offset)],
                             ctx=ast.Load())
            node.iter = ast.Call(func=ast.Name(id="__ttl_loop__", ctx=ast.Load()), args=[node.iter, site], keywords=[])
            for sub in node.body:
                for n in ast.walk(sub):
                    if (isinstance(n, ast.Call) and isinstance(n.func, ast.Attribute) and n.func.attr == "pop"
                            and not n.args and not n.keywords):
                        n.args = [n.func.value]
                        n.func = ast.Name(id="__ttl_pop__", ctx=ast.Load())
            self.changed += 1
        return node

    def _batchable(self, node: ast.For, after: List[ast.stmt]) -> bool:
        if node.orelse:
            return False
        targets = _target_names(node.target)
        if targets is None:
            return False
        stored: Set[str] = set(targets)

        def scan(stmts: Sequence[ast.stmt], own_loop: bool) -> bool:
            for s in stmts:
                for n in ast.walk(s) if not isinstance(s, (ast.For, ast.While)) else [s]:
                    if isinstance(n, (ast.Return, ast.Yield, ast.YieldFrom, ast.Await, ast.Global, ast.Nonlocal, ast.Delete,
                                      ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef, ast.NamedExpr, ast.Try,
                                      ast.Import, ast.ImportFrom)):
                        return False
                    if isinstance(n, ast.Break) and own_loop:
                        return False
                    if isinstance(n, (ast.For, ast.AsyncFor)):    # a loop nested in an if / with statement
                        tn = _target_names(n.target)
                        if tn is None:
                            return False
                        stored.update(tn)
                    if isinstance(n, (ast.Assign, ast.AugAssign, ast.AnnAssign)):
                        for t in (n.targets if isinstance(n, ast.Assign) else [n.target]):
                            tn = _target_names(t)
                            if tn is None:
                                return False
                            stored.update(tn)
                    if isinstance(n, (ast.With, ast.AsyncWith)):
                        for item in n.items:
                            if item.optional_vars is not None:
                                tn = _target_names(item.optional_vars)
                                if tn is None:
                                    return False
                                stored.update(tn)
                    if isinstance(n, ast.Call) and isinstance(n.func, ast.Attribute):
                        if n.func.attr in _MUTATORS or (n.func.attr == "pop" and (n.args or n.keywords)):
                            return False
                if isinstance(s, (ast.For, ast.While)):
                    # an inner loop: its own break is fine, everything else is checked the same way
                    if isinstance(s, ast.For):
                        tn = _target_names(s.target)
                        if tn is None:
                            return False
                        stored.update(tn)
                    if not scan([ast.Expr(s.iter if isinstance(s, ast.For) else s.test)], own_loop):
                        return False
                    if not scan(list(s.body) + list(s.orelse), False):
                        return False
                else:
                    # `break` / `continue` nested in if / with belong to this loop when own_loop
                    pass
            return True

        if not scan(node.body, True):
            return False
        # carried from one iteration to the next: read in the body before the body has written it
        carried, _ = _reads_before_write(node.body, stored, set(targets))
        if carried:
            return False
        # read after the loop before anything else writes it
        live_out, _ = _reads_before_write(after, stored, set())
        return not live_out


_CACHE: Dict[types.CodeType, Optional[types.CodeType]] = {}


def _find_code(code: types.CodeType, name: str, depth: int = 0) -> Optional[types.CodeType]:
    for c in code.co_consts:
        if isinstance(c, types.CodeType):
            if c.co_name == name and depth >= 1:
                return c
            hit = _find_code(c, name, depth + 1)
            if hit is not None:
                return hit
    return None


def transform(fn: types.FunctionType) -> types.FunctionType:
    """`fn` with its batchable loops rewritten, sharing `fn`'s closure cells and globals; `fn` itself when its
    source is not available or nothing in it can be batched."""
    code = fn.__code__
    if code not in _CACHE:
        _CACHE[code] = _transform_code(fn)
    new = _CACHE[code]
    if new is None:
        return fn
    cells = dict(zip(code.co_freevars, fn.__closure__ or ()))
    if any(v not in cells for v in new.co_freevars):
        return fn
    fn.__globals__.setdefault("__ttl_loop__", loop)
    fn.__globals__.setdefault("__ttl_pop__", pop_call)
    out = types.FunctionType(new, fn.__globals__, fn.__name__, fn.__defaults__, tuple(cells[v] for v in new.co_freevars))
    out.__kwdefaults__ = fn.__kwdefaults__
    return out


def _transform_code(fn: types.FunctionType) -> Optional[types.CodeType]:
    try:
        lines, first = inspect.getsourcelines(fn)
        tree = ast.parse(textwrap.dedent("".join(lines)))
    except (OSError, TypeError, SyntaxError, IndentationError):
        return None
    if not tree.body or not isinstance(tree.body[0], ast.FunctionDef):
        return None
    fdef = tree.body[0]
    fdef.decorator_list = []
    filename = fn.__code__.co_filename
    ast.increment_lineno(tree, first - 1)
    tr = _Transformer(filename)
    fdef = tr.visit(fdef)
    if not tr.changed:
        return None
    free = fn.__code__.co_freevars
    factory = ast.FunctionDef(
        name="__ttl_factory__",
        args=ast.arguments(posonlyargs=[], args=[ast.arg(arg=v) for v in free], vararg=None, kwonlyargs=[], kw_defaults=[],
                           kwarg=None, defaults=[]),
        body=[fdef, ast.Return(value=ast.Name(id=fdef.name, ctx=ast.Load()))], decorator_list=[], type_params=[])
    mod = ast.Module(body=[factory], type_ignores=[])
    ast.fix_missing_locations(mod)
    try:
        compiled = compile(mod, filename, "exec")
    except (SyntaxError, ValueError):
        return None
    return _find_code(compiled, fdef.name)
