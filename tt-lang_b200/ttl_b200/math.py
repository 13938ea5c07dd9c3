"""`ttl.math`: block math functions.

`broadcast` follows the simulator (python/sim/math.py:20-106): it checks that the
named block dims have size 1 and returns the block; the broadcasting itself happens
in the binary op that consumes it.  Both call forms found in the reference are
accepted, `broadcast(blk, dims=[..])` and the compiler's `broadcast(blk, out_blk, dims=[..])`
(python/ttl/operators.py:332-360).  The unary functions and `max`/`min` are the compiler's
element-wise op table (include/ttlang/Dialect/TTL/TTLElementwiseOps.def:61-82).
"""

from __future__ import annotations

from typing import Any, List, Optional

from .trace import Block, Leaf, Red, _as_block, _tag


# Which meaning `broadcast` has on FULL (non-degenerate) tiles.  The two reference front ends disagree:
# the simulator returns the block unchanged and lets the consuming op repeat the whole tile over the
# tile grid (python/sim/math.py:62-80); the compiler lowers to ttl.bcast, which spreads the tile's first
# row / column / element over the tile (TTLOps.td:570-597, test/python/test_bcast_ops.py:31-55).
# The simulator is the oracle, so its meaning is the default; on degenerate tensors ([1,N], [N,1],
# [1,1]) the two agree.
_hardware_broadcast = False


def set_hardware_broadcast(enabled: bool) -> None:
    """Follow the compiler front end where it differs from the simulator: `ttl.math.broadcast` has the hardware
    meaning on full tiles, and `ttl.grid_size()` keeps answering after a kernel call has returned."""
    global _hardware_broadcast
    _hardware_broadcast = bool(enabled)
    # programs written for the compiler also read the grid back after a kernel call (trace.GRID_OUTLIVES_KERNEL)
    from . import trace
    trace.set_grid_outlives_kernel(enabled)


def broadcast(block: Any, out_block: Optional[Any] = None, dims: Optional[List[int]] = None) -> Block:
    if dims is None:
        raise ValueError("dims parameter is required for broadcast()")
    b = _as_block(block)
    shape = b.shape
    v = b.value()
    for dim in dims:
        if dim >= len(shape):
            raise ValueError(
                f"Cannot broadcast along dimension {dim}: block has shape {shape} "
                f"with only {len(shape)} dimensions")
    if _hardware_broadcast and isinstance(v, Leaf) and any(v.tensor.shape[dim] != 1 for dim in dims):
        # hardware convention (compiler form `broadcast(inp, out_blk, dims=[..])`, ttl.bcast Row / Col / Scalar,
        # python/ttl/operators.py:332-360, test/python/test_bcast_ops.py:31-55): FULL tiles whose first row
        # (dims=[0]) / first column (dims=[1]) / element [0,0] carries the data; every tile of the block is
        # broadcast within itself, and a block dim of one tile expands to the output block's
        first = (0 in dims and v.tensor.shape[0] != 1, 1 in dims and v.tensor.shape[1] != 1)
        out_shape = shape
        if out_block is not None:
            out_shape = _as_block(out_block).shape
            for d in (0, 1):
                if shape[d] != out_shape[d] and shape[d] != 1:
                    raise ValueError(f"Cannot broadcast block of shape {shape} to output block of shape {out_shape}")
        leaf = Leaf(v.tensor, v.r0, v.r1, v.c0, v.c1, first)
        leaf.shape = v.shape
        return Block(out_shape, b.dtype, leaf, "FULL", "temp", temporary=True, nest=b.nest)
    for dim in dims:
        if shape[dim] != 1:
            raise ValueError(
                f"Cannot broadcast along dimension {dim}: dimension must have size 1, "
                f"but has size {shape[dim]}")
    return Block(shape, b.dtype, v, "FULL", "temp", temporary=True, nest=b.nest)


def _unary(name: str):
    def fn(block: Any) -> Block:
        return _as_block(block)._unary(name)
    fn.__name__ = name
    fn.__doc__ = f"Element-wise {name} of a block."
    return fn


exp = _unary("exp")
log = _unary("log")
sqrt = _unary("sqrt")
rsqrt = _unary("rsqrt")
tanh = _unary("tanh")
sigmoid = _unary("sigmoid")
neg = _unary("neg")
abs = _unary("abs")  # noqa: A001 - reference spelling
relu = _unary("relu")


# The rest of the specification's Appendix B (docs/sphinx/specs/TTLangSpecification.md:700-748); neither the
# reference compiler's op table nor its simulator has these yet.
exp2 = _unary("exp2")
expm1 = _unary("expm1")
logp1 = _unary("logp1")
square = _unary("square")
recip = _unary("recip")
tan = _unary("tan")
atan = _unary("atan")
atanh = _unary("atanh")
sin = _unary("sin")
asin = _unary("asin")
asinh = _unary("asinh")
cos = _unary("cos")
acos = _unary("acos")
acosh = _unary("acosh")
gelu = _unary("gelu")
silu = _unary("silu")
softsign = _unary("softsign")
hardsigmoid = _unary("hardsigmoid")


def _with_params(name: str, op: str, block: Any, *params: Any) -> Block:
    for v in params:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise TypeError(f"{name}(): scalar parameters must be numbers, got {type(v).__name__}")
    return _as_block(block)._unary(op, tuple(float(v) for v in params))


def rsub(a: Any, b: Any) -> Block:
    """`b - a` with a scalar `b`."""
    return _with_params("rsub", "rsub_imm", a, b)


def relu_max(expr: Any, upper_limit: Any) -> Block:
    """relu(min(x, upper_limit))."""
    return _with_params("relu_max", "relu_max", expr, upper_limit)


def relu_min(expr: Any, lower_limit: Any) -> Block:
    """relu(max(x, lower_limit))."""
    return _with_params("relu_min", "relu_min", expr, lower_limit)


def leaky_relu(expr: Any, slope: Any) -> Block:
    return _with_params("leaky_relu", "leaky_relu", expr, slope)


def prelu(expr: Any, alpha: Any) -> Block:
    """PReLU with one scalar weight: the same function as leaky_relu."""
    return _with_params("prelu", "leaky_relu", expr, alpha)


def elu(expr: Any, slope: Any) -> Block:
    return _with_params("elu", "elu", expr, slope)


def celu(expr: Any, alpha: Any, alpha_recip: Any) -> Block:
    return _with_params("celu", "celu", expr, alpha, alpha_recip)


def softplus(expr: Any, beta: Any, beta_reciprocal: Any, threshold: Any) -> Block:
    return _with_params("softplus", "softplus", expr, beta, beta_reciprocal, threshold)


def hardtanh(expr: Any, min: Any, max: Any) -> Block:  # noqa: A002 - reference spelling
    return _with_params("hardtanh", "hardtanh", expr, min, max)


def selu(expr: Any, scale: Any, alpha: Any) -> Block:
    return _with_params("selu", "selu", expr, scale, alpha)


def max(a: Any, b: Any) -> Block:  # noqa: A001 - reference spelling
    return _as_block(a)._binary(b, "max")


def min(a: Any, b: Any) -> Block:  # noqa: A001
    return _as_block(a)._binary(b, "min")


def _reduce(op: str, block: Any, scaler: Any, dims: Optional[List[int]]) -> Block:
    if dims is None:
        raise ValueError(f"dims parameter is required for reduce_{op}()")
    b = _as_block(block)
    if not isinstance(b, Block):
        raise TypeError(f"reduce_{op}() takes a block or a block expression")
    ds = tuple(sorted(set(int(d) for d in dims)))
    if not ds or any(d not in (0, 1) for d in ds):
        raise ValueError(f"reduce_{op}(): dims must name block dimensions 0 and/or 1, got {list(dims)}")
    sc = None
    if scaler is not None:
        sb = _as_block(scaler)
        if not isinstance(sb, Block):
            raise TypeError(f"reduce_{op}(): the scaler must be a block")
        if sb.shape != (1, 1):
            raise ValueError(f"reduce_{op}(): the scaler must be a block of one tile, got shape {sb.shape}")
        sc = sb.value()
    e = _tag(Red(op, b.value(), sc, ds))
    return Block(e.shape, b.dtype, e, "FULL", "temp", temporary=True, nest=b.nest)


def reduce_sum(block: Any, scaler: Any = None, dims: Optional[List[int]] = None) -> Block:
    """Scaled sum over block dims (docs/sphinx/specs/TTLangSpecification.md:754): dims=[0] sums over rows
    (a block of (R, C) tiles gives (1, C) tiles), dims=[1] over columns, dims=[0, 1] over both.  The sum of
    the elements, formed in fp32, is multiplied by element [0, 0] of the one-tile `scaler` block and rounded
    once to the block's element type."""
    return _reduce("sum", block, scaler, dims)


def reduce_max(block: Any, scaler: Any = None, dims: Optional[List[int]] = None) -> Block:
    """Scaled maximum over block dims (docs/sphinx/specs/TTLangSpecification.md:755); same conventions as
    `reduce_sum`."""
    return _reduce("max", block, scaler, dims)
