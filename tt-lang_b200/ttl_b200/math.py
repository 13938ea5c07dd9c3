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

from .trace import Block, _as_block


def broadcast(block: Any, _unused_arg: Optional[Any] = None, dims: Optional[List[int]] = None) -> Block:
    if dims is None:
        raise ValueError("dims parameter is required for broadcast()")
    b = _as_block(block)
    shape = b.shape
    for dim in dims:
        if dim >= len(shape):
            raise ValueError(
                f"Cannot broadcast along dimension {dim}: block has shape {shape} "
                f"with only {len(shape)} dimensions")
        if shape[dim] != 1:
            raise ValueError(
                f"Cannot broadcast along dimension {dim}: dimension must have size 1, "
                f"but has size {shape[dim]}")
    return Block(shape, b.dtype, b.value(), "FULL", "temp", temporary=True)


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


def max(a: Any, b: Any) -> Block:  # noqa: A001 - reference spelling
    return _as_block(a)._binary(b, "max")


def min(a: Any, b: Any) -> Block:  # noqa: A001
    return _as_block(a)._binary(b, "min")
