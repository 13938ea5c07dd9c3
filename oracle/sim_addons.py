"""Extra block math for the reference simulator, in the simulator's own idiom.

TEST INFRASTRUCTURE ONLY.  The reference simulator's `ttl.math` has only `broadcast`
(python/sim/__init__.py:22-29); the element-wise functions exist on the compiler side
(include/ttlang/Dialect/TTL/TTLElementwiseOps.def:61-82) with torch goldens
(test/me2e/ops/__init__.py:27-41).  To obtain simulator outputs for programs that use them,
this module adds `ttl.math.{exp,log,sqrt,rsqrt,tanh,sigmoid,neg,abs,relu,max,min}` to an
imported simulator: each applies the torch golden per tile and returns a temporary block,
keeping the source-block tracking the way python/sim/math.py:87-106 does for `broadcast`.
`reduce_sum` / `reduce_max` (docs/sphinx/specs/TTLangSpecification.md:750-755; implemented nowhere in
the reference) are added the same way: the block's tiles are assembled, combined in fp32 along the
named dims with torch.sum / torch.amax, multiplied by element [0, 0] of the scaler tile and rounded
once to the tile dtype; the result block holds degenerate tiles ((1,32), (32,1) or (1,1)), the
simulator's form of a broadcast source (python/sim/copyhandlers.py:103-131).  **Parity unpinned**:
this is the build's reading of the specification, no reference implementation exists to compare with.
Nothing under the reference tree is modified.
"""

from __future__ import annotations

from typing import Any, Callable

import torch

# torch goldens, as test/me2e/ops/__init__.py:27-41 pairs them with the op names
UNARY_GOLDEN = {
    "exp": torch.exp,
    "log": torch.log,
    "sqrt": torch.sqrt,
    "rsqrt": torch.rsqrt,
    "tanh": torch.tanh,
    "sigmoid": torch.sigmoid,
    "neg": torch.neg,
    "abs": torch.abs,
    "relu": torch.relu,
}
BINARY_GOLDEN = {"max": torch.maximum, "min": torch.minimum}


def _appendix_b() -> Any:
    """The other functions of the specification's Appendix B, as the oracle defines them (one block op each)."""
    from . import tile_oracle
    extra = {k: v for k, v in tile_oracle.UNARY.items() if k not in UNARY_GOLDEN}
    return extra, tile_oracle.PARAM_UNARY, tile_oracle.MATH_NAMES


def install(sim_module: Any) -> None:
    """Add the functions to `sim_module.ttl.math` (sim_module is the imported `sim` package)."""
    from sim.block import Block, BlockAcquisition, ThreadType  # type: ignore
    from sim.ttnnsim import Tensor  # type: ignore

    def track(result: Any, actual: Any) -> None:
        result._source_blocks = list(getattr(actual, "_source_blocks", []))
        if (not actual._is_temporary and actual._acquisition == BlockAcquisition.WAIT
                and actual._thread_type == ThreadType.COMPUTE):
            result._source_blocks.append(actual)

    def make_unary(fn: Callable[[torch.Tensor], torch.Tensor]) -> Callable[[Any], Any]:
        def op(block: Any) -> Any:
            actual = block.block() if hasattr(block, "block") else block
            tiles = [Tensor(fn(t.to_torch())) for t in actual.to_list()]
            res = Block.from_list(tiles, actual._shape)
            track(res, actual)
            return res
        return op

    def make_binary(fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor]) -> Callable[[Any, Any], Any]:
        def tile_op(a: Any, b: Any) -> Any:
            if isinstance(a, Tensor):
                return Tensor(fn(a.to_torch(), b.to_torch()))
            return fn(a, b)

        def op(a: Any, b: Any) -> Any:
            la = a.block() if hasattr(a, "block") else a
            lb = b.block() if hasattr(b, "block") else b
            return la._binary_op(lb, tile_op)
        return op

    def make_reduce(kind: str) -> Callable[..., Any]:
        def op(block: Any, scaler: Any = None, dims: Any = None) -> Any:
            if dims is None:
                raise ValueError(f"dims parameter is required for reduce_{kind}()")
            actual = block.block() if hasattr(block, "block") else block
            rows, cols = actual._shape
            tiles = [t.to_torch() for t in actual.to_list()]
            dt = tiles[0].dtype
            full = torch.cat([torch.cat(tiles[r * cols:(r + 1) * cols], dim=1) for r in range(rows)], dim=0)
            full = full.to(torch.float32)
            ds = sorted(set(int(d) for d in dims))
            res = full.sum(dim=ds, keepdim=True) if kind == "sum" else full.amax(dim=ds, keepdim=True)
            sc_block = None
            if scaler is not None:
                sc_block = scaler.block() if hasattr(scaler, "block") else scaler
                res = res * sc_block.to_list()[0].to_torch()[0, 0].to(torch.float32)
            res = res.to(dt)
            shape = (1 if 0 in ds else rows, 1 if 1 in ds else cols)
            th, tw = (1 if 0 in ds else 32), (1 if 1 in ds else 32)
            out_tiles = [Tensor(res[r * th:(r + 1) * th, c * tw:(c + 1) * tw].contiguous())
                         for r in range(shape[0]) for c in range(shape[1])]
            result = Block.from_list(out_tiles, shape)
            track(result, actual)
            if sc_block is not None:
                mine = list(result._source_blocks)
                track(result, sc_block)
                result._source_blocks = mine + [b for b in result._source_blocks if b not in mine]
            return result
        return op

    def make_param_unary(fn: Callable[..., torch.Tensor]) -> Callable[..., Any]:
        def op(block: Any, *params: float) -> Any:
            return make_unary(lambda t: fn(t, *params))(block)
        return op

    m = sim_module.ttl.math
    extra_unary, param_unary, spellings = _appendix_b()
    for name, fn in extra_unary.items():
        setattr(m, name, make_unary(fn))
    for name, fn in param_unary.items():
        setattr(m, name, make_param_unary(fn))
    for spelling, name in spellings.items():
        setattr(m, spelling, make_param_unary(param_unary[name]))
    m.reduce_sum = make_reduce("sum")
    m.reduce_max = make_reduce("max")
    for name, fn in UNARY_GOLDEN.items():
        setattr(m, name, make_unary(fn))
    for name, fn in BINARY_GOLDEN.items():
        setattr(m, name, make_binary(fn))
