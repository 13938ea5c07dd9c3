"""`@ttl.kernel`, `@ttl.compute`, `@ttl.datamovement`, `ttl.core`, `ttl.grid_size`.

Same call shapes as the reference decorator (python/ttl/ttl_api.py:1125-1249; the
simulator's twin python/sim/kernel.py:202-293): calling the decorated function runs
the kernel body once to create circular buffers and collect the three thread
functions, then executes the program on the grid.  Here "executes" means: trace the
threads symbolically on every core (trace.py), recognise the result as a fused
element-wise program or a matmul (recognize.py), cache that plan per tensor signature
(as python/ttl/ttl_api.py:1189-1230 caches compiled kernels), and launch the CUDA
kernels through the C ABI.  Outputs are written in place; the call returns None.
"""

from __future__ import annotations

import os
import types
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

from . import trace as _trace
from . import ttnn as _ttnn

_thread_registry: List[Tuple[str, types.FunctionType]] = []


class _ThreadTemplate:
    def __init__(self, func: types.FunctionType, kind: str):
        self.__name__ = func.__name__
        self.__wrapped__ = func
        self.thread_type = kind

    def __call__(self, *a: Any, **k: Any) -> Any:
        raise RuntimeError(f"{self.__name__} is a kernel thread; it runs when the kernel is called")


def compute() -> Callable[[types.FunctionType], _ThreadTemplate]:
    def decorator(func: types.FunctionType) -> _ThreadTemplate:
        _thread_registry.append(("compute", func))
        return _ThreadTemplate(func, "compute")
    return decorator


def datamovement() -> Callable[[types.FunctionType], _ThreadTemplate]:
    def decorator(func: types.FunctionType) -> _ThreadTemplate:
        _thread_registry.append(("dm", func))
        return _ThreadTemplate(func, "dm")
    return decorator


def grid_size(dims: int = 2) -> Any:
    return _trace.grid_size_of(_trace.current_grid(), dims)


def core(dims: int = 2) -> Any:
    return _trace.core_coords(_trace.current_core(), _trace.current_grid(), dims)


def _signature(args: Tuple[Any, ...]) -> Tuple[Any, ...]:
    sig = []
    for a in args:
        if isinstance(a, _ttnn.Tensor):
            sig.append(("T", tuple(a.shape), str(a.dtype), tuple(a._tensor.stride()) if a._packed is None else ()))
        else:
            try:
                hash(a)
                sig.append(("V", a))
            except TypeError:
                sig.append(("V", repr(a)))
    return tuple(sig)


def kernel(grid: Union[str, Tuple[int, ...], Callable[..., Any]] = "auto", memory_space: str = "L1", tiled: bool = True,
           fp32_dest_acc_en: Optional[bool] = None, dst_full_sync_en: Optional[bool] = None,
           num_outs: int = 1, **_ignored: Any) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
    """Decorator turning a tile-program builder into a callable GPU program.

    grid: "auto" (8x8, as the simulator), a tuple, or a callable returning a tuple.
    fp32_dest_acc_en: True keeps fp32 intermediates through a fused element-wise chain
      and rounds once at the end; otherwise (default) every op rounds to the tensor's
      element type, which is what the simulator computes on bf16 tensors.
    memory_space / tiled / dst_full_sync_en / num_outs: accepted for source
      compatibility with python/ttl/ttl_api.py:1125-1170; they describe Tensix
      resources and have no effect here.
    """
    if num_outs != 1:
        raise ValueError("num_outs must be 1")

    def decorator(func: Callable[..., Any]) -> Callable[..., Any]:
        plans: Dict[Tuple[Any, ...], Any] = {}

        def _resolve_grid() -> Tuple[int, ...]:
            if grid == "auto":
                return (8, 8)
            if callable(grid):
                return tuple(grid())
            if isinstance(grid, str):
                raise ValueError(f"Unknown grid specification {grid!r}")
            return tuple(grid)  # type: ignore[arg-type]

        def get_plan(*args: Any, **kwargs: Any) -> Any:
            from . import recognize as _rec

            g = _resolve_grid()
            key = (_signature(args), tuple(sorted(kwargs.items())) if kwargs else (), g)
            plan = plans.get(key)
            if plan is None:
                # `grid` is visible as a global inside the kernel body, as in the simulator
                new_globals = func.__globals__
                had, old = "grid" in new_globals, new_globals.get("grid")
                new_globals["grid"] = g
                _thread_registry.clear()
                _trace.set_grid(g)
                try:
                    func(*args, **kwargs)
                    threads = list(_thread_registry)
                finally:
                    _thread_registry.clear()
                    if had:
                        new_globals["grid"] = old
                    else:
                        new_globals.pop("grid", None)
                if len(threads) != 3:
                    _trace.set_grid(None)
                    raise ValueError(
                        f"Kernel must define exactly 3 threads (compute, dm0, dm1), got {len(threads)}")
                n_compute = sum(1 for k, _ in threads if k == "compute")
                if n_compute != 1:
                    _trace.set_grid(None)
                    raise ValueError(f"Kernel must define exactly 1 compute thread, got {n_compute}")
                if len(threads) - n_compute != 2:
                    _trace.set_grid(None)
                    raise ValueError(
                        f"Kernel must define exactly 2 datamovement threads, got {len(threads) - n_compute}")
                try:
                    tr = _trace.run_program(threads, g, strict_cb=os.environ.get("TTLB200_STRICT_CB") == "1")
                finally:
                    _trace.set_grid(None)
                tensors = [a for a in args if isinstance(a, _ttnn.Tensor)]
                plan = _rec.build_plan(tr, tensors, fp32_intermediates=bool(fp32_dest_acc_en))
                if plan.cacheable:  # programs that derive tensors inside the body are re-traced every call
                    plans[key] = plan
            return plan

        def wrapper(*args: Any, **kwargs: Any) -> None:
            plan = get_plan(*args, **kwargs)
            plan.run([a for a in args if isinstance(a, _ttnn.Tensor)])

        wrapper.__name__ = getattr(func, "__name__", "kernel")
        wrapper.__doc__ = func.__doc__
        wrapper.__wrapped__ = func  # type: ignore[attr-defined]
        wrapper.__pykernel_config__ = {"grid": grid}  # type: ignore[attr-defined]
        wrapper._plans = plans  # type: ignore[attr-defined]
        wrapper.plan = get_plan  # type: ignore[attr-defined]  # trace + recognise without launching
        return wrapper

    return decorator
