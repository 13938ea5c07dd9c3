"""Operator-level entry points over the C ABI (used by recognised programs and by
callers that already know which kernel they want)."""

from __future__ import annotations

from typing import Any, Tuple

from . import capi
from .recognize import Unsupported


def launch_gemm(ctx: capi.Context, a: Any, b: Any, out: Any, rect: Tuple[int, int, int, int], stream: int) -> None:
    raise Unsupported("matmul kernels are not built into this library yet")
