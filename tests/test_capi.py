"""The C-ABI library loads and exports every symbol include/ttlb200.h declares (no GPU needed)."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "ttlb200.h").read_text()
    return sorted(set(re.findall(r"TTLB_EXPORT\s+[\w\s\*]+?\b(ttlb_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for s in ("ttlb_init", "ttlb_destroy", "ttlb_last_error", "ttlb_eltwise"):
        assert s in syms


def test_library_exports_every_declared_symbol():
    from ttl_b200 import capi
    lib = capi.lib()
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} is declared in include/ttlb200.h but not exported"
    assert b"sm_100a" in lib.ttlb_version()


def test_descriptor_layout_matches_header():
    from ttl_b200 import capi
    # ttlb_operand: ptr, ld, 2 x int32, 2 x int64; ttlb_instr: 2 x int16
    assert ctypes.sizeof(capi.Operand) == 40
    assert ctypes.sizeof(capi.Instr) == 4
    assert ctypes.sizeof(capi.EltwiseDesc) == 16 + 6 * 40 + 32 * 4 + 8 + 8 + 32


def test_init_without_gpu_returns_error():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from ttl_b200 import capi
    h = ctypes.c_void_p()
    assert capi.lib().ttlb_init(0, ctypes.byref(h)) == capi.TTLB_ERR_CUDA
    assert not h.value
    with pytest.raises(capi.BackendError):
        capi.context()
