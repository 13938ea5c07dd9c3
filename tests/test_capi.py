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
    assert ctypes.sizeof(capi.EltwiseDesc) == 16 + 6 * 40 + 32 * 4 + 8 + 8 + 32 + 8 * 4   # ... + imm[8]


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


def test_specialised_kernel_source_is_generated_without_a_gpu():
    """ttlb_eltwise_source: the streaming skeleton instantiated for one program."""
    from ttl_b200 import capi
    d = capi.EltwiseDesc()
    d.dtype, d.round_each_op, d.n_in = capi.TTLB_BF16, 0, 4
    modes = [(capi.IDX_SAME, capi.IDX_SAME), (capi.IDX_ZERO, capi.IDX_ZERO), (capi.IDX_ZERO, capi.IDX_SAME),
             (capi.IDX_SAME, capi.IDX_SAME)]
    for k, (rm, cm) in enumerate(modes):
        d.inp[k].ptr, d.inp[k].ld, d.inp[k].row_mode, d.inp[k].col_mode = 0x10000, 8192, rm, cm
    ops = [("load", 0), ("mul", 1), ("exp", 0), ("mul", 2), ("add", 3), ("relu", 0)]
    d.n_ops = len(ops)
    for k, (op, arg) in enumerate(ops):
        d.ops[k].opcode, d.ops[k].arg = capi.OPCODES[op], arg
    d.out, d.out_ld, d.rows, d.cols = 0x20000, 8192, 8192, 8192
    src = capi.eltwise_source(d)
    assert 'extern "C" __global__' in src and "expf(a)" in src
    assert src.count("ld_stream(") == 2 * 4 + 1   # A and C stream, 4 rows in flight per thread (+ the helper's definition)
    loop = src.index("for (u32 r")
    assert src.index("v2 = ld_cached") < loop    # the row vector is fetched once, before the row loop
    assert "pack_bf16x2(acc[e], acc[e + 1])" not in src   # fp32 intermediates: no per-op rounding
    d.round_each_op = 1
    assert "pack_bf16x2(acc[e], acc[e + 1])" in capi.eltwise_source(d)
    d.n_ops = 0
    with pytest.raises(capi.BackendError):
        capi.eltwise_source(d)
