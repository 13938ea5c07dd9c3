"""ctypes binding of libttlb200.so (declarations: include/ttlb200.h).

The reference reaches its native code through a compiled Python module
(python/TTLangModule.cpp:14-46 over lib/CAPI); here the native side is a plain C ABI
and this file is the whole binding.  There is no fallback: if the library is missing
or no B200 is present, calls raise.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Dict, Optional

TTLB_OK = 0
TTLB_ERR_INVALID_ARG = -1
TTLB_ERR_UNSUPPORTED = -2
TTLB_ERR_CUDA = -3
TTLB_ERR_TIMEOUT = -4
TTLB_ERR_NCCL = -5

TTLB_BF16, TTLB_F32, TTLB_BFP8_B = 0, 1, 2
TTLB_MAX_IN, TTLB_MAX_OPS, TTLB_ARG_STACK, TTLB_MAX_IMM = 6, 32, -1, 8
IDX_SAME, IDX_ZERO, IDX_TILE, IDX_FIRST = 0, 1, 2, 3

OPCODES = {
    "load": 0, "add": 1, "sub": 2, "rsub": 3, "mul": 4, "div": 5, "rdiv": 6, "max": 7, "min": 8,
    "floordiv": 9, "rfloordiv": 10, "mod": 11, "rmod": 12, "pow": 13, "rpow": 14,
    "exp": 16, "log": 17, "sqrt": 18, "rsqrt": 19, "tanh": 20, "sigmoid": 21, "neg": 22, "abs": 23, "relu": 24,
    "push": 32,
    # the specification's Appendix B beyond the compiler's op table (specialised kernel only)
    "exp2": 40, "expm1": 41, "logp1": 42, "square": 43, "recip": 44, "tan": 45, "atan": 46, "atanh": 47, "sin": 48,
    "asin": 49, "asinh": 50, "cos": 51, "acos": 52, "acosh": 53, "gelu": 54, "silu": 55, "softsign": 56,
    "hardsigmoid": 57,
    # with scalar parameters (arg = index of the first one in EltwiseDesc.imm)
    "rsub_imm": 64, "relu_max": 65, "relu_min": 66, "leaky_relu": 67, "elu": 68, "celu": 69, "softplus": 70,
    "hardtanh": 71, "selu": 72, "pow_imm": 73,
}
# number of scalar parameters of the parametrised functions
IMM_PARAMS = {"rsub_imm": 1, "relu_max": 1, "relu_min": 1, "leaky_relu": 1, "elu": 1, "celu": 2, "softplus": 3,
              "hardtanh": 2, "selu": 2, "pow_imm": 1}


class Operand(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("ld", C.c_int64), ("row_mode", C.c_int32), ("col_mode", C.c_int32),
                ("row_off", C.c_int64), ("col_off", C.c_int64)]


class Instr(C.Structure):
    _fields_ = [("opcode", C.c_int16), ("arg", C.c_int16)]


class EltwiseDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("round_each_op", C.c_int32), ("n_in", C.c_int32), ("n_ops", C.c_int32),
                ("inp", Operand * TTLB_MAX_IN), ("ops", Instr * TTLB_MAX_OPS),
                ("out", C.c_void_p), ("out_ld", C.c_int64),
                ("row0", C.c_int64), ("col0", C.c_int64), ("rows", C.c_int64), ("cols", C.c_int64),
                ("imm", C.c_float * TTLB_MAX_IMM)]


REDUCE_SUM, REDUCE_MAX = 0, 1
REDUCE_ROWS, REDUCE_COLS = 1, 2


class ReduceDesc(C.Structure):
    _fields_ = [("src", EltwiseDesc), ("op", C.c_int32), ("dims", C.c_int32), ("scaler", C.c_void_p),
                ("out", C.c_void_p), ("out_ld", C.c_int64), ("fill_rows", C.c_int32), ("fill_cols", C.c_int32)]


TTLB_MAX_PHASES, IDX_PHASE = 3, 4


class RowFusedDesc(C.Structure):
    _fields_ = [("n_phases", C.c_int32), ("phase", ReduceDesc * TTLB_MAX_PHASES), ("final", EltwiseDesc)]


class GemmDesc(C.Structure):
    _fields_ = [("a", C.c_void_p), ("lda", C.c_int64), ("b", C.c_void_p), ("ldb", C.c_int64),
                ("c", C.c_void_p), ("ldc", C.c_int64), ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64)]


class GemmBfp8Desc(C.Structure):
    _fields_ = [("a", C.c_void_p), ("lda", C.c_int64), ("b_tiles", C.c_void_p), ("b_tile_cols", C.c_int64),
                ("b_tile_col0", C.c_int64), ("c", C.c_void_p), ("ldc", C.c_int64),
                ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64)]


class AttnDesc(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
                ("batch_heads", C.c_int64), ("seq", C.c_int64), ("head_dim", C.c_int64),
                ("causal", C.c_int32), ("scale", C.c_float)]


ELTWISE_AUTO, ELTWISE_GENERIC, ELTWISE_SPECIALISED = 0, 1, 2


def eltwise_source(desc: "EltwiseDesc") -> str:
    """CUDA source of the kernel specialised for `desc` (works without a GPU)."""
    l = lib()
    n = l.ttlb_eltwise_source(C.byref(desc), None, 0)
    if n < 0:
        raise BackendError(int(n), "invalid element-wise descriptor")
    buf = C.create_string_buffer(int(n))
    l.ttlb_eltwise_source(C.byref(desc), buf, int(n))
    return buf.value.decode()


def reduce_source(desc: "ReduceDesc") -> str:
    """CUDA source of the reduction kernel specialised for `desc` (works without a GPU)."""
    l = lib()
    n = l.ttlb_reduce_source(C.byref(desc), None, 0)
    if n < 0:
        raise BackendError(int(n), "invalid reduction descriptor")
    buf = C.create_string_buffer(int(n))
    l.ttlb_reduce_source(C.byref(desc), buf, int(n))
    return buf.value.decode()


def rowfused_source(desc: "RowFusedDesc") -> str:
    """CUDA source of the row-resident kernel specialised for `desc` (works without a GPU)."""
    l = lib()
    n = l.ttlb_rowfused_source(C.byref(desc), None, 0)
    if n < 0:
        raise BackendError(int(n), "invalid or unsupported row-fusion descriptor")
    buf = C.create_string_buffer(int(n))
    l.ttlb_rowfused_source(C.byref(desc), buf, int(n))
    return buf.value.decode()


ACTIVATIONS = {"relu": 1, "gelu": 2, "silu": 3, "sigmoid": 4, "tanh": 5}   # TTLB_ACT_*

BFP8_MODE_DEFAULT = 1


class BackendError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"ttlb200 error {code}: {message}")
        self.code = code


_LIB: Optional[C.CDLL] = None
LIB_PATH = Path(__file__).resolve().parent / "libttlb200.so"


def lib() -> C.CDLL:
    """Load the native library (once).  Raises if it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build the CUDA extension first (python tt-lang_b200/build.py). "
            "The B200 backend has no CPU fallback.")
    l = C.CDLL(str(LIB_PATH))
    l.ttlb_version.restype = C.c_char_p
    l.ttlb_init.argtypes = [C.c_int, C.POINTER(C.c_void_p)]
    l.ttlb_init.restype = C.c_int
    l.ttlb_destroy.argtypes = [C.c_void_p]
    l.ttlb_destroy.restype = None
    l.ttlb_last_error.argtypes = [C.c_void_p]
    l.ttlb_last_error.restype = C.c_char_p
    l.ttlb_launch_count.argtypes = [C.c_void_p]
    l.ttlb_launch_count.restype = C.c_int64
    l.ttlb_eltwise.argtypes = [C.c_void_p, C.POINTER(EltwiseDesc), C.c_void_p]
    l.ttlb_eltwise.restype = C.c_int
    l.ttlb_eltwise_set_mode.argtypes = [C.c_void_p, C.c_int]
    l.ttlb_eltwise_set_mode.restype = C.c_int
    l.ttlb_eltwise_last_path.argtypes = [C.c_void_p]
    l.ttlb_eltwise_last_path.restype = C.c_int
    l.ttlb_eltwise_source.argtypes = [C.POINTER(EltwiseDesc), C.c_char_p, C.c_size_t]
    l.ttlb_eltwise_source.restype = C.c_int64
    l.ttlb_reduce.argtypes = [C.c_void_p, C.POINTER(ReduceDesc), C.c_void_p]
    l.ttlb_reduce.restype = C.c_int
    l.ttlb_reduce_source.argtypes = [C.POINTER(ReduceDesc), C.c_char_p, C.c_size_t]
    l.ttlb_reduce_source.restype = C.c_int64
    l.ttlb_rowfused.argtypes = [C.c_void_p, C.POINTER(RowFusedDesc), C.c_void_p]
    l.ttlb_rowfused.restype = C.c_int
    l.ttlb_rowfused_source.argtypes = [C.POINTER(RowFusedDesc), C.c_char_p, C.c_size_t]
    l.ttlb_rowfused_source.restype = C.c_int64
    l.ttlb_matmul_bf16.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p]
    l.ttlb_matmul_bf16.restype = C.c_int
    l.ttlb_matmul_bf16_bias.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p, C.c_int64, C.c_void_p]
    l.ttlb_matmul_bf16_bias.restype = C.c_int
    l.ttlb_matmul_bf16_epilogue.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
    l.ttlb_matmul_bf16_epilogue.restype = C.c_int
    l.ttlb_matmul_bfp8w_epilogue.argtypes = [C.c_void_p, C.POINTER(GemmBfp8Desc), C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
    l.ttlb_matmul_bfp8w_epilogue.restype = C.c_int
    l.ttlb_pack_bfp8_b.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
    l.ttlb_pack_bfp8_b.restype = C.c_int
    l.ttlb_unpack_bfp8_b.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
    l.ttlb_unpack_bfp8_b.restype = C.c_int
    l.ttlb_unpack_bfp8_b_device.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                            C.c_void_p, C.c_int64, C.c_void_p]
    l.ttlb_unpack_bfp8_b_device.restype = C.c_int
    for name in ("ttlb_pack_bfp4_b", "ttlb_unpack_bfp4_b"):
        getattr(l, name).argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        getattr(l, name).restype = C.c_int
    l.ttlb_unpack_bfp4_b_device.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                            C.c_void_p, C.c_int64, C.c_void_p]
    l.ttlb_unpack_bfp4_b_device.restype = C.c_int
    l.ttlb_matmul_bfp4w.argtypes = [C.c_void_p, C.POINTER(GemmBfp8Desc), C.c_void_p]
    l.ttlb_matmul_bfp4w.restype = C.c_int
    l.ttlb_matmul_bfp4w_epilogue.argtypes = [C.c_void_p, C.POINTER(GemmBfp8Desc), C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
    l.ttlb_matmul_bfp4w_epilogue.restype = C.c_int
    l.ttlb_matmul_bfp8w.argtypes = [C.c_void_p, C.POINTER(GemmBfp8Desc), C.c_void_p]
    l.ttlb_matmul_bfp8w.restype = C.c_int
    l.ttlb_matmul_bfp8w_noalloc.argtypes = [C.POINTER(GemmBfp8Desc), C.c_void_p, C.c_int, C.c_char_p, C.c_size_t]
    l.ttlb_matmul_bfp8w_noalloc.restype = C.c_int
    l.ttlb_attention.argtypes = [C.c_void_p, C.POINTER(AttnDesc), C.c_void_p]
    l.ttlb_attention.restype = C.c_int
    l.ttlb_matmul_f32.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p]
    l.ttlb_matmul_f32.restype = C.c_int
    l.ttlb_check_status.argtypes = [C.c_void_p, C.c_void_p]
    l.ttlb_check_status.restype = C.c_int
    l.ttlb_matmul_bf16_multicast.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p]
    l.ttlb_matmul_bf16_multicast.restype = C.c_int
    l.ttlb_matmul_bfp8w_multicast.argtypes = [C.c_void_p, C.POINTER(GemmBfp8Desc), C.c_void_p]
    l.ttlb_matmul_bfp8w_multicast.restype = C.c_int
    l.ttlb_matmul_bf16_peers.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.POINTER(C.c_void_p), C.c_int, C.c_void_p]
    l.ttlb_matmul_bf16_peers.restype = C.c_int
    l.ttlb_matmul_bfp8w_peers.argtypes = [C.c_void_p, C.POINTER(GemmBfp8Desc), C.POINTER(C.c_void_p), C.c_int, C.c_void_p]
    l.ttlb_matmul_bfp8w_peers.restype = C.c_int
    l.ttlb_attention_multicast.argtypes = [C.c_void_p, C.POINTER(AttnDesc), C.c_void_p]
    l.ttlb_attention_multicast.restype = C.c_int
    l.ttlb_attention_peers.argtypes = [C.c_void_p, C.POINTER(AttnDesc), C.POINTER(C.c_void_p), C.c_int, C.c_void_p]
    l.ttlb_attention_peers.restype = C.c_int
    l.ttlb_multimem_bcast.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                      C.c_void_p]
    l.ttlb_multimem_bcast.restype = C.c_int
    l.ttlb_selftest_wait_timeout.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
    l.ttlb_selftest_wait_timeout.restype = C.c_int
    l.ttlb_set_gemm_variant.argtypes = [C.c_void_p, C.c_int]
    l.ttlb_set_gemm_variant.restype = C.c_int
    l.ttlb_set_bfp8_chunks.argtypes = [C.c_void_p, C.c_int]
    l.ttlb_set_bfp8_chunks.restype = C.c_int
    l.ttlb_set_bfp8_mode.argtypes = [C.c_void_p, C.c_int]
    l.ttlb_set_bfp8_mode.restype = C.c_int
    l.ttlb_set_wait_limit.argtypes = [C.c_void_p, C.c_int64]
    l.ttlb_set_wait_limit.restype = C.c_int
    _LIB = l
    return l


class Context:
    """One ttlb_ctx, bound to one CUDA device."""

    def __init__(self, device: int):
        self._lib = lib()
        h = C.c_void_p()
        rc = self._lib.ttlb_init(device, C.byref(h))
        if rc != TTLB_OK:
            raise BackendError(rc, f"ttlb_init(device={device}) failed: no usable B200 "
                                   "(this backend has no CPU fallback)")
        self.handle = h
        self.device = device

    def check(self, rc: int) -> None:
        if rc != TTLB_OK:
            raise BackendError(rc, (self._lib.ttlb_last_error(self.handle) or b"").decode())

    def launch_count(self) -> int:
        return int(self._lib.ttlb_launch_count(self.handle))

    def eltwise(self, desc: EltwiseDesc, stream: int) -> None:
        self.check(self._lib.ttlb_eltwise(self.handle, C.byref(desc), C.c_void_p(stream)))

    def reduce(self, desc: "ReduceDesc", stream: int) -> None:
        self.check(self._lib.ttlb_reduce(self.handle, C.byref(desc), C.c_void_p(stream)))

    def rowfused(self, desc: "RowFusedDesc", stream: int) -> None:
        self.check(self._lib.ttlb_rowfused(self.handle, C.byref(desc), C.c_void_p(stream)))

    def matmul_bf16(self, desc: "GemmDesc", stream: int) -> None:
        self.check(self._lib.ttlb_matmul_bf16(self.handle, C.byref(desc), C.c_void_p(stream)))

    def matmul_bf16_bias(self, desc: "GemmDesc", bias_ptr: int, ldbias: int, stream: int) -> None:
        """C = A @ B + bias (bias: bf16 [m, n], added in fp32 before the rounding)."""
        self.check(self._lib.ttlb_matmul_bf16_bias(self.handle, C.byref(desc), C.c_void_p(bias_ptr), ldbias,
                                                   C.c_void_p(stream)))

    def matmul_bf16_epilogue(self, desc: "GemmDesc", bias_ptr: int, ldbias: int, act: int, stream: int) -> None:
        """C = act(A @ B + bias); bias_ptr 0: no bias; ldbias 0: the bias is one row added to every output row."""
        self.check(self._lib.ttlb_matmul_bf16_epilogue(self.handle, C.byref(desc), C.c_void_p(bias_ptr or None), ldbias, act,
                                                       C.c_void_p(stream)))

    def matmul_bfp8w_epilogue(self, desc: "GemmBfp8Desc", bias_ptr: int, ldbias: int, act: int, stream: int) -> None:
        self.check(self._lib.ttlb_matmul_bfp8w_epilogue(self.handle, C.byref(desc), C.c_void_p(bias_ptr or None), ldbias, act,
                                                        C.c_void_p(stream)))

    def matmul_f32(self, desc: "GemmDesc", stream: int) -> None:
        self.check(self._lib.ttlb_matmul_f32(self.handle, C.byref(desc), C.c_void_p(stream)))

    def matmul_bfp8w(self, desc: "GemmBfp8Desc", stream: int) -> None:
        self.check(self._lib.ttlb_matmul_bfp8w(self.handle, C.byref(desc), C.c_void_p(stream)))

    def matmul_bfp4w(self, desc: "GemmBfp8Desc", stream: int) -> None:
        self.check(self._lib.ttlb_matmul_bfp4w(self.handle, C.byref(desc), C.c_void_p(stream)))

    def matmul_bfp4w_epilogue(self, desc: "GemmBfp8Desc", bias_ptr: int, ldbias: int, act: int, stream: int) -> None:
        self.check(self._lib.ttlb_matmul_bfp4w_epilogue(self.handle, C.byref(desc), C.c_void_p(bias_ptr or None), ldbias, act,
                                                        C.c_void_p(stream)))

    def unpack_bfp4_b(self, tiles_ptr: int, tile_cols_total: int, tile_col0: int, k: int, n: int, out_ptr: int,
                      ld: int, stream: int) -> None:
        self.check(self._lib.ttlb_unpack_bfp4_b_device(self.handle, C.c_void_p(tiles_ptr), tile_cols_total, tile_col0,
                                                       k, n, C.c_void_p(out_ptr), ld, C.c_void_p(stream)))

    def unpack_bfp8_b(self, tiles_ptr: int, tile_cols_total: int, tile_col0: int, k: int, n: int, out_ptr: int,
                      ld: int, stream: int) -> None:
        self.check(self._lib.ttlb_unpack_bfp8_b_device(self.handle, C.c_void_p(tiles_ptr), tile_cols_total, tile_col0,
                                                       k, n, C.c_void_p(out_ptr), ld, C.c_void_p(stream)))

    def attention(self, desc: "AttnDesc", stream: int) -> None:
        self.check(self._lib.ttlb_attention(self.handle, C.byref(desc), C.c_void_p(stream)))

    def attention_multicast(self, desc: "AttnDesc", stream: int) -> None:
        self.check(self._lib.ttlb_attention_multicast(self.handle, C.byref(desc), C.c_void_p(stream)))

    def attention_peers(self, desc: "AttnDesc", peers: "list[int]", stream: int) -> None:
        arr = (C.c_void_p * len(peers))(*peers)
        self.check(self._lib.ttlb_attention_peers(self.handle, C.byref(desc), arr, len(peers), C.c_void_p(stream)))

    def check_status(self, stream: int = 0) -> None:
        """Synchronise `stream` and raise if a bounded device-side wait ran out since the last check."""
        self.check(self._lib.ttlb_check_status(self.handle, C.c_void_p(stream)))

    def matmul_bf16_multicast(self, desc: "GemmDesc", stream: int) -> None:
        self.check(self._lib.ttlb_matmul_bf16_multicast(self.handle, C.byref(desc), C.c_void_p(stream)))

    def matmul_bfp8w_multicast(self, desc: "GemmBfp8Desc", stream: int) -> None:
        self.check(self._lib.ttlb_matmul_bfp8w_multicast(self.handle, C.byref(desc), C.c_void_p(stream)))

    def matmul_bf16_peers(self, desc: "GemmDesc", peers: "list[int]", stream: int) -> None:
        """C = A @ B stored into the output region of every buffer in `peers` (peer-mapped copies, own copy included)."""
        arr = (C.c_void_p * len(peers))(*peers)
        self.check(self._lib.ttlb_matmul_bf16_peers(self.handle, C.byref(desc), arr, len(peers), C.c_void_p(stream)))

    def matmul_bfp8w_peers(self, desc: "GemmBfp8Desc", peers: "list[int]", stream: int) -> None:
        arr = (C.c_void_p * len(peers))(*peers)
        self.check(self._lib.ttlb_matmul_bfp8w_peers(self.handle, C.byref(desc), arr, len(peers), C.c_void_p(stream)))

    def multimem_bcast(self, src_ptr: int, src_ld_bytes: int, mc_dst_ptr: int, dst_ld_bytes: int, rows: int,
                       row_bytes: int, stream: int) -> None:
        self.check(self._lib.ttlb_multimem_bcast(self.handle, C.c_void_p(src_ptr), src_ld_bytes, C.c_void_p(mc_dst_ptr),
                                                 dst_ld_bytes, rows, row_bytes, C.c_void_p(stream)))

    def selftest_wait_timeout(self, limit_cycles: int, stream: int = 0) -> None:
        """Launch the bounded-wait self-test (a wait that nothing satisfies, with a short limit)."""
        self.check(self._lib.ttlb_selftest_wait_timeout(self.handle, limit_cycles, C.c_void_p(stream)))

    def set_gemm_variant(self, variant: int) -> None:
        """0: one-CTA 128x256 tiles; 1 (default): two-CTA 256x256 tiles for large outputs; 2: two-CTA always."""
        self.check(self._lib.ttlb_set_gemm_variant(self.handle, variant))

    def set_bfp8_chunks(self, chunks: int) -> None:
        """Column chunks (1..4) of the two-step bfp8 matmul: expansion of chunk i+1 under the GEMM of chunk i."""
        self.check(self._lib.ttlb_set_bfp8_chunks(self.handle, chunks))

    def set_bfp8_mode(self, mode: int) -> None:
        """0: unpack kernel + GEMM; 1: unpack inside the GEMM mainloop for large outputs; 2: always inside."""
        self.check(self._lib.ttlb_set_bfp8_mode(self.handle, mode))

    def set_wait_limit(self, cycles: int) -> None:
        self.check(self._lib.ttlb_set_wait_limit(self.handle, cycles))

    def set_eltwise_mode(self, mode: int) -> None:
        """ELTWISE_AUTO / ELTWISE_GENERIC / ELTWISE_SPECIALISED (include/ttlb200.h)."""
        self.check(self._lib.ttlb_eltwise_set_mode(self.handle, mode))

    def eltwise_last_path(self) -> int:
        return int(self._lib.ttlb_eltwise_last_path(self.handle))

    def close(self) -> None:
        if self.handle:
            self._lib.ttlb_destroy(self.handle)
            self.handle = C.c_void_p()


_CONTEXTS: Dict[int, Context] = {}


def context(device: Optional[int] = None) -> Context:
    """Context of `device` (default: torch's current CUDA device), created on first use."""
    import torch

    if device is None:
        if not torch.cuda.is_available():
            raise BackendError(TTLB_ERR_CUDA, "no CUDA device: the B200 backend has no CPU fallback")
        device = torch.cuda.current_device()
    ctx = _CONTEXTS.get(device)
    if ctx is None:
        ctx = Context(device)
        _CONTEXTS[device] = ctx
    return ctx


def current_stream(device: Optional[int] = None) -> int:
    """Handle of torch's current stream on `device` (default: the current CUDA device)."""
    import torch

    return int(torch.cuda.current_stream(device).cuda_stream)
