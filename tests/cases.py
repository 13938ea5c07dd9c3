"""Seeded parity cases shared by the golden generator and the tests.

Inputs are generated on the CPU with torch.Generator().manual_seed(seed) in fp32 and cast,
the way the reference's own tests seed theirs (examples/broadcast.py:126-133,
test/me2e/ops/__init__.py:141-148).
"""

from __future__ import annotations

from typing import Any, Callable, Dict, List, Tuple

import torch


def gen(shape: Tuple[int, int], dist: str, seed: int, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    if dist.startswith("bf16:"):      # values that bfloat16 represents exactly, whatever dtype carries them
        return gen(shape, dist[5:], seed, torch.bfloat16).to(dtype)
    g = torch.Generator().manual_seed(seed)
    if dist == "normal":
        t = torch.randn(shape, generator=g, dtype=torch.float32)
    elif dist == "uniform":           # U(-1, 1)
        t = torch.rand(shape, generator=g, dtype=torch.float32) * 2 - 1
    elif dist == "positive":          # U(0.01, 10): log / sqrt / rsqrt domain (test/me2e/ops/__init__.py:44-48)
        t = torch.rand(shape, generator=g, dtype=torch.float32) * 9.99 + 0.01
    elif dist == "ge1":               # U(1, 10): acosh domain
        t = torch.rand(shape, generator=g, dtype=torch.float32) * 9 + 1
    elif dist == "causal_mask":       # 0 where key <= query, a large negative number above the diagonal
        t = torch.triu(torch.full(shape, -1e4, dtype=torch.float32), diagonal=1)
    elif dist.startswith("const:"):
        t = torch.full(shape, float(dist.split(":")[1]), dtype=torch.float32)
    elif dist.startswith("normal*"):  # N(0, sigma)
        t = torch.randn(shape, generator=g, dtype=torch.float32) * float(dist.split("*")[1])
    else:
        raise ValueError(dist)
    return t.to(dtype)


class Case:
    def __init__(self, name: str, module: str, program: str, inputs: List[Tuple[Tuple[int, int], str, int]],
                 out_shape: Tuple[int, int], mode: str, expr: Any, check: str, factory_args: Tuple = (),
                 dtype: torch.dtype = torch.bfloat16, store: str = "full", reduce: Any = None):
        self.reduce = reduce   # (op, dims, index of the scaler input, shape of the reduced values) for reductions
        self.name, self.module, self.program, self.inputs, self.out_shape = name, module, program, inputs, out_shape
        self.mode, self.expr, self.check, self.factory_args, self.dtype, self.store = (
            mode, expr, check, factory_args, dtype, store)

    def make_inputs(self) -> List[torch.Tensor]:
        return [gen(s, d, seed, self.dtype) for (s, d, seed) in self.inputs]

    def get_program(self, modules: Dict[str, Any], f32acc: bool = False) -> Callable[..., None]:
        obj = getattr(modules[self.module], self.program)
        if self.factory_args or self.program.startswith("make_"):
            args = self.factory_args
            if self.program in ("make_unary_chain", "make_operator") or self.module == "reduce":
                return obj(*args, fp32_dest_acc_en=f32acc)
            return obj(*args)
        if f32acc and hasattr(modules[self.module], self.program + "_f32acc"):
            return getattr(modules[self.module], self.program + "_f32acc")
        return obj


_FUSED = ("relu", ("add", ("mul", ("exp", ("mul", 0, 1)), 2), 3))
_MAB = ("add", ("mul", 0, 1), 2)

CASES: List[Case] = [
    # configs[0]: eltwise add 1024x1024 bf16, seeds 0/1, simulator-native numerics
    Case("add_1024", "eltwise", "eltwise_add", [((1024, 1024), "normal", 0), ((1024, 1024), "normal", 1)],
         (1024, 1024), "native", ("add", 0, 1), "exact", store="digest"),
    Case("add_f32_256", "eltwise", "eltwise_add", [((256, 256), "normal", 0), ((256, 256), "normal", 1)],
         (256, 256), "native", ("add", 0, 1), "exact", dtype=torch.float32),
    # configs[1] at reduced size: Y = relu(exp(s*A) * b + C), both numerics modes
    Case("fused_native_256x512", "eltwise", "fused_exp_bcast",
         [((256, 512), "normal", 0), ((1, 1), "const:0.1", 0), ((1, 512), "uniform", 1), ((256, 512), "normal", 2)],
         (256, 512), "native", _FUSED, "ulp1"),
    Case("fused_f32_256x512", "eltwise", "fused_exp_bcast",
         [((256, 512), "normal", 0), ((1, 1), "const:0.1", 0), ((1, 512), "uniform", 1), ((256, 512), "normal", 2)],
         (256, 512), "f32", _FUSED, "ulp1"),
    Case("fused_f32_ragged_96x160", "eltwise", "fused_exp_bcast",
         [((96, 160), "normal", 3), ((1, 1), "const:0.1", 0), ((1, 160), "uniform", 4), ((96, 160), "normal", 5)],
         (96, 160), "f32", _FUSED, "ulp1"),
    # broadcast forms of A*B + C (general_broadcast.py): column, row vector, one tile row/col, scalar
    Case("bcast_col", "eltwise", "mul_add_bcast", [((128, 128), "uniform", 10), ((128, 128), "uniform", 11), ((128, 1), "uniform", 12)],
         (128, 128), "native", _MAB, "exact"),
    Case("bcast_row_tilecol", "eltwise", "mul_add_bcast", [((128, 128), "uniform", 13), ((1, 128), "uniform", 14), ((128, 32), "uniform", 15)],
         (128, 128), "native", _MAB, "exact"),
    Case("bcast_tilerow_scalar", "eltwise", "mul_add_bcast", [((128, 128), "uniform", 16), ((32, 128), "uniform", 17), ((1, 1), "uniform", 18)],
         (128, 128), "native", _MAB, "exact"),
    Case("bcast_tile_full", "eltwise", "mul_add_bcast", [((128, 128), "uniform", 19), ((32, 32), "uniform", 20), ((128, 128), "uniform", 21)],
         (128, 128), "native", _MAB, "exact"),
    Case("bcast_col_f32", "eltwise", "mul_add_bcast", [((128, 128), "uniform", 10), ((128, 128), "uniform", 11), ((128, 1), "uniform", 12)],
         (128, 128), "native", _MAB, "exact", dtype=torch.float32),
    # expression with temporaries
    Case("sum_of_products", "eltwise", "sum_of_products",
         [((64, 96), "uniform", 30), ((64, 96), "uniform", 31), ((64, 96), "uniform", 32), ((64, 96), "positive", 33)],
         (64, 96), "native", ("div", ("sub", ("mul", 0, 1), ("mul", 2, 3)), ("add", ("mul", 0, 0), 3)), "exact"),
    # intermediate circular buffer filled and drained by the compute thread; rows dealt out over 2 cores
    Case("intermediate_cb", "eltwise", "intermediate_cb", [((160, 96), "uniform", 34), ((160, 96), "uniform", 35)],
         (160, 96), "native", ("mul", ("exp", 0), 1), "ulp1"),
    # multicast pipe: only the 4 cores of the pipe compute (columns 0..3 of the output)
    Case("eltwise_pipe", "eltwise", "eltwise_pipe", [((128, 2048), "uniform", 40), ((128, 2048), "uniform", 41), ((32, 32), "uniform", 42)],
         (128, 2048), "native", _MAB, "exact"),
]

# one case per element-wise function of the compiler's op table
for _i, (_op, _dist, _check) in enumerate([
        ("exp", "uniform", "ulp1"), ("log", "positive", "ulp1"), ("sqrt", "positive", "exact"),
        ("rsqrt", "positive", "exact"), ("tanh", "normal", "ulp1"), ("sigmoid", "normal", "ulp1"),
        ("neg", "normal", "exact"), ("abs", "normal", "exact"), ("relu", "normal", "exact")]):
    CASES.append(Case(f"unary_{_op}", "eltwise", "make_unary_chain", [((64, 64), _dist, 50 + _i), ((64, 64), "uniform", 70 + _i)],
                      (64, 64), "native", ("add", (_op, 0), 1), _check, factory_args=([_op],)))

# the rest of the specification's Appendix B: one case per function, Y = f(A) + B (run by the specialised kernel only)
MATH_CASES: List[Case] = []
for _i, (_op, _dist, _check) in enumerate([
        ("exp2", "uniform", "ulp1"), ("expm1", "uniform", "ulp1"), ("logp1", "positive", "ulp1"),
        ("square", "normal", "exact"), ("recip", "positive", "exact"), ("tan", "uniform", "ulp1"),
        ("atan", "normal", "ulp1"), ("atanh", "uniform", "ulp1"), ("sin", "normal", "ulp1"), ("asin", "uniform", "ulp1"),
        ("asinh", "normal", "ulp1"), ("cos", "normal", "ulp1"), ("acos", "uniform", "ulp1"), ("acosh", "ge1", "ulp1"),
        ("gelu", "normal", "ulp1"), ("silu", "normal", "ulp1"), ("softsign", "normal", "exact"),
        ("hardsigmoid", "normal*3", "ulp1"),
        (("rsub", 2), "normal", "exact"), (("relu_max", 1), "normal", "exact"), (("relu_min", 1), "normal", "exact"),
        (("leaky_relu", 0.25), "normal", "exact"), (("prelu", 0.125), "normal", "exact"), (("elu", 1.5), "normal", "ulp1"),
        (("celu", 2, 0.5), "normal", "ulp1"), (("softplus", 2, 0.5, 4), "normal*3", "ulp1"),
        (("hardtanh", -0.5, 0.75), "normal", "exact"), (("selu", 1.0507, 1.67326), "normal", "ulp1")]):
    _name = _op if isinstance(_op, str) else _op[0]
    MATH_CASES.append(Case(f"math_{_name}", "eltwise", "make_unary_chain", [((64, 96), _dist, 100 + _i), ((64, 96), "uniform", 140 + _i)],
                           (64, 96), "native", ("add", (_op, 0), 1), _check, factory_args=([_op],)))

# the block operators // % ** (torch semantics through the simulator); inputs away from zero divisors
OPERATOR_CASES: List[Case] = [
    Case("op_floordiv", "eltwise", "make_operator", [((96, 128), "normal*3", 170), ((96, 128), "positive", 171)],
         (96, 128), "native", ("floordiv", 0, 1), "exact", factory_args=("floordiv",)),
    Case("op_floordiv_f32_negdiv", "eltwise", "make_operator", [((64, 96), "normal*3", 172), ((64, 96), "uniform", 173)],
         (64, 96), "native", ("floordiv", 0, 1), "exact", factory_args=("floordiv",), dtype=torch.float32),
    Case("op_mod", "eltwise", "make_operator", [((96, 128), "normal*3", 174), ((96, 128), "uniform", 175)],
         (96, 128), "native", ("mod", 0, 1), "exact", factory_args=("mod",)),
    Case("op_mod_f32", "eltwise", "make_operator", [((64, 96), "normal*3", 176), ((64, 96), "uniform", 177)],
         (64, 96), "native", ("mod", 0, 1), "exact", factory_args=("mod",), dtype=torch.float32),
    Case("op_pow_block", "eltwise", "make_operator", [((96, 128), "positive", 178), ((96, 128), "uniform", 179)],
         (96, 128), "native", ("pow", 0, 1), "ulp1", factory_args=("pow",)),
    Case("op_pow_2", "eltwise", "make_operator", [((64, 96), "normal", 180), ((64, 96), "uniform", 181)],
         (64, 96), "native", ("add", (("pow_imm", 2), 0), 1), "exact", factory_args=("pow", 2)),
    Case("op_pow_3", "eltwise", "make_operator", [((64, 96), "normal", 182), ((64, 96), "uniform", 183)],
         (64, 96), "native", ("add", (("pow_imm", 3), 0), 1), "exact", factory_args=("pow", 3)),
    Case("op_pow_5", "eltwise", "make_operator", [((64, 96), "normal", 184), ((64, 96), "uniform", 185)],
         (64, 96), "native", ("add", (("pow_imm", 5), 0), 1), "ulp1", factory_args=("pow", 5)),
]

MATMUL_CASES: List[Case] = [
    # the reference's own simulator test sizes (examples/metal_examples/*/ttlang: 256^3) and smaller
    Case("mm_single_128x256x64", "matmul", "singlecore_matmul", [((128, 256), "normal*0.0625", 0), ((256, 64), "normal*0.0625", 1)],
         (128, 64), "f32", None, "rel1e-2"),
    Case("mm_multi_256", "matmul", "multicore_matmul", [((256, 256), "normal*0.0625", 2), ((256, 256), "normal*0.0625", 3)],
         (256, 256), "f32", None, "rel1e-2"),
    Case("mm_blocked_256x512x256", "matmul", "make_blocked_matmul", [((256, 512), "normal*0.0442", 4), ((512, 256), "normal*0.0442", 5)],
         (256, 256), "f32", None, "rel1e-2", factory_args=(2, 4)),
    Case("mm_multi_native_128", "matmul", "multicore_matmul", [((128, 128), "normal*0.09", 6), ((128, 128), "normal*0.09", 7)],
         (128, 128), "native", None, "rel1e-2"),
    # the specification's matmul with bias (third input = C)
    Case("mm_bias_96x160x128", "matmul", "matmul_bias", [((96, 160), "normal*0.08", 8), ((160, 128), "normal*0.08", 9),
                                                         ((96, 128), "normal", 10)],
         (96, 128), "f32", None, "rel1e-2"),
]


# reductions (ttl.math.reduce_sum / reduce_max): the last-but-one input of the single-operand programs is the
# scaler tile; "native" = one block per result (fp32 combine, one rounding), "f32" = fp32 intermediates
def _red(name, program, args, in_shape, out_shape, op, dims, mode, check, dtype=torch.bfloat16, dist="normal", scaler="const:0.5"):
    return Case(name, "reduce", program, [(in_shape, dist, 80), ((32, 32), scaler, 0)], out_shape, mode, 0, check,
                factory_args=args, dtype=dtype, reduce=(op, dims, 1, in_shape))


REDUCE_CASES: List[Case] = [
    _red("red_sum_rows_256x160", "make_reduce", ("sum", [0]), (256, 160), (1, 160), "sum", [0], "native", "ulp1"),
    _red("red_sum_cols_160x256", "make_reduce", ("sum", [1]), (160, 256), (160, 1), "sum", [1], "native", "ulp1"),
    _red("red_sum_all_96x128", "make_reduce", ("sum", [0, 1]), (96, 128), (1, 1), "sum", [0, 1], "native", "ulp1"),
    _red("red_max_rows_256x160", "make_reduce", ("max", [0]), (256, 160), (1, 160), "max", [0], "native", "exact"),
    _red("red_max_cols_160x256", "make_reduce", ("max", [1]), (160, 256), (160, 1), "max", [1], "native", "exact"),
    _red("red_max_all_96x128", "make_reduce", ("max", [0, 1]), (96, 128), (1, 1), "max", [0, 1], "native", "exact",
         scaler="const:2.0"),
    _red("red_sum_rows_f32_128x96", "make_reduce", ("sum", [0]), (128, 96), (1, 96), "sum", [0], "native", "rel1e-5",
         dtype=torch.float32),
    _red("red_max_cols_f32_128x96", "make_reduce", ("max", [1]), (128, 96), (128, 1), "max", [1], "native", "exact",
         dtype=torch.float32),
    # accumulated over blocks of 2 row tiles with store(acc=True): fp32 partial sums
    _red("red_colsum_acc_256x96", "make_colsum_acc", (2,), (256, 96), (1, 96), "sum", [0], "f32", "ulp1"),
    _red("red_colsum_acc_f32_256x96", "make_colsum_acc", (2,), (256, 96), (1, 96), "sum", [0], "native", "rel1e-5",
         dtype=torch.float32),
    # element-wise chain + broadcast row vector reduced over columns: sum_j exp(a_ij) * b_j
    Case("red_rowsum_exp_128x256", "reduce", "make_rowsum_exp",
         [((128, 256), "uniform", 81), ((1, 256), "uniform", 82), ((32, 32), "const:0.25", 0)], (128, 1), "f32",
         ("mul", ("exp", 0), 1), "ulp1", factory_args=(), reduce=("sum", [1], 2, (128, 256))),
]


# tile programs whose reductions feed further element-wise ops (results pass through circular buffers)
_SM_E = ("exp", ("sub", 0, ("reduce_max", 0, 1, [1])))
_SOFTMAX = ("div", _SM_E, ("reduce_sum", _SM_E, 1, [1]))
_ST_C = ("sub", 0, ("reduce_sum", 0, 1, [1]))
_STANDARDIZE = ("mul", _ST_C, ("rsqrt", ("reduce_sum", ("mul", _ST_C, _ST_C), 1, [1])))
COMPOSITE_CASES: List[Case] = [
    Case("softmax_128x256", "reduce", "make_softmax", [((128, 256), "normal", 85), ((32, 32), "const:1.0", 0)],
         (128, 256), "native", _SOFTMAX, "ulp2", factory_args=()),
    Case("softmax_f32_96x160", "reduce", "make_softmax", [((96, 160), "normal", 86), ((32, 32), "const:1.0", 0)],
         (96, 160), "native", _SOFTMAX, "rel1e-5", factory_args=(), dtype=torch.float32),
    Case("standardize_128x256", "reduce", "make_standardize", [((128, 256), "normal", 87), ((32, 32), "const:0.00390625", 0)],
         (128, 256), "native", _STANDARDIZE, "ulp2", factory_args=()),
    Case("standardize_f32_96x128", "reduce", "make_standardize", [((96, 128), "normal", 88), ((32, 32), "const:0.0078125", 0)],
         (96, 128), "native", _STANDARDIZE, "rel1e-5", factory_args=(), dtype=torch.float32),
]


# matmul whose result is used further: product through an intermediate circular buffer, then bias + activation.
# `expr` is the epilogue over [product, further inputs...]
EPILOGUE_CASES: List[Case] = [
    Case("linear_relu_96x160x128", "matmul", "linear_relu",
         [((96, 160), "normal*0.08", 11), ((160, 128), "normal*0.08", 12), ((1, 128), "normal", 13)],
         (96, 128), "native", ("relu", ("add", 0, 1)), "rel1e-2"),
]


# attention written as a tile program (tests/programs/attention.py); the one-tile size is what the reference
# simulator can run (its block matmul needs K = 1 tile); inputs: q, k^T, v, additive causal mask, scale tile, ones tile
def _attn_inputs(s, d, exact_in_bf16=False):
    pre = "bf16:" if exact_in_bf16 else ""
    return [((s, d), pre + "normal", 200), ((d, s), pre + "normal", 201), ((s, d), pre + "normal", 202),
            ((s, s), "causal_mask", 0), ((32, 32), f"{pre}const:{d ** -0.5}", 0), ((32, 32), "const:1.0", 0)]


ATTENTION_CASES: List[Case] = [
    Case("attention_tile_32", "attention", "attention_rows", _attn_inputs(32, 32), (32, 32), "native", None, "rel1e-2"),
    Case("attention_tile_32_f32", "attention", "attention_rows", _attn_inputs(32, 32), (32, 32), "native", None, "rel1e-5",
         dtype=torch.float32),
]

# the same attention as three kernels (scores, masked softmax, probabilities @ V) in 1x1-tile block matmuls, which the
# simulator runs at the fused kernel's head dimension: these fixtures pin the fused attention kernel to the simulator
ATTENTION_PIPELINE_CASES: List[Case] = [
    Case("attention_pipeline_256x128_f32", "attention", "attention_pipeline", _attn_inputs(256, 128, True), (256, 128), "native",
         None, "rel1e-5", dtype=torch.float32),
    Case("attention_pipeline_256x128", "attention", "attention_pipeline", _attn_inputs(256, 128), (256, 128), "native",
         None, "rel1e-2"),
    Case("attention_pipeline_128x128_f32", "attention", "attention_pipeline", _attn_inputs(128, 128, True), (128, 128), "native",
         None, "rel1e-5", dtype=torch.float32),
]


def by_name(name: str) -> Case:
    for c in (CASES + MATMUL_CASES + REDUCE_CASES + COMPOSITE_CASES + MATH_CASES + EPILOGUE_CASES + OPERATOR_CASES + ATTENTION_CASES
              + ATTENTION_PIPELINE_CASES):
        if c.name == name:
            return c
    raise KeyError(name)
