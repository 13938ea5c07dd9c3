"""CPU restatement of what the reference simulator computes for the recognised tile programs.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  Pinned by tests/golden/*.npz, which hold
outputs of the unmodified reference simulator (python/sim) on the programs in tests/programs/
(generator: tests/golden/make_golden.py), and by tests/test_oracle.py which, when the reference
tree is present, also runs the simulator live beside these functions.

Numerics follow the simulator: every block op is a torch CPU op on tiles held in the tensor's
own dtype (python/sim/block.py:870-920, python/sim/ttnnsim.py:67-109, 384-460), so on bf16
tensors each op rounds to bf16 (mode "native"); "f32" mode is the same program run on the
values upcast to fp32 with one final round-to-nearest-even to bf16 - which is what "fp32
intermediate / fp32 accumulate, bf16 out" means for a simulator that computes in the
tensor dtype.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Sequence, Tuple

from typing import Optional

import torch

TILE = 32

UNARY: Dict[str, Callable[[torch.Tensor], torch.Tensor]] = {
    # torch goldens of the element-wise op table (test/me2e/ops/__init__.py:27-41)
    "exp": torch.exp, "log": torch.log, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "tanh": torch.tanh,
    "sigmoid": torch.sigmoid, "neg": torch.neg, "abs": torch.abs, "relu": torch.relu,
}


def _in_f32(fn: Callable[..., torch.Tensor]) -> Callable[..., torch.Tensor]:
    """A function of the specification's Appendix B is ONE block op: evaluated in fp32, rounded once."""
    def wrapped(x: torch.Tensor, *params: float) -> torch.Tensor:
        return fn(x.to(torch.float32), *params).to(x.dtype)
    return wrapped


_F = torch.nn.functional
# The rest of the specification's Appendix B (docs/sphinx/specs/TTLangSpecification.md:700-748), paired with the
# torch functions the specification links to.  No reference implementation exists: parity unpinned.
UNARY.update({name: _in_f32(fn) for name, fn in {
    "exp2": torch.exp2, "expm1": torch.expm1, "logp1": torch.log1p, "square": torch.square, "recip": torch.reciprocal,
    "tan": torch.tan, "atan": torch.atan, "atanh": torch.atanh, "sin": torch.sin, "asin": torch.asin,
    "asinh": torch.asinh, "cos": torch.cos, "acos": torch.acos, "acosh": torch.acosh, "gelu": _F.gelu,
    "silu": _F.silu, "softsign": _F.softsign, "hardsigmoid": _F.hardsigmoid}.items()})
# functions with scalar parameters: name -> fn(x, *params)
PARAM_UNARY: Dict[str, Callable[..., torch.Tensor]] = {name: _in_f32(fn) for name, fn in {
    "rsub_imm": lambda x, b: b - x,
    "relu_max": lambda x, hi: torch.relu(torch.clamp(x, max=hi)),
    "relu_min": lambda x, lo: torch.relu(torch.clamp(x, min=lo)),
    "leaky_relu": lambda x, slope: _F.leaky_relu(x, slope),
    "elu": lambda x, alpha: _F.elu(x, alpha),
    "celu": lambda x, alpha, _alpha_recip: _F.celu(x, alpha),
    "softplus": lambda x, beta, _beta_recip, threshold: _F.softplus(x, beta, threshold),
    "hardtanh": lambda x, lo, hi: _F.hardtanh(x, lo, hi),
    "selu": lambda x, scale, alpha: scale * torch.where(x > 0, x, alpha * torch.expm1(x)),
}.items()}
# block ** integer is torch.pow on the tile in the tile's own type (python/sim/block.py:986-989): torch squares and
# cubes by multiplying in that type, so a bfloat16 cube rounds twice
PARAM_UNARY["pow_imm"] = lambda x, n: torch.pow(x, int(n) if float(n).is_integer() else n)
# spelling in ttl.math -> op name
MATH_NAMES = {"rsub": "rsub_imm", "prelu": "leaky_relu"}

BINARY: Dict[str, Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = {
    "add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div,
    "max": torch.maximum, "min": torch.minimum,
    # the simulator's other block operators are torch's `//`, `%`, `**` on the tile tensors
    # (python/sim/ttnnsim.py:424-450)
    "floordiv": torch.floor_divide, "mod": torch.remainder, "pow": torch.pow,
}


def expand_operand(t: torch.Tensor, out_shape: Tuple[int, int]) -> torch.Tensor:
    """Bring an operand to the output's shape the way the simulator's tile-grid broadcast does
    (python/sim/ttnnsim.py:67-109 with tiles cut by python/sim/copyhandlers.py:312-333):
    a size-1 dim broadcasts element-wise (degenerate tiles); a dim of exactly one tile (32)
    repeats that tile along the tile grid; otherwise the dim must match."""
    out = t
    for dim in (0, 1):
        n, want = out.shape[dim], out_shape[dim]
        if n == want:
            continue
        if n == 1:
            shape = list(out.shape)
            shape[dim] = want
            out = out.expand(*shape)
        elif n == TILE and want % TILE == 0:
            reps = [1, 1]
            reps[dim] = want // TILE
            out = out.repeat(*reps)
        else:
            raise ValueError(f"operand dim {dim} of size {n} cannot be broadcast to {want}")
    return out


def eval_expression(expr: Sequence, inputs: Sequence[torch.Tensor], out_shape: Tuple[int, int], mode: str) -> torch.Tensor:
    """Evaluate a nested-tuple expression, e.g. ("relu", ("add", ("mul", ("exp", ("mul", 0, 1)), 2), 3)),
    integers naming inputs.  mode "native": ops run in the inputs' dtype (bf16 ops round each
    time, as the simulator on bf16 tensors); mode "f32": inputs upcast to fp32, result rounded
    once to the inputs' dtype."""
    dt = inputs[0].dtype
    work = [t.to(torch.float32) if mode == "f32" else t for t in inputs]

    def ev(e):
        if isinstance(e, int):
            return expand_operand(work[e], out_shape)
        op = e[0]
        if isinstance(op, (tuple, list)):   # ((name, p0, ...), operand): a function with scalar parameters
            return PARAM_UNARY[MATH_NAMES.get(op[0], op[0])](ev(e[1]), *op[1:])
        if op in UNARY:
            return UNARY[op](ev(e[1]))
        if op in ("reduce_sum", "reduce_max"):
            # ("reduce_sum", expr, index of the scaler input, dims): fp32 combine, times scaler[0, 0], one
            # rounding to the working dtype; reduced dims keep length 1 and broadcast in the ops that follow
            x = ev(e[1])
            v = x.to(torch.float32)
            r = v.sum(dim=list(e[3]), keepdim=True) if op == "reduce_sum" else v.amax(dim=list(e[3]), keepdim=True)
            return (r * work[e[2]][0, 0].to(torch.float32)).to(x.dtype)
        return BINARY[op](ev(e[1]), ev(e[2]))

    return ev(expr).to(dt).contiguous()


def reduce_expression(expr: Sequence, inputs: Sequence[torch.Tensor], in_shape: Tuple[int, int], mode: str,
                      op: str, dims: Sequence[int], scaler: Optional[torch.Tensor]) -> torch.Tensor:
    """`reduce_sum / reduce_max(expr, scaler, dims)` (docs/sphinx/specs/TTLangSpecification.md:750-755; no
    reference implementation - this is the meaning the build gives it, see oracle/sim_addons.py): the
    expression's values (evaluated as `eval_expression` does, in `mode`) are combined in fp32 along `dims`,
    multiplied by the scaler's element [0, 0], and rounded once to the inputs' dtype.  Reduced dims keep
    length 1."""
    dt = inputs[0].dtype
    work = [t.to(torch.float32) if mode == "f32" else t for t in inputs]

    def ev(e):
        if isinstance(e, int):
            return expand_operand(work[e], in_shape)
        if e[0] in UNARY:
            return UNARY[e[0]](ev(e[1]))
        return BINARY[e[0]](ev(e[1]), ev(e[2]))

    vals = ev(expr).to(torch.float32)
    ds = sorted(set(dims))
    res = vals.sum(dim=ds, keepdim=True) if op == "sum" else vals.amax(dim=ds, keepdim=True)
    if scaler is not None:
        res = res * scaler[0, 0].to(torch.float32)
    return res.to(dt).contiguous()


def matmul_tiles(a: torch.Tensor, b: torch.Tensor, mode: str, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`for k: out_blk.store(a_blk @ b_blk, acc=True)` for every output tile
    (examples/singlecore_matmul.py:36-45; accumulate rule python/sim/block.py:856-864):
    the first K tile assigns, later ones add, every partial product and every running sum held
    in the tensor dtype ("native") or in fp32 with one final rounding ("f32").  All output tiles
    of one K step are computed at once as a slab product.  With `bias` the accumulation starts from
    `out_blk.store(c_blk, acc=True)` (docs/sphinx/specs/TTLangSpecification.md:290-312)."""
    dt = a.dtype
    if mode == "f32":
        a, b = a.to(torch.float32), b.to(torch.float32)
        bias = None if bias is None else bias.to(torch.float32)
    kt = -(-a.shape[1] // TILE)   # a ragged last K slab (C-ABI callers may pass K % 32 != 0) is one more step
    acc = None if bias is None else bias.clone()
    for k in range(kt):
        p = a[:, k * TILE:(k + 1) * TILE] @ b[k * TILE:(k + 1) * TILE, :]
        acc = p if acc is None else acc + p
    assert acc is not None
    return acc.to(dt)


def attention_rows(q: torch.Tensor, kt: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, scale: torch.Tensor,
                   one: torch.Tensor, mode: str = "native") -> torch.Tensor:
    """The attention tile program of tests/programs/attention.py op by op, the way the simulator evaluates it: every
    block op in the tensors' dtype ("native") - S = Q @ K^T accumulated over K tiles, z = S * scale + mask,
    m = reduce_max(z), e = exp(z - m), d = reduce_sum(e), O = (e / d) @ V; reductions as `reduce_expression`."""
    s = matmul_tiles(q, kt, mode)
    z = s * scale[0, 0] + mask
    m = (z.to(torch.float32).amax(dim=1, keepdim=True) * one[0, 0].to(torch.float32)).to(z.dtype)
    e = torch.exp(z - m)
    d = (e.to(torch.float32).sum(dim=1, keepdim=True) * one[0, 0].to(torch.float32)).to(z.dtype)
    return matmul_tiles(e / d, v, mode)


def bf16_ulp_diff(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """Distance in bf16 units-in-the-last-place between two bf16 tensors (monotone integer map)."""
    def key(t: torch.Tensor) -> torch.Tensor:
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return (key(x) - key(y)).abs()
