"""Differential test of the kernel generators at the C ABI: seeded random accumulator programs (operand index
modes, offsets, ragged rectangles, stack use) run by ttlb_eltwise (specialised and generic kernel) and by
ttlb_reduce (all three forms), against the host evaluation of the same descriptor (oracle/plan_oracle.py).

Inputs are small integers and the ops are add / sub / mul / max / min / relu / abs / neg, so every fp32
intermediate is exact: results must be bit-identical whatever the order of a sum, in both rounding modes."""

import random

import pytest
import torch

from oracle import plan_oracle

pytestmark = pytest.mark.gpu

SAME, ZERO, TILE, FIRST = 0, 1, 2, 3
BINARY = ["add", "sub", "rsub", "mul", "max", "min"]
UNARY = ["relu", "abs", "neg"]


def make_program(rng, n_in, max_steps=8, allow_mul=True):
    """A random valid accumulator program: the stack is never deeper than 2 and is empty at the end."""
    ops = [("load", rng.randrange(n_in))]
    depth = 0
    muls = 0
    for _ in range(rng.randrange(1, max_steps + 1)):
        kind = rng.random()
        if kind < 0.45:
            op = rng.choice(BINARY)
            if op == "mul":
                muls += 1
                if muls > 2 or not allow_mul:   # keep the integers small enough for exact fp32 arithmetic
                    op = "add"
            ops.append((op, rng.randrange(n_in)))
        elif kind < 0.65:
            ops.append((rng.choice(UNARY), 0))
        elif kind < 0.85 and depth < 2:
            ops += [("push", 0), ("load", rng.randrange(n_in))]
            depth += 1
        elif depth > 0:
            ops.append((rng.choice(["add", "sub", "rsub", "max", "min"]), -1))
            depth -= 1
    while depth > 0:
        ops.append((rng.choice(["add", "sub", "max"]), -1))
        depth -= 1
    return ops


def make_operand(rng, row0, rows, col0, cols, dtype, vec):
    """A tensor and index modes under which every access of the rectangle is in range."""
    def dim(mode, lo, n, align):
        if mode == SAME:        # index = i + off
            off = rng.choice([0, align, 2 * align] + ([-align * (lo // align)] if lo >= align else []))
            return off, lo + n + off
        if mode == ZERO:        # index = off
            off = rng.randrange(0, 40)
            return off, off + 1
        if mode == TILE:        # index = off + i mod 32
            off = rng.randrange(0, 3) * 32
            return off, off + 32
        off = rng.choice([0, 32] + ([-32 * (lo // 32)] if lo >= 32 else []))   # FIRST: index = off + i - i mod 32
        return off, off + ((lo + n - 1) // 32) * 32 + 1
    rm, cm = rng.choice([SAME, SAME, ZERO, TILE, FIRST]), rng.choice([SAME, SAME, ZERO, TILE, FIRST])
    ro, need_r = dim(rm, row0, rows, 1)
    co, need_c = dim(cm, col0, cols, vec)
    ld = -(-max(need_c, 1) // vec) * vec + vec * rng.randrange(0, 2)
    t = torch.randint(-3, 4, (need_r + rng.randrange(0, 2), ld), generator=torch.Generator().manual_seed(rng.randrange(1 << 30)))
    return t.to(dtype), (rm, ro, cm, co)


def build(seed, dtype, small=False):
    """small: sizes and programs whose SUM over the whole rectangle stays exact in fp32."""
    rng = random.Random(seed)
    vec = 8 if dtype == torch.bfloat16 else 4
    rows = rng.choice([1, 7, 32, 33, 96] + ([] if small else [200]))
    cols = rng.choice([1, 2, 5, 16] + ([] if small else [40])) * vec
    row0, col0 = rng.choice([0, 0, 3, 32]), rng.choice([0, 0, 1, 4]) * vec
    n_in = rng.randrange(1, 5)
    tensors, inputs = [], []
    for k in range(n_in):
        t, (rm, ro, cm, co) = make_operand(rng, row0, rows, col0, cols, dtype, vec)
        tensors.append(t)
        inputs.append((k, rm, ro, cm, co))
    ops = make_program(rng, n_in, 4, False) if small else make_program(rng, n_in)
    return rng, ops, tensors, inputs, (row0, rows, col0, cols)


def fill_desc(capi, d, ops, dev, inputs, rect, dtype, round_each_op):
    row0, rows, col0, cols = rect
    d.dtype = capi.TTLB_BF16 if dtype == torch.bfloat16 else capi.TTLB_F32
    d.round_each_op = 1 if round_each_op else 0
    d.n_in, d.n_ops = len(inputs), len(ops)
    for k, (ti, rm, ro, cm, co) in enumerate(inputs):
        d.inp[k].ptr, d.inp[k].ld = dev[ti].data_ptr(), dev[ti].stride(0)
        d.inp[k].row_mode, d.inp[k].row_off, d.inp[k].col_mode, d.inp[k].col_off = rm, ro, cm, co
    for k, (op, arg) in enumerate(ops):
        d.ops[k].opcode, d.ops[k].arg = capi.OPCODES[op], arg
    d.row0, d.rows, d.col0, d.cols = row0, rows, col0, cols


def expected(ops, tensors, inputs, rect, rnd):
    row0, rows, col0, cols = rect
    return plan_oracle._evaluate(inputs, ops, tensors, torch.arange(row0, row0 + rows), torch.arange(col0, col0 + cols), rnd)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32"])
@pytest.mark.parametrize("seed", range(16))
def test_random_elementwise_programs(seed, dtype, backend):
    from ttl_b200 import capi
    ctx = capi.context()
    rng, ops, tensors, inputs, rect = build(seed, dtype)
    row0, rows, col0, cols = rect
    rnd = dtype == torch.bfloat16 and seed % 2 == 0
    want = expected(ops, tensors, inputs, rect, rnd).to(dtype)
    dev = [t.cuda() for t in tensors]
    vec = 8 if dtype == torch.bfloat16 else 4
    for mode in (capi.ELTWISE_SPECIALISED, capi.ELTWISE_GENERIC):
        out = torch.full((row0 + rows + 2, col0 + cols + vec), 9.0, dtype=dtype, device="cuda")
        d = capi.EltwiseDesc()
        fill_desc(capi, d, ops, dev, inputs, rect, dtype, rnd)
        d.out, d.out_ld = out.data_ptr(), out.stride(0)
        ctx.set_eltwise_mode(mode)
        try:
            ctx.eltwise(d, capi.current_stream())
        finally:
            ctx.set_eltwise_mode(capi.ELTWISE_AUTO)
        got = out.cpu()
        assert torch.equal(got[row0:row0 + rows, col0:col0 + cols].float(), want.float()), (seed, mode, ops, inputs, rect)
        got[row0:row0 + rows, col0:col0 + cols] = 9.0
        assert (got == 9.0).all(), "the kernel wrote outside its rectangle"


@pytest.mark.parametrize("dims", [1, 2, 3], ids=["rows", "cols", "all"])
@pytest.mark.parametrize("op", ["sum", "max"])
@pytest.mark.parametrize("seed", range(8))
def test_random_reductions(seed, op, dims, backend):
    from ttl_b200 import capi
    ctx = capi.context()
    dtype = torch.bfloat16 if seed % 2 else torch.float32
    rng, ops, tensors, inputs, rect = build(1000 + seed * 7 + dims, dtype, small=True)
    row0, rows, col0, cols = rect
    rnd = dtype == torch.bfloat16 and seed % 4 == 1
    vals = expected(ops, tensors, inputs, rect, rnd)
    ds = [d for d, bit in ((0, 1), (1, 2)) if dims & bit]
    res = vals.sum(dim=ds, keepdim=True) if op == "sum" else vals.amax(dim=ds, keepdim=True)
    scale = rng.choice([1.0, 0.5, 2.0])
    want = (res * scale).to(dtype)
    fill_r, fill_c = rng.choice([1, 32]), rng.choice([1, 32])
    out_rows = fill_r if dims & 1 else rows
    out_cols = fill_c if dims & 2 else cols
    vec = 8 if dtype == torch.bfloat16 else 4
    out = torch.full((out_rows + 1, -(-out_cols // vec) * vec + vec), 9.0, dtype=dtype, device="cuda")
    scaler = torch.full((1, 1), scale, dtype=dtype, device="cuda")
    dev = [t.cuda() for t in tensors]
    r = capi.ReduceDesc()
    fill_desc(capi, r.src, ops, dev, inputs, rect, dtype, rnd)
    r.op = capi.REDUCE_SUM if op == "sum" else capi.REDUCE_MAX
    r.dims, r.scaler, r.out, r.out_ld, r.fill_rows, r.fill_cols = dims, scaler.data_ptr(), out.data_ptr(), out.stride(0), fill_r, fill_c
    for _ in range(2):     # twice: the scratch and its counters are reused
        ctx.reduce(r, capi.current_stream())
    got = out.cpu()
    block = torch.zeros(out_rows, out_cols)
    block[:want.shape[0], :want.shape[1]] = want.float()
    assert torch.equal(got[:out_rows, :out_cols].float(), block), (seed, op, dims, ops, inputs, rect)
    got[:out_rows, :out_cols] = 9.0
    assert (got == 9.0).all(), "the kernel wrote outside its result"


@pytest.mark.parametrize("seed", range(12))
def test_random_row_fused_programs(seed, backend):
    """ttlb_rowfused: one to three reductions over columns, each program free to read the results of the earlier
    ones, then a final element-wise program; against the same stages evaluated one after the other on the host."""
    from ttl_b200 import capi
    ctx = capi.context()
    rng = random.Random(5000 + seed)
    dtype = torch.bfloat16 if seed % 2 else torch.float32
    vec = 8 if dtype == torch.bfloat16 else 4
    rnd = dtype == torch.bfloat16 and seed % 4 == 1
    rows, cols = rng.choice([1, 7, 33, 96]), rng.choice([1, 2, 5]) * vec
    row0, col0 = rng.choice([0, 3, 32]), rng.choice([0, 1]) * vec
    rect = (row0, rows, col0, cols)
    n_mem = rng.randrange(1, 4)
    tensors, mem_inputs = [], []
    for k in range(n_mem):
        t, (rm, ro, cm, co) = make_operand(rng, row0, rows, col0, cols, dtype, vec)
        if k == 0:
            rm, cm, ro, co = SAME, SAME, 0, 0      # at least one operand that varies along both dims
            t = torch.randint(-3, 4, (row0 + rows, col0 + cols), generator=torch.Generator().manual_seed(seed)).to(dtype)
        tensors.append(t)
        mem_inputs.append((k, rm, ro, cm, co))
    dev = [t.cuda() for t in tensors]
    n_phases = rng.randrange(1, 4)
    f = capi.RowFusedDesc()
    f.n_phases = n_phases
    results = []                    # host tensors [row0 + rows, 1] holding the phase results
    scalers = []
    for st in range(n_phases + 1):
        # operands of this stage: the memory operands and the earlier results
        inputs = list(mem_inputs) + [(n_mem + q, SAME, 0, ZERO, 0) for q in range(len(results))]
        ops = make_program(rng, len(inputs), 2, False)
        vals = plan_oracle._evaluate(inputs, ops, tensors + results, torch.arange(row0, row0 + rows),
                                     torch.arange(col0, col0 + cols), rnd)
        d = f.phase[st].src if st < n_phases else f.final
        d.dtype = capi.TTLB_BF16 if dtype == torch.bfloat16 else capi.TTLB_F32
        d.round_each_op = 1 if rnd else 0
        d.n_in, d.n_ops = len(inputs), len(ops)
        for k, (ti, rm, ro, cm, co) in enumerate(inputs):
            if ti < n_mem:
                d.inp[k].ptr, d.inp[k].ld = dev[ti].data_ptr(), dev[ti].stride(0)
                d.inp[k].row_mode, d.inp[k].row_off, d.inp[k].col_mode, d.inp[k].col_off = rm, ro, cm, co
            else:
                d.inp[k].row_mode, d.inp[k].row_off = capi.IDX_PHASE, ti - n_mem
        for k, (op, arg) in enumerate(ops):
            d.ops[k].opcode, d.ops[k].arg = capi.OPCODES[op], arg
        d.row0, d.rows, d.col0, d.cols = rect
        if st == n_phases:
            want = vals.to(dtype)
            break
        op = rng.choice(["sum", "max"])
        scale = rng.choice([1.0, 0.5, 2.0])
        red = vals.sum(dim=1, keepdim=True) if op == "sum" else vals.amax(dim=1, keepdim=True)
        res = torch.zeros(row0 + rows, 1, dtype=dtype)
        res[row0:] = (red * scale).to(dtype)
        results.append(res)
        scalers.append(torch.full((1, 1), scale, dtype=dtype, device="cuda"))
        f.phase[st].op = capi.REDUCE_SUM if op == "sum" else capi.REDUCE_MAX
        f.phase[st].dims = capi.REDUCE_COLS
        f.phase[st].scaler = scalers[-1].data_ptr()
    out = torch.full((row0 + rows + 1, col0 + cols + vec), 9.0, dtype=dtype, device="cuda")
    # the second reduction's result is also written out, as ttlb_reduce would (fill 1)
    red_out = torch.full((rows + 1, vec), 9.0, dtype=dtype, device="cuda")
    if n_phases >= 2:
        f.phase[1].out, f.phase[1].out_ld, f.phase[1].fill_cols = red_out.data_ptr(), red_out.stride(0), 1
    f.final.out, f.final.out_ld = out.data_ptr(), out.stride(0)
    ctx.rowfused(f, capi.current_stream())
    got = out.cpu()
    assert torch.equal(got[row0:row0 + rows, col0:col0 + cols].float(), want.float()), (seed, n_phases, rect)
    got[row0:row0 + rows, col0:col0 + cols] = 9.0
    assert (got == 9.0).all(), "the kernel wrote outside its rectangle"
    if n_phases >= 2:
        r = red_out.cpu()
        assert torch.equal(r[:rows, 0].float(), results[1][row0:, 0].float())
        r[:rows, 0] = 9.0
        assert (r == 9.0).all()
