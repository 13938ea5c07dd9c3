"""GPU parity of the reduction kernels (`ttl.math.reduce_sum` / `reduce_max` -> ttlb_reduce), run the way a
user runs them: tt-lang program -> tracer -> recogniser -> C ABI -> CUDA kernel specialised for the program.
Checked against the simulator fixtures (simulator + the reduction add-on) and the CPU oracle."""


import pytest
import torch

import cases
from conftest import golden_tensor, load_golden
from test_oracle import oracle_output
from test_reduce import close

pytestmark = pytest.mark.gpu


def _launches():
    from ttl_b200 import capi
    return capi.context().launch_count()


@pytest.mark.parametrize("case", cases.REDUCE_CASES, ids=lambda c: c.name)
def test_program_matches_simulator_and_oracle(case, backend):
    _, mods = backend
    import ttnn
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    out = ttnn.from_torch(torch.full(case.out_shape, 7.0, dtype=case.dtype))
    before = _launches()
    case.get_program(mods, f32acc=(case.mode == "f32"))(*ins, out)
    assert _launches() == before + 1, "one reduction kernel per program"
    got = ttnn.to_torch(out)
    close(got, oracle_output(case), case.check, "vs oracle")
    close(got, golden_tensor(load_golden(case.name)["out"], case.dtype), case.check, "vs simulator golden")


@pytest.fixture(params=[True, False], ids=["row_fused", "launch_by_launch"])
def row_fusion(request):
    import ttl_b200
    ttl_b200.set_row_fusion(request.param)
    yield request.param
    ttl_b200.set_row_fusion(True)


@pytest.mark.parametrize("case", cases.COMPOSITE_CASES, ids=lambda c: c.name)
def test_reductions_inside_expressions(case, backend, row_fusion):
    """Softmax / row standardisation as tile programs: one row-resident launch, or three launches (two
    reductions into temporaries, one element-wise); against the simulator fixture and the oracle; a second
    call reuses the plan."""
    _, mods = backend
    import ttnn
    prog = case.get_program(mods)
    n_launches = 1 if row_fusion else 3
    want = golden_tensor(load_golden(case.name)["out"], case.dtype)
    for _ in range(2):
        ins = [ttnn.from_torch(t) for t in case.make_inputs()]
        out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
        before = _launches()
        prog(*ins, out)
        assert _launches() == before + n_launches
        got = ttnn.to_torch(out)
        close(got, oracle_output(case), case.check, "vs oracle")
        close(got, want, case.check, "vs simulator golden")


def test_softmax_full_size(backend, row_fusion):
    """Row softmax of a bf16 [8192, 8192] tensor as a tile program, fp32 tensors' worth of checks: rows sum
    to one, results within bf16 rounding of a float64 softmax."""
    _, mods = backend
    import ttnn
    n = 8192
    x = cases.gen((n, n), "normal", 93)
    s = ttnn.from_torch(torch.ones(32, 32, dtype=torch.bfloat16))
    out = ttnn.from_torch(torch.zeros((n, n), dtype=torch.bfloat16))
    before = _launches()
    mods["reduce"].make_softmax()(ttnn.from_torch(x), s, out)
    assert _launches() == before + (1 if row_fusion else 3)
    got = ttnn.to_torch(out).double()
    want = torch.softmax(x.double(), dim=1)
    # every op rounds to bf16: x - max (up to 2^-9 * 10 absolute, so 2 % in the exponential), exp, the row
    # sum, the quotient
    assert ((got - want).abs() <= 2.0 ** -5 * want + 1e-7).all()
    assert (got.sum(dim=1) - 1).abs().max() < 2e-2


def test_full_tile_output_and_repeat_calls(backend):
    """Output of full tiles: value in row 0 of the tile, zeros below.  The scratch (partial rows, arrival
    counters) is shared by all calls of a context: a second and third call must give the same bits."""
    _, mods = backend
    import ttnn
    case = cases.by_name("red_sum_rows_256x160")
    prog = case.get_program(mods)
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    first = None
    for i in range(3):
        out = ttnn.from_torch(torch.full((32, 160), float(i + 1), dtype=case.dtype))
        prog(*ins, out)
        got = ttnn.to_torch(out)
        close(got[0:1], oracle_output(case), case.check, "row 0")
        assert (got[1:] == 0).all()
        first = got if first is None else first
        assert torch.equal(got.view(torch.int16), first.view(torch.int16))


@pytest.mark.parametrize("dims", [[0], [1], [0, 1]], ids=["rows", "cols", "all"])
@pytest.mark.parametrize("op", ["sum", "max"])
def test_full_size_8192(backend, op, dims):
    """8192 x 8192 bf16 (134 MB, larger than L2): against a float64 reduction of the same values, bit-identical
    across launches, and exactly linear in a power-of-two scaler."""
    _, mods = backend
    import ttnn
    n = 8192
    a = cases.gen((n, n), "normal", 90)
    out_shape = (1 if 0 in dims else n, 1 if 1 in dims else n)
    prog = mods["reduce"].make_reduce(op, dims)
    a_dev = ttnn.from_torch(a)
    results = []
    for sval in (1.0, 1.0, 4.0):
        s = ttnn.from_torch(torch.full((32, 32), sval, dtype=torch.bfloat16))
        out = ttnn.from_torch(torch.zeros(out_shape, dtype=torch.bfloat16))
        before = _launches()
        prog(a_dev, s, out)
        assert _launches() == before + 1
        results.append(ttnn.to_torch(out))
    r1, r1b, r4 = results
    assert torch.equal(r1.view(torch.int16), r1b.view(torch.int16)), "the summation order must be fixed"
    assert torch.equal((r1.float() * 4).to(torch.bfloat16).view(torch.int16), r4.view(torch.int16))
    ref = a.double().sum(dim=dims, keepdim=True) if op == "sum" else a.double().amax(dim=dims, keepdim=True)
    if op == "max":
        assert torch.equal(r1.double(), ref)
    else:
        # fp32 accumulation of 8192 (or 67M) N(0,1) values, then one bf16 rounding (2^-9 relative)
        scale = (n ** 0.5) if len(dims) == 1 else float(n)
        err = (r1.double() - ref).abs().max().item()
        assert err <= 2.0 ** -8 * ref.abs().max().item() + 1e-3 * scale, f"abs err {err}"


def test_fused_chain_full_width(backend):
    """sum_j exp(a_ij) * b_j over 4096 columns, fp32 intermediates: the element-wise chain runs inside the
    reduction kernel (one launch, no intermediate tensor)."""
    _, mods = backend
    import ttnn
    a = cases.gen((512, 4096), "uniform", 91)
    b = cases.gen((1, 4096), "uniform", 92)
    s = cases.gen((32, 32), "const:0.5", 0)
    out = ttnn.from_torch(torch.zeros((512, 1), dtype=torch.bfloat16))
    before = _launches()
    mods["reduce"].make_rowsum_exp(fp32_dest_acc_en=True)(*(ttnn.from_torch(t) for t in (a, b, s)), out)
    assert _launches() == before + 1
    want = ((torch.exp(a.double()) * b.double()).sum(dim=1, keepdim=True) * 0.5)
    got = ttnn.to_torch(out).double()
    assert ((got - want).abs() <= 2.0 ** -8 * want.abs() + 1e-2).all()


def test_c_abi_rejects_bad_descriptors(backend):
    from ttl_b200 import capi
    ctx = capi.context()
    x = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    o = torch.zeros((1, 64), dtype=torch.bfloat16, device="cuda")

    def desc():
        r = capi.ReduceDesc()
        d = r.src
        d.dtype, d.n_in, d.n_ops = capi.TTLB_BF16, 1, 1
        d.inp[0].ptr, d.inp[0].ld = x.data_ptr(), 64
        d.ops[0].opcode, d.ops[0].arg = 0, 0
        d.rows, d.cols = 64, 64
        r.op, r.dims, r.out, r.out_ld, r.fill_rows, r.fill_cols = 0, 1, o.data_ptr(), 64, 1, 1
        return r

    ctx.reduce(desc(), 0)   # the well-formed descriptor runs
    for mutate, code in ((lambda r: setattr(r, "out", 0), capi.TTLB_ERR_INVALID_ARG),
                         (lambda r: setattr(r, "out", o.data_ptr() + 2), capi.TTLB_ERR_INVALID_ARG),
                         (lambda r: setattr(r, "dims", 7), capi.TTLB_ERR_INVALID_ARG),
                         (lambda r: setattr(r.src.inp[0], "ptr", 0), capi.TTLB_ERR_INVALID_ARG)):
        r = desc()
        mutate(r)
        with pytest.raises(capi.BackendError) as e:
            ctx.reduce(r, 0)
        assert e.value.code == code
    torch.cuda.synchronize()
    assert o.float().abs().sum().item() == 0.0


def test_rows_too_long_for_the_row_resident_kernel_fall_back(backend, monkeypatch):
    """The kernel itself refuses rows that do not fit in registers (TTLB_ERR_UNSUPPORTED, nothing launched);
    the launch then runs stage by stage.  Forced here by lifting the recogniser's own limit."""
    from ttl_b200 import capi, recognize
    _, mods = backend
    import ttnn
    monkeypatch.setattr(recognize, "MAX_FUSED_VECTORS_PER_ROW", 1 << 30)
    x = cases.gen((64, 16384), "normal", 94, torch.float32)       # 4096 vectors of 16 bytes per row
    s = ttnn.from_torch(torch.ones(32, 32, dtype=torch.float32))
    out = ttnn.from_torch(torch.zeros((64, 16384), dtype=torch.float32))
    prog = mods["reduce"].make_softmax()
    xin = ttnn.from_torch(x)
    plan = prog.plan(xin, s, out)
    assert [d["kind"] for d in plan.describe()] == ["row_fused"]
    before = _launches()
    prog(xin, s, out)
    assert _launches() == before + 3, "three stage launches after the fused launch was refused"
    assert plan.launches[0]._unfused
    want = torch.softmax(x.double(), dim=1)
    assert ((ttnn.to_torch(out).double() - want).abs() <= 1e-5 * want + 1e-9).all()
    prog(xin, s, out)                                            # the refusal is remembered
    assert _launches() == before + 6
