"""Reductions (`ttl.math.reduce_sum` / `reduce_max`) without a GPU: the oracle against the simulator
fixtures, the tracer and recogniser (the plan is evaluated on the host by the plan oracle), the
descriptor checks of the C ABI and the generated CUDA source."""

import ctypes

import pytest
import torch

import cases
from conftest import digest, golden_tensor, load_golden
from oracle import plan_oracle, tile_oracle
from test_oracle import oracle_output


def close(got, want, how, what):
    """exact: bit-identical.  ulp1: the fp32 sum may be formed in another order, so a result may land on
    the other side of a bf16 rounding boundary: at most 1 bf16 ulp.  rel1e-5: fp32 results."""
    if how == "exact":
        assert torch.equal(got.view(torch.int16) if got.dtype == torch.bfloat16 else got,
                           want.view(torch.int16) if want.dtype == torch.bfloat16 else want), what
    elif how in ("ulp1", "ulp2"):
        # ulp2: programs that pass a rounded reduction result on (softmax, standardisation) - a one-ulp
        # difference in a row's maximum or sum moves every element of the row
        ulp = tile_oracle.bf16_ulp_diff(got, want)
        # near a zero crossing ulps are meaningless: allow the ulps or 1e-3 of the largest result
        bad = (ulp > int(how[3])) & ((got.float() - want.float()).abs() > 1e-3 * want.float().abs().max())
        assert not bad.any(), f"{what}: max ulp {int(ulp.max())}"
    else:
        err = (got.float() - want.float()).abs().max() / want.float().abs().max()
        assert err <= 1e-5, f"{what}: rel err {err}"


@pytest.mark.parametrize("case", cases.REDUCE_CASES, ids=lambda c: c.name)
def test_oracle_matches_simulator_golden(case):
    g = load_golden(case.name)
    assert str(g["input_digest"]) == digest(case.make_inputs()), "seeded inputs drifted from the fixture"
    close(oracle_output(case), golden_tensor(g["out"], case.dtype), case.check, case.name)


@pytest.mark.parametrize("case", cases.REDUCE_CASES, ids=lambda c: c.name)
def test_program_is_recognised_and_plan_matches_simulator(case, backend):
    _, mods = backend
    import ttnn
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    out = ttnn.from_torch(torch.full(case.out_shape, 7.0, dtype=case.dtype))
    plan = case.get_program(mods, f32acc=(case.mode == "f32")).plan(*ins, out)
    d = plan.describe()
    op, dims, _si, in_shape = case.reduce
    assert {x["kind"] for x in d} == {"reduce_" + op}
    assert len(d) == 1, "the per-core reductions of neighbouring strips merge into one launch"
    assert d[0]["dims"] == dims
    assert d[0]["reduced_tiles"] == (in_shape[0] // 32 if 0 in dims else 0, in_shape[1] // 32 if 1 in dims else 0)
    plan_oracle.run_plan(plan, [t._tensor for t in ins] + [out._tensor])
    close(out._tensor, golden_tensor(load_golden(case.name)["out"], case.dtype), case.check, case.name)


@pytest.mark.parametrize("case", cases.COMPOSITE_CASES, ids=lambda c: c.name)
def test_reductions_inside_expressions(case, backend):
    """Softmax and row standardisation written as tile programs: the reductions become launches of their own
    into temporaries of the plan (the element-wise ops in front of a reduction fused into it), the last
    launch is element-wise and reads the temporaries as broadcast columns."""
    g = load_golden(case.name)
    assert str(g["input_digest"]) == digest(case.make_inputs())
    want = golden_tensor(g["out"], case.dtype)
    close(oracle_output(case), want, case.check, "oracle vs simulator")
    _, mods = backend
    import ttnn
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
    import ttl_b200
    stages = ["reduce_max", "reduce_sum", "eltwise"] if "softmax" in case.name else ["reduce_sum", "reduce_sum", "eltwise"]
    for fusion in (False, True):
        ttl_b200.set_row_fusion(fusion)
        try:
            plan = case.get_program(mods).plan(*ins, out)
        finally:
            ttl_b200.set_row_fusion(True)
        d = plan.describe()
        if fusion:   # the three stages as one row-resident launch
            assert [x["kind"] for x in d] == ["row_fused"]
            assert [x["kind"] for x in d[0]["phases"]] + [d[0]["final"]["kind"]] == stages
        else:
            assert [x["kind"] for x in d] == stages
        assert len(plan.temps) == 2 and all(t.shape == (case.out_shape[0], 1) for t in plan.temps)
        out._tensor.zero_()
        plan_oracle.run_plan(plan, [t._tensor for t in ins] + [out._tensor])
        close(out._tensor, want, case.check, "plan vs simulator")
    if "softmax" in case.name:
        assert (out._tensor.float().sum(dim=1) - 1).abs().max() < 2e-2


def test_row_fused_source_reads_each_operand_once(backend):
    from ttl_b200 import capi
    _, mods = backend
    import ttnn
    z = lambda s: ttnn.from_torch(torch.zeros(s, dtype=torch.bfloat16))  # noqa: E731
    args = [z((8192, 8192)), z((32, 32)), z((8192, 8192))]
    plan = mods["reduce"].make_softmax(fp32_dest_acc_en=True).plan(*args)
    src = capi.rowfused_source(plan.launches[0].desc(plan.indexed(args), with_pointers=False))
    body = src.split("ttlb_rowfused_jit", 1)[1]
    # x: 1024 vectors per row on 512 threads = 2 vectors per thread, loaded once for all three stages (written
    # twice in the source: the first row, and inside the loop the prefetch of the CTA's next row)
    assert "__launch_bounds__(512)" in src
    assert body.count("ld_stream(") == 4 and body.count("g0_0 = h0_0") == 1
    assert body.count("expf(") == 2, "exp(x - max) is evaluated once per vector and carried over to the last stage"
    assert body.count("__shfl_xor_sync") == 2 and "phv0" in body and "phv1" in body
    # rows too long to hold on chip are left as separate launches
    args = [z((32, 32768)), z((32, 32)), z((32, 32768))]
    kinds = [d["kind"] for d in mods["reduce"].make_softmax().plan(*args).describe()]
    assert kinds == ["reduce_max", "reduce_sum", "eltwise"]


def test_full_tile_output_has_the_value_in_row_zero(backend):
    """An output of full tiles gets the result in the first row of its tiles and zeros below (the layout a
    hardware broadcast source has)."""
    _, mods = backend
    import ttnn
    case = cases.by_name("red_sum_rows_256x160")
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    out = ttnn.from_torch(torch.full((32, 160), 7.0, dtype=case.dtype))
    plan = case.get_program(mods).plan(*ins, out)
    plan_oracle.run_plan(plan, [t._tensor for t in ins] + [out._tensor])
    close(out._tensor[0:1], oracle_output(case), "exact", "row 0")
    assert (out._tensor[1:] == 0).all()


def test_unsupported_forms_are_rejected_with_a_reason(backend):
    import ttl
    import ttnn
    from ttl_b200 import Unsupported
    _, mods = backend
    z = lambda s, dt=torch.bfloat16: ttnn.from_torch(torch.zeros(s, dtype=dt))  # noqa: E731
    # accumulating over blocks of a bf16 tensor rounds each partial in the simulator: needs fp32_dest_acc_en
    with pytest.raises(Unsupported, match="fp32_dest_acc_en"):
        mods["reduce"].make_colsum_acc(2).plan(z((128, 64)), z((32, 32)), z((1, 64)))
    with pytest.raises(ValueError, match="dims"):
        ttl.math.reduce_sum(None, None, dims=None)

    @ttl.kernel(grid=(1, 1))
    def red_in_expr(a, s, out):
        a_cb = ttl.make_circular_buffer_like(a, shape=(2, 1), buffer_factor=2)
        s_cb = ttl.make_circular_buffer_like(s, shape=(1, 1), buffer_factor=2)
        o_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)

        @ttl.compute()
        def compute():
            with a_cb.wait() as ab, s_cb.wait() as sb, o_cb.reserve() as ob:
                ob.store(ttl.math.exp(ttl.math.reduce_max(ab, sb, dims=[0, 1])))

        @ttl.datamovement()
        def dm0():
            with a_cb.reserve() as ab:
                tx = ttl.copy(a[0:2, 0:1], ab)
                tx.wait()
            with s_cb.reserve() as sb:
                tx = ttl.copy(s[0:1, 0:1], sb)
                tx.wait()

        @ttl.datamovement()
        def dm1():
            with o_cb.wait() as ob:
                tx = ttl.copy(ob, out[0:1, 0:1])
                tx.wait()

    with pytest.raises(Unsupported, match="both dimensions inside a larger expression"):
        red_in_expr.plan(z((64, 32)), z((32, 32)), z((1, 1)))


def _desc(capi, dims=1, op=0, rows=64, cols=64):
    r = capi.ReduceDesc()
    d = r.src
    d.dtype, d.n_in, d.n_ops = capi.TTLB_BF16, 1, 1
    d.inp[0].ptr, d.inp[0].ld = 4096, cols
    d.ops[0].opcode, d.ops[0].arg = 0, 0
    d.rows, d.cols = rows, cols
    r.op, r.dims, r.out, r.out_ld, r.fill_rows, r.fill_cols = op, dims, 8192, cols, 1, 1
    return r


def test_generated_source_per_form():
    from ttl_b200 import capi
    rows = capi.reduce_source(_desc(capi, dims=1))
    assert "ttlb_reduce_jit" in rows and "atomicAdd(&q.counter[blockIdx.x]" in rows and "q.counter2" not in rows.split("ttlb_reduce_jit")[1]
    cols = capi.reduce_source(_desc(capi, dims=2, op=1))
    assert "__shfl_xor_sync" in cols and "nan_max" in cols and "atomicAdd" not in cols
    both = capi.reduce_source(_desc(capi, dims=3))
    assert "atomicAdd(q.counter2" in both


def test_bad_descriptors_are_rejected_before_any_launch():
    from ttl_b200 import capi
    l = capi.lib()
    for mutate in (lambda r: setattr(r, "dims", 0), lambda r: setattr(r, "dims", 4), lambda r: setattr(r, "op", 2),
                   lambda r: setattr(r, "fill_rows", 33),
                   lambda r: setattr(r.src, "cols", 60), lambda r: setattr(r.src, "rows", 0)):
        r = _desc(capi)
        mutate(r)
        assert l.ttlb_reduce_source(ctypes.byref(r), None, 0) == capi.TTLB_ERR_INVALID_ARG
