"""The math functions of the specification's Appendix B beyond the compiler's op table
(docs/sphinx/specs/TTLangSpecification.md:700-748: exp2, expm1, logp1, square, recip, rsub, the trigonometric
family, gelu, silu, leaky_relu, elu, celu, softplus, hardtanh, selu, ...).  Each is one block op: evaluated in
fp32 and rounded once.  CPU: oracle against the simulator fixtures (simulator + add-on), recognised plan
evaluated by the plan oracle.  GPU: the specialised kernel against both."""

import pytest
import torch

import cases
from conftest import digest, golden_tensor, load_golden
from oracle import plan_oracle
from test_oracle import oracle_output


def _same(a, b):
    return torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("case", cases.MATH_CASES + cases.OPERATOR_CASES, ids=lambda c: c.name)
def test_oracle_and_plan_match_simulator_golden(case, backend):
    g = load_golden(case.name)
    assert str(g["input_digest"]) == digest(case.make_inputs())
    want = golden_tensor(g["out"], case.dtype)
    assert _same(oracle_output(case), want), "oracle vs simulator"
    _, mods = backend
    import ttnn
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
    plan = case.get_program(mods).plan(*ins, out)
    d = plan.describe()
    assert len(d) == 1 and d[0]["kind"] == "eltwise" and len(d[0]["ops"]) in (2, 3)
    plan_oracle.run_plan(plan, [t._tensor for t in ins] + [out._tensor])
    assert _same(out._tensor, want), "plan vs simulator"


def test_scalar_parameters_are_checked(backend):
    import ttl
    with pytest.raises(TypeError, match="scalar parameters must be numbers"):
        ttl.math.leaky_relu(None, "0.1")


def test_generated_source_reads_parameters_from_the_launch():
    """Scalar parameters are launch parameters, not part of the compiled kernel: one kernel per function."""
    from ttl_b200 import capi
    d = capi.EltwiseDesc()
    d.dtype, d.n_in, d.n_ops = capi.TTLB_BF16, 1, 2
    d.inp[0].ptr, d.inp[0].ld = 4096, 64
    d.ops[0].opcode, d.ops[0].arg = capi.OPCODES["load"], 0
    d.ops[1].opcode, d.ops[1].arg = capi.OPCODES["hardtanh"], 2
    d.out, d.out_ld, d.rows, d.cols = 8192, 64, 64, 64
    src = capi.eltwise_source(d)
    assert "P0 = p.imm[2], P1 = p.imm[3]" in src and "fminf(fmaxf(a, P0), P1)" in src
    d.ops[1].arg = 7   # needs parameters 7 and 8 of 8
    with pytest.raises(capi.BackendError):
        capi.eltwise_source(d)


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.MATH_CASES + cases.OPERATOR_CASES, ids=lambda c: c.name)
def test_gpu_matches_simulator_and_oracle(case, backend):
    from test_gpu_eltwise import check, run_case
    from ttl_b200 import capi
    _, mods = backend
    import ttnn
    before = capi.context().launch_count()
    got = run_case(case, mods, ttnn)
    assert capi.context().launch_count() == before + 1
    assert capi.context().eltwise_last_path() == capi.ELTWISE_SPECIALISED
    check(got, oracle_output(case), case.check, "vs oracle", case.mode)
    check(got, golden_tensor(load_golden(case.name)["out"], case.dtype), case.check, "vs simulator golden", case.mode)


@pytest.mark.gpu
def test_generic_kernel_rejects_the_new_functions(backend):
    from ttl_b200 import capi
    _, mods = backend
    import ttnn
    ctx = capi.context()
    ctx.set_eltwise_mode(capi.ELTWISE_GENERIC)
    try:
        case = cases.by_name("math_gelu")
        ins = [ttnn.from_torch(t) for t in case.make_inputs()]
        out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
        with pytest.raises(capi.BackendError, match="specialised kernel only"):
            case.get_program(mods)(*ins, out)
    finally:
        ctx.set_eltwise_mode(capi.ELTWISE_AUTO)
