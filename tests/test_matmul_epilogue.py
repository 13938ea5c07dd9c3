"""A block matmul whose result is used further in the same kernel (bias vector + activation): the product
passes through an intermediate circular buffer, i.e. a block of the output's element type.  The plan is the
tensor-core GEMM into a temporary followed by one fused element-wise launch."""

import pytest
import torch

import cases
from conftest import golden_tensor, load_golden
from oracle import plan_oracle
from test_oracle import oracle_output


def _rel(got, want):
    return ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()


@pytest.mark.parametrize("case", cases.EPILOGUE_CASES, ids=lambda c: c.name)
def test_plan_and_oracle_match_simulator(case, backend):
    want = golden_tensor(load_golden(case.name)["out"], case.dtype)
    # the simulator adds the K tiles in bf16, the oracle's slab product differs in summation order only
    assert _rel(oracle_output(case), want) <= 1e-2
    _, mods = backend
    import ttnn
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
    plan = case.get_program(mods).plan(*ins, out)
    d = plan.describe()
    assert [x["kind"] for x in d] == ["matmul_bf16", "eltwise"]
    assert d[0]["out"] >= 1000 and d[1]["inputs"][0][0] == d[0]["out"], "the product goes through a temporary"
    assert len(plan.temps) == 1 and tuple(plan.temps[0].shape) == case.out_shape
    plan_oracle.run_plan(plan, [t._tensor for t in ins] + [out._tensor])
    assert _rel(out._tensor, want) <= 1e-2
    assert (out._tensor.float() >= 0).all()


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.EPILOGUE_CASES, ids=lambda c: c.name)
def test_gpu_matches_simulator_and_oracle(case, backend):
    from ttl_b200 import capi
    _, mods = backend
    import ttnn
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
    before = capi.context().launch_count()
    case.get_program(mods)(*ins, out)
    assert capi.context().launch_count() == before + 2
    got = ttnn.to_torch(out)
    assert _rel(got, oracle_output(case)) <= 1e-2
    assert _rel(got, golden_tensor(load_golden(case.name)["out"], case.dtype)) <= 1e-2
    assert (got.float() >= 0).all()


@pytest.mark.gpu
def test_gpu_linear_relu_1024(backend):
    """1024 x 2048 x 1024 against an fp32 torch reference computed on the GPU."""
    _, mods = backend
    import ttnn
    a = cases.gen((1024, 2048), "normal*0.022", 14)
    b = cases.gen((2048, 1024), "normal", 15)
    v = cases.gen((1, 1024), "normal", 16)
    out = ttnn.from_torch(torch.zeros((1024, 1024), dtype=torch.bfloat16))
    mods["matmul"].linear_relu(*(ttnn.from_torch(t) for t in (a, b, v)), out)
    want = torch.relu(a.cuda().float() @ b.cuda().float() + v.cuda().float())
    got = out._tensor.float()
    assert ((got - want).abs().max() / want.abs().max()).item() <= 1e-2


@pytest.mark.parametrize("act", ["relu", "gelu", "silu", "sigmoid", "tanh"])
def test_fp32_intermediates_fuse_bias_and_activation_into_the_gemm(act, backend):
    """With fp32_dest_acc_en the element-wise launch disappears: one GEMM launch with the bias row and the
    activation in its epilogue; its temporary gives its memory back."""
    _, mods = backend
    import ttnn
    a, b, v = cases.gen((96, 160), "normal*0.08", 11), cases.gen((160, 128), "normal*0.08", 12), cases.gen((1, 128), "normal", 13)
    ins = [ttnn.from_torch(t) for t in (a, b, v)]
    out = ttnn.from_torch(torch.zeros((96, 128), dtype=torch.bfloat16))
    plan = mods["matmul"].make_linear(act, fp32_dest_acc_en=True).plan(*ins, out)
    d = plan.describe()
    assert len(d) == 1 and d[0]["kind"] == "matmul_bf16" and d[0]["bias"] == 2 and d[0]["act"] == act and d[0]["out"] == 3
    assert plan.temps[0]._tensor.numel() == 0
    plan_oracle.run_plan(plan, [t._tensor for t in ins] + [out._tensor])
    from oracle import tile_oracle
    want = tile_oracle.UNARY[act](a.float() @ b.float() + v.float())
    assert _rel(out._tensor, want) <= 1e-2
    # without fp32 intermediates every op rounds to bf16: two launches
    kinds = [x["kind"] for x in mods["matmul"].make_linear(act).plan(*ins, out).describe()]
    assert kinds == ["matmul_bf16", "eltwise"]


@pytest.mark.gpu
@pytest.mark.parametrize("act", ["relu", "gelu", "silu", "sigmoid", "tanh"])
@pytest.mark.parametrize("shape", [(96, 160, 128), (2048, 256, 4096)], ids=["small_one_cta", "large_two_cta"])
def test_gpu_fused_epilogue(act, shape, backend):
    """The fused epilogue on both GEMM kernels (the large shape takes the two-CTA kernel) against fp32 torch."""
    from ttl_b200 import capi
    from oracle import tile_oracle
    _, mods = backend
    import ttnn
    m, k, n = shape
    a, b, v = cases.gen((m, k), f"normal*{k ** -0.5}", 21), cases.gen((k, n), "normal", 22), cases.gen((1, n), "normal", 23)
    out = ttnn.from_torch(torch.zeros((m, n), dtype=torch.bfloat16))
    prog = mods["matmul"].make_linear(act, fp32_dest_acc_en=True)
    before = capi.context().launch_count()
    prog(*(ttnn.from_torch(t) for t in (a, b, v)), out)
    assert capi.context().launch_count() == before + 1
    want = tile_oracle.UNARY[act](a.cuda().float() @ b.cuda().float() + v.cuda().float())
    got = out._tensor.float()
    assert ((got - want).abs().max() / want.abs().max()).item() <= 1e-2
    capi.context().check_status()
