"""Attention written as a tt-lang tile program with block matmuls and reductions (tests/programs/attention.py).

Front half only (no GPU): the program is traced, its computed matmul operand (the softmax) and the score matrix
become temporaries, and the plan - GEMM, row-resident softmax, GEMM - is evaluated by the plan oracle.  The
one-tile size is pinned to the reference simulator (its block matmul accepts K = 1 tile only); the larger sizes are
checked against a float64 attention.  The kernels this plan launches are each covered by the GPU parity tests."""

import pytest
import torch

import cases
from conftest import digest, golden_tensor, load_golden
from oracle import plan_oracle
from test_oracle import oracle_output


def _rel(got, want):
    return ((got.double() - want.double()).abs().max() / want.double().abs().max()).item()


@pytest.mark.parametrize("case", cases.ATTENTION_CASES, ids=lambda c: c.name)
def test_one_tile_attention_matches_simulator(case, backend):
    g = load_golden(case.name)
    assert str(g["input_digest"]) == digest(case.make_inputs())
    want = golden_tensor(g["out"], case.dtype)
    tol = 1e-2 if case.dtype == torch.bfloat16 else 1e-5
    assert _rel(oracle_output(case), want) <= tol
    _, mods = backend
    import ttnn
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
    plan = case.get_program(mods).plan(*ins, out)
    kinds = [d["kind"] for d in plan.describe()]
    mm = "matmul_bf16" if case.dtype == torch.bfloat16 else "matmul_f32"
    # one tile row: the operands are "one tile repeated", which the row fusion leaves as separate launches
    assert kinds in ([mm, "row_fused", mm], [mm, "reduce_max", "reduce_sum", "eltwise", mm])
    plan_oracle.run_plan(plan, [t._tensor for t in ins] + [out._tensor])
    assert _rel(out._tensor, want) <= tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)], ids=["f32", "bf16"])
@pytest.mark.parametrize("s,d", [(128, 64), (256, 128)])
def test_multi_tile_attention_plan(s, d, dtype, tol, backend):
    """(1, D) @ (D, S) scores, softmax over S, (1, S) @ (S, D): three launches for the whole head."""
    _, mods = backend
    import ttnn
    g = torch.Generator().manual_seed(s + d)
    q, k, v = (torch.randn(s, d, generator=g).to(dtype) for _ in range(3))
    mask = torch.triu(torch.full((s, s), -1e4), diagonal=1).to(dtype)
    scale = torch.full((32, 32), d ** -0.5).to(dtype)
    one = torch.ones(32, 32).to(dtype)
    out = ttnn.from_torch(torch.zeros(s, d, dtype=dtype))
    ins = [ttnn.from_torch(t) for t in (q, k.t().contiguous(), v, mask, scale, one)]
    plan = mods["attention"].attention_rows.plan(*ins, out)
    desc = plan.describe()
    assert [x["kind"] for x in desc][1] == "row_fused" and len(desc) == 3
    assert [p["kind"] for p in desc[1]["phases"]] == ["reduce_max", "reduce_sum"]
    # the score matrix and the softmax are temporaries of the plan: [S, S] each; the reductions stay on chip
    big = [t for t in plan.temps if t._tensor.numel() > 0 and t.shape == (s, s)]
    assert len(big) == 2
    plan_oracle.run_plan(plan, [t._tensor for t in ins] + [out._tensor])
    want = torch.softmax(q.double() @ k.double().t() * scale[0, 0].double() + mask.double(), dim=1) @ v.double()
    assert _rel(out._tensor, want) <= tol


def test_computed_operand_without_a_k_range_is_refused(backend):
    import ttl
    import ttnn
    from ttl_b200 import Unsupported
    z = lambda shape: ttnn.from_torch(torch.zeros(shape, dtype=torch.bfloat16))  # noqa: E731

    @ttl.kernel(grid=(1, 1))
    def both_computed(a, b, out):
        a_cb = ttl.make_circular_buffer_like(a, shape=(1, 2), buffer_factor=2)
        b_cb = ttl.make_circular_buffer_like(b, shape=(1, 1), buffer_factor=2)
        o_cb = ttl.make_circular_buffer_like(out, shape=(1, 1), buffer_factor=2)

        @ttl.compute()
        def compute():
            with a_cb.wait() as ab, b_cb.wait() as bb, o_cb.reserve() as ob:
                # (1, 2) @ (2, 1) where the right operand is a reduction result with no block of its own shape inside
                ob.store(ttl.math.relu(ab) @ ttl.math.reduce_sum(ab, bb, dims=[0, 1]))

        @ttl.datamovement()
        def dm0():
            with a_cb.reserve() as ab:
                tx = ttl.copy(a[0:1, 0:2], ab)
                tx.wait()
            with b_cb.reserve() as bb:
                tx = ttl.copy(b[0:1, 0:1], bb)
                tx.wait()

        @ttl.datamovement()
        def dm1():
            with o_cb.wait() as ob:
                tx = ttl.copy(ob, out[0:1, 0:1])
                tx.wait()

    with pytest.raises((Unsupported, ValueError)):
        both_computed.plan(z((32, 64)), z((32, 32)), z((32, 32)))
