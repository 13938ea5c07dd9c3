"""The attention oracle: tile-program form against the textbook form (no GPU)."""

import pytest
import torch

import cases
from oracle import attention_oracle


@pytest.mark.parametrize("seq,causal", [(128, True), (256, True), (200, True), (256, False), (96, False)])
def test_tiles_match_plain(seq, causal):
    q, k, v = (cases.gen((2 * seq, 128), "normal", s).reshape(2, seq, 128) for s in (0, 1, 2))
    a = attention_oracle.attention_tiles(q, k, v, causal, 128 ** -0.5)
    b = attention_oracle.attention_plain(q, k, v, causal, 128 ** -0.5)
    assert (a.float() - b.float()).abs().max() <= 2 ** -7 * b.float().abs().max()


def test_causal_first_row_is_first_value():
    q, k, v = (cases.gen((256, 128), "normal", s).reshape(1, 256, 128) for s in (3, 4, 5))
    o = attention_oracle.attention_tiles(q, k, v, True, 128 ** -0.5)
    assert torch.equal(o[0, 0], v[0, 0])


@pytest.mark.parametrize("case", cases.ATTENTION_PIPELINE_CASES, ids=lambda c: c.name)
def test_attention_oracle_is_pinned_to_the_simulator(case):
    """The fixtures are outputs of the UNMODIFIED reference simulator (tests/golden/make_golden.py) running
    attention as three tile kernels - scores and probabilities @ V in 1x1-tile block matmuls accumulated with
    store(acc=True), the masked row softmax in between (tests/programs/attention.py) - at the fused kernel's head
    dimension.  The oracle of the fused kernel (online softmax over 128-key blocks, bf16 inputs and output) must
    agree with them within the tolerance stated for attention, max |diff| / max |want| <= 1e-2."""
    from conftest import digest, golden_tensor, load_golden
    g = load_golden(case.name)
    assert str(g["input_digest"]) == digest(case.make_inputs()), "seeded inputs drifted from the fixture"
    want = golden_tensor(g["out"], case.dtype)
    q, kt, v, _mask, scale, _one = case.make_inputs()
    bf = torch.bfloat16
    for fn in (attention_oracle.attention_tiles, attention_oracle.attention_plain):
        got = fn(q.to(bf)[None], kt.t().contiguous().to(bf)[None], v.to(bf)[None], True, float(scale[0, 0]))[0]
        err = ((got.double() - want.double()).abs().max() / want.double().abs().max()).item()
        assert err <= 1e-2, (fn.__name__, err)


@pytest.mark.parametrize("case", cases.ATTENTION_PIPELINE_CASES, ids=lambda c: c.name)
def test_attention_pipeline_plans_match_the_simulator(case, backend):
    """The same three kernels through this backend's tracer and recogniser: GEMM, row-resident softmax, GEMM,
    evaluated on the host by the plan oracle, against the simulator's output."""
    from conftest import golden_tensor, load_golden
    from oracle import plan_oracle
    _, mods = backend
    import ttnn
    want = golden_tensor(load_golden(case.name)["out"], case.dtype)
    q, kt, v, mask, scale, one = (ttnn.Tensor(t) for t in case.make_inputs())
    s = q.shape[0]
    scores, probs, out = (ttnn.Tensor(torch.zeros(shape, dtype=case.dtype)) for shape in ((s, s), (s, s), case.out_shape))
    prog = mods["attention"]
    kinds = []
    for kern, args in ((prog.tile_matmul, (q, kt, scores)), (prog.masked_softmax_rows, (scores, mask, scale, one, probs)),
                       (prog.tile_matmul, (probs, v, out))):
        plan = kern.plan(*args)
        kinds += [d["kind"] for d in plan.describe()]
        plan_oracle.run_plan(plan, [t._tensor for t in args])
    mm = "matmul_bf16" if case.dtype == torch.bfloat16 else "matmul_f32"
    assert kinds == [mm, "row_fused", mm]
    err = ((out._tensor.double() - want.double()).abs().max() / want.double().abs().max()).item()
    assert err <= (1e-2 if case.dtype == torch.bfloat16 else 1e-5), err
