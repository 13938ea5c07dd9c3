"""The CPU oracle against the committed simulator outputs (and, where the reference checkout is
present, against the simulator run live)."""

import sys
from pathlib import Path

import pytest
import torch

import cases
from conftest import reference_root, digest, golden_tensor, load_golden
from oracle import tile_oracle

REFERENCE = reference_root() or Path("reference-checkout-not-found")


def oracle_output(case):
    ins = case.make_inputs()
    if case.module == "attention":
        return tile_oracle.attention_rows(*ins, mode=case.mode)
    if case.module == "matmul" and case.expr is not None:   # product, then an element-wise epilogue
        prod = tile_oracle.matmul_tiles(ins[0], ins[1], case.mode)
        return tile_oracle.eval_expression(case.expr, [prod] + ins[2:], case.out_shape, case.mode)
    if case.module == "matmul":
        return tile_oracle.matmul_tiles(ins[0], ins[1], case.mode, bias=ins[2] if len(ins) > 2 else None)
    if case.reduce is not None:
        op, dims, si, in_shape = case.reduce
        data = [t for k, t in enumerate(ins) if k != si]
        return tile_oracle.reduce_expression(case.expr, data, in_shape, case.mode, op, dims, ins[si])
    out = tile_oracle.eval_expression(case.expr, ins, case.out_shape, case.mode)
    if case.name == "eltwise_pipe":  # only the pipe's four cores compute: tile columns 0..3
        full = torch.zeros(case.out_shape, dtype=case.dtype)
        full[:, :128] = out[:, :128]
        out = full
    return out


@pytest.mark.parametrize("case", cases.CASES + cases.MATMUL_CASES, ids=lambda c: c.name)
def test_oracle_matches_simulator_golden(case):
    g = load_golden(case.name)
    assert str(g["input_digest"]) == digest(case.make_inputs()), "seeded inputs drifted from the fixture"
    out = oracle_output(case)
    if case.store == "digest":
        assert digest([out]) == str(g["out_digest"])
        assert torch.equal(out[:64, :64], golden_tensor(g["corner"], case.dtype))
        return
    want = golden_tensor(g["out"], case.dtype)
    if case.module == "matmul":
        # slab products and per-tile products may sum the 32 inner terms in a different order
        tol = 1e-2 if case.mode == "native" else 1e-5
        err = (out.float() - want.float()).abs().max() / want.float().abs().max()
        assert err <= tol, f"rel err {err}"
    else:
        # same torch ops on the same values: bit-identical, transcendental functions included
        assert torch.equal(out.view(torch.int16) if out.dtype == torch.bfloat16 else out,
                           want.view(torch.int16) if want.dtype == torch.bfloat16 else want)


@pytest.mark.skipif(not (REFERENCE / "python" / "sim").exists(), reason="reference checkout not present")
def test_fixtures_reproduce_from_live_simulator():
    """Re-run two programs on the live simulator in a subprocess and compare with the fixtures."""
    import subprocess

    code = (
        "import sys; sys.argv=['x'];"
        "sys.path.insert(0, 'tests/golden'); import make_golden as m, numpy as np;"
        f"from pathlib import Path; sim = m.load_sim(Path({str(REFERENCE)!r})); import ttnn, cases;"
        "mods = m.load_programs('sim');\n"
        "for n in ['bcast_row_tilecol', 'unary_exp', 'mm_single_128x256x64']:\n"
        "    c = cases.by_name(n); out = m.run_case_on_sim(c, mods, ttnn);"
        " g = np.load(f'tests/golden/{n}.npz'); assert (m.bits(out) == g['out']).all(), n\n"
        "print('OK')"
    )
    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "OK" in r.stdout, r.stderr[-2000:]


def test_expand_operand_forms():
    t = torch.arange(32 * 64, dtype=torch.float32).reshape(32, 64)
    e = tile_oracle.expand_operand(t, (96, 64))
    assert torch.equal(e[32:64], t) and torch.equal(e[64:], t)
    r = torch.arange(64, dtype=torch.float32).reshape(1, 64)
    assert torch.equal(tile_oracle.expand_operand(r, (96, 64))[95], r[0])
    with pytest.raises(ValueError):
        tile_oracle.expand_operand(torch.zeros(64, 64), (96, 64))


def test_bf16_ulp_diff():
    a = torch.tensor([1.0, -1.0, 0.0], dtype=torch.bfloat16)
    b = torch.tensor([1.0078125, -1.0078125, -0.0], dtype=torch.bfloat16)
    assert tile_oracle.bf16_ulp_diff(a, b).tolist() == [1, 1, 0]
