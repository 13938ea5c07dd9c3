"""The native runner `ttlang-b200-run` (tt-lang_b200/cli/ttlang_b200_run.cpp) and the plan files
`python -m ttl_b200.translate --emit` writes for it: the run-time counterpart, without Python, of the reference's
native tool next to its Python front end (tools/ttlang-translate/ttlang-translate.cpp:24-29)."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import cases

ROOT = Path(__file__).resolve().parent.parent
RUNNER = ROOT / "tt-lang_b200" / "ttl_b200" / "ttlang-b200-run"

PROGRAM = '''
import sys
sys.path.insert(0, {tests!r})
sys.path.insert(0, {programs!r})
import torch, ttnn
import cases
import eltwise as E
import matmul as M
import reduce as R

case = cases.by_name("fused_f32_256x512")
ins = [ttnn.from_torch(t) for t in case.make_inputs()]
out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=torch.bfloat16))
E.fused_exp_bcast_f32acc(*ins, out)

a = cases.gen((256, 192), "normal*0.07", 0); b = cases.gen((192, 320), "normal", 1)
c = ttnn.from_torch(torch.zeros((256, 320), dtype=torch.bfloat16))
M.multicore_matmul(ttnn.from_torch(a), ttnn.from_torch(b), c)

w = cases.gen((192, 320), "normal*0.02", 2, torch.float32)
c2 = ttnn.from_torch(torch.zeros((256, 320), dtype=torch.bfloat16))
M.multicore_matmul(ttnn.from_torch(a), ttnn.from_torch(w, dtype=ttnn.bfloat8_b), c2)

x = cases.gen((128, 256), "normal", 7)
ones = ttnn.from_torch(torch.ones(32, 32, dtype=torch.bfloat16))
s1 = ttnn.from_torch(torch.zeros((128, 1), dtype=torch.bfloat16))
R.make_reduce("sum", [1])(ttnn.from_torch(x), ones, s1)
y = ttnn.from_torch(torch.zeros((128, 256), dtype=torch.bfloat16))
R.make_softmax(fp32_dest_acc_en=True)(ttnn.from_torch(x), ones, y)
'''


@pytest.fixture(scope="module")
def emitted(tmp_path_factory):
    d = tmp_path_factory.mktemp("emit")
    prog = d / "prog.py"
    prog.write_text(PROGRAM.format(tests=str(ROOT / "tests"), programs=str(ROOT / "tests" / "programs")))
    env = {"PYTHONPATH": str(ROOT / "tt-lang_b200"), "PATH": "/usr/bin:/bin", "CUDA_VISIBLE_DEVICES": ""}
    r = subprocess.run([sys.executable, "-m", "ttl_b200.translate", str(prog), "--no-source", "--emit", str(d / "plans")],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    return d / "plans"


def test_emitted_plans_describe_the_launches_and_tensors(emitted):
    kinds = []
    for i in range(5):
        plan = json.loads((emitted / f"call{i}" / "plan.json").read_text())
        kinds.append([l["kind"] for l in plan["launches"]])
        for t in plan["tensors"]:
            size = (emitted / f"call{i}" / t["file"]).stat().st_size
            r, c = t["shape"]
            assert size == {"bf16": r * c * 2, "f32": r * c * 4, "bfp8_b": (r // 32) * (c // 32) * 1088}[t["dtype"]]
    assert kinds[:3] == [["eltwise"], ["matmul_bf16"], ["matmul_bfp8w"]]
    more = [[l["kind"] for l in json.loads((emitted / f"call{i}" / "plan.json").read_text())["launches"]] for i in (3, 4)]
    assert more == [["reduce_sum"], ["row_fused"]]
    first = json.loads((emitted / "call0" / "plan.json").read_text())["launches"][0]
    assert len(first["opcodes"]) == len(first["ops"]) and first["round_each_op"] is False


def test_runner_is_built_and_fails_loudly_without_a_gpu(emitted):
    assert RUNNER.exists(), "ttlang-b200-run was not built (python tt-lang_b200/build.py)"
    r = subprocess.run([str(RUNNER), "--help"], capture_output=True, text=True)
    assert r.returncode == 0 and "usage: ttlang-b200-run" in r.stdout
    if not torch.cuda.is_available():
        r = subprocess.run([str(RUNNER), str(emitted / "call0" / "plan.json")], capture_output=True, text=True)
        assert r.returncode == 3 and "no CPU fallback" in r.stderr


@pytest.mark.gpu
def test_runner_reproduces_the_python_backend_bit_for_bit(emitted, backend):
    """The three emitted kernel calls run by the native tool: its outputs equal what the same programs give when
    called through `@ttl.kernel` in this process (the same kernels through the same C ABI), and match the oracle."""
    from oracle import bfp8_oracle, tile_oracle
    _, mods = backend
    import ttnn

    def run(i, out_index, shape):
        r = subprocess.run([str(RUNNER), str(emitted / f"call{i}" / "plan.json"), "--steps", "3", "--warmup", "1"],
                           capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        rec = json.loads(r.stdout.strip().splitlines()[-1])
        assert rec["launches"] == 1 and rec["ms_per_step"] > 0 and len(rec["outputs"]) == 1
        raw = np.fromfile(emitted / f"call{i}" / f"t{out_index}.bin.out", dtype=np.int16)
        return torch.from_numpy(raw.copy()).view(torch.bfloat16).reshape(shape)

    case = cases.by_name("fused_f32_256x512")
    ins = case.make_inputs()
    out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=torch.bfloat16))
    mods["eltwise"].fused_exp_bcast_f32acc(*[ttnn.from_torch(t) for t in ins], out)
    got = run(0, 4, case.out_shape)
    assert torch.equal(got, ttnn.to_torch(out))
    a, b = cases.gen((256, 192), "normal*0.07", 0), cases.gen((192, 320), "normal", 1)
    got = run(1, 2, (256, 320))
    want = tile_oracle.matmul_tiles(a, b, "f32")
    assert ((got.float() - want.float()).abs().max() / want.float().abs().max()).item() <= 1e-2
    w = cases.gen((192, 320), "normal*0.02", 2, torch.float32)
    wq = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w.numpy()), 192, 320))
    got = run(2, 2, (256, 320))
    want = tile_oracle.matmul_tiles(a.float(), wq, "f32")
    assert ((got.float() - want.float()).abs().max() / want.float().abs().max()).item() <= 1e-2
    # a reduction over columns and the row-resident softmax: the same bits as through `@ttl.kernel`
    x = cases.gen((128, 256), "normal", 7)
    ones = ttnn.from_torch(torch.ones(32, 32, dtype=torch.bfloat16))
    s1 = ttnn.from_torch(torch.zeros((128, 1), dtype=torch.bfloat16))
    mods["reduce"].make_reduce("sum", [1])(ttnn.from_torch(x), ones, s1)
    assert torch.equal(run(3, 2, (128, 1)), ttnn.to_torch(s1))
    y = ttnn.from_torch(torch.zeros((128, 256), dtype=torch.bfloat16))
    mods["reduce"].make_softmax(fp32_dest_acc_en=True)(ttnn.from_torch(x), ones, y)
    got = run(4, 2, (128, 256))
    assert torch.equal(got, ttnn.to_torch(y))
    want = torch.softmax(x.double(), dim=1)
    assert ((got.double() - want).abs() <= 2.0 ** -6 * want + 1e-7).all()
