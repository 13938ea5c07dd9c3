"""The per-launch / per-source-line timing report (counterpart of the reference's auto-profiler report,
docs/auto-profiler-examples/demo-one.txt): line attribution on the CPU with made-up times, real times on the GPU."""

import pytest
import torch

import cases


@pytest.fixture()
def profiling(backend):
    import ttl_b200
    ttl_b200.profile.reset()
    ttl_b200.profile.enable()
    yield ttl_b200.profile
    ttl_b200.profile.disable()
    ttl_b200.profile.reset()


def _source_lines(report, section):
    body = report.split(section, 1)[1]
    return [ln for ln in body.splitlines() if ln[:1].isdigit()]


def test_launches_are_reported_against_the_program_lines_they_implement(profiling, backend):
    _, mods = backend
    import ttnn
    import ttl_b200
    z = lambda s: ttnn.from_torch(torch.zeros(s, dtype=torch.bfloat16))  # noqa: E731
    ttl_b200.set_row_fusion(False)   # launch by launch: three launches to tell apart
    try:
        plan = mods["reduce"].make_softmax().plan(z((128, 256)), z((32, 32)), z((128, 256)))
    finally:
        ttl_b200.set_row_fusion(True)
    assert all(l.lines for l in plan.launches)
    report = profiling.summarize([(l, 10.0 * (i + 1)) for _ in range(2) for i, l in enumerate(plan.launches)], 2)
    assert "TTLANG-B200 PROFILE REPORT" in report and "GPU launches: 6" in report and "GPU time: 120.0 us" in report
    assert "LAUNCH 1: reduce_max dims=[1] -> ttlb_reduce_jit   (x2, avg=10.0 us" in report
    assert "LAUNCH 3: eltwise -> ttlb_eltwise_jit" in report
    by_line = _source_lines(report, "BY SOURCE LINE")
    text = "\n".join(by_line)
    # the store of the row maximum feeds launch 1 only; exp(x - max) is computed by launches 2 and 3;
    # the copy of x into its circular buffer feeds all three; 4 row strips -> 4 blocks per line
    assert any("reduce_max(xb, sb, dims=[1])" in ln and ln.rstrip().endswith("[L1]") for ln in by_line), text
    assert any("ttl.math.exp(xb - " in ln and ln.rstrip().endswith("[L2,L3]") for ln in by_line), text
    assert any("ttl.copy(x[r:r + 1, 0:ct], xb)" in ln and "100.0%" in ln and ln.rstrip().endswith("[L1,L2,L3]") for ln in by_line), text
    assert any("ttl.copy(yb, y[r:r + 1, 0:ct])" in ln and ln.rstrip().endswith("[L3]") for ln in by_line), text
    launch1 = report.split("LAUNCH 1:", 1)[1].split("LAUNCH 2:", 1)[0]
    assert "x4" in launch1


def test_plans_built_without_profiling_carry_no_lines(backend):
    _, mods = backend
    import ttl_b200
    import ttnn
    z = lambda s: ttnn.from_torch(torch.zeros(s, dtype=torch.bfloat16))  # noqa: E731
    plan = mods["reduce"].make_softmax().plan(z((64, 64)), z((32, 32)), z((64, 64)))
    assert not any(getattr(l, "lines", None) for l in plan.launches)
    assert "no line information" in ttl_b200.profile.summarize([(plan.launches[0], 1.0)], 1)


@pytest.mark.gpu
def test_gpu_report_has_measured_times(profiling, backend):
    _, mods = backend
    import ttnn
    case = cases.by_name("softmax_128x256")
    prog = case.get_program(mods)
    for _ in range(3):
        ins = [ttnn.from_torch(t) for t in case.make_inputs()]
        out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
        prog(*ins, out)
    report = profiling.report()
    assert "Kernel calls: 3" in report and "GPU launches: 3" in report and "LAUNCH 1: row_fused" in report
    import re
    totals = [float(x.replace(",", "")) for x in re.findall(r"total=([\d,\.]+) us", report)]
    assert len(totals) == 1 and all(t > 0 for t in totals)
    assert "reduce_max(xb, sb, dims=[1])" in report and "ttl.copy(yb, y[r:r + 1, 0:ct])" in report
    # the result is still right when every launch is bracketed by events
    from conftest import golden_tensor, load_golden
    from test_reduce import close
    close(ttnn.to_torch(out), golden_tensor(load_golden(case.name)["out"], case.dtype), case.check, "profiled run")
