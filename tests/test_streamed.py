"""ttl_b200.run_streamed: a row-parallel tile program on host tensors, in row chunks with the copies
overlapped.  Same bits as the plain call; programs that are not row-parallel are refused."""

import pytest
import torch

import cases
from test_oracle import oracle_output


def test_without_gpu_fails_loudly(backend):
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    import ttl_b200
    _, mods = backend
    with pytest.raises(ttl_b200.BackendError, match="no CPU fallback"):
        ttl_b200.run_streamed(mods["eltwise"].eltwise_add, [torch.zeros(64, 64)] * 2, torch.zeros(64, 64))


@pytest.mark.gpu
@pytest.mark.parametrize("chunks", [1, 3, 8])
def test_same_bits_as_the_plain_call(backend, chunks):
    import ttl_b200
    _, mods = backend
    case = cases.by_name("fused_f32_256x512")
    host = [t.pin_memory() for t in case.make_inputs()]
    out = torch.empty(case.out_shape, dtype=case.dtype).pin_memory()
    got = ttl_b200.run_streamed(case.get_program(mods, f32acc=True), host, out, chunks=chunks)
    assert got is out
    import ttnn
    plain = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
    case.get_program(mods, f32acc=True)(*[ttnn.from_torch(t) for t in host], plain)
    assert torch.equal(out.view(torch.int16), ttnn.to_torch(plain).view(torch.int16))
    from test_gpu_eltwise import check
    check(out, oracle_output(case), case.check, "vs oracle", case.mode)


@pytest.mark.gpu
def test_programs_that_mix_rows_are_refused(backend):
    import ttl_b200
    _, mods = backend
    a = torch.zeros(128, 128, dtype=torch.bfloat16)
    with pytest.raises(ttl_b200.Unsupported, match="rows are independent"):
        ttl_b200.run_streamed(mods["matmul"].singlecore_matmul,
                              [torch.zeros(128, 64, dtype=torch.bfloat16), torch.zeros(64, 128, dtype=torch.bfloat16)],
                              torch.zeros(128, 128, dtype=torch.bfloat16))
    with pytest.raises(ttl_b200.Unsupported, match="rows are independent"):
        ttl_b200.run_streamed(mods["reduce"].make_reduce("sum", [0]), [a, torch.ones(32, 32, dtype=torch.bfloat16)],
                              torch.zeros(32, 128, dtype=torch.bfloat16))


@pytest.mark.gpu
def test_row_softmax_streams_too(backend):
    """A row-fused program (softmax: reductions over columns + element-wise) is row-parallel as well."""
    import ttl_b200
    _, mods = backend
    case = cases.by_name("softmax_128x256")
    host = [t.pin_memory() for t in case.make_inputs()]
    out = torch.empty(case.out_shape, dtype=case.dtype).pin_memory()
    ttl_b200.run_streamed(case.get_program(mods), host, out, chunks=2)
    from conftest import golden_tensor, load_golden
    from test_reduce import close
    close(out, golden_tensor(load_golden(case.name)["out"], case.dtype), case.check, "streamed softmax")
