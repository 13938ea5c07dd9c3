"""Failure detection without a GPU fault: a device-side wait that nothing satisfies runs into its
short limit, the kernel returns normally with a status word, the host turns it into
TTLB_ERR_TIMEOUT, and the context stays usable."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_timeout_and_context_stays_usable():
    from ttl_b200 import capi, ops, ttnn
    ctx = capi.context()
    stream = capi.current_stream()
    ctx.check_status(stream)                       # clean before
    ctx.selftest_wait_timeout(2_000_000, stream)   # ~1 ms at 1.9 GHz
    with pytest.raises(capi.BackendError) as e:
        ctx.check_status(stream)
    assert e.value.code == capi.TTLB_ERR_TIMEOUT and "self-test" in str(e.value)
    ctx.check_status(stream)                       # the record was cleared by the failing check
    # the context and the GPU are fine: run a real matmul afterwards
    a = torch.ones(128, 64, dtype=torch.bfloat16)
    b = torch.ones(64, 256, dtype=torch.bfloat16)
    c = ttnn.to_torch(ops.matmul(ttnn.from_torch(a), ttnn.from_torch(b)))
    ctx.check_status(stream)
    assert (c == 64).all()
    with pytest.raises(capi.BackendError):
        ctx.selftest_wait_timeout(0, stream)       # limit out of range: rejected on the host
