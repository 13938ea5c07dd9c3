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


def test_timeout_surfaces_where_the_host_reads_results_back():
    """A device-side wait that ran out must not pass silently: `ttnn.to_torch`, `ttl_b200.synchronize` and
    `run_streamed` check the status word where they already wait for the GPU.  The wait that runs out is the
    self-test's (a barrier nothing arrives on, 1 ms limit): the kernel returns normally."""
    import ttl_b200
    from ttl_b200 import capi, ttnn
    ctx = capi.context()
    stream = capi.current_stream()
    ctx.check_status(stream)
    x = ttnn.from_torch(torch.ones(64, 64, dtype=torch.bfloat16))
    ctx.selftest_wait_timeout(2_000_000, stream)
    with pytest.raises(capi.BackendError) as e:
        ttnn.to_torch(x)
    assert e.value.code == capi.TTLB_ERR_TIMEOUT
    assert (ttnn.to_torch(x) == 1).all()           # reported once; the context carries on
    ctx.selftest_wait_timeout(2_000_000, stream)
    with pytest.raises(capi.BackendError) as e:
        ttl_b200.synchronize()
    assert e.value.code == capi.TTLB_ERR_TIMEOUT
    ttl_b200.synchronize()
    pinned = torch.empty(64, 64, dtype=torch.bfloat16).pin_memory()
    ctx.selftest_wait_timeout(2_000_000, stream)
    with pytest.raises(capi.BackendError):
        ttnn.to_torch(x, out=pinned)
    ttnn.to_torch(x, out=pinned)
    assert (pinned == 1).all()
