"""GPU parity of the fused element-wise / broadcast kernel, called the way a user calls it:
a tt-lang program run through the backend (tracer -> recogniser -> C ABI -> CUDA kernel),
checked against the simulator's committed outputs and against the CPU oracle."""

import ctypes

import pytest
import torch

import cases
from conftest import golden_tensor, load_golden
from oracle import tile_oracle
from test_oracle import oracle_output

pytestmark = pytest.mark.gpu


def run_case(case, mods, ttnn):
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
    case.get_program(mods, f32acc=(case.mode == "f32"))(*ins, out)
    assert out._tensor.is_cuda
    return ttnn.to_torch(out)


def check(got, want, how, what, mode="native"):
    """how="exact": bit-identical.  how="ulp1": for chains with a transcendental function.  The GPU's
    expf/logf/tanhf and the CPU's are both within 1 fp32 ulp of the true value but not of each other,
    so a few results land on the other side of a bf16 rounding boundary.  Allowed: at most 0.1% of
    elements differ at all, and each differing element is within 1 bf16 ulp, or - where a following
    add cancels (result much smaller than its operands, so ulps of the result are meaningless) -
    within an absolute error of one ulp of the intermediate that flipped: fp32 ulp of a value <= 16
    (1e-5 with margin) with fp32 intermediates, bf16 ulp of a value <= 4 (2**-6) when every op rounds."""
    if how == "exact":
        same = torch.equal(got.view(torch.int16), want.view(torch.int16)) if got.dtype == torch.bfloat16 \
            else torch.equal(got, want)
        assert same, f"{what}: not bit-identical ({(got != want).sum().item()} elements differ)"
        return
    ulp = tile_oracle.bf16_ulp_diff(got, want)
    frac = (ulp > 0).float().mean().item()
    assert frac <= 1e-3, f"{what}: {frac:.2e} of elements differ"
    atol = 1e-5 if mode == "f32" else 2.0 ** -6
    bad = (ulp > 1) & ((got.float() - want.float()).abs() > atol)
    assert not bad.any(), f"{what}: {int(bad.sum())} elements beyond 1 bf16 ulp and {atol} abs (max ulp {int(ulp.max())})"


@pytest.fixture(params=["specialised", "generic"])
def eltwise_path(request):
    """Run every program on both GPU execution paths of ttlb_eltwise: the kernel specialised for the
    program (NVRTC) and the generic interpreting kernel."""
    from ttl_b200 import capi
    ctx = capi.context()
    mode = capi.ELTWISE_SPECIALISED if request.param == "specialised" else capi.ELTWISE_GENERIC
    ctx.set_eltwise_mode(mode)
    yield mode
    ctx.set_eltwise_mode(capi.ELTWISE_AUTO)


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.name)
def test_program_matches_simulator_and_oracle(case, backend, eltwise_path):
    from ttl_b200 import capi
    _, mods = backend
    import ttnn
    before = _launches()
    got = run_case(case, mods, ttnn)
    assert _launches() > before, "no CUDA kernel was launched"
    assert capi.context().eltwise_last_path() == eltwise_path
    check(got, oracle_output(case), case.check, "vs oracle", case.mode)
    g = load_golden(case.name)
    if case.store == "digest":
        from conftest import digest
        assert digest([got]) == str(g["out_digest"]), "output bytes differ from the simulator's"
    else:
        check(got, golden_tensor(g["out"], case.dtype), case.check, "vs simulator golden", case.mode)


def _launches():
    from ttl_b200 import capi
    return capi.context().launch_count()


def test_config2_full_size_against_oracle(backend):
    """configs[1] at full size: 8192x8192, fp32 intermediates, bf16 out."""
    _, mods = backend
    import ttnn
    n = 8192
    a = cases.gen((n, n), "normal", 0)
    s = cases.gen((1, 1), "const:0.1", 0)
    b = cases.gen((1, n), "uniform", 1)
    c = cases.gen((n, n), "normal", 2)
    out = ttnn.from_torch(torch.zeros((n, n), dtype=torch.bfloat16))
    mods["eltwise"].fused_exp_bcast_f32acc(*[ttnn.from_torch(t) for t in (a, s, b, c)], out)
    got = ttnn.to_torch(out)
    want = tile_oracle.eval_expression(("relu", ("add", ("mul", ("exp", ("mul", 0, 1)), 2), 3)), [a, s, b, c], (n, n), "f32")
    check(got, want, "ulp1", "config 2 full size", "f32")
    # properties that hold at any size: relu output is non-negative; zero exactly where the pre-activation is <= 0
    assert (got.float() >= 0).all()
    pre = torch.exp(a.float() * s.float()) * b.float() + c.float()
    assert ((got == 0) == (pre.to(torch.bfloat16) <= 0)).float().mean().item() > 0.9999


def test_repeated_calls_reuse_plan_and_stay_correct(backend):
    _, mods = backend
    import ttnn
    case = cases.by_name("bcast_row_tilecol")
    want = oracle_output(case)
    prog = case.get_program(mods)
    n_plans = None
    for i in range(3):
        ins = [ttnn.from_torch(t) for t in case.make_inputs()]
        out = ttnn.from_torch(torch.full(case.out_shape, float(i), dtype=case.dtype))
        prog(*ins, out)
        assert torch.equal(ttnn.to_torch(out), want)
        if n_plans is None:
            n_plans = len(prog._plans)
    assert len(prog._plans) == n_plans, "the plan of an already-seen tensor signature must be reused"


def test_kernel_calls_can_be_captured_in_a_cuda_graph(backend):
    """Launch-bound inner loops: once a program has been seen (plan built, kernel compiled), calling it on a
    capturing stream records its launches and nothing else - no allocation, no synchronisation - so a CUDA graph
    of several kernel calls replays them without the host; new inputs written into the same tensors give new
    results on the next replay."""
    _, mods = backend
    import ttnn
    case = cases.by_name("bcast_row_tilecol")
    prog = case.get_program(mods)
    ins = [ttnn.from_torch(t) for t in case.make_inputs()]
    outs = [ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype)) for _ in range(3)]
    prog(*ins, outs[0])                                  # first call outside the capture: trace, compile
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for o in outs:
            prog(*ins, o)
    for o in outs:
        o._tensor.zero_()
    graph.replay()
    torch.cuda.synchronize()
    want = oracle_output(case)
    for o in outs:
        assert torch.equal(ttnn.to_torch(o), want)
    ins[0]._tensor.mul_(2)                               # same storage, new values
    torch.cuda.synchronize()
    graph.replay()
    prog(*ins, outs[0])
    direct = ttnn.to_torch(outs[0]).clone()
    assert torch.equal(ttnn.to_torch(outs[2]), direct) and not torch.equal(direct, want)


# ---- the C ABI itself: error behaviour and edge cases --------------------------------------
def _desc(capi, x, y, out, ops, rows, cols, n_in=2):
    d = capi.EltwiseDesc()
    d.dtype, d.round_each_op, d.n_in, d.n_ops = capi.TTLB_BF16, 1, n_in, len(ops)
    for k, t in enumerate((x, y)[:n_in]):
        d.inp[k].ptr, d.inp[k].ld = t.data_ptr(), t.stride(0)
    for k, (op, arg) in enumerate(ops):
        d.ops[k].opcode, d.ops[k].arg = capi.OPCODES[op], arg
    d.out, d.out_ld, d.rows, d.cols = out.data_ptr(), out.stride(0), rows, cols
    return d


def test_c_abi_rejects_malformed_descriptors_before_launching():
    from ttl_b200 import capi
    ctx = capi.context()
    lib = capi.lib()
    x = torch.ones(64, 64, dtype=torch.bfloat16, device="cuda")
    y = torch.ones(64, 64, dtype=torch.bfloat16, device="cuda")
    o = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    n0 = ctx.launch_count()

    def rc(d):
        return lib.ttlb_eltwise(ctx.handle, ctypes.byref(d), None)

    assert rc(_desc(capi, x, y, o, [("add", 1)], 64, 64)) == capi.TTLB_ERR_INVALID_ARG          # no LOAD first
    assert b"LOAD" in lib.ttlb_last_error(ctx.handle)
    assert rc(_desc(capi, x, y, o, [("load", 0), ("add", 5)], 64, 64)) == capi.TTLB_ERR_INVALID_ARG   # bad input index
    assert rc(_desc(capi, x, y, o, [("load", 0), ("add", -1)], 64, 64)) == capi.TTLB_ERR_INVALID_ARG  # pop of empty stack
    assert rc(_desc(capi, x, y, o, [("load", 0), ("push", 0)], 64, 64)) == capi.TTLB_ERR_INVALID_ARG  # value left on stack
    assert rc(_desc(capi, x, y, o, [("load", 0), ("add", 1)], 64, 60)) == capi.TTLB_ERR_INVALID_ARG   # cols not multiple of 8
    d = _desc(capi, x, y, o, [("load", 0), ("add", 1)], 64, 64)
    d.dtype = capi.TTLB_BFP8_B
    assert rc(d) == capi.TTLB_ERR_UNSUPPORTED
    d = _desc(capi, x, y, o, [("load", 0), ("add", 1)], 64, 64)
    d.inp[1].ptr = None
    assert rc(d) == capi.TTLB_ERR_INVALID_ARG
    assert lib.ttlb_eltwise(ctx.handle, None, None) == capi.TTLB_ERR_INVALID_ARG
    assert lib.ttlb_eltwise(None, ctypes.byref(d), None) == capi.TTLB_ERR_INVALID_ARG
    assert ctx.launch_count() == n0, "a rejected descriptor must not launch anything"
    # empty rectangle: accepted, nothing launched, output untouched
    assert rc(_desc(capi, x, y, o, [("load", 0), ("add", 1)], 0, 64)) == capi.TTLB_OK
    torch.cuda.synchronize()
    assert ctx.launch_count() == n0 and (o == 0).all()
    # and a valid one still works afterwards
    assert rc(_desc(capi, x, y, o, [("load", 0), ("add", 1)], 64, 64)) == capi.TTLB_OK
    torch.cuda.synchronize()
    assert (o == 2).all() and ctx.launch_count() == n0 + 1


def test_c_abi_sub_rectangle_and_offsets_leave_the_rest_untouched():
    from ttl_b200 import capi
    ctx = capi.context()
    g = torch.Generator().manual_seed(5)
    xc = torch.randn(96, 128, generator=g).to(torch.bfloat16)
    yc = torch.randn(96, 128, generator=g).to(torch.bfloat16)
    x, y = xc.cuda(), yc.cuda()
    o = torch.full((96, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    d = _desc(capi, x, y, o, [("load", 0), ("mul", 1)], 32, 64)
    d.row0, d.col0 = 32, 32
    d.inp[1].row_off, d.inp[1].col_off = 32, -32   # y is read shifted by one tile down / one tile left
    ctx.eltwise(d, 0)
    torch.cuda.synchronize()
    want = torch.full((96, 128), 7.0, dtype=torch.bfloat16)
    want[32:64, 32:96] = xc[32:64, 32:96] * yc[64:96, 0:64]
    assert torch.equal(o.cpu(), want)


@pytest.mark.parametrize("dims,in_block,out_block", [([0], (2, 2), (2, 2)), ([1], (2, 2), (2, 2)), ([0, 1], (2, 2), (2, 2)),
                                                      ([0], (1, 2), (2, 2)), ([1], (2, 1), (2, 3)), ([0, 1], (1, 1), (3, 2))])
def test_hardware_broadcast_of_full_tiles(dims, in_block, out_block, backend, eltwise_path):
    """The compiler's broadcast convention (first row / column / element of every FULL source tile,
    test/python/test_bcast_ops.py:31-55), selected with set_hardware_broadcast: index modes FIRST and
    ZERO-with-offset in both GPU kernels, against a torch restatement."""
    import ttl_b200
    _, mods = backend
    import ttnn
    g = torch.Generator().manual_seed(7)
    x = torch.randn(out_block[0] * 32, out_block[1] * 32, generator=g).to(torch.bfloat16)
    b = torch.randn(in_block[0] * 32, in_block[1] * 32, generator=g).to(torch.bfloat16)
    src = b.float().reshape(in_block[0], 32, in_block[1], 32)
    if 0 in dims:
        src = src[:, :1].expand(-1, 32, -1, -1)
    if 1 in dims:
        src = src[:, :, :, :1].expand(-1, -1, -1, 32)
    src = src.expand(out_block[0] if in_block[0] == 1 else -1, -1, out_block[1] if in_block[1] == 1 else -1, -1)
    xf = x.float()
    want = ((xf + xf).to(torch.bfloat16).float() + src.reshape(out_block[0] * 32, out_block[1] * 32)).to(torch.bfloat16)
    out = ttnn.from_torch(torch.zeros_like(x))
    ttl_b200.set_hardware_broadcast(True)
    try:
        mods["eltwise"].make_hw_broadcast(dims, in_block, out_block)(ttnn.from_torch(x), ttnn.from_torch(b), out)
    finally:
        ttl_b200.set_hardware_broadcast(False)
    assert torch.equal(ttnn.to_torch(out), want)
