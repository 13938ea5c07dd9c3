"""GPU parity of the tcgen05 bf16 GEMM: tt-lang matmul programs run through the backend, and the
C ABI called directly, against the simulator's committed outputs and the CPU oracle.
Tolerance (stated by the task for matmul): max |got - want| / max |want| <= 1e-2 against the
fp32-accumulated result, bf16 output."""

import ctypes

import pytest
import torch

import cases
from conftest import golden_tensor, load_golden
from oracle import tile_oracle

pytestmark = pytest.mark.gpu
TOL = 1e-2


def rel_err(got, want):
    return ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()


@pytest.mark.parametrize("case", cases.MATMUL_CASES, ids=lambda c: c.name)
def test_matmul_program_matches_simulator_and_oracle(case, backend):
    from ttl_b200 import capi
    _, mods = backend
    import ttnn
    ins = case.make_inputs()
    a, b = ins[0], ins[1]
    bias = ins[2] if len(ins) > 2 else None
    out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=torch.bfloat16))
    n0 = capi.context().launch_count()
    case.get_program(mods)(*[ttnn.from_torch(t) for t in ins], out)
    capi.context().check_status(capi.current_stream())
    assert capi.context().launch_count() == n0 + 1
    got = ttnn.to_torch(out)
    assert rel_err(got, tile_oracle.matmul_tiles(a, b, "f32", bias=bias)) <= TOL
    assert rel_err(got, golden_tensor(load_golden(case.name)["out"], torch.bfloat16)) <= TOL


@pytest.mark.parametrize("variant", [0, 1, 2], ids=["one_cta", "auto", "two_cta"])
@pytest.mark.parametrize("m,n,k", [(32, 32, 32), (128, 256, 64), (160, 96, 224), (384, 520, 72), (1024, 1536, 512),
                                   (96, 2048, 4096), (256, 256, 64), (300, 264, 136), (2304, 4352, 1024)])
def test_c_abi_matmul_shapes_with_ragged_tiles(m, n, k, variant):
    """Direct C-ABI calls: single tile, shapes that are not multiples of the CTA tile (TMA zero-fills
    the out-of-range part, the epilogue masks it), tall-K; with both tensor-core kernels (the default picks
    between them by output size)."""
    from ttl_b200 import capi, ops, ttnn
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    b = torch.randn(k, n, generator=g).to(torch.bfloat16)
    # canary rows/cols around the output: the kernel must not write outside [m, n]
    full = torch.full((m + 64, n + 64), 3.0, dtype=torch.bfloat16, device="cuda")
    d = capi.GemmDesc()
    A, B = a.cuda(), b.cuda()
    d.a, d.lda, d.b, d.ldb = A.data_ptr(), k, B.data_ptr(), n
    d.c, d.ldc = full.data_ptr() + (32 * full.stride(0) + 32) * 2, full.stride(0)
    d.m, d.n, d.k = m, n, k
    ctx = capi.context()
    ctx.set_gemm_variant(variant)
    try:
        ctx.matmul_bf16(d, capi.current_stream())
        ctx.check_status(capi.current_stream())
    finally:
        ctx.set_gemm_variant(1)
    got = full.cpu()
    assert rel_err(got[32:32 + m, 32:32 + n], tile_oracle.matmul_tiles(a, b, "f32")) <= TOL
    frame = got.clone()
    frame[32:32 + m, 32:32 + n] = 3.0
    assert (frame == 3.0).all(), "matmul wrote outside its output rectangle"


@pytest.mark.parametrize("variant", [0, 2], ids=["one_cta", "two_cta"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 264, 136), (2304, 4352, 512)])
def test_c_abi_matmul_with_bias(m, n, k, variant):
    """C = A B + bias through the C ABI with both tensor-core kernels, ragged tiles included; the bias is
    added in fp32 before the single rounding (checked exactly against a torch fp32 reference of the op)."""
    from ttl_b200 import capi
    g = torch.Generator().manual_seed(m + 2 * n + 3 * k)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    b = torch.randn(k, n, generator=g).to(torch.bfloat16)
    bias = (4 * torch.randn(m, n, generator=g)).to(torch.bfloat16)
    A, B, Cb = a.cuda(), b.cuda(), bias.cuda()
    out = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    d = capi.GemmDesc()
    d.a, d.lda, d.b, d.ldb, d.c, d.ldc = A.data_ptr(), k, B.data_ptr(), n, out.data_ptr(), n
    d.m, d.n, d.k = m, n, k
    ctx = capi.context()
    ctx.set_gemm_variant(variant)
    try:
        ctx.matmul_bf16_bias(d, Cb.data_ptr(), n, capi.current_stream())
        ctx.check_status(capi.current_stream())
    finally:
        ctx.set_gemm_variant(1)
    want = tile_oracle.matmul_tiles(a, b, "f32", bias=bias)
    assert rel_err(out.cpu(), want) <= TOL
    # the bias is not rounded away: with a zero product the output is the bias itself
    out.zero_()
    d.a = torch.zeros_like(A).data_ptr()
    ctx.matmul_bf16_bias(d, Cb.data_ptr(), n, capi.current_stream())
    assert torch.equal(out.cpu(), bias)


def test_c_abi_matmul_rejects_bad_descriptors():
    from ttl_b200 import capi
    ctx = capi.context()
    lib = capi.lib()
    x = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    n0 = ctx.launch_count()

    def desc(**kw):
        d = capi.GemmDesc()
        d.a = d.b = d.c = x.data_ptr()
        d.lda = d.ldb = d.ldc = 64
        d.m = d.n = d.k = 64
        for key, v in kw.items():
            setattr(d, key, v)
        return d

    def rc(d):
        return lib.ttlb_matmul_bf16(ctx.handle, ctypes.byref(d), None)

    assert rc(desc(a=None)) == capi.TTLB_ERR_INVALID_ARG
    assert rc(desc(k=0)) == capi.TTLB_ERR_INVALID_ARG
    assert rc(desc(k=60)) == capi.TTLB_ERR_INVALID_ARG            # K not a multiple of 8
    assert rc(desc(lda=32)) == capi.TTLB_ERR_INVALID_ARG          # pitch smaller than the row
    assert rc(desc(c=x.data_ptr() + 2)) == capi.TTLB_ERR_INVALID_ARG  # misaligned
    assert lib.ttlb_matmul_bf16(ctx.handle, None, None) == capi.TTLB_ERR_INVALID_ARG
    assert rc(desc(m=0)) == capi.TTLB_OK                           # empty output: nothing to do
    assert ctx.launch_count() == n0


def test_config3_full_size_slabs_and_scaling_property():
    """configs[2]: 8192^3, entries N(0, 1/sqrt(8192)) from seeds 0/1.  The oracle (fp32-accumulated tile
    matmul) is evaluated on three row slabs; a size-independent property covers the rest:
    scaling A by a power of two scales every output exactly."""
    from ttl_b200 import capi, ops, ttnn
    n = 8192
    a = cases.gen((n, n), f"normal*{n ** -0.5}", 0)
    b = cases.gen((n, n), f"normal*{n ** -0.5}", 1)
    A, B = ttnn.from_torch(a), ttnn.from_torch(b)
    C = ops.matmul(A, B)
    capi.context().check_status(capi.current_stream())
    got = ttnn.to_torch(C)
    for r0 in (0, 4064, 8128):
        want = tile_oracle.matmul_tiles(a[r0:r0 + 64], b, "f32")
        assert rel_err(got[r0:r0 + 64], want) <= TOL, f"rows {r0}..{r0 + 63}"
    C4 = ops.matmul(ttnn.from_torch(a * 4), B)
    assert torch.equal(ttnn.to_torch(C4), got * 4), "matmul(4A, B) must equal 4 * matmul(A, B) bit for bit"


@pytest.mark.parametrize("name", ["singlecore_matmul", "multicore_matmul"])
def test_fp32_matmul_program(backend, name):
    """The reference's matmul examples call their kernels on float32 tensors (128x256 @ 256x64) and
    check at rtol = atol = 1e-4 against an fp32 golden (examples/singlecore_matmul.py:73-88)."""
    from ttl_b200 import capi
    _, mods = backend
    import ttnn
    a = cases.gen((128, 256), "uniform", 0, torch.float32)
    b = cases.gen((256, 64), "uniform", 1, torch.float32)
    out = ttnn.from_torch(torch.zeros((128, 64), dtype=torch.float32))
    getattr(mods["matmul"], name)(ttnn.from_torch(a), ttnn.from_torch(b), out)
    got = ttnn.to_torch(out)
    assert torch.allclose(got, tile_oracle.matmul_tiles(a, b, "native"), rtol=1e-4, atol=1e-4)
    assert torch.allclose(got, a @ b, rtol=1e-4, atol=1e-4)


def test_c_abi_matmul_f32_ragged():
    from ttl_b200 import capi
    m, n, k = 100, 72, 40
    g = torch.Generator().manual_seed(3)
    a, b = torch.randn(m, k, generator=g), torch.randn(k, n, generator=g)
    A, B = a.cuda(), b.cuda()
    C = torch.full((m + 2, n + 3), 7.0, device="cuda")
    d = capi.GemmDesc()
    d.a, d.lda, d.b, d.ldb, d.c, d.ldc, d.m, d.n, d.k = A.data_ptr(), k, B.data_ptr(), n, C.data_ptr(), n + 3, m, n, k
    capi.context().matmul_f32(d, capi.current_stream())
    torch.cuda.synchronize()
    got = C.cpu()
    assert torch.allclose(got[:m, :n], a @ b, rtol=1e-5, atol=1e-5)
    assert (got[m:] == 7.0).all() and (got[:, n:] == 7.0).all()


def test_k_blocked_matmul_program(backend):
    """(bm, bk) @ (bk, bn) blocks (the reference's reuse matmul form, which its simulator cannot run): one GEMM
    launch; against fp32 torch."""
    _, mods = backend
    import ttnn
    from ttl_b200 import capi
    a = cases.gen((512, 768), "normal*0.036", 30)
    b = cases.gen((768, 384), "normal", 31)
    out = ttnn.from_torch(torch.zeros((512, 384), dtype=torch.bfloat16))
    prog = mods["matmul"].make_kblock_matmul(4, 3, 2)
    d = prog.plan(ttnn.from_torch(a), ttnn.from_torch(b), out).describe()
    assert len(d) == 1 and d[0]["kind"] == "matmul_bf16" and d[0]["k_tiles"] == 24
    before = capi.context().launch_count()
    prog(ttnn.from_torch(a), ttnn.from_torch(b), out)
    assert capi.context().launch_count() == before + 1
    want = a.float() @ b.float()
    got = ttnn.to_torch(out).float()
    assert ((got - want).abs().max() / want.abs().max()).item() <= 1e-2


def test_config3_as_the_unchanged_tile_program_at_full_size(backend):
    """configs[2] through `@ttl.kernel`: the reference's multicore matmul program in 1x1-tile blocks
    (examples/multicore_matmul.py:28-139, restated in tests/programs/matmul.py) on 8192^3 - 16.7 million tile
    multiply-accumulates traced with batched loops - becomes one GEMM launch; checked on three row slabs."""
    import time
    from ttl_b200 import capi
    _, mods = backend
    import ttnn
    n = 8192
    a = cases.gen((n, n), f"normal*{n ** -0.5}", 0)
    b = cases.gen((n, n), f"normal*{n ** -0.5}", 1)
    A, B = ttnn.from_torch(a), ttnn.from_torch(b)
    out = ttnn.from_torch(torch.zeros((n, n), dtype=torch.bfloat16))
    prog = mods["matmul"].multicore_matmul
    t0 = time.perf_counter()
    plan = prog.plan(A, B, out)
    assert time.perf_counter() - t0 < 10, "trace + recognise of the 8192^3 program took too long"
    assert [d["kind"] for d in plan.describe()] == ["matmul_bf16"]
    n0 = capi.context().launch_count()
    prog(A, B, out)
    capi.context().check_status(capi.current_stream())
    assert capi.context().launch_count() == n0 + 1
    got = ttnn.to_torch(out)
    for r0 in (0, 4064, 8128):
        assert rel_err(got[r0:r0 + 64], tile_oracle.matmul_tiles(a[r0:r0 + 64], b, "f32")) <= TOL, f"rows {r0}..{r0 + 63}"


@pytest.mark.parametrize("variant", [0, 2], ids=["one_cta", "two_cta"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 288, 136), (1024, 2048, 512)])
def test_c_abi_matmul_published_to_several_buffers(m, n, k, variant):
    """ttlb_matmul_bf16_peers: the epilogue that passes every tile through shared memory and stores it, whole
    256-byte row segments at a time, into the output region of several buffers (on a box with several GPUs: every
    GPU's copy of a shared output).  Here all buffers live on this GPU: each must hold exactly what the plain
    matmul gives, and nothing may be written around the output regions.  Both GEMM kernels have this epilogue
    (128x256 tiles of one CTA, 256x256 tiles of a CTA pair)."""
    from ttl_b200 import capi
    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    b = torch.randn(k, n, generator=g).to(torch.bfloat16)
    A, B = a.cuda(), b.cuda()
    ctx = capi.context()
    ctx.set_gemm_variant(variant)
    try:
        plain = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        d = capi.GemmDesc()
        d.a, d.lda, d.b, d.ldb, d.c, d.ldc, d.m, d.n, d.k = A.data_ptr(), k, B.data_ptr(), n, plain.data_ptr(), n, m, n, k
        ctx.matmul_bf16(d, capi.current_stream())
        bufs = [torch.full((m + 64, n + 64), 3.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
        d.c, d.ldc = None, n + 64
        ctx.matmul_bf16_peers(d, [x.data_ptr() + (32 * (n + 64) + 32) * 2 for x in bufs], capi.current_stream())
        ctx.check_status(capi.current_stream())
    finally:
        ctx.set_gemm_variant(1)
    assert rel_err(plain.cpu(), tile_oracle.matmul_tiles(a, b, "f32")) <= TOL
    for x in bufs:
        got = x.cpu()
        assert torch.equal(got[32:32 + m, 32:32 + n], plain.cpu()), "published tile differs from the plain matmul"
        got[32:32 + m, 32:32 + n] = 3.0
        assert (got == 3.0).all(), "the publishing epilogue wrote outside the output region"


def bf16_ulp_distance(golden: torch.Tensor, got: torch.Tensor) -> float:
    """max |got - golden| / ULP(golden), ULP = the gap from |golden| to the next bfloat16 above it: the measure of
    the reference's `assert_with_ulp` (python/utils/correctness.py:168-213)."""
    g = golden.to(torch.bfloat16)
    a = g.abs()
    gap = (torch.nextafter(a, torch.full_like(a, float("inf"))) - a).float()
    return ((got.float() - g.float()).abs() / gap).max().item()


@pytest.mark.parametrize("variant", [0, 2], ids=["one_cta", "two_cta"])
@pytest.mark.parametrize("n", [256, 512])
def test_matmul_within_10_bf16_ulp_of_torch_matmul(backend, n, variant):
    """The reference's own criterion for its matmul kernels
    (examples/metal_examples/singlecore_matmul/ttlang/singlecore_matmul.py:63-79): uniform [0, 1) bfloat16 operands,
    golden = torch.matmul in bfloat16, at most 10 bfloat16 ULP apart - next to the norm-wise 1e-2 bound, which
    would hide large relative errors on small outputs."""
    from ttl_b200 import capi
    _, mods = backend
    import ttnn
    torch.manual_seed(n)
    a, b = ttnn.rand((n, n), dtype=ttnn.bfloat16), ttnn.rand((n, n), dtype=ttnn.bfloat16)
    c = ttnn.empty((n, n), dtype=ttnn.bfloat16)
    ctx = capi.context()
    ctx.set_gemm_variant(variant)
    try:
        mods["matmul"].singlecore_matmul(a, b, c)
        ctx.check_status(capi.current_stream())
    finally:
        ctx.set_gemm_variant(1)
    golden = torch.matmul(ttnn.to_torch(a).to(torch.bfloat16), ttnn.to_torch(b).to(torch.bfloat16))
    result = ttnn.to_torch(c).to(torch.bfloat16)
    assert bf16_ulp_distance(golden, result) <= 10
    assert rel_err(result, golden) <= TOL
