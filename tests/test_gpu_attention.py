"""GPU parity of the fused attention kernel against the CPU oracle.  Tolerance (stated by the task
for attention): max |got - want| / max |want| <= 1e-2, fp32 row max / sum, bf16 output."""

import ctypes

import pytest
import torch

import cases
from oracle import attention_oracle

pytestmark = pytest.mark.gpu
TOL = 1e-2


def rel_err(got, want):
    return ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()


def qkv(shape, seeds=(0, 1, 2)):
    n = 1
    for s in shape[:-1]:
        n *= s
    return [cases.gen((n, shape[-1]), "normal", s).reshape(shape) for s in seeds]


@pytest.mark.parametrize("shape,causal", [((1, 1, 128, 128), True), ((1, 2, 256, 128), True), ((2, 3, 512, 128), True),
                                          ((1, 2, 384, 128), False), ((1, 1, 200, 128), True), ((1, 2, 72, 128), False),
                                          ((1, 1, 1000, 128), True), ((1, 2, 640, 128), True), ((1, 1, 128 * 7, 128), False)])
def test_attention_matches_oracle(shape, causal):
    """One tile, several KV blocks, several heads, non-causal, and sequence lengths that are not
    multiples of the 128-row tile (ragged last tile: out-of-range keys masked, rows not stored)."""
    from ttl_b200 import capi, ops, ttnn
    q, k, v = qkv(shape)
    scale = shape[-1] ** -0.5
    out = ttnn.from_torch(torch.full(shape, 5.0, dtype=torch.bfloat16))
    ops.attention(ttnn.from_torch(q), ttnn.from_torch(k), ttnn.from_torch(v), causal=causal, scale=scale, out=out)
    capi.context().check_status(capi.current_stream())
    got = ttnn.to_torch(out)
    assert torch.isfinite(got.float()).all()
    assert rel_err(got, attention_oracle.attention_tiles(q, k, v, causal, scale)) <= TOL
    assert rel_err(got, attention_oracle.attention_plain(q, k, v, causal, scale)) <= TOL


@pytest.mark.parametrize("causal", [True, False])
def test_attention_with_growing_scores(causal):
    """Keys whose magnitude grows along the sequence: the row max keeps jumping by far more than the
    kernel's lazy-rescaling threshold, so the output accumulators are corrected in place many times."""
    from ttl_b200 import capi, ops, ttnn
    shape = (1, 2, 1152, 128)
    q, k, v = qkv(shape, seeds=(3, 4, 5))
    ramp = torch.linspace(0.25, 6.0, shape[2]).reshape(1, 1, -1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    scale = shape[-1] ** -0.5
    got = ttnn.to_torch(ops.attention(ttnn.from_torch(q), ttnn.from_torch(k), ttnn.from_torch(v), causal=causal, scale=scale))
    capi.context().check_status(capi.current_stream())
    assert torch.isfinite(got.float()).all()
    assert rel_err(got, attention_oracle.attention_tiles(q, k, v, causal, scale)) <= TOL
    assert rel_err(got, attention_oracle.attention_plain(q, k, v, causal, scale)) <= TOL


def test_attention_properties_at_config5_shape_subset():
    """configs[4] geometry (seq 4096, head_dim 128, causal, scale 1/sqrt(128)) on 2 x 4 heads: sampled
    heads against the oracle, and properties that hold at any size - row 0 of a causal head equals
    V[0]; heads are independent (running a subset gives the same bits)."""
    from ttl_b200 import capi, ops, ttnn
    shape = (2, 4, 4096, 128)
    q, k, v = qkv(shape)
    scale = 128 ** -0.5
    O = ops.attention(ttnn.from_torch(q), ttnn.from_torch(k), ttnn.from_torch(v), causal=True, scale=scale)
    capi.context().check_status(capi.current_stream())
    got = ttnn.to_torch(O)
    for b, h in ((0, 0), (1, 3)):
        want = attention_oracle.attention_tiles(q[b, h], k[b, h], v[b, h], True, scale)
        assert rel_err(got[b, h], want) <= TOL, (b, h)
    assert torch.equal(got[:, :, 0, :], v[:, :, 0, :])
    sub = ops.attention(ttnn.from_torch(q[1:, 2:].contiguous()), ttnn.from_torch(k[1:, 2:].contiguous()),
                        ttnn.from_torch(v[1:, 2:].contiguous()), causal=True, scale=scale)
    assert torch.equal(ttnn.to_torch(sub), got[1:, 2:])


def test_c_abi_attention_rejects_bad_descriptors():
    from ttl_b200 import capi
    ctx = capi.context()
    lib = capi.lib()
    x = torch.zeros(1, 128, 128, dtype=torch.bfloat16, device="cuda")
    n0 = ctx.launch_count()

    def desc(**kw):
        d = capi.AttnDesc()
        d.q = d.k = d.v = d.o = x.data_ptr()
        d.batch_heads, d.seq, d.head_dim, d.causal, d.scale = 1, 128, 128, 1, 0.088
        for key, val in kw.items():
            setattr(d, key, val)
        return d

    def rc(d):
        return lib.ttlb_attention(ctx.handle, ctypes.byref(d), None)

    assert rc(desc(head_dim=64)) == capi.TTLB_ERR_UNSUPPORTED
    assert rc(desc(q=None)) == capi.TTLB_ERR_INVALID_ARG
    assert rc(desc(scale=0.0)) == capi.TTLB_ERR_INVALID_ARG
    assert rc(desc(o=x.data_ptr() + 2)) == capi.TTLB_ERR_INVALID_ARG
    assert rc(desc(seq=0)) == capi.TTLB_OK
    assert ctx.launch_count() == n0


@pytest.mark.parametrize("shape,causal", [((1, 2, 384, 128), True), ((1, 3, 200, 128), True), ((2, 2, 512, 128), False)])
def test_c_abi_attention_published_to_several_buffers(shape, causal):
    """ttlb_attention_peers: the epilogue that stages every tile's rows in shared memory and stores them, whole
    128-byte half rows at a time, into several buffers (on a box with several GPUs: every GPU's copy of a shared
    output).  Here all buffers live on this GPU: each must hold exactly what the plain kernel gives, and nothing
    may be written around the outputs (ragged last tile included)."""
    from ttl_b200 import capi, ops, ttnn
    q, k, v = qkv(shape)
    scale = shape[-1] ** -0.5
    Q, K, V = ttnn.from_torch(q), ttnn.from_torch(k), ttnn.from_torch(v)
    plain = ttnn.to_torch(ops.attention(Q, K, V, causal=causal, scale=scale))
    assert rel_err(plain, attention_oracle.attention_tiles(q, k, v, causal, scale)) <= TOL
    n = q.numel()
    bufs = [torch.full((n + 4096,), 3.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    out = ttnn.Tensor(bufs[0][2048:2048 + n].view(shape))
    ops.attention(Q, K, V, causal=causal, scale=scale, out=out, peer_ptrs=[b.data_ptr() + 4096 for b in bufs])
    capi.context().check_status(capi.current_stream())
    for b in bufs:
        got = b.cpu()
        assert torch.equal(got[2048:2048 + n].view(shape), plain), "published output differs from the plain kernel's"
        assert (got[:2048] == 3.0).all() and (got[2048 + n:] == 3.0).all(), "the publishing epilogue wrote outside the output"


@pytest.mark.parametrize("case", cases.ATTENTION_PIPELINE_CASES, ids=lambda c: c.name)
def test_fused_kernel_and_tile_programs_match_the_simulator(case, backend):
    """Pinned to the reference simulator: the fixtures are its outputs for attention run as three tile kernels (1x1-tile
    block matmuls accumulated over K, masked row softmax in between; tests/programs/attention.py, generated by
    tests/golden/make_golden.py) at head dimension 128.  Against them, within max |diff| / max |want| <= 1e-2:
    the fused kernel `ttlb_attention`; the same three kernels through `@ttl.kernel` on the GPU (GEMM, row-resident
    softmax, GEMM); and the single-kernel tile program with block matmuls whose plan has the same three launches."""
    from conftest import golden_tensor, load_golden
    from ttl_b200 import capi, ops
    _, mods = backend
    import ttnn
    want = golden_tensor(load_golden(case.name)["out"], case.dtype)
    host = case.make_inputs()
    q, kt, v, mask, scale, one = host
    bf = torch.bfloat16
    # 1. the fused kernel (bf16 in / out)
    shape = (1, 1) + tuple(q.shape)
    got = ttnn.to_torch(ops.attention(ttnn.from_torch(q.to(bf).reshape(shape)), ttnn.from_torch(kt.t().contiguous().to(bf).reshape(shape)),
                                      ttnn.from_torch(v.to(bf).reshape(shape)), causal=True, scale=float(scale[0, 0])))
    assert rel_err(got.reshape(q.shape), want) <= TOL
    # 2. three kernels, in the fixture's element type
    prog = mods["attention"]
    out = ttnn.from_torch(torch.zeros(case.out_shape, dtype=case.dtype))
    n0 = capi.context().launch_count()
    prog.attention_pipeline(*[ttnn.from_torch(t) for t in host], out)
    assert capi.context().launch_count() == n0 + 3
    assert rel_err(ttnn.to_torch(out), want) <= (TOL if case.dtype == bf else 1e-4)
    # 3. one kernel with block matmuls and reductions (bf16; the specification's block dot product)
    if case.dtype == bf:
        out2 = ttnn.from_torch(torch.zeros(case.out_shape, dtype=bf))
        plan = prog.attention_rows.plan(*[ttnn.from_torch(t) for t in host], out2)
        assert [d["kind"] for d in plan.describe()] == ["matmul_bf16", "row_fused", "matmul_bf16"]
        prog.attention_rows(*[ttnn.from_torch(t) for t in host], out2)
        capi.context().check_status(capi.current_stream())
        assert rel_err(ttnn.to_torch(out2), want) <= TOL


def test_config5_full_shape_properties_and_sampled_heads():
    """configs[4] at its full shape, B 8 x H 32 x S 4096 x D 128 (1 GB of tensors), checked on the whole output:
    with a causal mask row 0 of every head equals V's row 0 exactly; heads are independent (a second run with
    all other heads' Q / K / V changed leaves a head's output bits unchanged); and the oracle on sampled heads -
    the first and the last head of what each of 8 ranks would own (32 consecutive (batch, head) pairs)."""
    from ttl_b200 import capi, ops, ttnn
    B, H, S, D = 8, 32, 4096, 128
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(B * H, S, D, generator=g, dtype=torch.float32).to(torch.bfloat16) for _ in range(3))
    Q, K, V = (ttnn.from_torch(t) for t in (q, k, v))
    scale = D ** -0.5
    out = ttnn.to_torch(ops.attention(Q, K, V, causal=True, scale=scale))
    capi.context().check_status(capi.current_stream())
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out[:, 0, :], v[:, 0, :]), "row 0 of a causal head must be V's row 0"
    heads = sorted({0, 31, 32, 127, 128, 223, 224, 255})
    for h in heads[:4] + heads[-2:]:
        want = attention_oracle.attention_tiles(q[h:h + 1], k[h:h + 1], v[h:h + 1], True, scale)
        assert rel_err(out[h:h + 1], want) <= TOL, f"head {h}"
    # head independence: scramble every other head, the kept heads must not change by a bit
    keep = torch.tensor(heads)
    q2, k2, v2 = q.flip(0).clone(), k.flip(0).clone(), v.flip(0).clone()
    q2[keep], k2[keep], v2[keep] = q[keep], k[keep], v[keep]
    out2 = ttnn.to_torch(ops.attention(ttnn.from_torch(q2), ttnn.from_torch(k2), ttnn.from_torch(v2), causal=True, scale=scale))
    assert torch.equal(out2[keep], out[keep]), "a head's output depends on other heads"
