"""GPU parity for bfloat8_b weights: device unpack is bit-exact against the oracle, and the
bfp8-weight matmul matches the oracle (dequantised weights, fp32-accumulated tile matmul) within
1e-2, both through the C ABI and through a tt-lang matmul program whose B tensor is bfloat8_b."""

import numpy as np
import pytest
import torch

import cases
from oracle import bfp8_oracle, tile_oracle

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    return ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()


@pytest.mark.parametrize("k,n,col0,cols", [(32, 32, 0, 32), (96, 160, 0, 160), (128, 256, 64, 128), (4096, 512, 32, 448)])
def test_device_unpack_is_bit_exact(k, n, col0, cols):
    from ttl_b200 import bfp8, capi
    w = cases.gen((k, n), "normal*0.02", 1, torch.float32)
    w[0, :16] = torch.tensor([1e-30] * 8 + [3e-39] * 8)[: 16]   # a block with a tiny exponent
    w[1, :16] = torch.tensor([3e-38, -1.5e-38] + [2e-39] * 14)      # results that are bf16 denormals
    w[2, :16] = torch.tensor([-3e38, 1e38, 2.5e37, -7.0] + [1e30] * 12)   # the largest exponents
    w[3, :16] = torch.tensor([1.0, -1.0, 1.5, 1.9921875, -0.0078125, 0.0] + [0.33] * 10)   # exponent 127 / 128 boundary
    w[4, :16] = torch.tensor([2.0, -3.99, 2.5] + [1.0] * 13)
    w[5, :16] = 0.0                                             # an all-zero block (exponent 0)
    tiles = bfp8.pack_bfp8_b(w)
    want = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w.numpy()), k, n))[:, col0:col0 + cols]
    out = torch.full((k, cols + 8), 9.0, dtype=torch.bfloat16, device="cuda")
    dev = tiles.cuda()
    ctx = capi.context()
    ctx.unpack_bfp8_b(dev.data_ptr(), n // 32, col0 // 32, k, cols, out.data_ptr(), out.stride(0), capi.current_stream())
    torch.cuda.synchronize()
    got = out.cpu()
    assert torch.equal(got[:, :cols].float(), want), "device unpack differs from the oracle"
    assert (got[:, cols:] == 9.0).all(), "unpack wrote outside its window"


@pytest.fixture(params=[0, 1, 2], ids=["unpack_kernel", "auto", "in_mainloop"])
def bfp8_mode(request):
    """Run with the separate unpack kernel, the default choice, and the unpack fused into the GEMM mainloop."""
    from ttl_b200 import capi
    capi.context().set_bfp8_mode(request.param)
    yield request.param
    capi.context().set_bfp8_mode(capi.BFP8_MODE_DEFAULT)


@pytest.mark.parametrize("m,k,n", [(64, 128, 96), (256, 512, 1024), (160, 2048, 608), (300, 96, 416), (1280, 1056, 2336)])
def test_c_abi_matmul_bfp8w(m, k, n, bfp8_mode):
    from ttl_b200 import capi, ops, ttnn
    x = cases.gen((m, k), "normal", 0)
    w = cases.gen((k, n), "normal*0.02", 1, torch.float32)
    wq = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w.numpy()), k, n))
    want = tile_oracle.matmul_tiles(x.float(), wq, "f32")
    W = ttnn.from_torch(w, dtype=ttnn.bfloat8_b)
    got = ttnn.to_torch(ops.matmul(ttnn.from_torch(x), W))
    capi.context().check_status(capi.current_stream())
    assert rel_err(got, want) <= 1e-2
    # a column window of the same weights (what an N-sharded rank computes)
    if n >= 96:
        out = ttnn.from_torch(torch.zeros((m, n), dtype=torch.bfloat16))
        ops.launch_gemm(capi.context(), ttnn.from_torch(x), W, out, (0, m, 32, 96), capi.current_stream())
        got2 = ttnn.to_torch(out)
        assert rel_err(got2[:, 32:96], want[:, 32:96]) <= 1e-2
        assert (got2[:, :32] == 0).all() and (got2[:, 96:] == 0).all()


def test_matmul_program_with_bfloat8_b_weights(backend, bfp8_mode):
    """The multicore matmul tile program, unchanged, with B given as a bfloat8_b tensor."""
    _, mods = backend
    import ttnn
    from ttl_b200 import capi
    m, k, n = 128, 256, 192
    x = cases.gen((m, k), "normal", 2)
    w = cases.gen((k, n), "normal*0.02", 3, torch.float32)
    wq = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w.numpy()), k, n))
    out = ttnn.from_torch(torch.zeros((m, n), dtype=torch.bfloat16))
    W = ttnn.from_torch(w, dtype=ttnn.bfloat8_b)
    prog = mods["matmul"].multicore_matmul
    assert prog.plan(ttnn.from_torch(x), W, out).describe()[0]["kind"] == "matmul_bfp8w"
    prog(ttnn.from_torch(x), W, out)
    capi.context().check_status(capi.current_stream())
    assert rel_err(ttnn.to_torch(out), tile_oracle.matmul_tiles(x.float(), wq, "f32")) <= 1e-2


def test_in_mainloop_expansion_is_exact_for_every_exponent():
    """The kernel that expands the weights inside the mainloop multiplies by 2^(E-126), which is a bf16 only up to
    E = 253, and produces bf16 denormals for the smallest exponents.  With a one-hot activation matrix the product
    IS the expanded weight matrix: it must equal the oracle's unpack value for value, blocks with exponents 254 / 255
    (values of 2^121 and more, expanded the slow way), denormal results and all-zero blocks included."""
    from ttl_b200 import capi, ops, ttnn
    k, n = 256, 416
    w = cases.gen((k, n), "normal*0.02", 7, torch.float32)
    w[0, :16] = torch.tensor([1e-30] * 8 + [3e-39] * 8)
    w[1, :16] = torch.tensor([3e-38, -1.5e-38] + [2e-39] * 14)          # results that are bf16 denormals
    w[2, 16:32] = torch.tensor([-3e38, 1e38, 2.5e37, -7.0] + [1e30] * 12)   # exponent 254
    w[3, :16] = torch.tensor([1.0, -1.0, 1.5, 1.9921875, -0.0078125, 0.0] + [0.33] * 10)
    w[65, 32:48] = torch.tensor([2.0, -3.99, 2.5] + [1.0] * 13)
    w[66, 400:416] = torch.tensor([1.7e38, -1.7e38] + [5e37] * 14)
    w[129, :16] = 0.0                                                   # an all-zero block (exponent 0)
    want = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w.numpy()), k, n))
    x = torch.eye(k, dtype=torch.bfloat16)
    W = ttnn.from_torch(w, dtype=ttnn.bfloat8_b)
    ctx = capi.context()
    try:
        for mode in (2, 0):
            ctx.set_bfp8_mode(mode)
            got = ttnn.to_torch(ops.matmul(ttnn.from_torch(x), W))
            ctx.check_status(capi.current_stream())
            assert torch.equal(got.float(), want), f"mode {mode}"   # value for value (a sum does not keep the sign of -0)
    finally:
        ctx.set_bfp8_mode(capi.BFP8_MODE_DEFAULT)


@pytest.mark.parametrize("m,k,n", [(300, 96, 416), (512, 2048, 1024)])
def test_bfp8w_matmul_published_to_several_buffers(m, k, n, bfp8_mode):
    """ttlb_matmul_bfp8w_peers: the epilogue stores every tile, whole row segments at a time, into the output region
    of several buffers (on a box with several GPUs: every GPU's copy of a shared output).  Here all buffers live on
    this GPU: each must hold exactly what the plain call gives, and nothing may be written around the regions -
    with the separate unpack kernel and with the expansion inside the mainloop."""
    from ttl_b200 import capi, ops, ttnn
    x = cases.gen((m, k), "normal", 3)
    w = cases.gen((k, n), "normal*0.02", 4, torch.float32)
    W = ttnn.from_torch(w, dtype=ttnn.bfloat8_b)
    X = ttnn.from_torch(x)
    plain = ttnn.to_torch(ops.matmul(X, W))
    pad = 64
    bufs = [torch.full((m + pad, n + pad), 3.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    view = ttnn.Tensor(bufs[0][32:32 + m, 32:32 + n])          # shape and pitch of the output region
    ptrs = [b[32:, 32:].data_ptr() for b in bufs]
    ops.launch_gemm(capi.context(), X, W, view, (0, m, 0, n), capi.current_stream(), peer_ptrs=ptrs)
    capi.context().check_status(capi.current_stream())
    torch.cuda.synchronize()
    for b in bufs:
        got = b.cpu()
        assert torch.equal(got[32:32 + m, 32:32 + n], plain)
        got[32:32 + m, 32:32 + n] = 3.0
        assert (got == 3.0).all(), "the publishing epilogue wrote outside the output region"


def test_default_path_is_one_launch_for_large_outputs_and_two_for_small():
    """The default (`ttlb_set_bfp8_mode` 1): an output with at least one 256x256 tile per SM pair is computed by ONE
    launch that expands the weights inside the GEMM mainloop (no scratch, nothing written but the result); smaller
    outputs take the unpack kernel and the bf16 GEMM.  Same bits either way."""
    from ttl_b200 import capi, ops, ttnn
    ctx = capi.context()
    ctx.set_bfp8_mode(capi.BFP8_MODE_DEFAULT)
    k = 256
    w = cases.gen((k, 6144), "normal*0.02", 5, torch.float32)
    W = ttnn.from_torch(w, dtype=ttnn.bfloat8_b)
    for m, launches in ((1024, 1), (256, 2)):       # 4 x 24 = 96 tiles of 256 x 256 / 1 x 24
        X = ttnn.from_torch(cases.gen((m, k), "normal", 6))
        n0 = ctx.launch_count()
        got = ttnn.to_torch(ops.matmul(X, W))
        assert ctx.launch_count() - n0 == launches
        ctx.set_bfp8_mode(0)
        try:
            assert torch.equal(ttnn.to_torch(ops.matmul(X, W)), got)
        finally:
            ctx.set_bfp8_mode(capi.BFP8_MODE_DEFAULT)


def test_config4_shard_slab(bfp8_mode):
    """configs[3] shapes on one 2048-column stripe (what one of 14 column blocks looks like) with 256
    activation rows checked against the oracle, plus the full 4096 rows for the exact-scaling property."""
    from ttl_b200 import capi, ops, ttnn
    k, n = 8192, 2048
    x = cases.gen((4096, k), "normal", 0)
    w = cases.gen((k, n), "normal*0.02", 1, torch.float32)
    wq = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w.numpy()), k, n))
    W = ttnn.from_torch(w, dtype=ttnn.bfloat8_b)
    got = ttnn.to_torch(ops.matmul(ttnn.from_torch(x), W))
    capi.context().check_status(capi.current_stream())
    assert rel_err(got[:256], tile_oracle.matmul_tiles(x[:256].float(), wq, "f32")) <= 1e-2
    got2 = ttnn.to_torch(ops.matmul(ttnn.from_torch(x * 2), W))
    assert torch.equal(got2, got * 2)


def test_chunked_expansion_overlapping_the_gemm_gives_the_same_bits():
    """The two-step path can expand the weights in column chunks on a side stream under the GEMM of the
    previous chunk (ttlb_set_bfp8_chunks).  Same kernels, so the result must equal the unchunked one bit for bit - also on a second
    call that reuses the scratch buffer while the first may still be running, and with a different matrix."""
    from ttl_b200 import capi, ops, ttnn
    m, k, n = 4096, 256, 8192
    x = cases.gen((m, k), "normal", 20)
    ctx = capi.context()
    ctx.set_bfp8_mode(0)
    outs = {}
    for seed in (21, 22):
        w = cases.gen((k, n), "normal*0.02", seed, torch.float32)
        W = ttnn.from_torch(w, dtype=ttnn.bfloat8_b)
        X = ttnn.from_torch(x)
        for chunks in (4, 1):
            ctx.set_bfp8_chunks(chunks)
            a = ops.matmul(X, W)
            b = ops.matmul(X, W)          # back to back on the same stream
            outs[(seed, chunks)] = (ttnn.to_torch(a), ttnn.to_torch(b))
        ctx.set_bfp8_chunks(1)
        capi.context().check_status(capi.current_stream())
        assert torch.equal(outs[(seed, 4)][0], outs[(seed, 1)][0])
        assert torch.equal(outs[(seed, 4)][1], outs[(seed, 1)][0])
        wq = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w.numpy()), k, n))
        assert rel_err(outs[(seed, 4)][0][:256], tile_oracle.matmul_tiles(x[:256].float(), wq, "f32")) <= 1e-2
    assert not torch.equal(outs[(21, 4)][0], outs[(22, 4)][0])


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("act", ["gelu", "relu"])
def test_quantised_linear_program_with_bias_and_activation(backend, act, bits):
    """Y = act(X @ W + bias) as a tile program with W a bfloat8_b tensor and fp32 intermediates: one launch of
    the unpack kernel and one GEMM launch with the bias row and the activation in its epilogue."""
    _, mods = backend
    import ttnn
    from ttl_b200 import capi
    m, k, n = 128, 256, 192
    x = cases.gen((m, k), "normal", 4)
    w = cases.gen((k, n), "normal*0.02", 5, torch.float32)
    v = cases.gen((1, n), "normal", 6)
    if bits == 8:
        wq = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w.numpy()), k, n))
    else:
        wq = torch.from_numpy(bfp8_oracle.unpack4(bfp8_oracle.pack4(w.numpy()), k, n))
    out = ttnn.from_torch(torch.zeros((m, n), dtype=torch.bfloat16))
    W = ttnn.from_torch(w, dtype=ttnn.bfloat8_b if bits == 8 else ttnn.bfloat4_b)
    prog = mods["matmul"].make_linear(act, fp32_dest_acc_en=True)
    d = prog.plan(ttnn.from_torch(x), W, ttnn.from_torch(v), out).describe()
    assert len(d) == 1 and d[0]["kind"] == f"matmul_bfp{bits}w" and d[0]["act"] == act and d[0]["bias"] == 2
    before = capi.context().launch_count()
    prog(ttnn.from_torch(x), W, ttnn.from_torch(v), out)
    assert capi.context().launch_count() == before + 2     # weight expansion + GEMM
    capi.context().check_status(capi.current_stream())
    want = tile_oracle.UNARY[act](x.float() @ wq + v.float())
    assert rel_err(ttnn.to_torch(out), want) <= 1e-2


def test_config4_as_the_unchanged_tile_program_at_full_size(backend):
    """configs[3] through `@ttl.kernel`: the multicore matmul tile program in 1x1-tile blocks with the weights a
    bfloat8_b tensor [8192, 28672] (29.4 million tile multiply-accumulates, traced with batched loops): one
    weight expansion + one GEMM launch; 256 activation rows of two 1024-column stripes checked against the oracle."""
    import time
    _, mods = backend
    import ttnn
    from ttl_b200 import capi
    m, k, n = 4096, 8192, 28672
    x = cases.gen((m, k), "normal", 0)
    w = cases.gen((k, n), "normal*0.02", 1, torch.float32)
    W = ttnn.from_torch(w, dtype=ttnn.bfloat8_b)
    X = ttnn.from_torch(x)
    out = ttnn.from_torch(torch.zeros((m, n), dtype=torch.bfloat16))
    prog = mods["matmul"].multicore_matmul
    t0 = time.perf_counter()
    plan = prog.plan(X, W, out)
    assert time.perf_counter() - t0 < 10, "trace + recognise of the 4096 x 8192 x 28672 program took too long"
    assert [d["kind"] for d in plan.describe()] == ["matmul_bfp8w"]
    prog(X, W, out)
    capi.context().check_status(capi.current_stream())
    got = ttnn.to_torch(out)
    for c0 in (0, n - 1024):
        stripe = w[:, c0:c0 + 1024].contiguous()
        wq = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(stripe.numpy()), k, 1024))
        for r0 in (0, m - 256):
            want = tile_oracle.matmul_tiles(x[r0:r0 + 256].float(), wq, "f32")
            assert rel_err(got[r0:r0 + 256, c0:c0 + 1024], want) <= 1e-2, (r0, c0)
