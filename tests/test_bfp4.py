"""bfloat4_b (576-byte tiles): the library's CPU packer / unpacker against the independent NumPy oracle, the
ttnn surface, and on the GPU the device unpacker (bit-exact) and the bfp4-weight matmul."""

import numpy as np
import pytest
import torch

import cases
from oracle import bfp8_oracle, tile_oracle


def _rand(shape, seed, scale=0.02):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("shape,scale", [((32, 32), 0.02), ((64, 96), 0.02), ((128, 64), 1.0), ((32, 64), 1e-20), ((32, 32), 1e30)])
def test_pack_matches_oracle_bit_for_bit(shape, scale):
    from ttl_b200 import bfp8
    w = _rand(shape, 7, scale)
    got = bfp8.pack_bfp4_b(w).numpy()
    assert got.size == (shape[0] // 32) * (shape[1] // 32) * 576
    assert np.array_equal(got, bfp8_oracle.pack4(w.numpy()))
    back = bfp8.unpack_bfp4_b(torch.from_numpy(got), *shape).numpy()
    assert np.array_equal(back, bfp8_oracle.unpack4(got, *shape))


def test_quantisation_error_bound_idempotence_and_edges():
    from ttl_b200 import bfp8
    w = _rand((96, 160), 3)
    w[0, :16] = 0.0                                              # an all-zero block
    w[1, :16] = torch.tensor([1.0, -1.0, 1.75, 1.874, 1.876, 1.99, 0.124, 0.126, -0.25, 0.0] + [0.5] * 6)
    p = bfp8.pack_bfp4_b(w)
    u = bfp8.unpack_bfp4_b(p, 96, 160)
    # error <= half a step of the block (step = 2**(E-129)), one step where the magnitude saturates at 7
    blk_max = w.reshape(96, 10, 16).abs().amax(-1, keepdim=True).clamp_min(1e-30)
    step = torch.exp2(torch.floor(torch.log2(blk_max)) - 2)
    err = (u - w).reshape(96, 10, 16).abs()
    saturated = w.reshape(96, 10, 16).abs() >= 7.5 * step
    assert (err[~saturated] <= step.expand_as(err)[~saturated] / 2).all() and (err <= step).all()
    assert torch.equal(bfp8.pack_bfp4_b(u), p), "unpacked values are fixed points of the packer"
    assert torch.equal(u[1, :10], torch.tensor([1.0, -1.0, 1.75, 1.75, 1.75, 1.75, 0.0, 0.25, -0.25, 0.0]))
    with pytest.raises(ValueError):
        bfp8.pack_bfp4_b(torch.full((32, 32), float("inf")))
    with pytest.raises(ValueError):
        bfp8.pack_bfp4_b(torch.zeros(32, 48))


def test_ttnn_surface_and_plan(backend):
    _, mods = backend
    import ttnn
    w = _rand((64, 96), 5)
    t = ttnn.from_torch(w, dtype=ttnn.bfloat4_b)
    assert t.shape == (64, 96) and t.dtype is ttnn.bfloat4_b and repr(t.dtype) == "ttnn.bfloat4_b"
    assert np.array_equal(ttnn.to_torch(t).numpy(), bfp8_oracle.unpack4(bfp8_oracle.pack4(w.numpy()), 64, 96))
    x = ttnn.from_torch(torch.zeros((32, 64), dtype=torch.bfloat16))
    out = ttnn.from_torch(torch.zeros((32, 96), dtype=torch.bfloat16))
    d = mods["matmul"].singlecore_matmul.plan(x, t, out).describe()
    assert len(d) == 1 and d[0]["kind"] == "matmul_bfp4w" and d[0]["k_tiles"] == 2


@pytest.mark.gpu
@pytest.mark.parametrize("k,n,col0,cols", [(64, 96, 0, 96), (128, 256, 64, 128)])
def test_device_unpack_is_bit_exact(k, n, col0, cols):
    from ttl_b200 import bfp8, capi
    w = cases.gen((k, n), "normal*0.02", 1, torch.float32)
    w[0, :16] = torch.tensor([1e-30] * 8 + [3e-39] * 8)            # a block with a tiny exponent
    w[1, :16] = torch.tensor([3e-38, -1.5e-38] + [2e-39] * 14)      # results that are bf16 denormals
    w[2, :16] = torch.tensor([-3e38, 1e38, 2.5e37, -7.0] + [1e30] * 12)   # the largest exponents
    w[3, :16] = 0.0
    tiles = bfp8.pack_bfp4_b(w)
    want = torch.from_numpy(bfp8_oracle.unpack4(bfp8_oracle.pack4(w.numpy()), k, n))[:, col0:col0 + cols]
    out = torch.full((k, cols + 8), 9.0, dtype=torch.bfloat16, device="cuda")
    dev = tiles.cuda()
    capi.context().unpack_bfp4_b(dev.data_ptr(), n // 32, col0 // 32, k, cols, out.data_ptr(), out.stride(0), capi.current_stream())
    torch.cuda.synchronize()
    got = out.cpu()
    assert torch.equal(got[:, :cols].float(), want), "device unpack differs from the oracle"
    assert (got[:, cols:] == 9.0).all(), "unpack wrote outside its window"


@pytest.mark.gpu
def test_matmul_program_with_bfloat4_b_weights(backend):
    """The multicore matmul tile program, unchanged, with B given as a bfloat4_b tensor; and a large shape that
    takes the two-CTA GEMM."""
    _, mods = backend
    import ttnn
    from ttl_b200 import capi, ops
    for (m, k, n), prog in (((128, 256, 192), mods["matmul"].multicore_matmul), ((2048, 1024, 4096), None)):
        x = cases.gen((m, k), "normal", 2)
        w = cases.gen((k, n), "normal*0.02", 3, torch.float32)
        wq = torch.from_numpy(bfp8_oracle.unpack4(bfp8_oracle.pack4(w.numpy()), k, n))
        W = ttnn.from_torch(w, dtype=ttnn.bfloat4_b)
        if prog is not None:
            out = ttnn.from_torch(torch.zeros((m, n), dtype=torch.bfloat16))
            prog(ttnn.from_torch(x), W, out)
        else:
            out = ops.matmul(ttnn.from_torch(x), W)
        capi.context().check_status(capi.current_stream())
        want = tile_oracle.matmul_tiles(x.float(), wq, "f32")
        got = ttnn.to_torch(out).float()
        assert ((got - want).abs().max() / want.abs().max()).item() <= 1e-2
