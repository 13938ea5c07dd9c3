"""bfloat8_b: the library's CPU packer/unpacker against the independent NumPy oracle (no GPU)."""

import numpy as np
import pytest
import torch

from oracle import bfp8_oracle


def _rand(shape, seed, scale=0.02):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale)


@pytest.mark.parametrize("shape,scale", [((32, 32), 0.02), ((64, 96), 0.02), ((128, 64), 1.0), ((32, 64), 1e-20), ((32, 32), 1e30)])
def test_pack_matches_oracle_bit_for_bit(shape, scale):
    from ttl_b200 import bfp8
    w = _rand(shape, 7, scale)
    got = bfp8.pack_bfp8_b(w).numpy()
    assert got.size == (shape[0] // 32) * (shape[1] // 32) * 1088
    assert np.array_equal(got, bfp8_oracle.pack(w.numpy()))
    back = bfp8.unpack_bfp8_b(torch.from_numpy(got), *shape).numpy()
    assert np.array_equal(back, bfp8_oracle.unpack(got, *shape))


def test_quantisation_error_bound_and_idempotence():
    from ttl_b200 import bfp8
    w = _rand((96, 160), 3)
    p = bfp8.pack_bfp8_b(w)
    u = bfp8.unpack_bfp8_b(p, 96, 160)
    # error <= half a step of the block (step = 2**(E-133), E = exponent of the block maximum), except
    # where the magnitude saturates at 127 (a value within half a step of 2**(E-126)): there <= one step
    blk_max = w.reshape(96, 10, 16).abs().amax(-1, keepdim=True)
    step = torch.exp2(torch.floor(torch.log2(blk_max)) - 6)
    err = (u - w).reshape(96, 10, 16).abs()
    saturated = w.reshape(96, 10, 16).abs() >= 127.5 * step
    assert (err[~saturated] <= step.expand_as(err)[~saturated] / 2).all() and (err <= step).all()
    # unpacked values are fixed points of the packer
    assert torch.equal(bfp8.pack_bfp8_b(u), p)


def test_edge_cases():
    from ttl_b200 import bfp8
    w = torch.zeros(32, 32)
    p = bfp8.pack_bfp8_b(w)
    assert int(p.sum()) == 0 and torch.equal(bfp8.unpack_bfp8_b(p, 32, 32), w)
    # one block: large max, tiny others (flush to zero), exact halves (ties to even), saturation
    w = torch.zeros(32, 32)
    w[0, :6] = torch.tensor([1.0, -1.0, 1e-9, 1.9999999, 1.0 + 1 / 128, 1.0 + 3 / 128])
    p = bfp8.pack_bfp8_b(w).numpy()
    assert p[0] == 127                                     # exponent of 1.0
    assert list(p[64:70]) == [64, 0x80 | 64, 0, 127, 64, 66]   # 2.0 saturates to 127; 64.5 -> 64, 65.5 -> 66
    assert np.array_equal(p, bfp8_oracle.pack(w.numpy()))
    # negative zero keeps its sign bit, denormals flush
    w = torch.zeros(32, 32)
    w[0, 0], w[0, 1] = -0.0, 1e-42
    p = bfp8.pack_bfp8_b(w).numpy()
    assert p[64] == 0x80 and p[65] == 0 and p[0] == 0
    with pytest.raises(ValueError):
        bfp8.pack_bfp8_b(torch.full((32, 32), float("inf")))
    with pytest.raises(ValueError):
        bfp8.pack_bfp8_b(torch.zeros(32, 48))


def test_face_and_tile_order():
    """Element (r, c) of the matrix lands where the documented layout says."""
    from ttl_b200 import bfp8
    w = torch.zeros(64, 64)
    w[32 + 17, 32 + 5] = 1.0        # tile (1,1); face 2 (rows 16..31, cols 0..15); face row 1; value 5
    p = bfp8.pack_bfp8_b(w).numpy()
    tile = p[(1 * 2 + 1) * 1088:(1 * 2 + 2) * 1088]
    assert tile[2 * 16 + 1] == 127 and tile[64 + 2 * 256 + 1 * 16 + 5] == 64
    assert tile.sum() == 127 + 64 and p.sum() == 127 + 64


def test_ttnn_from_torch_bfloat8_b_roundtrip(backend):
    import ttnn
    w = _rand((64, 128), 11)
    t = ttnn.from_torch(w, dtype=ttnn.bfloat8_b)
    assert t.shape == (64, 128) and t.dtype is ttnn.bfloat8_b
    assert np.array_equal(ttnn.to_torch(t).numpy(), bfp8_oracle.unpack(bfp8_oracle.pack(w.numpy()), 64, 128))
