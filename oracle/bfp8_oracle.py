"""NumPy restatement of the bfloat8_b block-float format used by the B200 backend.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  PARITY UNPINNED: the reference contains no
pack/unpack code for bfloat8_b, only the tile size 1088 = 1024 + 64 bytes
(python/ttl/dtype_utils.py:174-175) and a dtype alias (python/ttl/dtype_utils.py:80-83); the byte
format itself belongs to tt-metal, which is not part of the reference checkout (pulled through
tt-mlir, pinned in third-party/tt-mlir.commit).  What is restated here is therefore this build's
own completion of the task's wording - "per 16-element block: shared 8-bit exponent, sign + 7-bit
mantissa per value, 32x32 tile / 16x16 face order":

  tile (tr, tc) of a [R, C] matrix at byte offset (tr * C/32 + tc) * 1088
  face f = 2*(r//16) + (c//16), block = one face row (16 consecutive values of a matrix row)
  bytes [0,64): block exponents E[f*16 + r%16] = max biased fp32 exponent in the block
  bytes [64,1088): value bytes at 64 + f*256 + (r%16)*16 + c%16 = sign<<7 | m,
      m = round_half_even(|x| * 2**(133-E)) saturated at 127;   x ~ (-1)**sign * m * 2**(E-133)

This oracle checks the library's CPU packer and GPU unpacker bit for bit against an independent
implementation; it cannot check compatibility with real Tenstorrent tensors.
"""

from __future__ import annotations

import numpy as np

TILE_BYTES = 1088


def _blocks(x: np.ndarray) -> np.ndarray:
    """[R, C] -> [R/32, C/32, 4 faces, 16 face rows, 16 values] in the storage order."""
    r, c = x.shape
    t = x.reshape(r // 32, 2, 16, c // 32, 2, 16)          # tr, fr_hi, fr, tc, fc_hi, j
    return t.transpose(0, 3, 1, 4, 2, 5).reshape(r // 32, c // 32, 4, 16, 16)


def pack(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.ndim == 2 and x.shape[0] % 32 == 0 and x.shape[1] % 32 == 0
    b = _blocks(x)
    bits = b.view(np.uint32)
    e = ((bits >> 23) & 0xFF).astype(np.int64)
    assert (e != 255).all(), "inf/nan cannot be represented"
    E = e.max(axis=-1, keepdims=True)                        # shared exponent per block
    # exact integer arithmetic on the 24-bit significand: |x| = sig * 2**(e-150), m = sig / 2**(17 + E - e)
    sig = np.where(e == 0, 0, (bits & 0x7FFFFF) | 0x800000).astype(np.int64)
    shift = np.minimum(17 + (E - e), 40)
    q = sig >> shift
    rem = sig & ((np.int64(1) << shift) - 1)
    half = np.int64(1) << (shift - 1)
    m = q + ((rem > half) | ((rem == half) & ((q & 1) == 1)))
    m = np.where(E == 0, 0, np.minimum(m, 127))
    val = ((bits >> 31).astype(np.int64) << 7) | m
    tr, tc = b.shape[:2]
    out = np.zeros((tr, tc, TILE_BYTES), dtype=np.uint8)
    out[:, :, :64] = E.reshape(tr, tc, 64)
    out[:, :, 64:] = val.reshape(tr, tc, 1024)
    return out.reshape(-1)


def unpack(tiles: np.ndarray, rows: int, cols: int) -> np.ndarray:
    tr, tc = rows // 32, cols // 32
    t = np.asarray(tiles, dtype=np.uint8).reshape(tr, tc, TILE_BYTES)
    E = t[:, :, :64].astype(np.int64).reshape(tr, tc, 4, 16, 1)
    v = t[:, :, 64:].astype(np.int64).reshape(tr, tc, 4, 16, 16)
    mag = np.ldexp((v & 0x7F).astype(np.float64), E - 133)
    x = np.where(v & 0x80, -mag, mag).astype(np.float32)
    # back from storage order to matrix order
    x = x.reshape(tr, tc, 2, 2, 16, 16).transpose(0, 2, 4, 1, 3, 5)
    return np.ascontiguousarray(x.reshape(rows, cols))


# --------------------------------------------------------------------------- #
# bfloat4_b: the same structure with 4-bit values (PARITY UNPINNED for the same reason: the reference gives only
# the tile size, 576 = 512 + 64 bytes, python/ttl/dtype_utils.py:178-179).  Completion used by this build:
#   bytes [0,64): block exponents as for bfloat8_b
#   bytes [64,576): 8 bytes per block at 64 + f*128 + (r%16)*8; value j in the low (j even) / high (j odd) nibble
#       of byte j//2; nibble = sign<<3 | m, m = round_half_even(|x| * 2**(129-E)) saturated at 7;
#       x ~ (-1)**sign * m * 2**(E-129)
# --------------------------------------------------------------------------- #
BFP4_TILE_BYTES = 576


def pack4(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.ndim == 2 and x.shape[0] % 32 == 0 and x.shape[1] % 32 == 0
    b = _blocks(x)
    bits = b.view(np.uint32)
    e = ((bits >> 23) & 0xFF).astype(np.int64)
    assert (e != 255).all(), "inf/nan cannot be represented"
    E = e.max(axis=-1, keepdims=True)
    sig = np.where(e == 0, 0, (bits & 0x7FFFFF) | 0x800000).astype(np.int64)
    shift = np.minimum(21 + (E - e), 40)
    q = sig >> shift
    rem = sig & ((np.int64(1) << shift) - 1)
    half = np.int64(1) << (shift - 1)
    m = q + ((rem > half) | ((rem == half) & ((q & 1) == 1)))
    m = np.where(E == 0, 0, np.minimum(m, 7))
    nib = ((bits >> 31).astype(np.int64) << 3) | m                   # [tr, tc, 4, 16, 16]
    byte = nib[..., 0::2] | (nib[..., 1::2] << 4)                    # two values per byte, even index low
    tr, tc = b.shape[:2]
    out = np.zeros((tr, tc, BFP4_TILE_BYTES), dtype=np.uint8)
    out[:, :, :64] = E.reshape(tr, tc, 64)
    out[:, :, 64:] = byte.reshape(tr, tc, 512)
    return out.reshape(-1)


def unpack4(tiles: np.ndarray, rows: int, cols: int) -> np.ndarray:
    tr, tc = rows // 32, cols // 32
    t = np.asarray(tiles, dtype=np.uint8).reshape(tr, tc, BFP4_TILE_BYTES)
    E = t[:, :, :64].astype(np.int64).reshape(tr, tc, 4, 16, 1)
    byte = t[:, :, 64:].astype(np.int64).reshape(tr, tc, 4, 16, 8)
    nib = np.stack([byte & 0xF, byte >> 4], axis=-1).reshape(tr, tc, 4, 16, 16)
    mag = np.ldexp((nib & 7).astype(np.float64), E - 129)
    x = np.where(nib & 8, -mag, mag).astype(np.float32)
    x = x.reshape(tr, tc, 2, 2, 16, 16).transpose(0, 2, 4, 1, 3, 5)
    return np.ascontiguousarray(x.reshape(rows, cols))
