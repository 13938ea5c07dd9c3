"""bfloat8_b packing on the host (thin wrapper over the library's CPU packer; the byte layout
is documented in csrc/bfp8.cu and include/ttlb200.h)."""

from __future__ import annotations

import torch

from . import capi

TILE_BYTES = 1088


def pack_bfp8_b(x: torch.Tensor) -> torch.Tensor:
    """fp32 [R, C] (multiples of 32) -> uint8 [(R/32)*(C/32)*1088] of bfloat8_b tiles."""
    if x.dim() != 2 or x.shape[0] % 32 or x.shape[1] % 32:
        raise ValueError("bfloat8_b needs a 2-D tensor whose dims are multiples of 32")
    x = x.detach().to(torch.float32).cpu().contiguous()
    out = torch.empty((x.shape[0] // 32) * (x.shape[1] // 32) * TILE_BYTES, dtype=torch.uint8)
    rc = capi.lib().ttlb_pack_bfp8_b(x.data_ptr(), x.shape[0], x.shape[1], out.data_ptr())
    if rc != 0:
        raise ValueError("bfloat8_b packing failed (inf/nan values cannot be represented)")
    return out


def unpack_bfp8_b(tiles: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """uint8 bfloat8_b tiles -> fp32 [rows, cols]."""
    tiles = tiles.cpu().contiguous()
    if tiles.numel() != (rows // 32) * (cols // 32) * TILE_BYTES:
        raise ValueError("tile buffer size does not match rows x cols")
    out = torch.empty((rows, cols), dtype=torch.float32)
    rc = capi.lib().ttlb_unpack_bfp8_b(tiles.data_ptr(), rows, cols, out.data_ptr())
    if rc != 0:
        raise ValueError("bfloat8_b unpacking failed")
    return out


BFP4_TILE_BYTES = 576


def pack_bfp4_b(x: torch.Tensor) -> torch.Tensor:
    """fp32 [R, C] (multiples of 32) -> uint8 [(R/32)*(C/32)*576] of bfloat4_b tiles (layout: csrc/bfp4.cu)."""
    if x.dim() != 2 or x.shape[0] % 32 or x.shape[1] % 32:
        raise ValueError("bfloat4_b needs a 2-D tensor whose dims are multiples of 32")
    x = x.detach().to(torch.float32).cpu().contiguous()
    out = torch.empty((x.shape[0] // 32) * (x.shape[1] // 32) * BFP4_TILE_BYTES, dtype=torch.uint8)
    if capi.lib().ttlb_pack_bfp4_b(x.data_ptr(), x.shape[0], x.shape[1], out.data_ptr()) != 0:
        raise ValueError("bfloat4_b packing failed (inf/nan values cannot be represented)")
    return out


def unpack_bfp4_b(tiles: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """uint8 bfloat4_b tiles -> fp32 [rows, cols]."""
    tiles = tiles.cpu().contiguous()
    if tiles.numel() != (rows // 32) * (cols // 32) * BFP4_TILE_BYTES:
        raise ValueError("tile buffer size does not match rows x cols")
    out = torch.empty((rows, cols), dtype=torch.float32)
    if capi.lib().ttlb_unpack_bfp4_b(tiles.data_ptr(), rows, cols, out.data_ptr()) != 0:
        raise ValueError("bfloat4_b unpacking failed")
    return out
