"""The allocation-free bfp8-weight matmul, ttlb_matmul_bfp8w_noalloc.

Some users of this library cannot allocate GPU memory at the moment they need a matmul: the serving
process around them has already handed every free byte to its own memory pool, or they sit on a
latency-critical path where cudaMalloc's device synchronisation is not acceptable.  For them the
library keeps a fixed 32 MiB scratch array in its device image, and this entry point uses it
instead of the context's cudaMalloc'ed scratch.  The test calls it through the C ABI twice in a
row, with different shapes and data, so that whatever the first call left in the shared array and
status word would show up in the second, and compares each result with the regular entry point,
ttlb_matmul_bfp8w, within the matmul tolerance used throughout the suite (1e-2 of the largest
magnitude; the two run the same kernels, so in practice the bits agree) and with the CPU oracle.  It also checks that a
weight window larger than the fixed array is refused with a message instead of overrunning it.
This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""

import ctypes

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu
TOL = 1e-2


def rel_err(got, want):
    return ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()


def _desc(capi, x_dev, tiles_dev, out_dev, m, k, n, tile_cols, col0):
    d = capi.GemmBfp8Desc()
    d.a, d.lda = x_dev.data_ptr(), x_dev.stride(0)
    d.b_tiles, d.b_tile_cols, d.b_tile_col0 = tiles_dev.data_ptr(), tile_cols, col0
    d.c, d.ldc = out_dev.data_ptr(), out_dev.stride(0)
    d.m, d.n, d.k = m, n, k
    return d


def test_noalloc_entry_point_matches_regular_one_on_two_calls_in_a_row():
    from ttl_b200 import bfp8, capi
    lib = capi.lib()
    ctx = capi.context()
    stream = capi.current_stream()
    err = ctypes.create_string_buffer(256)
    # second call: larger K, a column window that does not start at 0, different data
    for (m, k, n_total, col0_tiles, n, seed) in ((96, 256, 192, 0, 192, 0), (160, 1024, 512, 4, 320, 7)):
        x = cases.gen((m, k), "normal", seed).cuda()
        w = cases.gen((k, n_total), "normal*0.02", seed + 1, torch.float32)
        tiles = bfp8.pack_bfp8_b(w).cuda()
        want = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        ctx.matmul_bfp8w(_desc(capi, x, tiles, want, m, k, n, n_total // 32, col0_tiles), stream)
        ctx.check_status(stream)
        got = torch.full((m, n), 3.0, dtype=torch.bfloat16, device="cuda")
        rc = lib.ttlb_matmul_bfp8w_noalloc(ctypes.byref(_desc(capi, x, tiles, got, m, k, n, n_total // 32, col0_tiles)),
                                           ctypes.c_void_p(stream), 1, err, len(err))
        assert rc == capi.TTLB_OK, err.value.decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert rel_err(got.cpu(), want.cpu()) <= TOL
        # and against the CPU oracle (dequantised weights, fp32-accumulated tile matmul): a fault shared by both
        # entry points would not show in the comparison above
        from oracle import bfp8_oracle, tile_oracle
        wq = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w.numpy()), k, n_total))[:, col0_tiles * 32:col0_tiles * 32 + n]
        assert rel_err(got.cpu(), tile_oracle.matmul_tiles(x.cpu().float(), wq, "f32")) <= TOL


def test_noalloc_entry_point_rejects_windows_beyond_its_fixed_scratch():
    from ttl_b200 import capi
    lib = capi.lib()
    err = ctypes.create_string_buffer(256)
    x = torch.zeros((32, 8192), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((32, 4096), dtype=torch.bfloat16, device="cuda")
    dummy = torch.zeros(1088, dtype=torch.uint8, device="cuda")   # never read: the call is refused before any launch
    d = _desc(capi, x, dummy, out, 32, 8192, 4096, 128, 0)         # 8192 x 4096 = 32 Mi values > 16 Mi
    rc = lib.ttlb_matmul_bfp8w_noalloc(ctypes.byref(d), None, 0, err, len(err))
    assert rc == capi.TTLB_ERR_UNSUPPORTED
    assert b"exceeds the fixed scratch" in err.value
    d = _desc(capi, x, dummy, out, 32, 8192, 2048, 32, 0)          # column window runs past the packed matrix
    assert lib.ttlb_matmul_bfp8w_noalloc(ctypes.byref(d), None, 0, err, len(err)) == capi.TTLB_ERR_INVALID_ARG
    assert lib.ttlb_matmul_bfp8w_noalloc(None, None, 0, err, len(err)) == capi.TTLB_ERR_INVALID_ARG
