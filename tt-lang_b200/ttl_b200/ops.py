"""Operator-level entry points over the C ABI: used by recognised programs, and directly by
callers that already know which kernel they want (the way a `ttnn` op is called next to a
tt-lang kernel in the reference's examples, e.g. ttnn.multiply in examples/general_broadcast.py:184)."""

from __future__ import annotations

from typing import Any, Optional, Tuple

import torch

from . import capi
from . import ttnn as _ttnn
from .recognize import Unsupported


def _dev2d(t: "_ttnn.Tensor", what: str) -> torch.Tensor:
    x = t._tensor
    if not x.is_cuda:
        raise capi.BackendError(capi.TTLB_ERR_CUDA, f"{what} is not in GPU memory: the B200 backend has no CPU fallback")
    if x.dim() != 2 or x.stride(1) != 1:
        raise Unsupported(f"{what} must be 2-D with unit column stride")
    return x


def launch_gemm(ctx: capi.Context, a: "_ttnn.Tensor", b: "_ttnn.Tensor", out: "_ttnn.Tensor",
                rect: Tuple[int, int, int, int], stream: int, multicast_ptr: Optional[int] = None,
                bias: Optional["_ttnn.Tensor"] = None, act: int = 0, peer_ptrs: Optional[list] = None) -> None:
    """out[r0:r1, c0:c1] = a[r0:r1, :] @ b[:, c0:c1] (+ bias[r0:r1, c0:c1]) (element coordinates).  With
    `multicast_ptr` (the NVLink multicast address of out's element (0, 0)) the result is stored through the
    switch to every GPU of the multicast group instead of through out's own mapping; with `peer_ptrs` (the
    address of out's element (0, 0) in every GPU's copy of the buffer, own copy included) it is stored into each
    of them with ordinary stores."""
    r0, r1, c0, c1 = rect
    if peer_ptrs is not None and multicast_ptr is not None:
        raise ValueError("multicast_ptr and peer_ptrs are alternatives")
    if peer_ptrs is not None:
        multicast_ptr = peer_ptrs[0]     # the descriptor's output pointer; the kernel stores to every entry of peer_ptrs
    if (act or bias is not None) and (multicast_ptr is not None or a._tensor.dtype != torch.bfloat16):
        raise Unsupported("matmul with bias / activation: bfloat16 A, bias and output, own-memory output only")

    def bias_args(xo: torch.Tensor) -> Tuple[int, int]:
        if bias is None:
            return 0, 0
        xc = _dev2d(bias, "bias")
        row_vector = xc.shape[0] == 1 and xo.shape[0] != 1
        if xc.dtype != torch.bfloat16 or (not row_vector and tuple(xc.shape) != tuple(xo.shape)) or xc.shape[1] != xo.shape[1]:
            raise Unsupported("matmul with bias: the bias must be a bfloat16 tensor of the output's shape or one row of it")
        return xc.data_ptr() + ((0 if row_vector else r0 * xc.stride(0)) + c0) * 2, 0 if row_vector else xc.stride(0)

    if b._packed is not None:
        xa, xo = _dev2d(a, "A"), _dev2d(out, "out")
        if xa.dtype != torch.bfloat16 or xo.dtype != torch.bfloat16:
            raise Unsupported("matmul with bfloat8_b weights: bfloat16 activations and output only")
        if not b._packed.is_cuda:
            raise capi.BackendError(capi.TTLB_ERR_CUDA, "weights are not in GPU memory: the B200 backend has no CPU fallback")
        if c0 % 32 or c1 % 32:
            raise Unsupported("bfloat8_b weights are addressed in whole 32-column tiles")
        g = capi.GemmBfp8Desc()
        g.a, g.lda = xa.data_ptr() + r0 * xa.stride(0) * 2, xa.stride(0)
        g.b_tiles, g.b_tile_cols, g.b_tile_col0 = b._packed.data_ptr(), b.shape[1] // 32, c0 // 32
        c_base = xo.data_ptr() if multicast_ptr is None else multicast_ptr
        g.c, g.ldc = c_base + (r0 * xo.stride(0) + c0) * 2, xo.stride(0)
        g.m, g.n, g.k = r1 - r0, c1 - c0, xa.shape[1]
        if b._packed_bits == 4:
            if multicast_ptr is not None:
                raise Unsupported("matmul with bfloat4_b weights: no multicast output")
            ptr, ld = bias_args(xo)
            ctx.matmul_bfp4w_epilogue(g, ptr, ld, act, stream)
        elif bias is not None or act:
            ptr, ld = bias_args(xo)
            ctx.matmul_bfp8w_epilogue(g, ptr, ld, act, stream)
        elif multicast_ptr is None:
            ctx.matmul_bfp8w(g, stream)
        elif peer_ptrs is not None:
            ctx.matmul_bfp8w_peers(g, [p + (r0 * xo.stride(0) + c0) * 2 for p in peer_ptrs], stream)
        else:
            ctx.matmul_bfp8w_multicast(g, stream)
        return
    xa, xb, xo = _dev2d(a, "A"), _dev2d(b, "B"), _dev2d(out, "out")
    if not (xa.dtype == xb.dtype == xo.dtype) or xa.dtype not in (torch.bfloat16, torch.float32):
        raise Unsupported(f"matmul: A, B and the output must all be bfloat16 or all float32 "
                          f"(got {xa.dtype}, {xb.dtype}, {xo.dtype})")
    d = capi.GemmDesc()
    es = xa.element_size()
    d.a, d.lda = xa.data_ptr() + r0 * xa.stride(0) * es, xa.stride(0)
    d.b, d.ldb = xb.data_ptr() + c0 * es, xb.stride(0)
    c_base = xo.data_ptr() if multicast_ptr is None else multicast_ptr
    d.c, d.ldc = c_base + (r0 * xo.stride(0) + c0) * es, xo.stride(0)
    d.m, d.n, d.k = r1 - r0, c1 - c0, xa.shape[1]
    if xa.dtype == torch.float32:
        if multicast_ptr is not None:
            raise Unsupported("multicast output: bfloat16 matmuls only")
        ctx.matmul_f32(d, stream)
    elif peer_ptrs is not None:
        ctx.matmul_bf16_peers(d, [p + (r0 * xo.stride(0) + c0) * es for p in peer_ptrs], stream)
    elif multicast_ptr is not None:
        ctx.matmul_bf16_multicast(d, stream)
    elif bias is not None or act:
        ptr, ld = bias_args(xo)
        if act or ld == 0:
            ctx.matmul_bf16_epilogue(d, ptr, ld, act, stream)
        else:
            ctx.matmul_bf16_bias(d, ptr, ld, stream)
    else:
        ctx.matmul_bf16(d, stream)


def matmul(a: "_ttnn.Tensor", b: "_ttnn.Tensor", out: Optional["_ttnn.Tensor"] = None,
           multicast_ptr: Optional[int] = None, peer_ptrs: Optional[list] = None) -> "_ttnn.Tensor":
    """C = A @ B on the tensor cores (bf16 in, fp32 accumulate, bf16 out).  `multicast_ptr`, `peer_ptrs`: see
    launch_gemm."""
    m, n = a.shape[0], b.shape[1]
    if a.shape[1] != b.shape[0]:
        raise ValueError(f"Incompatible matrix shapes for multiplication: {a.shape} @ {b.shape}")
    if out is None:
        out = _ttnn.empty((m, n), dtype=a._tensor.dtype)
    dev = a._tensor.device.index if a._tensor.is_cuda else None
    launch_gemm(capi.context(dev), a, b, out, (0, m, 0, n), capi.current_stream(dev), multicast_ptr, peer_ptrs=peer_ptrs)
    return out


def attention(q: "_ttnn.Tensor", k: "_ttnn.Tensor", v: "_ttnn.Tensor", causal: bool = True,
              scale: Optional[float] = None, out: Optional["_ttnn.Tensor"] = None,
              multicast_ptr: Optional[int] = None, peer_ptrs: Optional[list] = None) -> "_ttnn.Tensor":
    """Fused attention forward on [B, H, S, D] (or [BH, S, D]) bf16 tensors, D = 128:
    softmax(scale * Q K^T + causal mask) V with fp32 scores and online softmax.  With `multicast_ptr` (the NVLink
    multicast address of out's first element) or `peer_ptrs` (the address of out's first element in every GPU's
    copy of a shared buffer, own copy included) the result is published to all those GPUs from the kernel's
    epilogue instead of being stored through out's own mapping."""
    xq, xk, xv = q._tensor, k._tensor, v._tensor
    for x, name in ((xq, "Q"), (xk, "K"), (xv, "V")):
        if not x.is_cuda:
            raise capi.BackendError(capi.TTLB_ERR_CUDA, f"{name} is not in GPU memory: the B200 backend has no CPU fallback")
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise Unsupported("attention: contiguous bfloat16 tensors only")
    if xq.shape != xk.shape or xq.shape != xv.shape or xq.dim() not in (3, 4):
        raise ValueError(f"attention: Q, K, V must share one [B, H, S, D] shape, got {tuple(xq.shape)}, "
                         f"{tuple(xk.shape)}, {tuple(xv.shape)}")
    seq, hd = xq.shape[-2], xq.shape[-1]
    bh = xq.numel() // (seq * hd) if seq * hd else 0
    if out is None:
        out = _ttnn.Tensor(torch.empty_like(xq))
    xo = out._tensor
    if xo.shape != xq.shape or xo.dtype != torch.bfloat16 or not xo.is_contiguous() or not xo.is_cuda:
        raise ValueError("attention: output must be a contiguous bfloat16 GPU tensor shaped like Q")
    d = capi.AttnDesc()
    d.q, d.k, d.v, d.o = xq.data_ptr(), xk.data_ptr(), xv.data_ptr(), xo.data_ptr()
    d.batch_heads, d.seq, d.head_dim = bh, seq, hd
    d.causal = 1 if causal else 0
    d.scale = float(scale) if scale is not None else float(hd) ** -0.5
    ctx = capi.context(xq.device.index)
    stream = capi.current_stream(xq.device.index)
    if peer_ptrs is not None:
        ctx.attention_peers(d, list(peer_ptrs), stream)
    elif multicast_ptr is not None:
        d.o = multicast_ptr
        ctx.attention_multicast(d, stream)
    else:
        ctx.attention(d, stream)
    return out
