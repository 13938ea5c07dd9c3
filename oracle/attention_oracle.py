"""CPU restatement of the flash-attention tile program.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  PARITY UNPINNED: the reference has no
attention kernel, example or test (README.md:83 names a flash-attention test file that is not in
the tree), so there is nothing of the reference's to pin this against.  `attention_tiles` is the
tile program as it would be written for the simulator - per 32x32-tile-aligned KV block:
S = Q @ K^T * scale (+ causal mask), running row max / row sum in fp32, O = O * alpha + P @ V -
evaluated with torch CPU ops on the bf16 values upcast to fp32 ("fp32 intermediates, bf16 out",
the same convention as the matmul oracle); `attention_plain` is the textbook
softmax(Q K^T * scale + mask) V used to cross-check it.
"""

from __future__ import annotations

import torch


def attention_plain(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, scale: float) -> torch.Tensor:
    qf, kf, vf = q.float(), k.float(), v.float()
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        n = s.shape[-1]
        s = s.masked_fill(torch.ones(n, n, dtype=torch.bool).triu(1), float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), vf).to(q.dtype)


def attention_tiles(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, scale: float,
                    block: int = 128) -> torch.Tensor:
    """Online-softmax attention over KV blocks of `block` keys (a multiple of the 32-row tile)."""
    qf, kf, vf = q.float(), k.float(), v.float()
    seq = q.shape[-2]
    o = torch.zeros_like(qf)
    m = torch.full(qf.shape[:-1] + (1,), float("-inf"))
    l = torch.zeros(qf.shape[:-1] + (1,))
    rows = torch.arange(seq).unsqueeze(-1)
    for j0 in range(0, seq, block):
        j1 = min(j0 + block, seq)
        s = torch.matmul(qf, kf[..., j0:j1, :].transpose(-1, -2)) * scale
        if causal:
            s = s.masked_fill(torch.arange(j0, j1).unsqueeze(0) > rows, float("-inf"))
        m_new = torch.maximum(m, s.amax(dim=-1, keepdim=True))
        # rows that have not seen a visible key yet keep m = -inf; exp(-inf - (-inf)) must not produce NaN
        alpha = torch.where(m == float("-inf"), torch.zeros_like(m), torch.exp(m - m_new))
        p = torch.where(m_new == float("-inf"), torch.zeros_like(s), torch.exp(s - m_new))
        l = l * alpha + p.sum(dim=-1, keepdim=True)
        o = o * alpha + torch.matmul(p, vf[..., j0:j1, :])
        m = m_new
    return (o / l).to(q.dtype)
