"""Sharding a recognised tile program over the GPUs of one box (one process per GPU).

The reference is single-chip: its only parallelism is splitting output tiles over the core grid
with `split_work_to_cores` (python/sim/ttnnsim.py:583-752), where the first `remainder` workers get
one unit more.  The same rule splits output row tiles (matmul), weight column tiles (bfp8-weight
matmul) or heads (attention) over ranks.  Each rank computes its shard with the single-GPU kernels;
no kernel reads another GPU's memory.  The only exchange is the final gather of the output shards
(NCCL all-gather over NVLink into this GPU's own HBM), followed by a local re-layout when the shards
are not contiguous in the full output (column shards, head shards).
"""

from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def split_units(n_units: int, world: int) -> List[Tuple[int, int]]:
    """(start, count) per rank: contiguous ranges, the first n_units % world ranks get one more."""
    if world <= 0:
        raise ValueError("world must be positive")
    base, rem = divmod(n_units, world)
    out, start = [], 0
    for r in range(world):
        c = base + (1 if r < rem else 0)
        out.append((start, c))
        start += c
    return out


def _world(group: Optional[dist.ProcessGroup]) -> Tuple[int, int]:
    if not dist.is_available() or not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def gather_shards(local: torch.Tensor, counts: List[int], dim: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather shards that differ only in their size along `dim` (counts[r] for rank r) and
    concatenate them along `dim`.  Shards are padded to the largest count for the collective."""
    rank, world = _world(group)
    if world == 1:
        return local
    if len(counts) != world or local.shape[dim] != counts[rank]:
        raise ValueError(f"rank {rank}: shard has {local.shape[dim]} units along dim {dim}, expected {counts[rank]}")
    mx = max(counts)
    moved = local.movedim(dim, 0).contiguous()
    if moved.shape[0] < mx:
        pad = torch.zeros((mx - moved.shape[0],) + tuple(moved.shape[1:]), dtype=moved.dtype, device=moved.device)
        moved = torch.cat([moved, pad], 0)
    staging = torch.empty((world * mx,) + tuple(moved.shape[1:]), dtype=moved.dtype, device=moved.device)
    dist.all_gather_into_tensor(staging, moved, group=group)   # concatenated form: rank r at rows [r*mx, (r+1)*mx)
    if all(c == mx for c in counts):
        full = staging
    else:
        full = torch.cat([staging[r * mx:r * mx + counts[r]] for r in range(world)], 0)
    return full.movedim(0, dim).contiguous() if dim != 0 else full


def sharded_matmul(a_rows: torch.Tensor, b: torch.Tensor, m_total: int, compute: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                   group: Optional[dist.ProcessGroup] = None, tile: int = 32) -> torch.Tensor:
    """C = A @ B with A's rows sharded: this rank holds `a_rows` = rows of the tile range
    split_units(m_total / tile, world)[rank]; B is replicated.  Returns the full C on every rank."""
    rank, world = _world(group)
    counts = [c * tile for _, c in split_units(m_total // tile, world)]
    if a_rows.shape[0] != counts[rank]:
        raise ValueError(f"rank {rank}: A shard has {a_rows.shape[0]} rows, expected {counts[rank]}")
    c_local = compute(a_rows, b)
    return gather_shards(c_local, counts, 0, group)


def sharded_matmul_cols(x: torch.Tensor, w_cols, n_total: int, compute: Callable, group: Optional[dist.ProcessGroup] = None,
                        tile: int = 32) -> torch.Tensor:
    """C = X @ W with W's columns sharded (tile columns split_units(n_total / tile, world)[rank]);
    X is replicated.  `compute(x, w_cols)` returns this rank's [M, n_local] block."""
    rank, world = _world(group)
    counts = [c * tile for _, c in split_units(n_total // tile, world)]
    c_local = compute(x, w_cols)
    if c_local.shape[1] != counts[rank]:
        raise ValueError(f"rank {rank}: output shard has {c_local.shape[1]} columns, expected {counts[rank]}")
    return gather_shards(c_local, counts, 1, group)


def sharded_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, h_total: int, compute: Callable,
                      group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Attention with heads sharded: this rank holds [B, h_local, S, D] slices of Q, K, V for the head
    range split_units(h_total, world)[rank].  Returns the full [B, H, S, D] output on every rank."""
    rank, world = _world(group)
    counts = [c for _, c in split_units(h_total, world)]
    if q.shape[1] != counts[rank]:
        raise ValueError(f"rank {rank}: Q shard has {q.shape[1]} heads, expected {counts[rank]}")
    o_local = compute(q, k, v)
    return gather_shards(o_local, counts, 1, group)
