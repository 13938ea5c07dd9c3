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


def cyclic_units(n_units: int, world: int, rank: int, chunks: int) -> List[Tuple[int, int]]:
    """Unit ranges (start, count) owned by `rank` when the units are dealt out in `chunks` rounds:
    round c hands units [c*world*uc + r*uc, +uc) to rank r (uc = n_units / (world*chunks)).  The shards
    of one round are then contiguous in the full output, so each round's all-gather writes straight into
    it, and round c's gather overlaps round c+1's compute.  chunks == 1 is the plain contiguous split."""
    if n_units % (world * chunks):
        raise ValueError(f"{n_units} units do not divide into {world} ranks x {chunks} rounds")
    uc = n_units // (world * chunks)
    return [((c * world + rank) * uc, uc) for c in range(chunks)]


def pick_chunks(n_units: int, world: int, want: int = 4) -> int:
    """Largest number of rounds <= want that divides the units evenly (0: not even one).  With many
    ranks the per-round pieces get small and per-copy overheads add up, so fewer rounds are asked for."""
    if world <= 1:
        return 1
    if world >= 8:
        want = min(want, 2)
    for c in range(want, 0, -1):
        if n_units % (world * c) == 0:
            return c
    return 0


def _pipelined_gather(local_chunks: int, out: torch.Tensor, compute_chunk: Callable[[int], torch.Tensor],
                      group: Optional[dist.ProcessGroup]) -> torch.Tensor:
    """Round c: compute this rank's piece, then start the all-gather of that round (async, on NCCL's
    stream) while the next round computes.  `out` is [chunks * world * rows_per_piece, ...]."""
    _, world = _world(group)
    per_round = out.shape[0] // local_chunks
    handles, keep = [], []
    for c in range(local_chunks):
        piece = compute_chunk(c)
        keep.append(piece)
        handles.append(dist.all_gather_into_tensor(out[c * per_round:(c + 1) * per_round], piece.contiguous(),
                                                   group=group, async_op=True))
    for h in handles:
        h.wait()
    return out


def sharded_matmul(a_rows: torch.Tensor, b: torch.Tensor, m_total: int, compute: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                   group: Optional[dist.ProcessGroup] = None, tile: int = 32, chunks: int = 1) -> torch.Tensor:
    """C = A @ B with A's row tiles sharded; B is replicated.  `a_rows` holds this rank's rows, round
    after round, for the unit ranges cyclic_units(m_total / tile, world, rank, chunks) (chunks == 1: one
    contiguous range, the first m % world ranks one tile more).  Returns the full C on every rank."""
    rank, world = _world(group)
    if world == 1:
        return compute(a_rows, b)
    if chunks >= 1 and (m_total // tile) % (world * chunks) == 0:
        mc = m_total // (world * chunks)
        if a_rows.shape[0] != mc * chunks:
            raise ValueError(f"rank {rank}: A shard has {a_rows.shape[0]} rows, expected {mc * chunks}")
        out = torch.empty((m_total, b.shape[1]), dtype=a_rows.dtype, device=a_rows.device)
        return _pipelined_gather(chunks, out, lambda c: compute(a_rows[c * mc:(c + 1) * mc], b), group)
    counts = [c * tile for _, c in split_units(m_total // tile, world)]
    if a_rows.shape[0] != counts[rank]:
        raise ValueError(f"rank {rank}: A shard has {a_rows.shape[0]} rows, expected {counts[rank]}")
    return gather_shards(compute(a_rows, b), counts, 0, group)


def sharded_matmul_cols(x: torch.Tensor, w_cols, n_total: int, compute: Callable, group: Optional[dist.ProcessGroup] = None,
                        tile: int = 32, chunks: int = 1) -> torch.Tensor:
    """C = X @ W with W's column tiles sharded (split_units(n_total / tile, world)[rank]); X is replicated.
    `compute(x_rows, w_cols)` returns this rank's [rows, n_local] block.  With chunks > 1 the rows of X are
    processed in rounds so that the gather of one round overlaps the next round's compute; the gathered
    [world, rows, n_local] pieces are interleaved into C by one strided copy per round."""
    rank, world = _world(group)
    if world == 1:
        return compute(x, w_cols)
    counts = [c * tile for _, c in split_units(n_total // tile, world)]
    m = x.shape[0]
    if chunks >= 1 and len(set(counts)) == 1 and m % chunks == 0:
        nl, mc = counts[0], m // chunks
        out = torch.empty((m, n_total), dtype=x.dtype, device=x.device)
        staging = torch.empty((chunks, world, mc, nl), dtype=x.dtype, device=x.device)
        handles, keep = [], []
        for c in range(chunks):
            piece = compute(x[c * mc:(c + 1) * mc], w_cols)
            if piece.shape != (mc, nl):
                raise ValueError(f"rank {rank}: output shard is {tuple(piece.shape)}, expected {(mc, nl)}")
            keep.append(piece)
            handles.append(dist.all_gather_into_tensor(staging[c].view(world * mc, nl), piece.contiguous(), group=group,
                                                       async_op=True))
        for c, h in enumerate(handles):
            h.wait()
            out[c * mc:(c + 1) * mc].view(mc, world, nl).copy_(staging[c].permute(1, 0, 2))
        return out
    c_local = compute(x, w_cols)
    if c_local.shape[1] != counts[rank]:
        raise ValueError(f"rank {rank}: output shard has {c_local.shape[1]} columns, expected {counts[rank]}")
    return gather_shards(c_local, counts, 1, group)


def sharded_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, units_total: int, compute: Callable,
                      group: Optional[dist.ProcessGroup] = None, chunks: int = 1) -> torch.Tensor:
    """Attention with the (batch, head) pairs sharded: Q, K, V are [units_local, S, D] slices of the
    flattened [B*H, S, D] tensors for the unit ranges cyclic_units(units_total, world, rank, chunks)
    (heads of one batch entry are independent, so any split of the flattened index is a head split).
    Returns the full [B*H, S, D] output on every rank."""
    rank, world = _world(group)
    if world == 1:
        return compute(q, k, v)
    if chunks >= 1 and units_total % (world * chunks) == 0:
        uc = units_total // (world * chunks)
        if q.shape[0] != uc * chunks:
            raise ValueError(f"rank {rank}: Q shard has {q.shape[0]} heads, expected {uc * chunks}")
        out = torch.empty((units_total,) + tuple(q.shape[1:]), dtype=q.dtype, device=q.device)
        return _pipelined_gather(chunks, out, lambda c: compute(q[c * uc:(c + 1) * uc], k[c * uc:(c + 1) * uc],
                                                                v[c * uc:(c + 1) * uc]), group)
    counts = [c for _, c in split_units(units_total, world)]
    if q.shape[0] != counts[rank]:
        raise ValueError(f"rank {rank}: Q shard has {q.shape[0]} heads, expected {counts[rank]}")
    return gather_shards(compute(q, k, v), counts, 0, group)


class SymmetricOutput:
    """Full-size output buffer that exists at the same place on every rank (torch symmetric memory over
    NVLink peer mappings).  A rank computes its shard straight into its own copy and then `push`es that
    region into every peer's copy with asynchronous peer-to-peer copies on a side stream: the copy engines
    do the gather while the SMs carry on with the next round of compute, instead of an SM-based
    all-gather that has to wait for the persistent GEMM CTAs to leave the SMs.  No kernel of this library
    reads or writes peer memory; `finish` joins the side stream and runs a cross-rank barrier."""

    def __init__(self, shape: Tuple[int, ...], dtype: torch.dtype, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.buf = symm.empty(tuple(shape), dtype=dtype, device=device)
        self.hdl = symm.rendezvous(self.buf, group=self.group)
        self.peers = [self.buf if r == self.rank else self.hdl.get_buffer(r, tuple(shape), dtype)
                      for r in range(self.world)]
        self.side = torch.cuda.Stream(device)

    @property
    def has_multicast(self) -> bool:
        return bool(self.hdl.multicast_ptr)

    def multicast_ptr_of(self, view: torch.Tensor) -> int:
        """Multicast address of element 0 of `view` (a view of this rank's buffer): a store there is
        replicated by the NVSwitch into the same place of every rank's buffer."""
        off = view.data_ptr() - self.buf.data_ptr()
        if not self.hdl.multicast_ptr or off < 0 or off >= self.buf.numel() * self.buf.element_size():
            raise ValueError("not a view of this symmetric buffer, or no multicast support")
        return int(self.hdl.multicast_ptr) + off

    def peer_ptrs_of(self, view: torch.Tensor) -> List[int]:
        """Address of element 0 of `view` (a view of this rank's buffer) in every rank's copy of the buffer, own
        copy first, then the other ranks starting with the next one (so that the ranks do not all write to the
        same GPU at the same moment)."""
        off = view.data_ptr() - self.buf.data_ptr()
        if off < 0 or off >= self.buf.numel() * self.buf.element_size():
            raise ValueError("not a view of this symmetric buffer")
        order = [(self.rank + k) % self.world for k in range(self.world)]
        return [int(self.peers[r].data_ptr()) + off for r in order]

    def barrier(self) -> torch.Tensor:
        self.hdl.barrier()
        return self.buf

    def push(self, index: Tuple[slice, ...]) -> None:
        """Send buf[index], just written on the current stream, to the same place on every peer."""
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev)
            for k in range(1, self.world):   # start with the next rank so that receivers are hit evenly
                r = (self.rank + k) % self.world
                self.peers[r][index].copy_(self.buf[index], non_blocking=True)

    def finish(self) -> torch.Tensor:
        torch.cuda.current_stream().wait_stream(self.side)
        self.hdl.barrier()
        return self.buf


def symmetric_matmul_rows(out: SymmetricOutput, a_rows: torch.Tensor, b: torch.Tensor,
                          compute_into: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], None], chunks: int) -> torch.Tensor:
    """Row-sharded C = A @ B into a SymmetricOutput: round c computes rows [(c*world + rank)*mc, +mc) in
    place and pushes them to the peers while round c+1 computes (unit layout of cyclic_units)."""
    m_total = out.buf.shape[0]
    mc = m_total // (out.world * chunks)
    if a_rows.shape[0] != mc * chunks:
        raise ValueError(f"rank {out.rank}: A shard has {a_rows.shape[0]} rows, expected {mc * chunks}")
    for c in range(chunks):
        r0 = (c * out.world + out.rank) * mc
        compute_into(a_rows[c * mc:(c + 1) * mc], b, out.buf[r0:r0 + mc])
        out.push((slice(r0, r0 + mc),))
    return out.finish()


def symmetric_matmul_cols(out: SymmetricOutput, x: torch.Tensor, w_cols, final: torch.Tensor,
                          compute_into: Callable, chunks: int) -> torch.Tensor:
    """Column-sharded C = X @ W.  `out` is a SymmetricOutput of shape [world, M, n_local]: every rank
    computes its column block into its own contiguous slab (rows of X in `chunks` rounds, each pushed to
    the peers as one contiguous copy while the next round computes); once all slabs have arrived, one
    local strided copy interleaves them into `final` [M, world * n_local]."""
    world, m, n_local = out.buf.shape
    mc = m // chunks
    for c in range(chunks):
        compute_into(x[c * mc:(c + 1) * mc], w_cols, out.buf[out.rank, c * mc:(c + 1) * mc])
        out.push((out.rank, slice(c * mc, (c + 1) * mc)))
    slabs = out.finish()
    final.view(m, world, n_local).copy_(slabs.permute(1, 0, 2))
    return final


def symmetric_attention(out: SymmetricOutput, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                        compute_into: Callable, chunks: int) -> torch.Tensor:
    """(batch, head)-sharded attention into a SymmetricOutput of shape [units_total, S, D]."""
    units_total = out.buf.shape[0]
    uc = units_total // (out.world * chunks)
    if q.shape[0] != uc * chunks:
        raise ValueError(f"rank {out.rank}: Q shard has {q.shape[0]} heads, expected {uc * chunks}")
    for c in range(chunks):
        u0 = (c * out.world + out.rank) * uc
        sl = slice(c * uc, (c + 1) * uc)
        compute_into(q[sl], k[sl], v[sl], out.buf[u0:u0 + uc])
        out.push((slice(u0, u0 + uc),))
    return out.finish()
