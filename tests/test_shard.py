"""Multi-rank logic of the sharded configs on CPU: two gloo ranks, the CPU oracle as the per-rank
compute, result compared with the unsharded oracle."""

import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def test_split_units():
    from ttl_b200.shard import split_units
    assert split_units(256, 8) == [(32 * r, 32) for r in range(8)]
    assert split_units(10, 4) == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert split_units(2, 4) == [(0, 1), (1, 1), (2, 0), (2, 0)]
    from ttl_b200.shard import cyclic_units, pick_chunks
    assert cyclic_units(16, 2, 1, 2) == [(4, 4), (12, 4)]
    assert cyclic_units(8, 4, 3, 1) == [(6, 2)]
    assert pick_chunks(256, 8) == 2 and pick_chunks(256, 4) == 4 and pick_chunks(6, 2) == 3 and pick_chunks(5, 2) == 0 and pick_chunks(7, 1) == 1
    assert sum(c for _, c in split_units(896, 8)) == 896
    with pytest.raises(ValueError):
        split_units(4, 0)


def _worker(rank, world, port, results):
    for p in (ROOT, ROOT / "tt-lang_b200", ROOT / "tests"):
        sys.path.insert(0, str(p))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cases
        from oracle import attention_oracle, tile_oracle
        from ttl_b200 import shard

        # matmul: rows sharded unevenly (5 row tiles over 2 ranks -> 3 + 2)
        a, b = cases.gen((160, 96), "normal*0.1", 0), cases.gen((96, 64), "normal", 1)
        (s0, c0) = shard.split_units(5, world)[rank]
        full = shard.sharded_matmul(a[s0 * 32:(s0 + c0) * 32], b, 160, lambda x, y: tile_oracle.matmul_tiles(x, y, "f32"))
        ok_mm = torch.equal(full, tile_oracle.matmul_tiles(a, b, "f32"))
        # weight columns sharded (4 column tiles -> 2 + 2)
        w = cases.gen((96, 128), "normal*0.02", 2)
        (s1, c1) = shard.split_units(4, world)[rank]
        full2 = shard.sharded_matmul_cols(a, w[:, s1 * 32:(s1 + c1) * 32], 128, lambda x, y: tile_oracle.matmul_tiles(x, y, "f32"))
        ok_cols = torch.equal(full2, tile_oracle.matmul_tiles(a, w, "f32"))
        # attention: (batch, head) pairs sharded unevenly (3 -> 2 + 1)
        q, k, v = (cases.gen((3 * 64, 128), "normal", s).reshape(3, 64, 128) for s in (3, 4, 5))
        (s2, c2) = shard.split_units(3, world)[rank]
        f = lambda x, y, z: attention_oracle.attention_tiles(x, y, z, True, 128 ** -0.5)
        full3 = shard.sharded_attention(q[s2:s2 + c2], k[s2:s2 + c2], v[s2:s2 + c2], 3, f)
        ok_attn = torch.equal(full3, f(q, k, v))
        # rounds (gather of round c overlaps compute of round c+1): units dealt out cyclically
        a8 = cases.gen((256, 96), "normal*0.1", 6)
        mine = shard.cyclic_units(8, world, rank, 2)
        a_loc = torch.cat([a8[u0 * 32:(u0 + n) * 32] for u0, n in mine])
        ok_mm = ok_mm and torch.equal(shard.sharded_matmul(a_loc, b, 256, lambda x, y: tile_oracle.matmul_tiles(x, y, "f32"), chunks=2),
                                      tile_oracle.matmul_tiles(a8, b, "f32"))
        ok_cols = ok_cols and torch.equal(shard.sharded_matmul_cols(a8, w[:, s1 * 32:(s1 + c1) * 32], 128,
                                                                    lambda x, y: tile_oracle.matmul_tiles(x, y, "f32"), chunks=4),
                                          tile_oracle.matmul_tiles(a8, w, "f32"))
        q4, k4, v4 = (cases.gen((4 * 64, 128), "normal", s).reshape(4, 64, 128) for s in (7, 8, 9))
        mine = shard.cyclic_units(4, world, rank, 2)
        pick = lambda t: torch.cat([t[u0:u0 + n] for u0, n in mine])
        ok_attn = ok_attn and torch.equal(shard.sharded_attention(pick(q4), pick(k4), pick(v4), 4, f, chunks=2), f(q4, k4, v4))
        # a shard of the wrong size is rejected before any collective
        try:
            shard.sharded_matmul(a[:32], b, 160, lambda x, y: x)
            ok_err = False
        except ValueError:
            ok_err = True
        results[rank] = (ok_mm, ok_cols, ok_attn, ok_err)
    finally:
        dist.destroy_process_group()


def test_sharded_configs_on_two_gloo_ranks():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: (True, True, True, True), 1: (True, True, True, True)}
