"""The (batch, head) sharding of the path on two and three CPU ranks (gloo): the partition covers
every unit once, and a sharded run gathered for verification equals the unsharded result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

import workloads
from sparseattention_b200 import sharding


def test_partition_covers_every_unit_once():
    for B, H, world in [(8, 32, 1), (8, 32, 2), (8, 32, 8), (2, 32, 8), (16, 32, 8), (3, 5, 4), (1, 4, 8)]:
        seen = []
        for r in range(world):
            for s in sharding.slabs_of(B, H, r, world):
                assert 0 <= s.b < B and 0 <= s.h0 < s.h1 <= H
                seen += [(s.b, h) for h in range(s.h0, s.h1)]
        assert sorted(seen) == [(b, h) for b in range(B) for h in range(H)]
        sizes = [sum(s.h1 - s.h0 for s in sharding.slabs_of(B, H, r, world)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1
    # whole batch elements when B is a multiple of the world size
    assert sharding.slabs_of(16, 32, 3, 8) == [sharding.Slab(6, 0, 32), sharding.Slab(7, 0, 32)]
    # heads of one batch element split when B < world
    assert sharding.slabs_of(2, 32, 5, 8) == [sharding.Slab(1, 8, 16)]
    with pytest.raises(ValueError):
        sharding.unit_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_attention(q, k, v, mask, bq, bk):
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask)


def _worker(rank, world, port, B, H, S, D, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v = workloads.make_qkv(B, H, S, D, torch.float32, seed=3)
        mask = workloads.random_block_mask(B, S, 0.5, 0.2, seed=4)
        local = sharding.sharded_forward(q, k, v, mask, 32, 32, rank, world, attention=_cpu_attention)
        full = sharding.gather_outputs(local, B, H)
        want = _cpu_attention(q, k, v, mask, 32, 32)
        ok = torch.allclose(full, want, atol=1e-6) and sum(o.shape[1] for _, o in local) in (
            (B * H) // world, (B * H) // world + 1)
        ret[rank] = bool(ok)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,B,H", [(2, 2, 4), (2, 1, 4), (3, 2, 5)])
def test_sharded_run_matches_unsharded(world, B, H):
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, B, H, 64, 16, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
