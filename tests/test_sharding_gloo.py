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


def _worker(rank, world, port, B, H, S, D, costs, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v = workloads.make_qkv(B, H, S, D, torch.float32, seed=3)
        mask = workloads.random_block_mask(B, S, 0.5, 0.2, seed=4)
        local = sharding.sharded_forward(q, k, v, mask, 32, 32, rank, world, attention=_cpu_attention, costs=costs)
        full = sharding.gather_outputs(local, B, H, costs=costs)
        want = _cpu_attention(q, k, v, mask, 32, 32)
        ok = torch.allclose(full, want, atol=1e-6)
        if costs is None:
            ok = ok and sum(o.shape[1] for _, o in local) in ((B * H) // world, (B * H) // world + 1)
        # the same partition through the rank-local interface (the rank fetches only its own slabs)
        fetched = []

        def fetch(slab):
            fetched.append(slab)
            sl = (slice(slab.b, slab.b + 1), slice(slab.h0, slab.h1))
            return q[sl], k[sl], v[sl], mask[slab.b:slab.b + 1]

        again = sharding.run_slabs(sharding.slabs_of(B, H, rank, world, costs), fetch, 32, 32,
                                   attention=lambda q, k, v, m, bq, bk, mask_metadata=None: _cpu_attention(q, k, v, m, bq, bk),
                                   classify=lambda m, bq, bk: None)
        ok = ok and [s for s, _ in again] == [s for s, _ in local] == fetched
        ok = ok and all(torch.equal(a, b) for (_, a), (_, b) in zip(again, local))
        ret[rank] = bool(ok)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,B,H,costs", [(2, 2, 4, None), (2, 1, 4, None), (3, 2, 5, None),
                                             (3, 1, 2, None),            # more ranks than (batch, head) units
                                             (2, 2, 4, [3.0, 1.0]), (3, 3, 4, [1.0, 5.0, 2.0])])
def test_sharded_run_matches_unsharded(world, B, H, costs):
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, B, H, 64, 16, costs, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_cost_balanced_partition():
    """Cuts by cost: every unit once, contiguous, and every rank within one unit's cost of the mean."""
    import random
    rnd = random.Random(5)
    for B, H, world in [(16, 32, 8), (16, 32, 4), (4, 32, 8), (3, 5, 4), (2, 2, 8)]:
        costs = [rnd.uniform(0.5, 2.0) for _ in range(B)]
        cuts = sharding.balanced_cuts(costs, H, world)
        assert cuts[0] == 0 and cuts[-1] == B * H and all(a <= b for a, b in zip(cuts, cuts[1:]))
        seen = []
        loads = []
        for r in range(world):
            slabs = sharding.slabs_of(B, H, r, world, costs)
            seen += [(s.b, h) for s in slabs for h in range(s.h0, s.h1)]
            loads.append(sum(costs[s.b] * (s.h1 - s.h0) for s in slabs))
        assert seen == [(b, h) for b in range(B) for h in range(H)]
        mean = sum(loads) / world
        assert max(abs(x - mean) for x in loads) <= max(costs) + 1e-9
    assert sharding.balanced_cuts([0.0, 0.0], 4, 2) == [0, 4, 8]          # no cost information: equal counts
