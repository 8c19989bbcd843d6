"""The (batch, head) sharding with the CUDA kernels behind it: the slabs of every rank of a 2-, 3- and
8-rank partition, run one after the other on one GPU and assembled, equal the unsharded call bit for bit
(every (batch, head) unit is independent: sparseattention/sparse_attn_kernel.py:94-96, mask_utils.py:60-62)."""
import pytest
import torch

import sparseattention_b200 as sa
import workloads
from sparseattention_b200 import sharding

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("world,costs", [(2, None), (3, None), (8, None), (3, "tiles")])
def test_slabs_of_all_ranks_equal_the_unsharded_run(native_lib, world, costs):
    B, H, S, D = 3, 4, 1024, 128
    q, k, v = (t.to(DEV) for t in workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=61))
    mask = workloads.document_causal_mask(B, S, (100, 600), 0.1, seed=62).to(DEV)       # [B,1,S,S]
    whole = sa.sparse_attention(q, k, v, mask, 128, 32, check_status=True)
    if costs == "tiles":                                 # listed tiles per batch element, from the lists
        md = sa.compute_mask_kernel(mask, 128, 32)
        costs = (md.unmasked_lens[:, 0].sum(-1) + md.masked_lens[:, 0].sum(-1)).tolist()
    out = torch.full_like(whole, float("nan"))
    for rank in range(world):
        for slab, o in sharding.sharded_forward(q, k, v, mask, 128, 32, rank, world, costs=costs):
            assert o.shape == (1, slab.h1 - slab.h0, S, D)
            out[slab.b, slab.h0:slab.h1] = o[0]
    assert torch.equal(out, whole)
    # the rank-local interface: stage 1 once per slab, stage 2 on its lists, with per-stage events
    events = []
    out2 = torch.full_like(whole, float("nan"))
    for rank in range(world):
        def fetch(slab):
            sl = (slice(slab.b, slab.b + 1), slice(slab.h0, slab.h1))
            return q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), mask[slab.b:slab.b + 1]
        for slab, o in sharding.run_slabs(sharding.slabs_of(B, H, rank, world, costs), fetch, 128, 32, events=events):
            out2[slab.b, slab.h0:slab.h1] = o[0]
    torch.cuda.synchronize()
    assert torch.equal(out2, whole)
    assert all(ev[0].elapsed_time(ev[2]) > 0 for _, ev in events)
