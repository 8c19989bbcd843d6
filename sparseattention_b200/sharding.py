"""Sharding of the forward path over the GPUs of one box.

Every (batch, head) slice of the attention (grid axis 1 of both reference kernels,
``mask_utils.py:60-62`` and ``sparse_attn_kernel.py:94-96``) and every distinct mask plane
of the classifier is independent, so the path shards with no data-path collective: the
flattened, batch-major list of (batch, head) units is cut into ``world`` contiguous ranges.
A rank that owns whole batch elements classifies only their mask planes; when a batch
element is split over ranks, each of them classifies that element's plane.

The only collective here is :func:`gather_outputs`, used to verify a sharded run against
an unsharded one; it is not on the hot path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class Slab:
    """Heads [h0, h1) of batch element b."""
    b: int
    h0: int
    h1: int


def unit_range(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous range of units of ``rank``; the first ``n_units % world`` ranks get one more."""
    if not (0 <= rank < world):
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def slabs_of(B: int, H: int, rank: int, world: int) -> List[Slab]:
    """The (batch, head-range) slabs of ``rank``: its range of the batch-major (b, h) list."""
    start, stop = unit_range(B * H, rank, world)
    out = []
    u = start
    while u < stop:
        b, h0 = divmod(u, H)
        h1 = min(H, h0 + (stop - u))
        out.append(Slab(b, h0, h1))
        u += h1 - h0
    return out


def _mask_of(mask: torch.Tensor, slab: Slab) -> torch.Tensor:
    mb = mask[slab.b:slab.b + 1] if mask.shape[0] > 1 else mask
    return mb[:, slab.h0:slab.h1] if mb.shape[1] > 1 else mb


def sharded_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, block_q: int,
                    block_k: int, rank: int, world: int, attention: Optional[Callable] = None
                    ) -> List[Tuple[Slab, torch.Tensor]]:
    """Runs the forward path on this rank's slabs of globally-indexed inputs ``[B,H,S,D]`` /
    mask ``[B or 1, H or 1, Sq, Sk]`` and returns ``[(slab, output [1, h1-h0, Sq, D])]``.
    ``attention(q, k, v, mask, block_q, block_k)`` defaults to :func:`sparse_attention`."""
    if attention is None:
        from .sparse_attn_kernel import sparse_attention as attention
    B, H = q.shape[0], q.shape[1]
    outs = []
    for slab in slabs_of(B, H, rank, world):
        sl = (slice(slab.b, slab.b + 1), slice(slab.h0, slab.h1))
        outs.append((slab, attention(q[sl], k[sl], v[sl], _mask_of(mask, slab), block_q, block_k)))
    return outs


def gather_outputs(local: List[Tuple[Slab, torch.Tensor]], B: int, H: int, group=None) -> torch.Tensor:
    """Verification only: assembles the full ``[B,H,Sq,D]`` output on every rank with one
    ``all_gather_object``-free exchange (padded ``all_gather`` of the flattened local units)."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    sample = local[0][1] if local else None
    shape = [None]
    if sample is not None:
        shape = [tuple(sample.shape[2:]), sample.dtype, sample.device]
    metas = [None] * world
    dist.all_gather_object(metas, shape, group=group)
    meta = next(m for m in metas if m[0] is not None)
    tail, dtype, device = meta
    if sample is not None:
        device = sample.device
    max_units = max(unit_range(B * H, r, world)[1] - unit_range(B * H, r, world)[0] for r in range(world))
    buf = torch.zeros((max_units,) + tuple(tail), dtype=dtype, device=device)
    n = 0
    for slab, o in local:
        cnt = slab.h1 - slab.h0
        buf[n:n + cnt] = o[0]
        n += cnt
    gathered = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(gathered, buf, group=group)
    full = torch.empty((B * H,) + tuple(tail), dtype=dtype, device=device)
    for r in range(world):
        s, e = unit_range(B * H, r, world)
        full[s:e] = gathered[r][: e - s]
    return full.reshape((B, H) + tuple(tail))
