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
from typing import Callable, List, Optional, Sequence, Tuple

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


def _slabs_of_range(start: int, stop: int, H: int) -> List[Slab]:
    out = []
    u = start
    while u < stop:
        b, h0 = divmod(u, H)
        h1 = min(H, h0 + (stop - u))
        out.append(Slab(b, h0, h1))
        u += h1 - h0
    return out


def balanced_cuts(costs: Sequence[float], H: int, world: int) -> List[int]:
    """Cut points of the batch-major (b, h) list for ``world`` ranks such that every rank's summed cost
    is as close to total / world as whole units allow.  ``costs[b]`` is the cost of ONE head of batch
    element b (every head of a batch element walks the same lists, so they cost the same) -- e.g. its
    listed-tile count, or an estimate such as the sum of squared document lengths.  Returns
    ``world + 1`` non-decreasing unit indices starting at 0 and ending at ``B * H``."""
    B = len(costs)
    total = float(sum(costs)) * H
    cuts = [0]
    if total <= 0:
        return [unit_range(B * H, r, world)[0] for r in range(world)] + [B * H]
    prefix = [0.0]
    for c in costs:
        prefix.append(prefix[-1] + float(c) * H)
    for r in range(1, world):
        target = total * r / world
        b = 0
        while b < B - 1 and prefix[b + 1] <= target:      # batch element that holds the target
            b += 1
        per_head = float(costs[b])
        h = int(round((target - prefix[b]) / per_head)) if per_head > 0 else 0
        cuts.append(max(cuts[-1], min(B * H, b * H + max(0, min(H, h)))))
    cuts.append(B * H)
    return cuts


def slabs_of(B: int, H: int, rank: int, world: int, costs: Optional[Sequence[float]] = None) -> List[Slab]:
    """The (batch, head-range) slabs of ``rank``: its contiguous range of the batch-major (b, h) list --
    equal unit counts by default, equal summed cost when per-batch-element ``costs`` are given (masks
    whose batch elements differ in density, e.g. documents of different lengths)."""
    if costs is None:
        start, stop = unit_range(B * H, rank, world)
    else:
        if len(costs) != B:
            raise ValueError("costs must hold one entry per batch element")
        if not (0 <= rank < world):
            raise ValueError("rank must be in [0, world)")
        cuts = balanced_cuts(costs, H, world)
        start, stop = cuts[rank], cuts[rank + 1]
    return _slabs_of_range(start, stop, H)


def _mask_of(mask: torch.Tensor, slab: Slab) -> torch.Tensor:
    mb = mask[slab.b:slab.b + 1] if mask.shape[0] > 1 else mask
    return mb[:, slab.h0:slab.h1] if mb.shape[1] > 1 else mb


def run_slabs(slabs: Sequence[Slab], fetch: Callable, block_q: int, block_k: int,
              attention: Optional[Callable] = None, classify: Optional[Callable] = None,
              events: Optional[list] = None) -> List[Tuple[Slab, torch.Tensor]]:
    """Both stages on rank-local inputs: ``fetch(slab)`` returns this slab's ``(q, k, v, mask)`` with
    q, k, v ``[1, h1-h0, S, D]`` and the mask ``[1, 1 or h1-h0, Sq, Sk]`` (the rank holds nothing of other
    ranks' units).  Each slab's mask planes are classified once (``classify(mask, bq, bk)``, default
    :func:`compute_mask_kernel`), then ``attention(q, k, v, mask, bq, bk, mask_metadata=md)`` runs on the
    lists (default :func:`sparse_attention`).  With ``events`` (a list), three CUDA events per slab --
    start, classified, attended -- are appended to it for per-stage timing."""
    if attention is None:
        from .sparse_attn_kernel import sparse_attention as attention
    if classify is None:
        from .mask_utils import compute_mask_kernel as classify
    outs = []
    for slab in slabs:
        q, k, v, mask = fetch(slab)
        ev = None
        if events is not None:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
        md = classify(mask.expand(q.shape[0], q.shape[1], mask.shape[2], mask.shape[3]), block_q, block_k)
        if ev is not None:
            ev[1].record()
        outs.append((slab, attention(q, k, v, mask, block_q, block_k, mask_metadata=md)))
        if ev is not None:
            ev[2].record()
            events.append((slab, ev))
    return outs


def sharded_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, block_q: int,
                    block_k: int, rank: int, world: int, attention: Optional[Callable] = None,
                    costs: Optional[Sequence[float]] = None) -> List[Tuple[Slab, torch.Tensor]]:
    """Runs the forward path on this rank's slabs of globally-indexed inputs ``[B,H,S,D]`` /
    mask ``[B or 1, H or 1, Sq, Sk]`` and returns ``[(slab, output [1, h1-h0, Sq, D])]``.
    ``attention(q, k, v, mask, block_q, block_k)`` defaults to :func:`sparse_attention` (which classifies
    the slab's mask planes itself)."""
    if attention is None:
        from .sparse_attn_kernel import sparse_attention as attention
    B, H = q.shape[0], q.shape[1]
    outs = []
    for slab in slabs_of(B, H, rank, world, costs):
        sl = (slice(slab.b, slab.b + 1), slice(slab.h0, slab.h1))
        outs.append((slab, attention(q[sl], k[sl], v[sl], _mask_of(mask, slab), block_q, block_k)))
    return outs


def gather_outputs(local: List[Tuple[Slab, torch.Tensor]], B: int, H: int, group=None,
                   device: Optional[torch.device] = None,
                   costs: Optional[Sequence[float]] = None) -> torch.Tensor:
    """Verification only: assembles the full ``[B,H,Sq,D]`` output on every rank with one padded
    ``all_gather`` of the flattened local units.  Ranks exchange only the per-unit shape and dtype; each
    allocates on its own device -- ``device``, else the device of its local outputs, else (a rank that
    owns no unit, ``world > B*H``) its current CUDA device under NCCL or the CPU under gloo."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    sample = local[0][1] if local else None
    mine = None if sample is None else (tuple(sample.shape[2:]), str(sample.dtype).replace("torch.", ""))
    metas = [None] * world
    dist.all_gather_object(metas, mine, group=group)
    known = [m for m in metas if m is not None]
    if not known:
        raise ValueError("no rank holds any output")
    tail, dtype_name = known[0]
    dtype = getattr(torch, dtype_name)
    if device is None:
        if sample is not None:
            device = sample.device
        elif dist.get_backend(group) == "nccl":
            device = torch.device("cuda", torch.cuda.current_device())
        else:
            device = torch.device("cpu")
    if costs is None:
        ranges = [unit_range(B * H, r, world) for r in range(world)]
    else:                                                   # the partition sharded_forward used
        cuts = balanced_cuts(costs, H, world)
        ranges = [(cuts[r], cuts[r + 1]) for r in range(world)]
    max_units = max(e - s for s, e in ranges)
    buf = torch.zeros((max_units,) + tuple(tail), dtype=dtype, device=device)
    n = 0
    for slab, o in local:
        cnt = slab.h1 - slab.h0
        buf[n:n + cnt] = o[0]
        n += cnt
    gathered = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(gathered, buf, group=group)
    full = torch.empty((B * H,) + tuple(tail), dtype=dtype, device=device)
    for r, (s, e) in enumerate(ranges):
        full[s:e] = gathered[r][: e - s]
    return full.reshape((B, H) + tuple(tail))
