"""Seeded synthetic workloads: the boolean attention masks and Q/K/V tensors the
benchmark and the tests run on, plus the FLOP / byte accounting.

The masks stand in for the reference's benchmark generator
(``sparseattention/test_attn.py:17-29`` ``random_blocked_mask``: a three-state
block map -- dropped / kept / internally random -- expanded to ``[B,1,Sq,Sk]``).
Two conventions differ from that script and are deliberate:

* ``drop_p`` here is the probability that a block is DROPPED; the reference's
  ``p`` is the probability that it is KEPT (``rand > 1-p``, test_attn.py:21).
* diagonal blocks are always kept and diagonal elements always True, so no query
  row is empty (the reference's generator can produce empty rows, for which its
  kernel returns NaN).

All block-level draws come from a CPU ``torch.Generator`` so that a (config, seed)
pair names the same block map on every machine; only the element-level Bernoulli
bits of partial blocks are drawn on the target device when it is a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch

MASK_GRANULE = 32  # side of the square blocks the synthetic masks are built from


@dataclass(frozen=True)
class WorkloadConfig:
    name: str
    B: int
    H: int
    S: int
    D: int
    dtype: str                     # "float32" | "bfloat16" | "float16"
    kind: str                      # "random_block" | "document" | "composed"
    drop_ps: Tuple[float, ...] = (0.5,)
    partial_frac: float = 0.1
    doc_len: Tuple[int, int] = (256, 2048)
    mask_batch: Optional[int] = None   # leading mask dim; None -> B
    extra: dict = field(default_factory=dict)


# The five configurations the benchmark definition names.
CONFIGS = {
    "correctness": WorkloadConfig("correctness", 1, 4, 512, 64, "float32", "random_block", (0.5,), 0.1),
    "headline": WorkloadConfig("headline", 8, 32, 4096, 128, "bfloat16", "random_block",
                               (0.0, 0.1, 0.3, 0.5, 0.7, 0.9), 0.1),
    "document": WorkloadConfig("document", 4, 32, 8192, 128, "bfloat16", "document", (0.0,), 0.0, (256, 2048)),
    "composed": WorkloadConfig("composed", 2, 32, 16384, 128, "bfloat16", "composed", (0.2,), 0.0, mask_batch=1),
    "scaling": WorkloadConfig("scaling", 16, 32, 32768, 128, "bfloat16", "document", (0.0,), 0.05, (1024, 8192)),
}

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def torch_dtype(name: str) -> torch.dtype:
    return _TORCH_DTYPES[name]


def _cpu_gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    return g


def _dev_gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def _expand_blocks(block_map: torch.Tensor, granule: int) -> torch.Tensor:
    """[nb, nb] -> [nb*granule, nb*granule] by repetition (test_attn.py:24)."""
    return block_map.repeat_interleave(granule, 0).repeat_interleave(granule, 1)


def _apply_partial_blocks(mask2d: torch.Tensor, partial_blocks: torch.Tensor, granule: int,
                          gen: torch.Generator) -> None:
    """AND Bernoulli(0.5) bits into the blocks flagged in ``partial_blocks`` and
    force their diagonal elements (q == k) True; in place on one [S,S] plane."""
    S = mask2d.shape[0]
    idx = partial_blocks.nonzero()
    if idx.numel() == 0:
        return
    dev = mask2d.device
    ar = torch.arange(granule, device=dev)
    # process in chunks so the temporary stays small for 32768^2 planes
    for start in range(0, idx.shape[0], 65536):
        part = idx[start:start + 65536].to(dev)
        n = part.shape[0]
        bits = torch.rand((n, granule, granule), generator=gen, device=dev) < 0.5
        rows = (part[:, 0] * granule)[:, None, None] + ar[None, :, None]
        cols = (part[:, 1] * granule)[:, None, None] + ar[None, None, :]
        bits = bits | (rows == cols)
        rows = rows.expand(n, granule, granule)
        cols = cols.expand(n, granule, granule)
        mask2d[rows, cols] = mask2d[rows, cols] & bits


def random_block_mask(batch: int, S: int, drop_p: float, partial_frac: float = 0.1, *, seed: int = 0,
                      device="cpu", granule: int = MASK_GRANULE) -> torch.Tensor:
    """``[batch,1,S,S]`` bool, True = attend.  Each granule x granule block is
    dropped with probability ``drop_p`` except diagonal blocks; each kept block is,
    with probability ``partial_frac``, internally Bernoulli(0.5) with its diagonal
    elements forced True."""
    nb = S // granule
    cg = _cpu_gen(seed)
    dg = cg if torch.device(device).type == "cpu" else _dev_gen(seed + 1, device)
    out = torch.empty((batch, 1, S, S), dtype=torch.bool, device=device)
    eye = torch.eye(nb, dtype=torch.bool)
    for b in range(batch):
        keep = (torch.rand((nb, nb), generator=cg) >= drop_p) | eye
        partial = keep & (torch.rand((nb, nb), generator=cg) < partial_frac)
        plane = _expand_blocks(keep.to(device), granule)
        _apply_partial_blocks(plane, partial, granule, dg)
        out[b, 0] = plane
    return out


def document_lengths(S: int, lo: int, hi: int, gen: torch.Generator) -> list:
    """Document lengths uniform in [lo, hi] until S is filled; the last is truncated."""
    lens, total = [], 0
    while total < S:
        n = int(torch.randint(lo, hi + 1, (1,), generator=gen))
        n = min(n, S - total)
        lens.append(n)
        total += n
    return lens


def document_causal_mask(batch: int, S: int, doc_len=(256, 2048), partial_frac: float = 0.0, *, seed: int = 0,
                         device="cpu", granule: int = MASK_GRANULE) -> torch.Tensor:
    """``[batch,1,S,S]``: same-document AND causal.  With ``partial_frac`` > 0 that
    fraction of the non-empty granule blocks is additionally ANDed with
    Bernoulli(0.5) bits (diagonal elements kept)."""
    cg = _cpu_gen(seed)
    dg = cg if torch.device(device).type == "cpu" else _dev_gen(seed + 1, device)
    out = torch.empty((batch, 1, S, S), dtype=torch.bool, device=device)
    pos = torch.arange(S, device=device)
    rows_per_chunk = max(granule, min(S, (1 << 28) // S // granule * granule))
    for b in range(batch):
        lens = document_lengths(S, doc_len[0], doc_len[1], cg)
        doc_id = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).to(device)
        plane = out[b, 0]
        for r0 in range(0, S, rows_per_chunk):
            r1 = min(S, r0 + rows_per_chunk)
            plane[r0:r1] = (doc_id[r0:r1, None] == doc_id[None, :]) & (pos[r0:r1, None] >= pos[None, :])
        if partial_frac > 0:
            nb = S // granule
            # non-empty blocks of a document-causal mask: same test on block corners
            blk_first_doc = doc_id[::granule].cpu()
            blk_last_doc = doc_id[granule - 1::granule].cpu()
            bi = torch.arange(nb)
            nonempty = (bi[:, None] >= bi[None, :]) & (blk_first_doc[:, None] <= blk_last_doc[None, :])
            partial = nonempty & (torch.rand((nb, nb), generator=cg) < partial_frac)
            _apply_partial_blocks(plane, partial, granule, dg)
    return out


def composed_mask(S: int, prefix: int = 1024, window: int = 2048, drop_p: float = 0.2, *, seed: int = 0,
                  device="cpu", granule: int = MASK_GRANULE) -> torch.Tensor:
    """``[1,1,S,S]``: (prefix-LM block of the first ``prefix`` tokens, bidirectional)
    UNION (causal sliding window of width ``window``), INTERSECTED with a random
    granule-block dropout (diagonal blocks kept)."""
    cg = _cpu_gen(seed)
    nb = S // granule
    keep = (torch.rand((nb, nb), generator=cg) >= drop_p) | torch.eye(nb, dtype=torch.bool)
    out = torch.empty((1, 1, S, S), dtype=torch.bool, device=device)
    pos = torch.arange(S, device=device)
    rows_per_chunk = max(granule, min(S, (1 << 28) // S // granule * granule))
    keep_dev = keep.to(device)
    for r0 in range(0, S, rows_per_chunk):
        r1 = min(S, r0 + rows_per_chunk)
        q = pos[r0:r1, None]
        kk = pos[None, :]
        base = ((q < prefix) & (kk < prefix)) | ((q - kk >= 0) & (q - kk < window))
        kb = keep_dev[r0 // granule:(r1 + granule - 1) // granule].repeat_interleave(granule, 0)[: r1 - r0]
        out[0, 0, r0:r1] = base & kb.repeat_interleave(granule, 1)
    return out


def make_mask(cfg: WorkloadConfig, drop_p: Optional[float] = None, *, seed: int = 0, device="cpu",
              batch: Optional[int] = None) -> torch.Tensor:
    """Mask of one configuration; ``batch`` overrides the leading dim (sharded runs)."""
    nb = batch if batch is not None else (cfg.mask_batch if cfg.mask_batch is not None else cfg.B)
    p = cfg.drop_ps[0] if drop_p is None else drop_p
    if cfg.kind == "random_block":
        return random_block_mask(nb, cfg.S, p, cfg.partial_frac, seed=seed, device=device)
    if cfg.kind == "document":
        return document_causal_mask(nb, cfg.S, cfg.doc_len, cfg.partial_frac, seed=seed, device=device)
    if cfg.kind == "composed":
        return composed_mask(cfg.S, drop_p=p, seed=seed, device=device)
    raise ValueError(cfg.kind)


def make_qkv(B: int, H: int, S: int, D: int, dtype: torch.dtype, *, seed: int = 0, device="cpu"):
    """Q, K, V ~ N(0,1) (test_attn.py:33-35), drawn in fp32 on the CPU generator for
    small cases and on the device generator otherwise, then cast."""
    if torch.device(device).type == "cpu" or B * H * S * D <= (1 << 22):
        g = _cpu_gen(seed)
        return tuple(torch.randn((B, H, S, D), generator=g).to(dtype).to(device) for _ in range(3))
    g = _dev_gen(seed, device)
    return tuple(torch.randn((B, H, S, D), generator=g, device=device, dtype=torch.float32).to(dtype)
                 for _ in range(3))


# ----------------------------------------------------------------------------- accounting

def computed_tile_flops(unmasked_lens: torch.Tensor, masked_lens: torch.Tensor, block_q: int, block_k: int,
                        D: int) -> float:
    """FLOPs over non-skipped tiles: 4*D*BQ*BK per listed tile (two GEMMs, 2 flop/MAC),
    summed over every (batch, head, query block)."""
    n = int(unmasked_lens.sum(dtype=torch.int64)) + int(masked_lens.sum(dtype=torch.int64))
    return 4.0 * D * block_q * block_k * n


def dense_flops(B: int, H: int, Sq: int, Sk: int, D: int) -> float:
    """test_attn.py:84."""
    return 4.0 * B * H * Sq * Sk * D


def classifier_bytes(n_unique_slices: int, Sq: int, Sk: int, block_q: int, lens_sum: int) -> float:
    """Algorithmic HBM bytes of stage 1: every unique mask byte read once, every
    listed id written once (4 B), two counts per (slice, query block)."""
    return float(n_unique_slices) * Sq * Sk + 4.0 * lens_sum + 8.0 * n_unique_slices * (Sq // block_q)
