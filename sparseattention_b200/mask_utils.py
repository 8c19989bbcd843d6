"""Stage 1 entry points, mirroring ``sparseattention/mask_utils.py`` of the reference:
``MaskMetadata`` (lines 6-11), ``compute_mask_kernel`` (lines 85-107) and
``compute_mask_slow`` (lines 14-44).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _native


@dataclass
class MaskMetadata:
    """The four tensors of the reference's dataclass (mask_utils.py:6-11), in the same
    order, plus two optional extras that default to ``None``:

    ``packed_bits``  uint32-valued int32 tensor [Bu,Hu,Sk/32,Sq], bit j of word [.,.,c,r] =
                     mask[.,.,r,32c+j]; the Blackwell attention kernel stages partial tiles
                     from it.  When absent, ``sparse_attention`` derives it from the mask.
    ``block_sizes``  the (BLOCK_Q, BLOCK_K) the lists were built for.
    """
    unmasked_kv_ids: torch.Tensor
    unmasked_lens: torch.Tensor
    masked_kv_ids: torch.Tensor
    masked_lens: torch.Tensor
    packed_bits: Optional[torch.Tensor] = None
    block_sizes: Optional[tuple] = None


def compute_mask_kernel(mask: torch.Tensor, BLOCK_Q: int, BLOCK_K: int) -> MaskMetadata:
    """Classifies every BLOCK_Q x BLOCK_K tile of a ``[B,H,Sq,Sk]`` bool mask (True = attend)
    on the GPU and returns, per (batch, head, query block), the ascending kv-block ids of the
    fully-unmasked tiles and of the partially-masked tiles with their counts
    (mask_utils.py:85-107).

    Differences from the reference, all at the edges of its contract: a mask that is an
    expanded view over batch and/or heads (sparse_attn_kernel.py:154, test_attn.py:36) is read
    once per distinct plane and the returned tensors are expanded views of shape
    ``[B,H,nq,nk]`` / ``[B,H,nq]``; list tails beyond the count hold -1 (the reference leaves
    them uninitialised); BLOCK_Q and BLOCK_K must be multiples of 32.
    """
    B, H, Sq, Sk = mask.shape
    assert Sq % BLOCK_Q == 0      # mask_utils.py:89
    assert Sk % BLOCK_K == 0      # mask_utils.py:90
    f_ids, f_lens, p_ids, p_lens, bits = _native.classify(mask, BLOCK_Q, BLOCK_K, with_bits=True)
    nq, nk = Sq // BLOCK_Q, Sk // BLOCK_K
    return MaskMetadata(
        f_ids.expand(B, H, nq, nk), f_lens.expand(B, H, nq),
        p_ids.expand(B, H, nq, nk), p_lens.expand(B, H, nq),
        packed_bits=bits, block_sizes=(BLOCK_Q, BLOCK_K))


def compute_mask_slow(mask: torch.Tensor, BLOCK_Q: int, BLOCK_K: int) -> MaskMetadata:
    """Same result from plain torch ops on whatever device the mask lives on
    (mask_utils.py:14-44); list tails hold -1.  Kept for API parity: nothing in this
    package calls it."""
    B, H, Sq, Sk = mask.shape
    assert mask.dtype == torch.bool
    assert Sq % BLOCK_Q == 0
    assert Sk % BLOCK_K == 0
    nq, nk = Sq // BLOCK_Q, Sk // BLOCK_K
    counts = mask.reshape(B, H, nq, BLOCK_Q, nk, BLOCK_K).sum(dim=(3, 5))
    full = counts == BLOCK_Q * BLOCK_K
    part = (counts > 0) & ~full
    pos = torch.arange(nk, device=mask.device, dtype=torch.int32)

    def compact(flags):
        lens = flags.sum(dim=-1).to(torch.int32)
        order = torch.argsort((~flags).to(torch.int8), dim=-1, stable=True).to(torch.int32)
        ids = torch.where(pos < lens[..., None], order, torch.full_like(order, -1))
        return ids, lens

    f_ids, f_lens = compact(full)
    p_ids, p_lens = compact(part)
    return MaskMetadata(f_ids, f_lens, p_ids, p_lens, block_sizes=(BLOCK_Q, BLOCK_K))
