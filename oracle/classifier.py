"""CPU restatement of the reference block classifier (test infrastructure).

Follows ``sparseattention/mask_utils.py:14-44`` (``compute_mask_slow``) and the
Triton kernel ``sparseattention/mask_utils.py:47-82``: for every
(batch, head, query block, kv block) tile of the boolean mask,

* ``count == BLOCK_Q*BLOCK_K``  -> the kv-block id is appended to the
  "unmasked" (full) list of the query block,
* ``0 < count < BLOCK_Q*BLOCK_K`` -> appended to the "masked" (partial) list,
* ``count == 0`` -> skipped,

kv-block ids ascending (the reference scans ``k_idx`` serially,
mask_utils.py:66-79).  Only ``ids[..., :len]`` is defined by the reference
(``torch.empty`` outputs, mask_utils.py:91-94); this restatement fills the tail
with -1.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class OracleMetadata:
    unmasked_kv_ids: np.ndarray  # int32 [B,H,nq,nk], tail = -1
    unmasked_lens: np.ndarray    # int32 [B,H,nq]
    masked_kv_ids: np.ndarray    # int32 [B,H,nq,nk], tail = -1
    masked_lens: np.ndarray      # int32 [B,H,nq]


def tile_counts(mask: np.ndarray, block_q: int, block_k: int) -> np.ndarray:
    """Population count of every BLOCK_Q x BLOCK_K tile (mask_utils.py:32-33)."""
    B, H, Sq, Sk = mask.shape
    assert Sq % block_q == 0 and Sk % block_k == 0  # mask_utils.py:19-20
    nq, nk = Sq // block_q, Sk // block_k
    m = np.ascontiguousarray(mask).view(np.uint8) != 0
    return m.reshape(B, H, nq, block_q, nk, block_k).sum(axis=(3, 5), dtype=np.int64)


def classify(mask: np.ndarray, block_q: int, block_k: int) -> OracleMetadata:
    """Vectorised equivalent of ``compute_mask_slow`` (mask_utils.py:14-44)."""
    assert mask.dtype == np.bool_  # mask_utils.py:18
    counts = tile_counts(mask, block_q, block_k)
    B, H, nq, nk = counts.shape
    full = counts == block_q * block_k          # mask_utils.py:34
    part = (counts > 0) & ~full                 # mask_utils.py:37

    def compact(flags):
        # stable ascending compaction of the kv-block ids of each query block
        lens = flags.sum(axis=-1).astype(np.int32)
        order = np.argsort(~flags, axis=-1, kind="stable").astype(np.int32)
        pos = np.arange(nk, dtype=np.int32)
        ids = np.where(pos < lens[..., None], order, np.int32(-1)).astype(np.int32)
        return ids, lens

    f_ids, f_lens = compact(full)
    p_ids, p_lens = compact(part)
    return OracleMetadata(f_ids, f_lens, p_ids, p_lens)


def classify_loops(mask: np.ndarray, block_q: int, block_k: int) -> OracleMetadata:
    """Literal loop nest of mask_utils.py:27-42; for tiny cases only."""
    B, H, Sq, Sk = mask.shape
    nq, nk = Sq // block_q, Sk // block_k
    f_ids = np.full((B, H, nq, nk), -1, np.int32)
    p_ids = np.full((B, H, nq, nk), -1, np.int32)
    f_lens = np.zeros((B, H, nq), np.int32)
    p_lens = np.zeros((B, H, nq), np.int32)
    for b in range(B):
        for h in range(H):
            for i in range(nq):
                nf = npart = 0
                for j in range(nk):
                    c = int(mask[b, h, i * block_q:(i + 1) * block_q, j * block_k:(j + 1) * block_k].sum())
                    if c == block_q * block_k:
                        f_ids[b, h, i, nf] = j
                        nf += 1
                    elif c > 0:
                        p_ids[b, h, i, npart] = j
                        npart += 1
                f_lens[b, h, i] = nf
                p_lens[b, h, i] = npart
    return OracleMetadata(f_ids, f_lens, p_ids, p_lens)


def pack_bits(mask: np.ndarray) -> np.ndarray:
    """Bit-plane the CUDA classifier also emits: uint32 [B,H,Sk/32,Sq], bit j of
    word [b,h,c,r] = mask[b,h,r,32*c+j].  Not part of the reference; it is the
    staged form of the byte mask that mask_utils/sparse_attn_kernel.py:42-46 loads."""
    B, H, Sq, Sk = mask.shape
    assert Sk % 32 == 0
    m = (np.ascontiguousarray(mask).view(np.uint8) != 0).reshape(B, H, Sq, Sk // 32, 32)
    weights = (np.uint64(1) << np.arange(32, dtype=np.uint64))
    words = (m.astype(np.uint64) * weights).sum(axis=-1).astype(np.uint32)  # [B,H,Sq,Sk/32]
    return np.ascontiguousarray(words.transpose(0, 1, 3, 2))
