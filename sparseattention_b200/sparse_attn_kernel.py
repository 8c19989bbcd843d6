"""Stage 2 entry point, mirroring ``sparseattention/sparse_attn_kernel.py:149-185``."""
from __future__ import annotations

import os

import torch

from . import _native
from .mask_utils import MaskMetadata, compute_mask_kernel

_EMPTY_BITS = {}


def _no_bits(device) -> torch.Tensor:
    t = _EMPTY_BITS.get(device)
    if t is None:
        t = torch.empty((0,), dtype=torch.int32, device=device)
        _EMPTY_BITS[device] = t
    return t


def sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, BLOCK_Q, BLOCK_K,
                     mask_metadata: MaskMetadata = None, *, impl: str = "auto", check_status: bool = None):
    """Block-sparse attention forward: ``softmax(q k^T / sqrt(D) + where(mask, 0, -inf)) v``
    computed only over the kv blocks listed in ``mask_metadata`` (built from the mask when
    not given), exactly the call of sparse_attn_kernel.py:149.

    q: ``[B,H,Sq,D]``; k, v: ``[B,H,Sk,D]``; mask: bool, broadcastable to ``[B,H,Sq,Sk]``.
    fp16 / bf16 with D in {64,128}, BLOCK_Q = 128 (or 32 / 64 when the lists are built here rather
    than supplied) and BLOCK_K in {32,64,128} run the TMA + tcgen05 kernel; every other
    combination of fp32 / fp16 / bf16, D in {16,32,64,128} and block sizes that are multiples of
    32 runs the generic CUDA-core kernel.  ``impl``
    ("auto" | "tcgen05" | "simt") forces one of them.  Rows whose mask is all False return 0.

    ``check_status`` (default: the SPARSEATTN_B200_CHECK environment variable) makes the call
    read the kernel's device status word back, which synchronises; by default the call is
    asynchronous like the reference's.
    """
    B, H, Sq, D = q.shape                       # sparse_attn_kernel.py:150
    Sk = k.shape[-2]                            # line 151
    mask = mask.expand(B, H, Sq, Sk)            # line 154
    if check_status is None:
        check_status = os.environ.get("SPARSEATTN_B200_CHECK", "0") not in ("", "0")

    q, k, v = _native._tma_ready(q), _native._tma_ready(k), _native._tma_ready(v)
    impl_id = _native.IMPLS[impl]
    md = mask_metadata
    if md is None and int(BLOCK_Q) in (32, 64) and impl_id != _native.SA_IMPL_SIMT and \
            _native.uses_tcgen05(q, k, v, 128, int(BLOCK_K), True):
        # The tensor-core kernel works on 128 query rows at a time.  With no lists from the caller
        # the classification is done at that height: a 128-row tile is computed when any of its
        # BLOCK_Q-row blocks would be, and the bit plane masks the elements, so the result is the
        # one the finer lists would give.
        BLOCK_Q = 128
    if md is None:                              # lines 157-158
        md = compute_mask_kernel(mask, BLOCK_Q, BLOCK_K)
    bits = getattr(md, "packed_bits", None)
    if bits is None and impl_id != _native.SA_IMPL_SIMT and \
            _native.uses_tcgen05(q, k, v, int(BLOCK_Q), int(BLOCK_K), True):
        # caller-supplied lists without the packed plane: derive the plane from the mask
        bits = _native.classify(mask, int(BLOCK_Q), int(BLOCK_K), with_bits=True)[4]
    if bits is None:
        bits = _no_bits(q.device)

    def lists(t, nd):
        t = t if t.dtype == torch.int32 else t.to(torch.int32)
        return t.expand(*((B, H) + tuple(t.shape[2:]))) if t.dim() == nd else t

    return _native.attn_fwd_op(
        q, k, v, mask, bits,
        lists(md.unmasked_kv_ids, 4), lists(md.unmasked_lens, 3),
        lists(md.masked_kv_ids, 4), lists(md.masked_lens, 3),
        int(BLOCK_Q), int(BLOCK_K), impl_id, bool(check_status))
