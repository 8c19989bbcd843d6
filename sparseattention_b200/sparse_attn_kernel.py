"""Stage 2 entry point, mirroring ``sparseattention/sparse_attn_kernel.py:149-185``."""
from __future__ import annotations

import os
from collections import OrderedDict

import torch

from . import _native
from .mask_utils import MaskMetadata, compute_mask_kernel

_EMPTY_BITS = {}

# Opt-in reuse of stage 1 across calls (``sparse_attention(..., cache=True)``): the lists and the packed
# plane of a mask are kept under the identity of its memory -- address, in-place modification counter
# (shared by all views of the storage), shape, strides, block sizes -- so that every layer of a model
# that attends under the same mask classifies it once (the amortisation the reference's README assumes
# when it quotes stage 2 alone).  An entry holds a reference to the mask tensor: its memory cannot be
# freed and handed to another tensor while the entry lives, so an address can never name a different
# mask.  At most MASK_CACHE_ENTRIES entries, least recently used first out.
MASK_CACHE_ENTRIES = 8
_MASK_CACHE: "OrderedDict[tuple, tuple]" = OrderedDict()


def clear_mask_cache() -> None:
    """Drops every cached ``MaskMetadata`` (and the references to the masks they were made from)."""
    _MASK_CACHE.clear()


def _cache_key(mask: torch.Tensor, block_q: int, block_k: int) -> tuple:
    return (mask.device.type, mask.device.index, mask.data_ptr(), mask._version, tuple(mask.shape),
            tuple(mask.stride()), int(block_q), int(block_k))


def cached_mask_metadata(mask: torch.Tensor, block_q: int, block_k: int) -> MaskMetadata:
    """``compute_mask_kernel(mask, block_q, block_k)``, computed once per (mask memory, version, layout,
    block sizes).  Writing into the mask in place (``mask[...] = ...``, ``mask.logical_and_(...)``)
    changes its version and therefore misses; writes that bypass autograd's version counter (raw pointer
    writes from another library) do not -- call :func:`clear_mask_cache` after those."""
    key = _cache_key(mask, block_q, block_k)
    hit = _MASK_CACHE.get(key)
    if hit is not None:
        _MASK_CACHE.move_to_end(key)
        return hit[0]
    md = compute_mask_kernel(mask, block_q, block_k)
    _MASK_CACHE[key] = (md, mask)
    while len(_MASK_CACHE) > MASK_CACHE_ENTRIES:
        _MASK_CACHE.popitem(last=False)
    return md


def _no_bits(device) -> torch.Tensor:
    t = _EMPTY_BITS.get(device)
    if t is None:
        t = torch.empty((0,), dtype=torch.int32, device=device)
        _EMPTY_BITS[device] = t
    return t


def _distinct(t: torch.Tensor) -> torch.Tensor:
    """The distinct leading planes of a list tensor that may be an expanded view."""
    bu = 1 if (t.shape[0] == 1 or t.stride(0) == 0) else t.shape[0]
    hu = 1 if (t.shape[1] == 1 or t.stride(1) == 0) else t.shape[1]
    return t[:bu, :hu]


def _merged_to_128(md: MaskMetadata, mask: torch.Tensor, block_q: int, block_k: int):
    """Caller-supplied lists for BLOCK_Q = 32 / 64 (test_attn.py:32 builds them at (32, 128)) folded
    into lists for the 128-row tiles of the tensor-core kernel, with a bit plane made from the mask and
    brought in line with the lists, so that the result is the one a walk over the given lists gives.
    None when the lists and the mask are broadcast differently (the generic kernel then runs)."""
    lists = [_distinct(t) for t in (md.unmasked_kv_ids, md.unmasked_lens, md.masked_kv_ids, md.masked_lens)]
    planes = tuple(lists[0].shape[:2])
    if any(tuple(t.shape[:2]) != planes for t in lists):
        return None
    bits = _native.classify(mask, 128, block_k, with_bits=True)[4]          # fresh: it is patched below
    bu, hu = bits.shape[0], bits.shape[1]
    if planes[0] not in (1, bu) or planes[1] not in (1, hu):
        return None
    lists = [t.expand(bu, hu, *t.shape[2:]).to(torch.int32).contiguous() for t in lists]
    f_ids, f_lens, p_ids, p_lens = _native.merge_lists(lists[0], lists[1], lists[2], lists[3],
                                                       block_q, block_k, 128 // block_q, bits)
    B, H, Sq, Sk = mask.shape
    nq, nk = Sq // 128, Sk // block_k
    return MaskMetadata(f_ids.expand(B, H, nq, nk), f_lens.expand(B, H, nq),
                        p_ids.expand(B, H, nq, nk), p_lens.expand(B, H, nq),
                        packed_bits=bits, block_sizes=(128, block_k))


def _pad_rows(t: torch.Tensor, n: int) -> torch.Tensor:
    """``t`` [.., .., S, X] with ``n`` rows of zeros (False) appended along S."""
    return torch.cat([t, t.new_zeros(t.shape[:2] + (n, t.shape[3]))], dim=2)


_SM_COUNT = {}


def _sm_count(device) -> int:
    idx = torch.device(device).index
    idx = torch.cuda.current_device() if idx is None else idx
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, BLOCK_Q, BLOCK_K,
                     mask_metadata: MaskMetadata = None, *, impl: str = "auto", check_status: bool = None,
                     return_lse: bool = False, cache: bool = False, splits: int = None):
    """Block-sparse attention forward: ``softmax(q k^T / sqrt(D) + where(mask, 0, -inf)) v``
    computed only over the kv blocks listed in ``mask_metadata`` (built from the mask when
    not given), exactly the call of sparse_attn_kernel.py:149.

    q: ``[B,H,Sq,D]``; k, v: ``[B,H,Sk,D]``; mask: bool, broadcastable to ``[B,H,Sq,Sk]``.
    fp16 / bf16 with D in {64,128}, BLOCK_Q = 128 (or 32 / 64: lists for those are built, or folded
    from the caller's, at 128 rows) and BLOCK_K in {32,64,128} run the TMA + tcgen05 kernel; every other
    combination of fp32 / fp16 / bf16, D in {16,32,64,128} and block sizes that are multiples of
    32 runs the generic CUDA-core kernel.  ``impl``
    ("auto" | "tcgen05" | "simt") forces one of them.  Rows whose mask is all False return 0.

    ``return_lse=True`` returns ``(out, lse)`` with ``lse`` float32 ``[B,H,Sq]``: the natural-log sum of
    exp of each row's scaled scores over its attended keys (-inf for a row with none) -- what a backward
    pass or a merge of partial attentions needs; the reference does not produce it.

    Gradients: the call is differentiable with respect to q, k and v (``out.backward(...)``; also through
    ``lse``).  The backward pass -- which the reference does not have -- recomputes P from the forward's
    log-sum-exp and walks the same lists (CUDA-core kernels, fp32 math).  With caller-supplied lists for
    BLOCK_Q = 32 / 64 the forward then runs the generic kernel on exactly those lists, so that forward and
    backward see the same tiles.

    ``cache=True`` (with no ``mask_metadata``) keeps the lists and the packed plane of this mask and
    reuses them on every later call that passes the same mask memory, unmodified, with the same block
    sizes (see :func:`cached_mask_metadata`): stage 1 then runs once per mask, not once per layer.

    Few query rows against long key sequences (decoding, a short chunk of queries against a long cache):
    with no ``mask_metadata``, a query length that is not a multiple of 128 is padded to one for the
    tensor-core kernel (zero queries under an all-False mask; the padding rows are cut off again), and when
    the (query block, batch, head) units are fewer than the GPU's SMs every unit's walk over its lists is
    cut into ``splits`` ranges that run side by side and are combined by a second kernel -- the reference
    has no such path.  ``splits=None`` picks the number (about one range per SM, at least 512 keys each);
    ``splits=1`` switches the cutting off.

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
    # a backward pass needs the log-sum-exp of the forward
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    pad_rows = (-Sq) % 128
    if pad_rows and md is None and not needs_grad and impl_id != _native.SA_IMPL_SIMT and q.is_cuda and \
            Sq % int(BLOCK_Q) == 0 and Sk % int(BLOCK_K) == 0 and \
            _native.uses_tcgen05(k[:, :, :128], k, v, 128, int(BLOCK_K), True):   # the padded q is fresh and dense: k stands in
        q = _pad_rows(q, pad_rows)
        BLOCK_Q = 128
        hit = _MASK_CACHE.get(_cache_key(mask, 128, BLOCK_K) + ("padded",)) if cache else None
        if hit is not None:                     # the lists and the padded copy made for this mask memory before
            md, mask = hit[0], hit[2]
        else:
            padded = _pad_rows(_native._distinct_planes(mask), pad_rows).expand(B, H, Sq + pad_rows, Sk)
            if cache:
                md = compute_mask_kernel(padded, 128, BLOCK_K)
                _MASK_CACHE[_cache_key(mask, 128, BLOCK_K) + ("padded",)] = (md, mask, padded)
                while len(_MASK_CACHE) > MASK_CACHE_ENTRIES:
                    _MASK_CACHE.popitem(last=False)
            mask = padded
        cache = False
    else:
        pad_rows = 0
    if md is None and int(BLOCK_Q) in (32, 64) and impl_id != _native.SA_IMPL_SIMT and \
            _native.uses_tcgen05(q, k, v, 128, int(BLOCK_K), True):
        # The tensor-core kernel works on 128 query rows at a time.  With no lists from the caller
        # the classification is done at that height: a 128-row tile is computed when any of its
        # BLOCK_Q-row blocks would be, and the bit plane masks the elements, so the result is the
        # one the finer lists would give.
        BLOCK_Q = 128
    if md is not None and int(BLOCK_Q) in (32, 64) and impl_id != _native.SA_IMPL_SIMT and not needs_grad and \
            _native.uses_tcgen05(q, k, v, 128, int(BLOCK_K), True):
        merged = _merged_to_128(md, mask, int(BLOCK_Q), int(BLOCK_K))
        if merged is not None:
            md, BLOCK_Q = merged, 128
    if md is None:                              # lines 157-158
        md = cached_mask_metadata(mask, BLOCK_Q, BLOCK_K) if cache else compute_mask_kernel(mask, BLOCK_Q, BLOCK_K)
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

    n_splits = 1
    if int(BLOCK_Q) == 128 and impl_id != _native.SA_IMPL_SIMT and (splits is None or int(splits) > 1) and \
            _native.uses_tcgen05(q, k, v, 128, int(BLOCK_K), bits.numel() > 0):
        units = B * H * (q.shape[2] // 128)
        if splits is None:
            # Only for a single query block per (batch, head): the rounding of a split call depends on the
            # number of ranges, and calls on parts of a batch (shards) are to equal the call on the whole.
            sms = _sm_count(q.device)
            # one wave of work items: more ranges than that wait for a second turn on some SM
            n_splits = max(1, min(sms // units, Sk // 512, 64)) if q.shape[2] == 128 else 1
        else:
            n_splits = int(splits)
    elif splits is not None and int(splits) > 1:
        raise NotImplementedError("splits > 1 needs the tensor-core kernel (fp16 / bf16, D 64 or 128, BLOCK_Q 128)")

    out, lse = _native.attn_fwd(
        q, k, v, mask, bits,
        lists(md.unmasked_kv_ids, 4), lists(md.unmasked_lens, 3),
        lists(md.masked_kv_ids, 4), lists(md.masked_lens, 3),
        int(BLOCK_Q), int(BLOCK_K), impl_id, bool(check_status), bool(return_lse or needs_grad), n_splits,
        differentiable=needs_grad)
    if pad_rows:
        out, lse = out[:, :, :Sq], (lse[:, :, :Sq] if lse.numel() else lse)
    return (out, lse) if return_lse else out
