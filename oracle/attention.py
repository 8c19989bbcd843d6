"""CPU restatement of the reference block-sparse attention forward (test infrastructure).

Two checkers:

* :func:`sdpa_reference` -- ``torch.nn.functional.scaled_dot_product_attention``
  with the boolean mask on the host.  This is the reference's own ground truth
  (``sparseattention/test_attn.py:40``) and the numerical authority: fully
  masked rows come out as 0 there, whereas the reference Triton kernel emits
  NaN for them (author's todo at ``sparse_attn_kernel.py:53``).
* :func:`blocked_reference` -- a numpy restatement of the Triton kernel itself
  (``sparse_attn_kernel.py:72-146`` with the inner loop of lines 10-63): Q tile
  loaded once, running max / sum / accumulator in fp32, loop A over the full
  list without the mask, loop B over the partial list with the mask tile added
  as 0 / -inf, base-2 exponentials with ``sm_scale = D**-0.5 / ln 2``
  (line 152), row sum taken before P is cast to the V dtype (lines 57, 61).
  With ``nan_safe=False`` it reproduces the reference's NaN rows exactly; with
  ``nan_safe=True`` it applies the -inf guard the CUDA kernels use.
"""
from __future__ import annotations

import math

import numpy as np


def sdpa_reference(q, k, v, mask):
    """test_attn.py:40 on host tensors; computed in fp32, returned as fp32 numpy."""
    import torch
    import torch.nn.functional as F

    tq, tk, tv = (torch.as_tensor(np.asarray(x, dtype=np.float32)) if not isinstance(x, torch.Tensor)
                  else x.detach().to("cpu", torch.float32) for x in (q, k, v))
    tm = torch.as_tensor(np.asarray(mask)) if not isinstance(mask, torch.Tensor) else mask.detach().cpu()
    out = F.scaled_dot_product_attention(tq, tk, tv, attn_mask=tm)
    return out.numpy()


def _round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round fp32 values to the storage dtype of V (sparse_attn_kernel.py:61)."""
    if dtype == "float32":
        return x
    if dtype == "float16":
        return x.astype(np.float16).astype(np.float32)
    if dtype == "bfloat16":
        u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
        rounded = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000))
        return rounded.view(np.float32)
    raise ValueError(dtype)


def blocked_reference(q, k, v, mask, meta, block_q, block_k, p_dtype="float32", nan_safe=True):
    """Restatement of sparse_attn_kernel.py:72-146.

    q,k,v: float32 numpy [B,H,S,D] (already holding values representable in the
    storage dtype); mask: bool [B,H,Sq,Sk] (expanded); meta: object with the four
    list fields of ``MaskMetadata`` as numpy arrays.
    """
    B, H, Sq, D = q.shape
    sm_scale = np.float32(D ** -0.5 / math.log(2))  # sparse_attn_kernel.py:152
    nq = Sq // block_q
    out = np.zeros((B, H, Sq, D), np.float32)
    ninf = np.float32(-np.inf)
    for b in range(B):
        for h in range(H):
            for i in range(nq):
                rows = slice(i * block_q, (i + 1) * block_q)
                qt = q[b, h, rows].astype(np.float32)                       # lines 98-101
                m = np.full(block_q, ninf, np.float32)                       # line 103
                l = np.zeros(block_q, np.float32)                            # line 104
                acc = np.zeros((block_q, D), np.float32)                     # line 105
                lists = (
                    (meta.unmasked_kv_ids[b, h, i], int(meta.unmasked_lens[b, h, i]), False),  # lines 107-125
                    (meta.masked_kv_ids[b, h, i], int(meta.masked_lens[b, h, i]), True),       # lines 127-142
                )
                for ids, n, use_mask in lists:
                    for t in range(n):
                        j = int(ids[t])                                       # line 33
                        cols = slice(j * block_k, (j + 1) * block_k)
                        s = qt @ k[b, h, cols].astype(np.float32).T           # line 40
                        if use_mask:
                            s = s * sm_scale + np.where(mask[b, h, rows, cols], np.float32(0), ninf)  # line 47
                            mij = np.maximum(m, s.max(axis=-1))               # line 48
                        else:
                            mij = np.maximum(m, s.max(axis=-1) * sm_scale)    # line 50
                            s = s * sm_scale                                  # line 51
                        with np.errstate(invalid="ignore"):
                            if nan_safe:
                                ref = np.where(np.isneginf(mij), np.float32(0), mij)
                                p = np.exp2(s - ref[:, None])
                                alpha = np.where(np.isneginf(m), np.float32(1), np.exp2(m - ref))
                            else:
                                p = np.exp2(s - mij[:, None])                 # line 54
                                alpha = np.exp2(m - mij)                      # line 55
                        m = mij                                               # line 56
                        l = l * alpha + p.sum(axis=-1, dtype=np.float32)      # line 57
                        acc = acc * alpha[:, None]                            # line 58
                        acc = acc + _round_to(p.astype(np.float32), p_dtype) @ v[b, h, cols].astype(np.float32)  # line 61
                with np.errstate(invalid="ignore", divide="ignore"):
                    if nan_safe:
                        o = np.where(l[:, None] > 0, acc / np.where(l > 0, l, 1)[:, None], np.float32(0))
                    else:
                        o = acc / l[:, None]                                  # line 144
                out[b, h, rows] = o
    return out


def predicted_nan_rows(mask, meta, block_q, block_k):
    """Rows for which the reference Triton kernel returns NaN: a query block with
    both lists empty (0/0 at sparse_attn_kernel.py:144), or -- when the full list
    is empty -- a row with no True inside the first partial tile processed
    (running max still -inf at lines 54-55)."""
    B, H, Sq, _ = mask.shape
    nq = Sq // block_q
    bad = np.zeros((B, H, Sq), bool)
    for b in range(B):
        for h in range(H):
            for i in range(nq):
                rows = slice(i * block_q, (i + 1) * block_q)
                nf = int(meta.unmasked_lens[b, h, i])
                npart = int(meta.masked_lens[b, h, i])
                if nf == 0 and npart == 0:
                    bad[b, h, rows] = True
                elif nf == 0:
                    j0 = int(meta.masked_kv_ids[b, h, i, 0])
                    bad[b, h, rows] = ~mask[b, h, rows, j0 * block_k:(j0 + 1) * block_k].any(axis=-1)
    return bad
