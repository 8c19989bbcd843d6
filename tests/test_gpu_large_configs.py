"""The document, composed and scaling configurations at their real sequence lengths (a few heads
of one batch element): bit-exact lists against the C oracle, the tcgen05 kernel against the
CUDA-core kernel over every row, and against host SDPA on one head (S = 32768: on four query blocks
of one head, over every key)."""
import numpy as np
import pytest
import torch

import sparseattention_b200 as sa
from oracle import cclassify
import workloads
from _util import assert_close_attn, assert_lists_equal, sdpa_cpu, MAX_ABS_16, MEAN_ABS_16

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _check(mask, S, H, seed, sdpa_head=True, bk=32):
    q, k, v = workloads.make_qkv(1, H, S, 128, torch.bfloat16, seed=seed, device=DEV)
    md = sa.compute_mask_kernel(mask.expand(1, H, S, S), 128, bk)
    ref = cclassify.classify(mask.cpu().numpy(), 128, bk)
    assert_lists_equal(sa.MaskMetadata(md.unmasked_kv_ids[:, :1], md.unmasked_lens[:, :1],
                                       md.masked_kv_ids[:, :1], md.masked_lens[:, :1]), ref, "lists")
    out = sa.sparse_attention(q, k, v, mask, 128, bk, mask_metadata=md, impl="tcgen05", check_status=True)
    simt = sa.sparse_attention(q, k, v, mask, 128, bk, mask_metadata=md, impl="simt", check_status=True)
    d = (out.float() - simt.float()).abs()
    assert not torch.isnan(out.float()).any()
    assert d.max().item() <= MAX_ABS_16 and d.mean().item() <= MEAN_ABS_16
    if sdpa_head:
        want = sdpa_cpu(q[:, :1], k[:, :1], v[:, :1], mask)
        assert_close_attn(out[:, :1], want, torch.bfloat16, "vs SDPA")
    else:
        # host SDPA over every key for a few query blocks spread over the sequence (first, last, and two
        # that straddle document boundaries somewhere in between)
        for blk in (0, S // 128 // 3, 2 * (S // 128) // 3 + 1, S // 128 - 1):
            rows = slice(128 * blk, 128 * (blk + 1))
            want = sdpa_cpu(q[:, :1, rows], k[:, :1], v[:, :1], mask[:, :, rows])
            assert_close_attn(out[:, :1, rows], want, torch.bfloat16, f"vs SDPA, query block {blk}")
    # skipped tiles really are empty: the listed tiles cover every True element
    tiles = int(md.unmasked_lens[0, 0].sum()) + int(md.masked_lens[0, 0].sum())
    return tiles / ((S // 128) * (S // bk))


def test_document_config_S8192(native_lib):
    cfg = workloads.CONFIGS["document"]
    mask = workloads.document_causal_mask(1, cfg.S, cfg.doc_len, cfg.partial_frac, seed=51, device=DEV)
    frac = _check(mask, cfg.S, 4, 51)
    assert 0.02 < frac < 0.3


def test_composed_config_S16384(native_lib):
    cfg = workloads.CONFIGS["composed"]
    mask = workloads.composed_mask(cfg.S, drop_p=0.2, seed=52, device=DEV)       # [1,1,S,S], shared
    frac = _check(mask, cfg.S, 2, 52)
    assert 0.05 < frac < 0.3


def test_scaling_config_S32768(native_lib):
    cfg = workloads.CONFIGS["scaling"]
    mask = workloads.document_causal_mask(1, cfg.S, cfg.doc_len, cfg.partial_frac, seed=53, device=DEV)
    frac = _check(mask, cfg.S, 2, 53, sdpa_head=False)
    assert 0.01 < frac < 0.3
    # the other supported list granularity on the same mask (no host check: lists differ, math must not)
    _check(mask, cfg.S, 1, 54, sdpa_head=False, bk=128)
