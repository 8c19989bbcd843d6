"""The reference's own way of calling the package, with its import lines unchanged
(sparseattention/test_attn.py:11-12 and 36-41): lists built by ``compute_mask_kernel`` on the expanded
mask at the harness's default block sizes (32, 128) and at the ones its sweep uses (128, 32), passed to
``sparse_attention`` as ``mask_metadata``, compared with SDPA the way test_attn.py:51 does."""
import pytest
import torch
from torch.nn import functional as F

from sparseattention.sparse_attn_kernel import sparse_attention
from sparseattention.mask_utils import compute_mask_kernel

import workloads

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("BLOCK_Q,BLOCK_K", [(32, 128), (128, 32)])
def test_reference_harness_calls(native_lib, BLOCK_Q, BLOCK_K):
    B, H, Sq, Sk, D, dtype = 2, 4, 1024, 1024, 128, torch.bfloat16
    torch.manual_seed(1352)
    mask = workloads.random_block_mask(B, Sq, 0.5, 0.1, seed=1352, device="cuda")      # [B,1,Sq,Sk]

    q = torch.randn(B, H, Sq, D, dtype=dtype, device="cuda")
    k = torch.randn(B, H, Sk, D, dtype=dtype, device="cuda")
    v = torch.randn(B, H, Sk, D, dtype=dtype, device="cuda")
    mask_expanded = mask.expand(B, H, Sq, Sk)

    mask_metadata = compute_mask_kernel(mask_expanded, BLOCK_Q, BLOCK_K)

    ref_attn = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
    sparse_attn = sparse_attention(q, k, v, mask_expanded, BLOCK_Q, BLOCK_K, mask_metadata=mask_metadata)

    torch.testing.assert_close(ref_attn, sparse_attn, atol=1e-2, rtol=1e-4)
    # and without metadata (sparse_attn_kernel.py:157-158: stage 1 runs inside the call)
    torch.testing.assert_close(ref_attn, sparse_attention(q, k, v, mask_expanded, BLOCK_Q, BLOCK_K),
                               atol=1e-2, rtol=1e-4)


def test_ops_are_registered_under_the_package_name(native_lib):
    assert hasattr(torch.ops.sparseattention, "classify_mask") and hasattr(torch.ops.sparseattention, "attn_fwd")
    mask = workloads.random_block_mask(1, 256, 0.5, 0.2, seed=3, device="cuda")
    f_ids, f_lens, p_ids, p_lens, bits = torch.ops.sparseattention.classify_mask(mask, 128, 32, True)
    md = compute_mask_kernel(mask, 128, 32)
    assert torch.equal(f_ids, md.unmasked_kv_ids) and torch.equal(p_lens, md.masked_lens)
