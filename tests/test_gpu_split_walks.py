"""Few query rows against long key sequences: walks over the lists cut into ranges that run side by side
(``sa_attn_fwd_splitkv``), and query lengths below 128 padded for the tensor-core kernel.  The reference has
no such path; the authority is host SDPA with the bool mask (test_attn.py:40), and the unsplit kernel."""
import pytest
import torch

import sparseattention_b200 as sa
import workloads
from sparseattention_b200 import _native
from _util import assert_close_attn, sdpa_cpu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(q, k, v, mask, bq, bk, **kw):
    out = sa.sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), mask.to(DEV), bq, bk, check_status=True, **kw)
    torch.cuda.synchronize()
    return out


def _decode_mask(B, Sq, Sk, keep_p, seed):
    """[B,1,Sq,Sk]: kv blocks of 32 kept with probability keep_p, a few elements knocked out of some kept blocks
    (partial blocks), a causal edge over the last Sq keys, and the first block always kept."""
    g = torch.Generator().manual_seed(seed)
    keep = torch.rand((B, 1, 1, Sk // 32), generator=g) < keep_p
    keep[..., 0] = True
    m = keep.repeat_interleave(32, dim=-1).expand(B, 1, Sq, Sk).clone()
    holes = torch.rand((B, 1, Sq, Sk), generator=g) < 0.02
    m &= ~holes
    tri = torch.ones((Sq, Sq), dtype=torch.bool).tril()
    m[..., Sk - Sq:] &= tri
    return m


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Sq,D,bk,splits", [(128, 128, 32, 4), (128, 64, 64, 3), (256, 128, 128, 7), (128, 128, 32, 64)])
def test_split_walks_match_sdpa_and_the_unsplit_kernel(native_lib, dtype, Sq, D, bk, splits):
    """Explicit split counts, among them one that does not divide the number of steps and one larger than it
    (empty ranges): values of SDPA, log-sum-exp of the unsplit call."""
    B, H, Sk = 2, 3, 4096
    q = torch.randn((B, H, Sq, D), generator=torch.Generator().manual_seed(1)).to(dtype)
    k = torch.randn((B, H, Sk, D), generator=torch.Generator().manual_seed(2)).to(dtype)
    v = torch.randn((B, H, Sk, D), generator=torch.Generator().manual_seed(3)).to(dtype)
    mask = _decode_mask(B, Sq, Sk, 0.5, seed=splits)
    ref = sdpa_cpu(q, k, v, mask.expand(B, H, Sq, Sk))
    one, lse_one = _run(q, k, v, mask, 128, bk, splits=1, return_lse=True)
    out, lse = _run(q, k, v, mask, 128, bk, splits=splits, return_lse=True)
    assert out.dtype == dtype and out.shape == q.shape
    assert_close_attn(out, ref, dtype, f"splits={splits}")
    assert_close_attn(out, one.float().cpu(), dtype, f"splits={splits} vs unsplit")
    assert torch.allclose(lse, lse_one, atol=2e-3, rtol=1e-4)


def test_rows_without_keys_and_empty_lists(native_lib):
    """A batch element whose mask is all False (every range empty), rows masked out inside an attended
    block, and a range count far above the number of listed blocks: zeros and -inf, no NaN."""
    B, H, Sq, Sk, D = 2, 2, 128, 2048, 128
    q, k, v = (torch.randn((B, H, s, D), generator=torch.Generator().manual_seed(i)).to(torch.bfloat16)
               for i, s in ((1, Sq), (2, Sk), (3, Sk)))
    mask = _decode_mask(B, Sq, Sk, 0.3, seed=5)
    mask[1] = False
    mask[0, :, 5:9, :] = False
    out, lse = _run(q, k, v, mask, 128, 32, splits=16, return_lse=True)
    assert not torch.isnan(out).any()
    assert torch.all(out[1] == 0) and torch.all(out[0, :, 5:9] == 0)
    assert torch.all(torch.isinf(lse[1])) and torch.all(lse[1] < 0) and torch.all(torch.isinf(lse[0, :, 5:9]))
    assert_close_attn(out, sdpa_cpu(q, k, v, mask.expand(B, H, Sq, Sk)), torch.bfloat16, "empty ranges")


@pytest.mark.parametrize("Sq,bq", [(32, 32), (64, 32), (96, 32), (64, 64), (160, 32)])
def test_short_query_lengths_are_padded_for_the_tensor_core_kernel(native_lib, Sq, bq):
    """Query lengths that are not multiples of 128, no lists from the caller: the call pads to 128 rows, picks
    the number of ranges itself, and returns the caller's rows -- values of SDPA and of the generic kernel."""
    B, H, Sk, D = 1, 4, 8192, 128
    q, k, v = (torch.randn((B, H, s, D), generator=torch.Generator().manual_seed(i)).to(torch.bfloat16)
               for i, s in ((1, Sq), (2, Sk), (3, Sk)))
    mask = _decode_mask(B, Sq, Sk, 0.4, seed=Sq)
    ref = sdpa_cpu(q, k, v, mask.expand(B, H, Sq, Sk))
    out, lse = _run(q, k, v, mask, bq, 32, return_lse=True)
    assert tuple(out.shape) == (B, H, Sq, D) and tuple(lse.shape) == (B, H, Sq)
    assert_close_attn(out, ref, torch.bfloat16, f"padded Sq={Sq}")
    generic, lse_g = _run(q, k, v, mask, bq, 32, impl="simt", return_lse=True)
    assert_close_attn(out, generic.float().cpu(), torch.bfloat16, f"padded Sq={Sq} vs generic kernel")
    assert torch.allclose(lse, lse_g, atol=2e-3, rtol=1e-4)


def test_c_abi_refuses_what_it_cannot_split(native_lib):
    """fp32 has no tensor-core path: SA_ERR_UNSUPPORTED (-2); a workspace that is too small: SA_ERR_WORKSPACE (-3)."""
    lib = _native.load_library()
    assert lib.sa_attn_splitkv_workspace_bytes(_native.SA_DTYPE_BF16, 2, 3, 128, 128, 4) >= \
        4 * 2 * 3 * 128 * (128 * 2 + 4) + 16
    q = torch.randn((1, 1, 128, 64), device=DEV, dtype=torch.float32)
    mask = torch.ones((1, 1, 128, 512), dtype=torch.bool, device=DEV)
    kv = torch.randn((1, 1, 512, 64), device=DEV, dtype=torch.float32)
    with pytest.raises(NotImplementedError):
        sa.sparse_attention(q, kv, kv, mask, 128, 32, splits=2)


def test_cache_keeps_the_padded_mask_and_its_lists(native_lib):
    """``cache=True`` on a short query length: the second call finds the lists (and the padded copy of the
    mask) made by the first; an in-place edit of the caller's mask misses."""
    B, H, Sq, Sk, D = 1, 2, 32, 4096, 128
    q, k, v = (torch.randn((B, H, s, D), generator=torch.Generator().manual_seed(i)).to(torch.bfloat16).to(DEV)
               for i, s in ((1, Sq), (2, Sk), (3, Sk)))
    mask = _decode_mask(B, Sq, Sk, 0.4, seed=3).to(DEV)
    sa.clear_mask_cache()
    first = sa.sparse_attention(q, k, v, mask, 32, 32, cache=True)
    calls = []
    real = sa.sparse_attn_kernel.compute_mask_kernel
    sa.sparse_attn_kernel.compute_mask_kernel = lambda *a, **kw: (calls.append(1), real(*a, **kw))[1]
    try:
        second = sa.sparse_attention(q, k, v, mask, 32, 32, cache=True)
        assert not calls and torch.equal(first, second)
        mask[..., 100:200] = False
        third = sa.sparse_attention(q, k, v, mask, 32, 32, cache=True)
        assert calls
    finally:
        sa.sparse_attn_kernel.compute_mask_kernel = real
        sa.clear_mask_cache()
    ref = sdpa_cpu(q.cpu(), k.cpu(), v.cpu(), mask.cpu().expand(B, H, Sq, Sk))
    assert_close_attn(third, ref, torch.bfloat16, "after the edit")
