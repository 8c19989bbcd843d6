"""The backward pass (no counterpart in the reference, which lists it as future work, README.md:61-65):
gradients of ``sparse_attention`` with respect to q, k, v against ``torch.autograd`` through SDPA with the
bool mask on the host in fp32 -- the forward's own ground truth differentiated."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import sparseattention_b200 as sa
import workloads
from sparseattention_b200 import _native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _reference_grads(q, k, v, mask, w, w_lse=None):
    qf, kf, vf = (t.detach().float().cpu().requires_grad_(True) for t in (q, k, v))
    out = F.scaled_dot_product_attention(qf, kf, vf, attn_mask=mask.cpu())
    loss = (out * w.float().cpu()).sum()
    if w_lse is not None:
        s = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * qf.shape[-1] ** -0.5
        B, H, Sq, Sk = s.shape
        lse = torch.logsumexp(s.masked_fill(~mask.cpu().expand(B, H, Sq, Sk), float("-inf")), dim=-1)
        live = torch.isfinite(lse)
        loss = loss + (torch.where(live, lse, torch.zeros_like(lse)) * w_lse.float().cpu()).sum()
    loss.backward()
    return qf.grad, kf.grad, vf.grad


def _assert_grad_close(got, want, dtype, what):
    got = got.detach().float().cpu()
    assert torch.isfinite(got).all(), f"{what}: non-finite gradient"
    scale = max(1.0, want.abs().max().item())
    diff = (got - want).abs()
    if dtype == torch.float32:
        assert diff.max().item() <= 2e-4 * scale, f"{what}: max-abs {diff.max().item():.3e} (scale {scale:.2f})"
    else:   # gradients are rounded to the 16-bit dtype on the way out: the forward's bound, relative to the largest entry
        assert diff.max().item() <= 2e-2 * scale, f"{what}: max-abs {diff.max().item():.3e} (scale {scale:.2f})"
        assert diff.mean().item() <= 2e-3 * scale, f"{what}: mean-abs {diff.mean().item():.3e}"


@pytest.mark.parametrize("dtype,D,bq,bk", [(torch.bfloat16, 128, 128, 32), (torch.float16, 64, 128, 64),
                                          (torch.float32, 64, 32, 32), (torch.bfloat16, 128, 32, 128)])
def test_gradients_match_autograd_through_sdpa(native_lib, dtype, D, bq, bk):
    B, H, S = 2, 2, 512
    q, k, v = workloads.make_qkv(B, H, S, D, dtype, seed=300 + D + bk)
    mask = workloads.random_block_mask(B, S, 0.5, 0.2, seed=301 + bq)
    mask[0, 0, 7] = False                                    # a row with no attended key: no gradient
    mask[1, 0, 128:256] = False                              # a whole query block with none
    g = torch.Generator().manual_seed(5)
    w = torch.randn((B, H, S, D), generator=g).to(dtype)
    want = _reference_grads(q, k, v, mask, w)
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = sa.sparse_attention(qd, kd, vd, mask.to(DEV), bq, bk, check_status=True)
    out.backward(w.to(DEV))
    torch.cuda.synchronize()
    for name, got, ref in zip(("dq", "dk", "dv"), (qd.grad, kd.grad, vd.grad), want):
        _assert_grad_close(got, ref, dtype, f"{name} {dtype} D={D} ({bq},{bk})")
    assert bool((qd.grad[0, :, 7] == 0).all()) and bool((qd.grad[1, :, 128:256] == 0).all())


def test_gradient_through_lse_and_caller_metadata(native_lib):
    """A loss that also uses the log-sum-exp output, with lists passed in by the caller (stage 1 amortised)."""
    B, H, S, D = 1, 3, 512, 128
    q, k, v = workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=310)
    mask = workloads.document_causal_mask(B, S, (60, 200), 0.1, seed=311)
    g = torch.Generator().manual_seed(6)
    w = torch.randn((B, H, S, D), generator=g).to(torch.bfloat16)
    w_lse = torch.randn((B, H, S), generator=g)
    want = _reference_grads(q, k, v, mask, w, w_lse)
    md = sa.compute_mask_kernel(mask.to(DEV).expand(B, H, S, S), 128, 32)
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out, lse = sa.sparse_attention(qd, kd, vd, mask.to(DEV), 128, 32, mask_metadata=md, return_lse=True)
    loss = (out.float() * w.to(DEV).float()).sum() + (lse * w_lse.to(DEV)).sum()
    loss.backward()
    for name, got, ref in zip(("dq", "dk", "dv"), (qd.grad, kd.grad, vd.grad), want):
        _assert_grad_close(got, ref, torch.bfloat16, name)


def test_shared_kv_heads_gradients_are_summed_over_the_heads(native_lib):
    B, H, S, D = 1, 4, 256, 64
    g = torch.Generator().manual_seed(7)
    q = torch.randn((B, H, S, D), generator=g).to(torch.float16)
    k1 = torch.randn((B, 1, S, D), generator=g).to(torch.float16)
    v1 = torch.randn((B, 1, S, D), generator=g).to(torch.float16)
    w = torch.randn((B, H, S, D), generator=g).to(torch.float16)
    mask = workloads.random_block_mask(B, S, 0.4, 0.2, seed=312)
    dq, dk, dv = _reference_grads(q, k1.expand(B, H, S, D), v1.expand(B, H, S, D), mask, w)
    qd, kd, vd = q.to(DEV).requires_grad_(True), k1.to(DEV).requires_grad_(True), v1.to(DEV).requires_grad_(True)
    out = sa.sparse_attention(qd, kd.expand(B, H, S, D), vd.expand(B, H, S, D), mask.to(DEV), 128, 32)
    out.backward(w.to(DEV))
    _assert_grad_close(qd.grad, dq, torch.float16, "dq")
    _assert_grad_close(kd.grad, dk.sum(1, keepdim=True), torch.float16, "dk summed over heads")
    _assert_grad_close(vd.grad, dv.sum(1, keepdim=True), torch.float16, "dv summed over heads")


def test_transposed_lists(native_lib):
    """kv-major lists: for every kv block the ascending query blocks that list it."""
    mask = workloads.random_block_mask(2, 1024, 0.6, 0.3, seed=313).to(DEV)
    md = sa.compute_mask_kernel(mask, 128, 32)
    planes = [t[:, :1].contiguous() for t in (md.unmasked_kv_ids, md.unmasked_lens, md.masked_kv_ids, md.masked_lens)]
    tf_ids, tf_lens, tp_ids, tp_lens = (t.cpu().numpy() for t in _native.transpose_lists(*planes))
    f_ids, f_lens, p_ids, p_lens = (t.cpu().numpy() for t in planes)
    nq, nk = f_ids.shape[2], f_ids.shape[3]
    for b in range(2):
        for ids, lens, t_ids, t_lens in ((f_ids, f_lens, tf_ids, tf_lens), (p_ids, p_lens, tp_ids, tp_lens)):
            member = np.zeros((nq, nk), dtype=bool)
            for i in range(nq):
                member[i, ids[b, 0, i, :lens[b, 0, i]]] = True
            for j in range(nk):
                want = np.nonzero(member[:, j])[0]
                assert t_lens[b, 0, j] == len(want)
                assert np.array_equal(t_ids[b, 0, j, :len(want)], want)
                assert (t_ids[b, 0, j, len(want):] == -1).all()


def test_backward_op_passes_opcheck(native_lib):
    B, H, S, D = 1, 2, 256, 64
    q, k, v = (t.to(DEV) for t in workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=314))
    mask = workloads.random_block_mask(B, S, 0.5, 0.2, seed=315).to(DEV)
    f_ids, f_lens, p_ids, p_lens, bits = _native.classify(mask, 128, 32)
    ex = lambda t: t.expand(*((B, H) + tuple(t.shape[2:])))
    o, lse = _native.attn_fwd_op(q, k, v, mask.expand(B, H, S, S), bits, ex(f_ids), ex(f_lens), ex(p_ids), ex(p_lens),
                                 128, 32, _native.SA_IMPL_AUTO, False, True)
    t = _native.transpose_lists(f_ids, f_lens, p_ids, p_lens)
    args = (q, k, v, o, torch.ones_like(o), lse, None, mask.expand(B, H, S, S), ex(f_ids), ex(f_lens), ex(p_ids),
            ex(p_lens), ex(t[0]), ex(t[1]), ex(t[2]), ex(t[3]), 128, 32)
    torch.library.opcheck(_native.attn_bwd_op, args, test_utils=("test_schema", "test_faketensor"))


@pytest.mark.parametrize("dtype,D,bq,bk", [(torch.bfloat16, 128, 64, 64), (torch.float16, 128, 128, 128),
                                          (torch.bfloat16, 64, 32, 32)])
def test_tensor_core_backward_on_a_mask_with_unaligned_rows(native_lib, dtype, D, bq, bk):
    """The tensor-core backward kernels with 64 and 32 rows per CTA on either side, and a mask whose rows
    are not 16-byte aligned (a view into a wider buffer): the mask bytes are then read one by one."""
    B, H, S = 1, 3, 768
    q, k, v = workloads.make_qkv(B, H, S, D, dtype, seed=330 + bq)
    wide = torch.zeros((B, 1, S, S + 8), dtype=torch.bool)
    wide[..., 4:S + 4] = workloads.document_causal_mask(B, S, (90, 300), 0.15, seed=331 + bk)
    mask = wide[..., 4:S + 4]
    g = torch.Generator().manual_seed(9)
    w = torch.randn((B, H, S, D), generator=g).to(dtype)
    want = _reference_grads(q, k, v, mask, w)
    for m_dev in (mask.to(DEV).contiguous(), wide.to(DEV)[..., 4:S + 4]):
        qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
        out = sa.sparse_attention(qd, kd, vd, m_dev, bq, bk, check_status=True)
        out.backward(w.to(DEV))
        torch.cuda.synchronize()
        for name, got, ref in zip(("dq", "dk", "dv"), (qd.grad, kd.grad, vd.grad), want):
            _assert_grad_close(got, ref, dtype, f"{name} {dtype} D={D} ({bq},{bk}) mask stride {m_dev.stride(2)}")
