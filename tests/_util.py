"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import attention as oa
from oracle import classifier as oc

# Tolerances the benchmark definition states for fp16 / bf16 inputs with fp32 accumulation.
MAX_ABS_16 = 2e-2
MEAN_ABS_16 = 2e-3
# fp32 inputs through the CUDA-core kernel (true fp32 math, exp2 in place of exp).
MAX_ABS_32 = 2e-4


def oracle_lists(mask_t: torch.Tensor, bq: int, bk: int):
    return oc.classify(np.ascontiguousarray(mask_t.cpu().numpy()), bq, bk)


def assert_lists_equal(md, ref, what=""):
    """Bit-exact: counts, and every id including the -1 tails."""
    f_ids, f_lens = md.unmasked_kv_ids.cpu().numpy(), md.unmasked_lens.cpu().numpy()
    p_ids, p_lens = md.masked_kv_ids.cpu().numpy(), md.masked_lens.cpu().numpy()
    assert f_ids.dtype == np.int32 and f_lens.dtype == np.int32
    assert np.array_equal(f_lens, ref.unmasked_lens), f"{what}: full counts differ"
    assert np.array_equal(p_lens, ref.masked_lens), f"{what}: partial counts differ"
    assert np.array_equal(f_ids, ref.unmasked_kv_ids), f"{what}: full ids differ"
    assert np.array_equal(p_ids, ref.masked_kv_ids), f"{what}: partial ids differ"


def sdpa_cpu(q, k, v, mask):
    return torch.from_numpy(oa.sdpa_reference(q, k, v, mask))


def assert_close_attn(out: torch.Tensor, ref: torch.Tensor, dtype, what=""):
    out = out.detach().float().cpu()
    assert not torch.isnan(out).any(), f"{what}: NaN in output"
    diff = (out - ref).abs()
    if dtype == torch.float32:
        assert diff.max().item() <= MAX_ABS_32, f"{what}: max-abs {diff.max().item():.3e}"
    else:
        assert diff.max().item() <= MAX_ABS_16, f"{what}: max-abs {diff.max().item():.3e}"
        assert diff.mean().item() <= MEAN_ABS_16, f"{what}: mean-abs {diff.mean().item():.3e}"
