"""CPU-side checks: the C-ABI library exports what the header declares, the workload
generators are well formed, and the Python entry points refuse CPU tensors."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from oracle import classifier as oc
import workloads
from sparseattention_b200 import _native
import sparseattention_b200 as sa

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(native_lib):
    header = open(os.path.join(ROOT, "include", "sa_b200.h")).read()
    declared = set(re.findall(r"\b(sa_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_native.SYMBOLS), declared ^ set(_native.SYMBOLS)
    for name in declared:
        assert hasattr(native_lib, name), name
    assert native_lib.sa_abi_version() == _native.SA_ABI_VERSION
    assert native_lib.sa_status_str(0) == b"ok"
    assert b"unsupported" in native_lib.sa_status_str(-2)


def test_argument_validation_needs_no_gpu(native_lib):
    bu, hu = ctypes.c_int(), ctypes.c_int()
    assert native_lib.sa_unique_planes(8, 32, 4096 * 4096, 0, ctypes.byref(bu), ctypes.byref(hu)) == 0
    assert (bu.value, hu.value) == (8, 1)
    assert native_lib.sa_unique_planes(0, 1, 0, 0, ctypes.byref(bu), ctypes.byref(hu)) == -1
    # headline mask: per (plane, 32-row slice) a 4-byte counter and eight 8-byte words (one per
    # 512-column strip), rounded up to 256 B
    assert native_lib.sa_classify_workspace_bytes(8, 1, 4096, 4096) == (8 * 128 * (4 + 8 * 8) + 255) // 256 * 256
    assert native_lib.sa_classify_workspace_bytes(1, 1, 64, 64) == 256
    # null pointers / non-dividing block sizes are rejected before anything is launched
    assert native_lib.sa_classify_mask(None, 0, 0, 64, 1, 1, 1, 64, 64, 32, 32, None, None, None, None, None,
                                       None, 0, 0, None) == -1
    buf = (ctypes.c_uint8 * 64)()
    p = ctypes.addressof(buf)
    p -= p % 16
    assert native_lib.sa_classify_mask(p, 0, 0, 64, 1, 1, 1, 64, 64, 48, 32, p, p, p, p, None, p, 1 << 20, 0, None) == -1
    assert native_lib.sa_classify_mask(p, 0, 0, 64, 1, 1, 1, 64, 64, 16, 32, p, p, p, p, None, p, 1 << 20, 0, None) == -2
    assert native_lib.sa_classify_mask(p, 0, 0, 64, 1, 1, 1, 64, 64, 32, 32, p, p, p, p, None, p, 0, 0, None) == -3
    assert native_lib.sa_classify_mask(p, 0, 0, 64, 1, 1, 1, 64, 64, 32, 32, p, p, p, p, None, p, 1 << 20, 7, None) == -1
    assert native_lib.sa_classify_mask(p, 0, 0, 2048, 1, 1, 1, 2048, 64, 2048, 32, p, p, p, p, None, p, 1 << 20, 0,
                                       None) == -2     # BLOCK_Q above 1024


def test_entry_points_refuse_cpu_tensors(native_lib):
    mask = torch.ones(1, 1, 64, 64, dtype=torch.bool)
    with pytest.raises(RuntimeError, match="CUDA"):
        sa.compute_mask_kernel(mask, 32, 32)
    q = torch.randn(1, 1, 64, 16)
    md = sa.compute_mask_slow(mask, 32, 32)
    with pytest.raises(RuntimeError, match="CUDA"):
        sa.sparse_attention(q, q, q, mask, 32, 32, mask_metadata=md)


def test_compute_mask_slow_matches_oracle():
    m = workloads.random_block_mask(2, 256, 0.5, 0.2, seed=3)
    for bq, bk in [(128, 32), (32, 128), (64, 64)]:
        md = sa.compute_mask_slow(m.expand(2, 3, 256, 256), bq, bk)
        ref = oc.classify(np.ascontiguousarray(m.expand(2, 3, 256, 256).numpy()), bq, bk)
        assert np.array_equal(md.unmasked_kv_ids.numpy(), ref.unmasked_kv_ids)
        assert np.array_equal(md.masked_kv_ids.numpy(), ref.masked_kv_ids)
        assert np.array_equal(md.unmasked_lens.numpy(), ref.unmasked_lens)
        assert np.array_equal(md.masked_lens.numpy(), ref.masked_lens)


def test_mask_metadata_keeps_reference_field_order():
    t = torch.zeros(1)
    md = sa.MaskMetadata(t, t + 1, t + 2, t + 3)
    assert md.unmasked_kv_ids is t and float(md.unmasked_lens) == 1 and float(md.masked_kv_ids) == 2
    assert float(md.masked_lens) == 3 and md.packed_bits is None


def test_random_block_mask_properties():
    m = workloads.random_block_mask(2, 512, 0.5, 0.1, seed=5)
    assert m.shape == (2, 1, 512, 512) and m.dtype == torch.bool
    assert torch.equal(m, workloads.random_block_mask(2, 512, 0.5, 0.1, seed=5))
    assert m.diagonal(dim1=-2, dim2=-1).all()                 # no empty row
    blocks = m.reshape(2, 16, 32, 16, 32).float().mean(dim=(2, 4))
    assert (blocks[:, range(16), range(16)] > 0).all()         # diagonal blocks kept
    empty = (blocks == 0).float().mean().item()
    assert 0.35 < empty < 0.6
    partial = ((blocks > 0) & (blocks < 1)).float().mean().item()
    assert 0.01 < partial < 0.12
    dense = workloads.random_block_mask(1, 256, 0.0, 0.0, seed=1)
    assert dense.all()


def test_document_and_composed_masks():
    m = workloads.document_causal_mask(2, 512, (40, 100), 0.0, seed=7)
    assert m.diagonal(dim1=-2, dim2=-1).all()
    assert not torch.triu(m[0, 0], diagonal=1).any()           # causal
    g = torch.Generator().manual_seed(7)
    lens = workloads.document_lengths(512, 40, 100, g)
    assert sum(lens) == 512 and all(1 <= n <= 100 for n in lens)
    assert not m[0, 0, lens[0], lens[0] - 1]                   # document boundary
    mp = workloads.document_causal_mask(1, 512, (64, 200), 0.3, seed=9)
    assert mp.diagonal(dim1=-2, dim2=-1).all()
    c = workloads.composed_mask(4096, prefix=1024, window=2048, drop_p=0.0, seed=1)
    assert c[0, 0, 10, 1000] and c[0, 0, 3000, 1000] and not c[0, 0, 3100, 1000] and not c[0, 0, 10, 2000]
    cd = workloads.composed_mask(4096, drop_p=0.2, seed=1)
    assert cd.diagonal(dim1=-2, dim2=-1).all() and cd.sum() < c.sum()


def test_flop_accounting():
    lens = torch.tensor([[[3, 1]]])
    assert workloads.computed_tile_flops(lens, lens, 128, 32, 128) == 4 * 128 * 128 * 32 * 8
    assert workloads.dense_flops(8, 32, 4096, 4096, 128) == pytest.approx(2.199e12, rel=1e-3)
    assert workloads.classifier_bytes(8, 4096, 4096, 128, 0) == 8 * 4096 * 4096 + 8 * 8 * 32


def test_reference_module_names_resolve_to_this_library():
    """``sparseattention.mask_utils`` / ``sparseattention.sparse_attn_kernel`` (the reference's module
    paths) export the reference's names, backed by this package; the torch ops carry the package name."""
    import sparseattention.mask_utils as mu
    import sparseattention.sparse_attn_kernel as sak
    import sparseattention_b200 as impl
    assert mu.MaskMetadata is impl.MaskMetadata and mu.compute_mask_kernel is impl.compute_mask_kernel
    assert mu.compute_mask_slow is impl.compute_mask_slow and sak.sparse_attention is impl.sparse_attention
    assert sak.compute_mask_kernel is impl.compute_mask_kernel
    assert hasattr(torch.ops.sparseattention, "classify_mask") and hasattr(torch.ops.sparseattention, "attn_fwd")
    with pytest.raises(RuntimeError):           # CUDA tensors only: no CPU implementation is registered
        mu.compute_mask_kernel(torch.ones((1, 1, 128, 128), dtype=torch.bool), 128, 32)


def test_reference_arm_of_the_bench_prints_one_contract_line():
    """``bench.py --impl reference`` needs no GPU: one JSON line with the contract's keys, the CPU arm's
    own figures in ``value`` / ``cpu_baseline`` / ``e2e``, no GPU launches claimed."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "1", "--cpu-heads", "1"], capture_output=True, text=True, timeout=600, cwd=root)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "impl"):
        assert key in line, key
    assert line["impl"] == "reference" and line["value"] > 0 and line["gpu_launches"] == 0
    assert line["e2e"]["value"] == line["value"] and line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["cpu_baseline"]["kind"] in ("port", "reference") and line["cpu_baseline"]["cores"] >= 1
