"""The CPU oracle against the outputs of the reference itself (tests/golden)."""
import numpy as np
import pytest

from oracle import attention as oa
from oracle import cclassify
from oracle import classifier as oc


def _expand(m, H):
    return np.broadcast_to(m, (m.shape[0], H) + m.shape[2:])


@pytest.mark.parametrize("impl", ["numpy", "c", "loops"])
def test_classifier_matches_reference_lists(golden, impl):
    H = golden.q.shape[1]
    for name, kind, bq, bk in golden.cases:
        mask = np.ascontiguousarray(_expand(golden.mask(kind), H))
        if impl == "numpy":
            md = oc.classify(mask, bq, bk)
        elif impl == "c":
            md = cclassify.classify(mask, bq, bk)
        else:
            md = oc.classify_loops(mask, bq, bk)
        for tag in ("slow", "triton"):       # compute_mask_slow and the Triton kernel under the interpreter
            assert np.array_equal(md.unmasked_lens, golden.get(f"{name}/{tag}/full_lens")), (name, tag)
            assert np.array_equal(md.masked_lens, golden.get(f"{name}/{tag}/part_lens")), (name, tag)
            assert np.array_equal(md.unmasked_kv_ids, golden.get(f"{name}/{tag}/full_ids")), (name, tag)
            assert np.array_equal(md.masked_kv_ids, golden.get(f"{name}/{tag}/part_ids")), (name, tag)


def test_blocked_restatement_matches_reference_kernel(golden):
    """The literal restatement (nan_safe=False) reproduces the Triton kernel, NaN rows included."""
    q, k, v = (x.astype(np.float32) for x in (golden.q, golden.k, golden.v))
    H = q.shape[1]
    for name, kind, bq, bk in golden.cases:
        mask = _expand(golden.mask(kind), H)
        md = oc.classify(np.ascontiguousarray(mask), bq, bk)
        ref = golden.get(f"{name}/attn_out")
        got = oa.blocked_reference(q, k, v, mask, md, bq, bk, nan_safe=False)
        nan_ref = np.isnan(ref).any(-1)
        assert np.array_equal(np.isnan(got).any(-1), nan_ref), name
        assert np.array_equal(oa.predicted_nan_rows(mask, md, bq, bk), nan_ref), name
        fin = ~nan_ref
        assert np.abs(got[fin] - ref[fin]).max() < 2e-5, name


def test_sdpa_agrees_with_reference_on_finite_rows(golden):
    """torch SDPA (the numerical authority) equals the reference kernel wherever the latter is finite,
    and the guarded restatement equals SDPA on every row."""
    q, k, v = (x.astype(np.float32) for x in (golden.q, golden.k, golden.v))
    H = q.shape[1]
    for name, kind, bq, bk in golden.cases:
        mask = _expand(golden.mask(kind), H)
        md = oc.classify(np.ascontiguousarray(mask), bq, bk)
        ref = golden.get(f"{name}/attn_out")
        sdpa = oa.sdpa_reference(q, k, v, golden.mask(kind))
        fin = ~np.isnan(ref).any(-1)
        assert np.abs(sdpa[fin] - ref[fin]).max() < 2e-5, name
        safe = oa.blocked_reference(q, k, v, mask, md, bq, bk, nan_safe=True)
        assert not np.isnan(safe).any()
        assert np.abs(safe - sdpa).max() < 2e-5, name


def test_fully_masked_rows_are_zero():
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((1, 1, 64, 16)).astype(np.float32) for _ in range(3))
    mask = rng.random((1, 1, 64, 64)) < 0.5
    mask[0, 0, 5] = False
    mask[0, 0, 32:64] = False
    md = oc.classify(mask, 32, 32)
    out = oa.blocked_reference(q, k, v, mask, md, 32, 32)
    assert np.all(out[0, 0, 5] == 0) and np.all(out[0, 0, 32:] == 0)
    assert np.abs(out - oa.sdpa_reference(q, k, v, mask)).max() < 2e-5


def test_pack_bits_layout():
    rng = np.random.default_rng(1)
    mask = rng.random((2, 1, 64, 96)) < 0.3
    bits = oc.pack_bits(mask)
    assert bits.shape == (2, 1, 3, 64) and bits.dtype == np.uint32
    for (b, r, c) in [(0, 0, 0), (1, 63, 95), (0, 17, 40), (1, 5, 33)]:
        assert bool((bits[b, 0, c // 32, r] >> (c % 32)) & 1) == bool(mask[b, 0, r, c])


def test_classifier_edge_cases():
    # all False, all True, a single True element, block sizes equal to S
    for S, bq, bk in [(64, 32, 32), (128, 128, 32), (128, 32, 128), (64, 64, 64)]:
        z = np.zeros((1, 1, S, S), bool)
        md = oc.classify(z, bq, bk)
        assert md.unmasked_lens.sum() == 0 and md.masked_lens.sum() == 0 and (md.unmasked_kv_ids == -1).all()
        o = np.ones((1, 1, S, S), bool)
        md = oc.classify(o, bq, bk)
        assert (md.unmasked_lens == S // bk).all() and md.masked_lens.sum() == 0
        assert np.array_equal(md.unmasked_kv_ids[0, 0, 0], np.arange(S // bk))
        one = z.copy()
        one[0, 0, S - 1, S - 1] = True
        md = oc.classify(one, bq, bk)
        assert md.masked_lens.sum() == 1 and md.masked_kv_ids[0, 0, -1, 0] == S // bk - 1
        c = cclassify.classify(one, bq, bk)
        assert np.array_equal(c.masked_kv_ids, md.masked_kv_ids) and np.array_equal(c.masked_lens, md.masked_lens)
    with pytest.raises(AssertionError):
        oc.classify(np.zeros((1, 1, 48, 64), bool), 32, 32)
