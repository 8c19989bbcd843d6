"""Stage 1 on the GPU against the CPU oracle and the recorded reference outputs: bit-exact lists."""
import ctypes

import numpy as np
import pytest
import torch

import sparseattention_b200 as sa
from oracle import cclassify
from oracle import classifier as oc
import workloads
from sparseattention_b200 import _native
from _util import assert_lists_equal, oracle_lists

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_golden_lists(golden, native_lib):
    H = golden.q.shape[1]
    for name, kind, bq, bk in golden.cases:
        m = torch.from_numpy(golden.mask(kind)).to(DEV)
        md = sa.compute_mask_kernel(m.expand(m.shape[0], H, *m.shape[2:]), bq, bk)
        assert md.unmasked_kv_ids.shape == (1, H, 256 // bq, 256 // bk)
        for tag in ("slow", "triton"):
            assert np.array_equal(md.unmasked_lens.cpu().numpy(), golden.get(f"{name}/{tag}/full_lens"))
            assert np.array_equal(md.masked_lens.cpu().numpy(), golden.get(f"{name}/{tag}/part_lens"))
            assert np.array_equal(md.unmasked_kv_ids.cpu().numpy(), golden.get(f"{name}/{tag}/full_ids"))
            assert np.array_equal(md.masked_kv_ids.cpu().numpy(), golden.get(f"{name}/{tag}/part_ids"))


@pytest.mark.parametrize("bq,bk", [(128, 32), (32, 128), (32, 32), (64, 64), (128, 128), (256, 64), (64, 512)])
def test_correctness_config_all_block_sizes(native_lib, bq, bk):
    cfg = workloads.CONFIGS["correctness"]
    m = workloads.make_mask(cfg, seed=1).to(DEV)            # [1,1,512,512]
    mask = m.expand(cfg.B, cfg.H, cfg.S, cfg.S)
    md = sa.compute_mask_kernel(mask, bq, bk)
    assert_lists_equal(md, oracle_lists(mask, bq, bk), f"({bq},{bk})")
    bits = md.packed_bits.cpu().numpy().view(np.uint32)
    assert np.array_equal(bits, oc.pack_bits(m.cpu().numpy()))


def test_broadcast_planes_are_read_once(native_lib):
    m = workloads.random_block_mask(2, 256, 0.4, 0.2, seed=2).to(DEV)      # [2,1,S,S]
    md = sa.compute_mask_kernel(m.expand(2, 5, 256, 256), 128, 32)
    assert md.unmasked_kv_ids.shape == (2, 5, 2, 8) and md.unmasked_kv_ids.stride(1) == 0
    assert md.packed_bits.shape == (2, 1, 8, 256)
    assert_lists_equal(md, oracle_lists(m.expand(2, 5, 256, 256), 128, 32))
    shared = workloads.composed_mask(512, prefix=64, window=128, drop_p=0.2, seed=3).to(DEV)   # [1,1,S,S]
    md = sa.compute_mask_kernel(shared.expand(3, 2, 512, 512), 128, 64)
    assert md.unmasked_kv_ids.stride(0) == 0 and md.unmasked_kv_ids.stride(1) == 0
    assert_lists_equal(md, oracle_lists(shared.expand(3, 2, 512, 512), 128, 64))


def test_per_head_masks_and_strided_rows(native_lib):
    g = torch.Generator().manual_seed(4)
    full = torch.rand((2, 3, 128, 256), generator=g) < 0.02
    full[:, :, :64, :96] = True
    full[0, 1, 64:, :] = False
    m = full.to(DEV)
    md = sa.compute_mask_kernel(m, 32, 32)
    assert_lists_equal(md, oracle_lists(m, 32, 32))
    # a column window of a wider buffer: row stride 512, still 16-byte aligned
    wide = torch.zeros((1, 1, 128, 512), dtype=torch.bool, device=DEV)
    wide[..., 128:384] = m[0:1, 0:1]
    view = wide[..., 128:384]
    md = sa.compute_mask_kernel(view, 64, 64)
    assert_lists_equal(md, oracle_lists(view, 64, 64))
    # a misaligned window is handled by an internal copy
    view2 = wide[..., 127:383]
    md = sa.compute_mask_kernel(view2, 64, 64)
    assert_lists_equal(md, oracle_lists(view2, 64, 64))


def test_edge_masks(native_lib):
    for S, bq, bk in [(64, 32, 32), (128, 128, 32), (1024, 128, 32), (96, 32, 96)]:
        z = torch.zeros((1, 1, S, S), dtype=torch.bool, device=DEV)
        md = sa.compute_mask_kernel(z, bq, bk)
        assert int(md.unmasked_lens.sum()) == 0 and int(md.masked_lens.sum()) == 0
        assert bool((md.unmasked_kv_ids == -1).all()) and bool((md.masked_kv_ids == -1).all())
        o = torch.ones((1, 1, S, S), dtype=torch.bool, device=DEV)
        md = sa.compute_mask_kernel(o, bq, bk)
        assert bool((md.unmasked_lens == S // bk).all()) and int(md.masked_lens.sum()) == 0
        one = z.clone()
        one[0, 0, S - 1, S - 1] = True
        one[0, 0, 0, 0] = True
        assert_lists_equal(sa.compute_mask_kernel(one, bq, bk), oracle_lists(one, bq, bk))
    with pytest.raises(AssertionError):
        sa.compute_mask_kernel(torch.zeros((1, 1, 48, 64), dtype=torch.bool, device=DEV), 32, 32)
    with pytest.raises(NotImplementedError):
        sa.compute_mask_kernel(torch.zeros((1, 1, 64, 64), dtype=torch.bool, device=DEV), 16, 32)


def test_long_rows_with_tiles_that_straddle_word_groups(native_lib):
    """Sk = 33792 (66 strips of 512 columns: more than one group of 32 flag words) with BLOCK_K = 96, whose
    tiles do not line up with the groups, and with BLOCK_K = 32 and 1024, which do."""
    g = torch.Generator().manual_seed(12)
    Sq, Sk = 64, 33792
    blocks = torch.rand((1, 1, Sq // 32, Sk // 32), generator=g)
    m = (blocks < 0.6).repeat_interleave(32, 2).repeat_interleave(32, 3)
    noisy = torch.rand((1, 1, Sq, Sk), generator=g) < 0.5
    part = (blocks < 0.15).repeat_interleave(32, 2).repeat_interleave(32, 3)
    m = (m & (~part | noisy)).to(DEV)
    for bq, bk in [(32, 96), (64, 96), (32, 32), (64, 1024), (32, 16896)]:
        assert_lists_equal(sa.compute_mask_kernel(m, bq, bk), oracle_lists(m, bq, bk), f"({bq},{bk})")


def test_nonzero_bytes_count_as_true(native_lib):
    raw = torch.zeros((1, 1, 64, 64), dtype=torch.uint8, device=DEV)
    raw[0, 0, :32, :32] = 255
    raw[0, 0, 32:, 32:] = 2
    raw[0, 0, 40, 40] = 0
    md = sa.compute_mask_kernel(raw.view(torch.bool), 32, 32)
    assert md.unmasked_lens.flatten().tolist() == [1, 0] and md.masked_lens.flatten().tolist() == [0, 1]
    # arbitrary byte values over a whole plane: the lists and the packed plane are those of (byte != 0)
    g = torch.Generator().manual_seed(3)
    raw = torch.randint(0, 256, (2, 1, 256, 1024), generator=g, dtype=torch.uint8)
    raw[torch.rand((2, 1, 256, 1024), generator=g) < 0.7] = 0
    raw[:, :, :64, :128] = 128
    raw[:, :, 64:128, 512:] = 0
    want = raw != 0
    md = sa.compute_mask_kernel(raw.to(DEV).view(torch.bool), 64, 32)
    assert_lists_equal(md, oracle_lists(want, 64, 32), "raw bytes")
    assert np.array_equal(md.packed_bits.cpu().numpy().view(np.uint32), oc.pack_bits(want.numpy()))


@pytest.mark.parametrize("name", ["document", "composed"])
def test_slices_of_large_configs(native_lib, name):
    """One plane of the document / composed configurations at S=4096 against the C oracle."""
    cfg = workloads.CONFIGS[name]
    if name == "document":
        m = workloads.document_causal_mask(1, 4096, cfg.doc_len, 0.05, seed=21, device=DEV)
    else:
        m = workloads.composed_mask(4096, drop_p=0.2, seed=22, device=DEV)
    md = sa.compute_mask_kernel(m, 128, 32)
    ref = cclassify.classify(m.cpu().numpy(), 128, 32)
    assert_lists_equal(md, ref, name)


def test_headline_shape_properties(native_lib):
    """Full headline size (B=8, S=4096, one plane per batch element, expanded over 32 heads)."""
    m = workloads.random_block_mask(8, 4096, 0.5, 0.1, seed=31, device=DEV)
    md = sa.compute_mask_kernel(m.expand(8, 32, 4096, 4096), 128, 32)
    assert md.unmasked_kv_ids.shape == (8, 32, 32, 128)
    ref = cclassify.classify(m.cpu().numpy(), 128, 32)                     # [8,1,...]
    assert np.array_equal(md.unmasked_lens[:, 0:1].cpu().numpy(), ref.unmasked_lens)
    assert np.array_equal(md.masked_lens[:, 0:1].cpu().numpy(), ref.masked_lens)
    assert np.array_equal(md.unmasked_kv_ids[:, 0:1].cpu().numpy(), ref.unmasked_kv_ids)
    assert np.array_equal(md.masked_kv_ids[:, 0:1].cpu().numpy(), ref.masked_kv_ids)
    # size-independent properties: ascending ids, counts bounded, every tile in exactly one class
    ids = md.unmasked_kv_ids[:, 0].long()
    lens = md.unmasked_lens[:, 0].long()
    pos = torch.arange(128, device=DEV)
    valid = pos < lens[..., None]
    assert bool(((ids[..., 1:] > ids[..., :-1]) | ~valid[..., 1:]).all())
    tiles = m[:, 0].reshape(8, 32, 128, 128, 32).sum(dim=(2, 4))
    assert int((tiles == 128 * 32).sum()) == int(md.unmasked_lens[:, 0].sum())
    assert int(((tiles > 0) & (tiles < 128 * 32)).sum()) == int(md.masked_lens[:, 0].sum())
    # the packed plane reproduces the mask bit for bit
    bits = md.packed_bits[:, 0]                                             # [8, 128, 4096] int32
    shifts = torch.arange(32, device=DEV, dtype=torch.int32)
    for b in (0, 7):
        unpacked = ((bits[b].unsqueeze(-1) >> shifts) & 1).bool()          # [Sk/32, Sq, 32]
        assert torch.equal(unpacked.permute(1, 0, 2).reshape(4096, 4096), m[b, 0])


def test_c_abi_direct_call(native_lib):
    """The same classification through raw pointers, as a non-Python host would call it."""
    m = workloads.random_block_mask(1, 256, 0.5, 0.2, seed=5).to(DEV).contiguous()
    nq, nk = 2, 8
    f_ids = torch.full((1, 1, nq, nk), 7, dtype=torch.int32, device=DEV)
    p_ids = torch.full((1, 1, nq, nk), 7, dtype=torch.int32, device=DEV)
    f_lens = torch.zeros((1, 1, nq), dtype=torch.int32, device=DEV)
    p_lens = torch.zeros((1, 1, nq), dtype=torch.int32, device=DEV)
    ws_bytes = native_lib.sa_classify_workspace_bytes(1, 1, 256, 256)
    ref = oracle_lists(m, 128, 32)
    # a workspace of unknown contents (the call clears it), then a zero-filled one declared clean, used twice:
    # the kernel hands a workspace back zero-filled
    dirty = torch.full((ws_bytes,), 0xAB, dtype=torch.uint8, device=DEV)
    clean = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    for ws, state in ((dirty, _native.SA_WS_UNKNOWN), (clean, _native.SA_WS_CLEAN), (clean, _native.SA_WS_CLEAN)):
        for t in (f_ids, p_ids, f_lens, p_lens):
            t.fill_(7)
        rc = native_lib.sa_classify_mask(m.data_ptr(), 0, 0, 256, 1, 1, 1, 256, 256, 128, 32,
                                         f_ids.data_ptr(), f_lens.data_ptr(), p_ids.data_ptr(), p_lens.data_ptr(),
                                         None, ws.data_ptr(), ws_bytes, state,
                                         torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert np.array_equal(f_ids.cpu().numpy(), ref.unmasked_kv_ids)
        assert np.array_equal(p_ids.cpu().numpy(), ref.masked_kv_ids)
        assert np.array_equal(f_lens.cpu().numpy(), ref.unmasked_lens)
        assert np.array_equal(p_lens.cpu().numpy(), ref.masked_lens)
    assert int(clean.sum()) == 0
    ws = clean
    # too small a workspace is refused before any launch
    rc = native_lib.sa_classify_mask(m.data_ptr(), 0, 0, 256, 1, 1, 1, 256, 256, 128, 32,
                                     f_ids.data_ptr(), f_lens.data_ptr(), p_ids.data_ptr(), p_lens.data_ptr(),
                                     None, ws.data_ptr(), 1, _native.SA_WS_UNKNOWN,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == -3
