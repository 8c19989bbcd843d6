"""Stage 2 on the GPU against the CPU oracle (torch SDPA with the bool mask on the host,
the reference's own ground truth) and against the recorded outputs of the reference kernel."""
import numpy as np
import pytest
import torch

import sparseattention_b200 as sa
from oracle import attention as oa
from oracle import classifier as oc
import workloads
from sparseattention_b200 import _native
from _util import assert_close_attn, assert_lists_equal, sdpa_cpu, MAX_ABS_16

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(q, k, v, mask, bq, bk, impl="auto", md=None):
    out = sa.sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), mask.to(DEV), bq, bk, mask_metadata=md,
                              impl=impl, check_status=True)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("bq,bk", [(128, 32), (32, 128), (32, 32), (64, 64)])
def test_correctness_config_fp32(native_lib, bq, bk):
    """B=1, H=4, S=512, D=64, fp32 inputs, 32x32-block mask with p=0.5: the CPU-runnable case."""
    cfg = workloads.CONFIGS["correctness"]
    q, k, v = workloads.make_qkv(cfg.B, cfg.H, cfg.S, cfg.D, torch.float32, seed=1)
    mask = workloads.make_mask(cfg, seed=1)
    ref = sdpa_cpu(q, k, v, mask)
    out = _run(q, k, v, mask, bq, bk)
    assert out.dtype == torch.float32 and out.shape == q.shape
    assert_close_attn(out, ref, torch.float32, f"fp32 ({bq},{bk})")


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,bk", [(128, 32), (128, 64), (128, 128), (64, 32), (64, 128)])
def test_half_precision_vs_sdpa(native_lib, impl, dtype, D, bk):
    B, H, S = 2, 2, 512
    q, k, v = workloads.make_qkv(B, H, S, D, dtype, seed=D + bk)
    mask = workloads.random_block_mask(B, S, 0.5, 0.15, seed=bk)
    ref = sdpa_cpu(q, k, v, mask)
    assert _native.uses_tcgen05(q.to(DEV), k.to(DEV), v.to(DEV), 128, bk)
    out = _run(q, k, v, mask, 128, bk, impl=impl)
    assert out.dtype == dtype
    assert_close_attn(out, ref, dtype, f"{impl} {dtype} D={D} bk={bk}")


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
def test_golden_reference_outputs(golden, native_lib, impl):
    """fp16 inputs of the recorded cases: equal to the reference kernel on its finite rows,
    to SDPA on all rows, 0 where a row has no attended key."""
    q, k, v = (torch.from_numpy(x) for x in (golden.q, golden.k, golden.v))     # fp16, D=64
    for name, kind, bq, bk in golden.cases:
        if impl == "tcgen05" and bq != 128:
            continue
        mask = torch.from_numpy(golden.mask(kind))
        out = _run(q, k, v, mask, bq, bk, impl=impl).float().cpu()
        ref = torch.from_numpy(golden.get(f"{name}/attn_out"))
        fin = ~torch.isnan(ref).any(-1)
        assert (out[fin] - ref[fin]).abs().max().item() <= MAX_ABS_16, name
        assert_close_attn(out, sdpa_cpu(q, k, v, mask), torch.float16, name)


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
def test_masked_rows_empty_blocks_and_dense(native_lib, impl):
    B, H, S, D = 1, 2, 512, 128
    q, k, v = workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=3)
    mask = workloads.random_block_mask(B, S, 0.6, 0.3, seed=3)
    mask[0, 0, 5] = False                 # a fully masked row inside a live query block
    mask[0, 0, 128:256] = False           # a query block with both lists empty
    mask[0, 0, 256:384, :] = False
    mask[0, 0, 256:384, 32:64] = True     # a query block with exactly one full tile
    out = _run(q, k, v, mask, 128, 32, impl=impl)
    assert_close_attn(out, sdpa_cpu(q, k, v, mask), torch.bfloat16, "edge rows")
    o = out.float().cpu()
    assert bool((o[:, :, 5] == 0).all()) and bool((o[:, :, 128:256] == 0).all())
    dense = torch.ones((1, 1, S, S), dtype=torch.bool)
    out = _run(q, k, v, dense, 128, 32, impl=impl)
    assert_close_attn(out, sdpa_cpu(q, k, v, dense), torch.bfloat16, "dense")
    causal = torch.tril(torch.ones((S, S), dtype=torch.bool))[None, None]
    for bk in (32, 64, 128):
        out = _run(q, k, v, causal, 128, bk, impl=impl)
        assert_close_attn(out, sdpa_cpu(q, k, v, causal), torch.bfloat16, f"causal bk={bk}")


def test_list_lengths_not_multiple_of_step(native_lib):
    """Query blocks whose full / partial counts leave ragged 128-row steps (1..7 listed blocks)."""
    B, H, S, D = 1, 1, 1024, 128
    q, k, v = workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=9)
    mask = torch.zeros((1, 1, S, S), dtype=torch.bool)
    g = torch.Generator().manual_seed(9)
    for i in range(8):                       # query block i: i+1 listed blocks, first (i+1)//2 full
        rows = slice(128 * i, 128 * (i + 1))
        cols = torch.randperm(32, generator=g)[: i + 1]
        for n, c in enumerate(cols.tolist()):
            if n < (i + 1) // 2:
                mask[0, 0, rows, 32 * c:32 * c + 32] = True
            else:
                mask[0, 0, rows, 32 * c:32 * c + 32] = torch.rand((128, 32), generator=g) < 0.5
    ref = sdpa_cpu(q, k, v, mask)
    for impl in ("simt", "tcgen05"):
        out = _run(q, k, v, mask, 128, 32, impl=impl)
        assert_close_attn(out, ref, torch.bfloat16, impl)


def test_strided_inputs_and_broadcast_mask(native_lib):
    B, H, S, D = 2, 3, 256, 128
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn((B, S, 3, H, D), generator=g).to(torch.bfloat16).to(DEV)   # packed projection layout
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))               # [B,H,S,D] views
    assert not q.is_contiguous()
    mask = workloads.composed_mask(S, prefix=64, window=96, drop_p=0.2, seed=5)  # [1,1,S,S]
    ref = sdpa_cpu(q, k, v, mask)
    for impl in ("simt", "tcgen05"):
        out = _run(q, k, v, mask, 128, 32, impl=impl)
        assert_close_attn(out, ref, torch.bfloat16, impl)


def test_caller_supplied_metadata(native_lib):
    """Lists built elsewhere (here: by compute_mask_slow on the GPU, int32, no packed plane) are honoured."""
    B, H, S, D = 1, 2, 512, 128
    q, k, v = workloads.make_qkv(B, H, S, D, torch.float16, seed=6)
    mask = workloads.random_block_mask(B, S, 0.5, 0.2, seed=6).to(DEV)
    md = sa.compute_mask_slow(mask.expand(B, H, S, S), 128, 32)
    assert md.packed_bits is None
    ref = sdpa_cpu(q, k, v, mask)
    out = _run(q, k, v, mask, 128, 32, md=md)
    assert_close_attn(out, ref, torch.float16, "metadata from compute_mask_slow")
    md2 = sa.compute_mask_kernel(mask.expand(B, H, S, S), 128, 32)
    out2 = _run(q, k, v, mask, 128, 32, md=md2)
    assert torch.equal(out, out2)


def test_deterministic_and_no_unwritten_rows(native_lib):
    B, H, S, D = 2, 4, 1024, 128
    q, k, v = workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=7)
    mask = workloads.document_causal_mask(B, S, (100, 400), 0.1, seed=7)
    a = _run(q, k, v, mask, 128, 32, impl="tcgen05")
    b = _run(q, k, v, mask, 128, 32, impl="tcgen05")
    assert torch.equal(a, b)
    assert_close_attn(a, sdpa_cpu(q, k, v, mask), torch.bfloat16, "document")


def test_unsupported_calls_raise(native_lib):
    q = torch.randn((1, 1, 128, 48), device=DEV, dtype=torch.bfloat16)
    mask = torch.ones((1, 1, 128, 128), dtype=torch.bool, device=DEV)
    with pytest.raises(NotImplementedError):
        sa.sparse_attention(q, q, q, mask, 128, 32)                 # head dim 48
    q = torch.randn((1, 1, 128, 64), device=DEV, dtype=torch.float32)
    with pytest.raises(NotImplementedError):
        sa.sparse_attention(q, q, q, mask, 128, 32, impl="tcgen05")  # fp32 has no tensor-core path
    with pytest.raises(TypeError):
        sa.sparse_attention(q.double(), q.double(), q.double(), mask, 128, 32)


@pytest.mark.parametrize("drop_p", [0.0, 0.1, 0.3, 0.5, 0.7, 0.9])
def test_headline_shape_slice(native_lib, drop_p):
    """One batch element of the headline shape (H=32, S=4096, D=128, bf16) at every drop probability of
    the sweep: the tensor-core kernel against host SDPA on two heads, and (at p = 0.5 and 0.9, the dense
    and the ragged regime of the lists) against the CUDA-core kernel over all heads."""
    H, S, D = 32, 4096, 128
    seed = 8 + int(drop_p * 10)
    q, k, v = workloads.make_qkv(1, H, S, D, torch.bfloat16, seed=seed, device=DEV)
    mask = workloads.random_block_mask(1, S, drop_p, 0.1, seed=seed, device=DEV)
    md = sa.compute_mask_kernel(mask.expand(1, H, S, S), 128, 32)
    out = sa.sparse_attention(q, k, v, mask, 128, 32, mask_metadata=md, impl="tcgen05", check_status=True)
    hs = [0, 31]
    ref = sdpa_cpu(q[:, hs], k[:, hs], v[:, hs], mask)
    assert_close_attn(out[:, hs], ref, torch.bfloat16, f"headline slice vs SDPA, p={drop_p}")
    if drop_p in (0.5, 0.9):
        simt = sa.sparse_attention(q, k, v, mask, 128, 32, mask_metadata=md, impl="simt", check_status=True)
        d = (out.float() - simt.float()).abs()
        assert d.max().item() <= MAX_ABS_16 and d.mean().item() <= 2e-3


def test_custom_ops_pass_opcheck(native_lib):
    """The two torch.library ops: schema and fake-tensor (shape / dtype propagation) checks."""
    B, H, S, D = 1, 2, 256, 128
    q, k, v = (t.to(DEV) for t in workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=11))
    mask = workloads.random_block_mask(B, S, 0.5, 0.2, seed=11).to(DEV)
    checks = ("test_schema", "test_faketensor")
    torch.library.opcheck(_native.classify_mask_op, (mask, 128, 32, True), test_utils=checks)
    f_ids, f_lens, p_ids, p_lens, bits = _native.classify(mask, 128, 32)
    ex = lambda t, nd: t.expand(*((B, H) + tuple(t.shape[2:])))
    args = (q, k, v, mask.expand(B, H, S, S), bits, ex(f_ids, 4), ex(f_lens, 3), ex(p_ids, 4), ex(p_lens, 3),
            128, 32, _native.SA_IMPL_AUTO, False, True)
    torch.library.opcheck(_native.attn_fwd_op, args, test_utils=checks)


def test_both_stages_replay_from_a_cuda_graph(native_lib):
    """Stage 1 + stage 2 captured once and replayed: nothing on the path allocates outside torch's
    capture-aware allocator or synchronises, so a layer loop can replay it (the amortisation the
    reference's README assumes when it quotes stage 2 alone)."""
    B, H, S, D = 2, 4, 1024, 128
    q, k, v = (t.to(DEV) for t in workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=21))
    mask = workloads.random_block_mask(B, S, 0.6, 0.2, seed=22).to(DEV)

    def both():
        md = sa.compute_mask_kernel(mask.expand(B, H, S, S), 128, 32)
        return sa.sparse_attention(q, k, v, mask, 128, 32, mask_metadata=md, check_status=False)

    eager = both()                                  # also the warm-up the capture needs
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        both()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            out = both()
    for _ in range(3):
        out.zero_()
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    ref = sdpa_cpu(q.cpu(), k.cpu(), v.cpu(), mask.cpu())
    assert_close_attn(out, ref, torch.bfloat16, "graph replay")


def test_uneven_tiles_are_all_written(native_lib):
    """Tiles of very different length (document mask: 1 to S/128 steps) with more tiles than SMs: the
    CTAs draw tiles from the shared counter; every query block must come out once and right."""
    B, H, S, D = 1, 6, 4096, 128                    # 6 * 32 = 192 tiles > 148 CTAs
    q, k, v = workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=31)
    mask = workloads.document_causal_mask(B, S, (256, 2048), seed=32)
    ref = sdpa_cpu(q, k, v, mask)
    for _ in range(2):
        out = _run(q, k, v, mask, 128, 32, impl="tcgen05")
        assert_close_attn(out, ref, torch.bfloat16, "uneven tiles")


@pytest.mark.parametrize("bq,bk", [(32, 32), (64, 64), (32, 128)])
def test_finer_query_blocks_take_the_tensor_core_kernel(native_lib, bq, bk):
    """BLOCK_Q of 32 / 64 (the reference's other defaults, test_attn.py:32) without caller lists: the
    lists are built 128 rows high and the bit plane masks the elements -- same values as SDPA and as
    the generic kernel walking the finer lists."""
    B, H, S, D = 2, 2, 512, 128
    q, k, v = workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=bq + bk)
    mask = workloads.random_block_mask(B, S, 0.5, 0.2, seed=bq)
    ref = sdpa_cpu(q, k, v, mask)
    out = _run(q, k, v, mask, bq, bk)
    assert_close_attn(out, ref, torch.bfloat16, f"auto ({bq},{bk})")
    fine = _run(q, k, v, mask, bq, bk, impl="simt")
    assert_close_attn(out, fine.float().cpu(), torch.bfloat16, f"auto vs simt ({bq},{bk})")


@pytest.mark.parametrize("bq,bk", [(32, 128), (64, 32), (32, 32)])
def test_caller_lists_for_short_query_blocks_are_folded(native_lib, bq, bk):
    """Lists supplied by the caller for BLOCK_Q = 32 / 64 -- the way the reference's own harness calls it
    (test_attn.py:38-41, lists built at (32, 128) and passed in): folded into 128-row lists on the device.
    The folded lists must be the ones the classifier gives at 128 rows, and the values those of SDPA."""
    B, H, S, D = 2, 3, 1024, 128
    q, k, v = workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=3 * bq + bk)
    mask = workloads.random_block_mask(B, S, 0.5, 0.2, seed=bq + 7).to(DEV)
    md = sa.compute_mask_kernel(mask.expand(B, H, S, S), bq, bk)
    short = [t[:, :1].contiguous() for t in (md.unmasked_kv_ids, md.unmasked_lens, md.masked_kv_ids, md.masked_lens)]
    f128, fl128, p128, pl128, bits = _native.classify(mask, 128, bk, with_bits=True)
    before = bits.clone()
    f_ids, f_lens, p_ids, p_lens = _native.merge_lists(*short, bq, bk, 128 // bq, bits)
    torch.cuda.synchronize()
    assert torch.equal(f_lens, fl128) and torch.equal(p_lens, pl128)
    assert torch.equal(f_ids, f128) and torch.equal(p_ids, p128)          # tails are -1 in both
    assert torch.equal(bits, before)                                      # lists from the same mask: no change
    ref = sdpa_cpu(q, k, v, mask.cpu())
    md.packed_bits = None                                                 # as if the reference had made it
    out = _run(q, k, v, mask, bq, bk, md=md)
    assert_close_attn(out, ref, torch.bfloat16, f"folded ({bq},{bk})")


def test_pruned_caller_lists_are_honoured_after_folding(native_lib):
    """A caller that drops kv blocks from the short lists (block selection on top of the mask) gets what a
    walk over those lists gives -- the generic kernel is that walk -- not what the mask alone would give."""
    B, H, S, D, bq, bk = 1, 2, 1024, 128, 32, 32
    q, k, v = workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=77)
    mask = workloads.random_block_mask(B, S, 0.3, 0.2, seed=78).to(DEV)
    md = sa.compute_mask_kernel(mask.expand(B, H, S, S), bq, bk)
    # drop the last listed block of every list that has more than one entry
    md.unmasked_lens = torch.where(md.unmasked_lens > 1, md.unmasked_lens - 1, md.unmasked_lens).contiguous()
    md.masked_lens = torch.where(md.masked_lens > 1, md.masked_lens - 1, md.masked_lens).contiguous()
    md.packed_bits = None
    walk = _run(q, k, v, mask, bq, bk, impl="simt", md=md).float().cpu()
    out = _run(q, k, v, mask, bq, bk, md=md)
    assert_close_attn(out, walk, torch.bfloat16, "pruned lists")
    full = sdpa_cpu(q, k, v, mask.cpu())
    assert (walk - full).abs().max().item() > 5e-2          # the pruning does change the answer


def test_without_a_workspace_the_tiles_are_dealt_round_robin(native_lib, monkeypatch):
    """sa_attn_fwd with workspace = NULL (a host that binds the C ABI without one): the CTAs step through
    the tiles by the grid size instead of drawing them from the counter; same values."""
    B, H, S, D = 1, 6, 4096, 128                    # 192 tiles > 148 CTAs
    q, k, v = workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=41)
    mask = workloads.document_causal_mask(B, S, (256, 2048), seed=42)
    with_ws = _run(q, k, v, mask, 128, 32, impl="tcgen05")
    monkeypatch.setattr(native_lib, "sa_attn_workspace_bytes", lambda: 0)
    without = _run(q, k, v, mask, 128, 32, impl="tcgen05")
    assert torch.equal(with_ws, without)


@pytest.mark.parametrize("impl,dtype", [("tcgen05", torch.bfloat16), ("simt", torch.bfloat16), ("simt", torch.float32)])
def test_lse_output(native_lib, impl, dtype):
    """The optional log-sum-exp of a row's scaled scores over its attended keys (natural log), against
    torch.logsumexp of the masked score matrix in fp32; -inf where a row attends to nothing."""
    B, H, S, D = 1, 2, 512, 128
    q, k, v = workloads.make_qkv(B, H, S, D, dtype, seed=51)
    mask = workloads.random_block_mask(B, S, 0.5, 0.2, seed=52)
    mask[:, :, 5, :] = False                                        # a row with no key
    mask[:, :, 128:256, :] = False                                  # a whole query block with none
    scores = torch.einsum("bhqd,bhkd->bhqk", q.float(), k.float()) * D ** -0.5
    ref = torch.logsumexp(scores.masked_fill(~mask.expand(B, H, S, S), float("-inf")), dim=-1)
    out, lse = sa.sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), mask.to(DEV), 128, 32, impl=impl,
                                   check_status=True, return_lse=True)
    torch.cuda.synchronize()
    lse = lse.cpu()
    assert lse.shape == (B, H, S) and lse.dtype == torch.float32
    empty = ~mask.expand(B, H, S, S).any(-1)
    assert torch.isneginf(lse[empty]).all() and torch.isfinite(lse[~empty]).all()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert (lse[~empty] - ref[~empty]).abs().max().item() <= tol
    assert_close_attn(out, sdpa_cpu(q, k, v, mask), dtype, f"lse run {impl}")


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
@pytest.mark.parametrize("Sq,Sk", [(256, 1024), (1024, 384)])
def test_rectangular_attention(native_lib, impl, Sq, Sk):
    """Sq != Sk (cross attention / a decode chunk against a longer cache): the reference's kernels take the
    two lengths separately (sparse_attn_kernel.py:150-151); lists, bit plane and tiles must too."""
    B, H, D = 2, 3, 128
    g = torch.Generator().manual_seed(Sq + Sk)
    q = torch.randn((B, H, Sq, D), generator=g).to(torch.bfloat16)
    k = torch.randn((B, H, Sk, D), generator=g).to(torch.bfloat16)
    v = torch.randn((B, H, Sk, D), generator=g).to(torch.bfloat16)
    blocks = torch.rand((B, 1, Sq // 32, Sk // 32), generator=g) < 0.5
    mask = blocks.repeat_interleave(32, 2).repeat_interleave(32, 3)
    noisy = torch.rand((B, 1, Sq, Sk), generator=g) < 0.5
    part = (torch.rand((B, 1, Sq // 32, Sk // 32), generator=g) < 0.2).repeat_interleave(32, 2).repeat_interleave(32, 3)
    mask = mask & (~part | noisy)
    ref = sdpa_cpu(q, k, v, mask)
    md = sa.compute_mask_kernel(mask.to(DEV).expand(B, H, Sq, Sk), 128, 32)
    assert_lists_equal(md, oc.classify(mask.expand(B, H, Sq, Sk).numpy(), 128, 32), f"rectangular {Sq}x{Sk}")
    out = _run(q, k, v, mask, 128, 32, impl=impl, md=md)
    assert out.shape == (B, H, Sq, D)
    assert_close_attn(out, ref, torch.bfloat16, f"rectangular {impl} {Sq}x{Sk}")


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
def test_shared_key_value_heads(native_lib, impl):
    """K and V given as views expanded over the heads (one kv head shared by all query heads, stride 0):
    read in place, no copy; same values as with the heads materialised."""
    B, H, S, D = 2, 4, 512, 128
    g = torch.Generator().manual_seed(91)
    q = torch.randn((B, H, S, D), generator=g).to(torch.bfloat16)
    k1 = torch.randn((B, 1, S, D), generator=g).to(torch.bfloat16)
    v1 = torch.randn((B, 1, S, D), generator=g).to(torch.bfloat16)
    mask = workloads.random_block_mask(B, S, 0.4, 0.2, seed=92)
    ref = sdpa_cpu(q, k1.expand(B, H, S, D).contiguous(), v1.expand(B, H, S, D).contiguous(), mask)
    kd, vd = k1.to(DEV).expand(B, H, S, D), v1.to(DEV).expand(B, H, S, D)
    assert kd.stride(1) == 0
    out = sa.sparse_attention(q.to(DEV), kd, vd, mask.to(DEV), 128, 32, impl=impl, check_status=True)
    torch.cuda.synchronize()
    assert_close_attn(out, ref, torch.bfloat16, f"shared kv heads {impl}")


def test_mask_metadata_cache(native_lib, monkeypatch):
    """``cache=True``: a second call on the same, unmodified mask runs no classifier and returns the same
    bits; an in-place edit of the mask (or other block sizes, or another mask) classifies again."""
    B, H, S, D = 2, 4, 1024, 128
    q, k, v = (t.to(DEV) for t in workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=71))
    mask = workloads.random_block_mask(B, S, 0.5, 0.2, seed=72).to(DEV)
    sa.clear_mask_cache()
    calls = []
    real = native_lib.sa_classify_mask
    monkeypatch.setattr(native_lib, "sa_classify_mask", lambda *a: (calls.append(1), real(*a))[1])

    plain = sa.sparse_attention(q, k, v, mask, 128, 32, check_status=True)
    assert len(calls) == 1
    first = sa.sparse_attention(q, k, v, mask, 128, 32, cache=True, check_status=True)
    assert len(calls) == 2
    for _ in range(3):                                        # "layers" sharing the mask
        again = sa.sparse_attention(q, k, v, mask.expand(B, H, S, S), 128, 32, cache=True, check_status=True)
        assert torch.equal(again, first)
    assert len(calls) == 2 and torch.equal(first, plain)
    sa.sparse_attention(q, k, v, mask, 128, 64, cache=True)   # other block sizes: another entry
    assert len(calls) == 3
    mask[0, 0, :128, :] = False                               # in-place edit: the version moves
    edited = sa.sparse_attention(q, k, v, mask, 128, 32, cache=True, check_status=True)
    assert len(calls) == 4
    assert_close_attn(edited, sdpa_cpu(q, k, v, mask), torch.bfloat16, "after the edit")
    assert bool((edited[0, :, :128] == 0).all())
    # the kernel list of a cached call holds no classifier kernel (when the profiler can see kernels here)
    try:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            sa.sparse_attention(q, k, v, mask, 128, 32, cache=True)
            torch.cuda.synchronize()
        names = [e.key for e in prof.key_averages()]
    except Exception:
        names = []
    if any("attn_fwd" in n for n in names):
        assert not any("classify" in n for n in names), names
    sa.clear_mask_cache()
    sa.sparse_attention(q, k, v, mask, 128, 32, cache=True)
    assert len(calls) == 5
    sa.clear_mask_cache()


def test_bounded_wait_runs_out_and_reports(native_lib):
    """Every mbarrier wait of the tensor-core kernel is bounded.  The library's self-test waits, with a limit
    of 1 ms, on a barrier nothing arrives on: the kernel must come back by itself, set the status word to
    "wait expired", and have waited about as long as the limit (not the kernel's 1 s default)."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    waited = torch.zeros(1, dtype=torch.int64, device=DEV)
    rc = native_lib.sa_selftest_bounded_wait(1_000_000, status.data_ptr(), waited.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == _native.SA_DEV_WAIT_EXPIRED
    assert 1_000_000 <= int(waited.item()) < 50_000_000
    # the context is still usable
    assert int((torch.ones(4, device=DEV) * 2).sum().item()) == 8
    assert native_lib.sa_selftest_bounded_wait(0, status.data_ptr(), None, None) == -1          # limits are bounded
    assert native_lib.sa_selftest_bounded_wait(10**12, status.data_ptr(), None, None) == -1
