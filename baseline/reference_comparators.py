#!/usr/bin/env python
"""Same-GPU comparators that need the reference package itself: its Triton classifier and attention
kernels (sparseattention/mask_utils.py:85, sparse_attn_kernel.py:149) and FlexAttention the way its
harness sets it up (test_attn.py:14, 45-48), timed on the headline inputs of ``bench.py``.

Run by ``bench.py`` as a child process, because the reference package and this repository's drop-in
package share the name ``sparseattention``: here ``baseline/_ref`` (an unmodified copy of the reference
package; not tracked, placed there by ``__graft_entry__.build()``) comes first on ``sys.path``.
Prints one JSON object per finished part on stdout: ``{"row": {"p": ..., ...}}`` per drop probability
and part (rows of the same p are merged by the reader), and
``{"triton": ...}`` / ``{"flex": ...}`` notes (``unavailable`` with the exception text when a part cannot
run on this machine).  Timing as in the reference harness: a warm-up (the first call of the reference
kernel also runs its autotuner over 8 configurations; excluded), then the best of a few CUDA-event
timings; the attention timing is given the lists and excludes stage 1 (test_attn.py:65).
"""
import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, os.path.join(HERE, "_ref"))          # the reference's `sparseattention`
sys.path.append(ROOT)                                   # `workloads` only; the drop-in package must not shadow

import torch  # noqa: E402


def emit(obj):
    print(json.dumps(obj), flush=True)


def best_ms(fn, n=3, warm=1):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(n):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return min(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--B", type=int, default=8)
    ap.add_argument("--H", type=int, default=32)
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--D", type=int, default=128)
    ap.add_argument("--ps", default="0.0,0.1,0.3,0.5,0.7,0.9")
    ap.add_argument("--no-flex", action="store_true")
    args = ap.parse_args()
    B, H, S, D = args.B, args.H, args.S, args.D
    ps = [float(x) for x in args.ps.split(",")]
    BQ, BK = 128, 32

    import workloads
    dev = torch.device("cuda", 0)
    q, k, v = workloads.make_qkv(B, H, S, D, torch.bfloat16, seed=1000, device=dev)          # bench.py, rank 0
    masks = [workloads.random_block_mask(B, S, p, 0.1, seed=2000 + i, device=dev) for i, p in enumerate(ps)]

    rows = {p: {"p": p} for p in ps}
    # ---- the reference's Triton kernels
    try:
        import sparseattention
        assert os.path.realpath(os.path.dirname(sparseattention.__file__)).startswith(os.path.realpath(os.path.join(HERE, "_ref")))
        from sparseattention.mask_utils import compute_mask_kernel
        from sparseattention.sparse_attn_kernel import sparse_attention
        import torch.nn.functional as F
        t0 = time.time()
        note = {}
        for p, m in zip(ps, masks):
            me = m.expand(B, H, S, S)
            md = compute_mask_kernel(me, BQ, BK)
            rows[p]["triton_mask_ms"] = best_ms(lambda: compute_mask_kernel(me, BQ, BK))
            rows[p]["triton_attn_ms"] = best_ms(lambda: sparse_attention(q, k, v, me, BQ, BK, mask_metadata=md))
            if p == 0.5:                           # its output against SDPA on the rows where it is finite
                out = sparse_attention(q[:1, :2], k[:1, :2], v[:1, :2], me[:1, :2], BQ, BK)
                ref = F.scaled_dot_product_attention(q[:1, :2], k[:1, :2], v[:1, :2], attn_mask=m[:1])
                fin = ~torch.isnan(out.float()).any(-1)
                note["nan_row_fraction"] = float((~fin).float().mean())
                note["max_abs_vs_sdpa_on_finite_rows"] = float((out.float() - ref.float())[fin].abs().max())
        note["seconds"] = round(time.time() - t0, 1)
        import triton
        note["triton_version"] = triton.__version__
        emit({"triton": note})
        for p in ps:
            emit({"row": rows[p]})
    except Exception as e:
        emit({"triton": {"unavailable": f"{type(e).__name__}: {e}"[:400]}})

    # ---- FlexAttention as the reference harness builds it (mask_mod indexing the dense mask)
    if not args.no_flex:
        try:
            from torch.nn.attention.flex_attention import create_block_mask, flex_attention
            flex = torch.compile(flex_attention)
            t0 = time.time()
            for p, m in zip(ps, masks):
                def mask_mod(b, h, q_idx, kv_idx, m=m):
                    return m[b, 0, q_idx, kv_idx]
                block_mask = create_block_mask(mask_mod, B, None, S, S, device="cuda")
                emit({"row": {"p": p, "flex_ms": best_ms(lambda: flex(q, k, v, block_mask=block_mask))}})
            emit({"flex": {"seconds": round(time.time() - t0, 1), "torch_version": torch.__version__}})
        except Exception as e:
            emit({"flex": {"unavailable": f"{type(e).__name__}: {e}"[:400]}})


if __name__ == "__main__":
    main()
