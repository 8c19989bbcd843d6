"""Generates ``reference_vectors.npz``: inputs and the outputs of the REFERENCE itself.

Run where a checkout of the reference (tomatillos/sparseattention) and triton are available; no GPU
is needed:

    python tests/golden/make_golden.py --reference /path/to/sparseattention-checkout

What it records, per case:

* the lists of the reference's pure-torch ``compute_mask_slow`` (mask_utils.py:14-44),
* the lists of its Triton classifier ``compute_mask_kernel`` (mask_utils.py:85-107) run
  under the Triton CPU interpreter (only ``ids[..., :len]`` is defined there; the tails
  are overwritten with -1 before saving),
* the output of its Triton attention kernel ``sparse_attention``
  (sparse_attn_kernel.py:149-185) under the interpreter in fp32, with the autotuner
  wrapper bypassed (it needs a GPU driver).  NaN rows are kept as they come out.

Inputs: Q, K, V ~ N(0,1) rounded to fp16 (so the same values feed fp16 and fp32 runs);
masks from this repository's seeded generators.  The script is the only thing that reads
the reference; the tests read the ``.npz`` only.
"""
import argparse
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import workloads  # noqa: E402

CASES = [
    # name, mask kind, BLOCK_Q, BLOCK_K
    ("random_128x32", "random", 128, 32),
    ("random_32x32", "random", 32, 32),
    ("random_32x128", "random", 32, 128),
    ("document_64x64", "document", 64, 64),
    ("document_128x32", "document", 128, 32),
]
B, H, S, D = 1, 2, 256, 64


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import sparseattention.mask_utils as mu
    import sparseattention.sparse_attn_kernel as sak

    # the autotuner needs an active GPU driver; its wrapped function is the kernel itself
    sak.sparse_attention_kernel = sak.sparse_attention_kernel.fn

    g = torch.Generator().manual_seed(20240607)
    q, k, v = (torch.randn((B, H, S, D), generator=g).to(torch.float16) for _ in range(3))
    masks = {
        "random": workloads.random_block_mask(B, S, 0.5, 0.1, seed=11),
        "document": workloads.document_causal_mask(B, S, (40, 100), 0.0, seed=12),
    }
    out = {"q": q.numpy(), "k": k.numpy(), "v": v.numpy()}
    for name, m in masks.items():
        out[f"mask_{name}"] = np.packbits(m.numpy().astype(np.uint8), axis=-1)

    def trim(ids, lens):
        ids = ids.clone()
        pos = torch.arange(ids.shape[-1])
        ids[pos >= lens[..., None]] = -1
        return ids.numpy().astype(np.int32)

    for name, kind, bq, bk in CASES:
        mask = masks[kind].expand(B, H, S, S)
        slow = mu.compute_mask_slow(mask, bq, bk)
        kern = mu.compute_mask_kernel(mask, bq, bk)
        for tag, md in (("slow", slow), ("triton", kern)):
            out[f"{name}/{tag}/full_ids"] = trim(md.unmasked_kv_ids, md.unmasked_lens)
            out[f"{name}/{tag}/full_lens"] = md.unmasked_lens.numpy().astype(np.int32)
            out[f"{name}/{tag}/part_ids"] = trim(md.masked_kv_ids, md.masked_lens)
            out[f"{name}/{tag}/part_lens"] = md.masked_lens.numpy().astype(np.int32)
        o = sak.sparse_attention(q.float(), k.float(), v.float(), mask, bq, bk, mask_metadata=kern)
        out[f"{name}/attn_out"] = o.numpy().astype(np.float32)
        print(name, "nan rows:", int(torch.isnan(o).any(-1).sum()), "of", B * H * S)

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
