"""``sparseattention.sparse_attn_kernel`` of the reference (``sparseattention/sparse_attn_kernel.py:149``),
served by the sm_100a library: ``sparse_attention`` with the reference's positional signature.  The
implementation lives in :mod:`sparseattention_b200.sparse_attn_kernel`."""
from sparseattention.mask_utils import compute_mask_kernel  # the reference module exposes it too (line 7)
from sparseattention_b200.sparse_attn_kernel import sparse_attention

__all__ = ["sparse_attention", "compute_mask_kernel"]
