"""B200-native two-stage block-sparse attention forward, a drop-in for the Python entry
points of ``tomatillos/sparseattention``:

* ``sparseattention_b200.mask_utils``: ``MaskMetadata``, ``compute_mask_kernel``, ``compute_mask_slow``
* ``sparseattention_b200.sparse_attn_kernel``: ``sparse_attention``

The kernels are hand-written sm_100a CUDA behind a C ABI (``include/sa_b200.h``,
``libsparseattn_b200.so``).  There is no CPU fallback.
"""
from .mask_utils import MaskMetadata, compute_mask_kernel, compute_mask_slow
from .sparse_attn_kernel import cached_mask_metadata, clear_mask_cache, sparse_attention

__all__ = ["MaskMetadata", "compute_mask_kernel", "compute_mask_slow", "sparse_attention",
           "cached_mask_metadata", "clear_mask_cache"]
