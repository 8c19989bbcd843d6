"""``sparseattention.mask_utils`` of the reference (``sparseattention/mask_utils.py``), served by the
sm_100a library: the same three names, so a caller's ``from sparseattention.mask_utils import ...``
lines stay as they are.  The implementation lives in :mod:`sparseattention_b200.mask_utils`."""
from sparseattention_b200.mask_utils import MaskMetadata, compute_mask_kernel, compute_mask_slow

__all__ = ["MaskMetadata", "compute_mask_kernel", "compute_mask_slow"]
