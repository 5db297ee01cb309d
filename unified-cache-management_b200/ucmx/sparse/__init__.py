"""Sparse-attention plug-ins behind the reference's hook interface, running on the CUDA kernels."""
from .base import INVALID_SLOT, UcmSparseBase, UcmSparseMetadata, UcmSparseRole  # noqa: F401
