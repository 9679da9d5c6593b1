"""Inference helpers of the sparse decode path."""

from relation_lm.inference.packed_cache import (
    SPARSE_CACHE_NAMES,
    PackedSparseCacheProjection,
    pack_sparse_cache_projection_weights,
)

__all__ = [
    "SPARSE_CACHE_NAMES",
    "PackedSparseCacheProjection",
    "pack_sparse_cache_projection_weights",
]
