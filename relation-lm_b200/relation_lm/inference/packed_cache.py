"""Packed sparse-cache projection: six token-local projections as one matrix product.

Names, field order and validation follow the reference project's
``src/relation_lm/inference/packed_cache.py:10-94``.
"""
from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import Tensor

SPARSE_CACHE_NAMES = (
    "anchor_key",
    "partner_key",
    "operand",
    "partner_anchor",
    "anchor_router_key",
    "partner_router_key",
)


@dataclass(frozen=True)
class PackedSparseCacheProjection:
    """A ``[sum(split_sizes), d]`` weight whose product with a memory vector yields every
    per-token cache feature of sparse decode at once."""

    weight: Tensor
    split_sizes: tuple[int, ...]
    names: tuple[str, ...] = SPARSE_CACHE_NAMES

    def __post_init__(self) -> None:
        if self.weight.dim() != 2:
            raise ValueError("weight must be a 2D tensor")
        if len(self.split_sizes) != len(self.names):
            raise ValueError("split_sizes and names must have the same length")
        if min(self.split_sizes) <= 0:
            raise ValueError("split sizes must be positive")
        if sum(self.split_sizes) != self.weight.size(0):
            raise ValueError("split sizes must sum to the packed output width")

    @property
    def input_width(self) -> int:
        return int(self.weight.size(1))

    @property
    def output_width(self) -> int:
        return int(self.weight.size(0))

    def project(self, memory: Tensor) -> tuple[Tensor, ...]:
        """Project ``memory [..., d]``; the pieces come back in ``names`` order as views of
        one packed result (so the router slices keep the packed row stride)."""
        if memory.size(-1) != self.input_width:
            raise ValueError("memory width does not match packed projection input")
        if memory.is_cuda and memory.dtype in (torch.bfloat16, torch.float16) \
                and self.weight.dtype == memory.dtype and self.output_width % 32 == 0 \
                and self.input_width % 8 == 0:
            # tensor-core kernel of this library (tcgen05); fp32 operands use the library GEMM
            from relation_lm.kernels.packed_projection import packed_projection

            rows = memory.reshape(-1, self.input_width) if memory.dim() != 2 else memory
            if rows.stride(-1) != 1 or rows.stride(0) % 8 != 0:
                rows = rows.contiguous()
            packed = packed_projection(rows, self.weight).view(*memory.shape[:-1], self.output_width)
        else:
            packed = F.linear(memory, self.weight)
        return packed.split(self.split_sizes, dim=-1)

    def project_dict(self, memory: Tensor) -> dict[str, Tensor]:
        return dict(zip(self.names, self.project(memory), strict=True))


def pack_sparse_cache_projection_weights(
    weights: Sequence[Tensor],
    *,
    names: Sequence[str] = SPARSE_CACHE_NAMES,
) -> PackedSparseCacheProjection:
    """Stack per-feature projection weights (anchor key, partner key, operand, partner-anchor
    factor, anchor-router key, partner-router key) into one packed projection."""
    parts = tuple(weights)
    labels = tuple(names)
    if not parts:
        raise ValueError("at least one weight is required")
    if len(parts) != len(labels):
        raise ValueError("weights and names must have the same length")
    if any(w.dim() != 2 for w in parts):
        raise ValueError("every weight must be a 2D tensor")
    first = parts[0]
    if any(w.size(1) != first.size(1) for w in parts):
        raise ValueError("all weights must have the same input width")
    if any(w.device != first.device or w.dtype != first.dtype for w in parts):
        raise ValueError("all weights must share device and dtype")
    return PackedSparseCacheProjection(
        weight=torch.cat(parts, dim=0).contiguous(),
        split_sizes=tuple(int(w.size(0)) for w in parts),
        names=labels,
    )
