"""``relation_lm::router_cache_update`` — stateful router-key update for one position.

Same operator name, schema and mutated arguments as the reference project's
``src/relation_lm/kernels/router_cache.py:175-241``; one launch of the sm_100a
kernel ``router_cache_update_kernel`` through the C ABI.
"""
from __future__ import annotations

import torch
from torch import Tensor

from relation_lm.kernels import _abi

_MUTATED = ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache",
            "anchor_mean", "anchor_std", "partner_mean", "partner_std")


@torch.library.custom_op("relation_lm::router_cache_update", mutates_args=_MUTATED,
                         device_types="cuda")
def router_cache_update(
    anchor_raw: Tensor,
    partner_raw: Tensor,
    anchor_raw_cache: Tensor,
    partner_raw_cache: Tensor,
    anchor_conv_cache: Tensor,
    partner_conv_cache: Tensor,
    anchor_mean: Tensor,
    anchor_std: Tensor,
    partner_mean: Tensor,
    partner_std: Tensor,
    anchor_conv_weight: Tensor,
    partner_conv_weight: Tensor,
    position: Tensor,
    block_size: int,
) -> Tensor:
    """Write raw and causally convolved router keys at ``position`` and refresh that block's
    mean / biased std for both streams.  ``anchor_raw`` / ``partner_raw`` may be column slices
    of a wider packed projection (row stride is honoured, inner stride must be 1).
    Returns the convolved keys ``[B, 2, 64]`` in fp32."""
    device = _abi.require_cuda_contiguous(
        anchor_raw_cache=anchor_raw_cache, partner_raw_cache=partner_raw_cache,
        anchor_conv_cache=anchor_conv_cache, partner_conv_cache=partner_conv_cache,
        anchor_mean=anchor_mean, anchor_std=anchor_std, partner_mean=partner_mean,
        partner_std=partner_std, anchor_conv_weight=anchor_conv_weight,
        partner_conv_weight=partner_conv_weight)
    for name, raw in (("anchor_raw", anchor_raw), ("partner_raw", partner_raw)):
        if raw.device != device or raw.dim() != 2 or raw.size(1) != 64 or raw.stride(1) != 1:
            raise ValueError(f"{name} must be a [B, 64] CUDA tensor with unit inner stride")
    _abi.require_position(position, device)
    batch = anchor_raw.size(0)
    if anchor_raw_cache.size(2) != 64 or anchor_mean[0, 0].numel() != 64:
        raise ValueError("this build supports router width 64")
    out = torch.empty((batch, 2, 64), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_router_cache_update(
            _abi.ptr(anchor_raw), anchor_raw.stride(0), _abi.ptr(partner_raw), partner_raw.stride(0),
            _abi.ptr(anchor_raw_cache), _abi.ptr(partner_raw_cache), _abi.ptr(anchor_conv_cache),
            _abi.ptr(partner_conv_cache), _abi.ptr(anchor_mean), _abi.ptr(anchor_std),
            _abi.ptr(partner_mean), _abi.ptr(partner_std), _abi.ptr(anchor_conv_weight),
            _abi.ptr(partner_conv_weight), _abi.ptr(position), _abi.ptr(out), batch,
            anchor_raw_cache.size(1), anchor_mean.size(1), int(block_size),
            _abi.same_dtype("raw key", anchor_raw, partner_raw),
            _abi.same_dtype("router cache", anchor_raw_cache, partner_raw_cache,
                            anchor_conv_cache, partner_conv_cache),
            _abi.same_dtype("block statistics", anchor_mean, anchor_std, partner_mean, partner_std),
            _abi.same_dtype("conv weight", anchor_conv_weight, partner_conv_weight),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out


@router_cache_update.register_fake
def _(anchor_raw, partner_raw, anchor_raw_cache, partner_raw_cache, anchor_conv_cache,
      partner_conv_cache, anchor_mean, anchor_std, partner_mean, partner_std,
      anchor_conv_weight, partner_conv_weight, position, block_size):
    return anchor_raw.new_empty((anchor_raw.size(0), 2, anchor_raw.size(1)), dtype=torch.float32)


_APPEND_MUTATED = ("anchor_keys", "partner_keys", "operand_cache", "partner_anchor_cache") + _MUTATED


@torch.library.custom_op("relation_lm::sparse_cache_append", mutates_args=_APPEND_MUTATED,
                         device_types="cuda")
def sparse_cache_append(
    packed: Tensor,
    anchor_keys: Tensor,
    partner_keys: Tensor,
    operand_cache: Tensor,
    partner_anchor_cache: Tensor,
    anchor_raw_cache: Tensor,
    partner_raw_cache: Tensor,
    anchor_conv_cache: Tensor,
    partner_conv_cache: Tensor,
    anchor_mean: Tensor,
    anchor_std: Tensor,
    partner_mean: Tensor,
    partner_std: Tensor,
    anchor_conv_weight: Tensor,
    partner_conv_weight: Tensor,
    position: Tensor,
    block_size: int,
) -> None:
    """All layers of a stack at once: write the packed projection's token features into row
    ``position`` of their caches and update both router streams (extension of
    ``router_cache_update``; every cache carries a leading layer dimension and ``packed`` is
    ``[B, layers * (384 + R)]`` in the packed column order)."""
    device = _abi.require_cuda_contiguous(
        anchor_keys=anchor_keys, partner_keys=partner_keys, operand_cache=operand_cache,
        partner_anchor_cache=partner_anchor_cache, anchor_raw_cache=anchor_raw_cache,
        partner_raw_cache=partner_raw_cache, anchor_conv_cache=anchor_conv_cache,
        partner_conv_cache=partner_conv_cache, anchor_mean=anchor_mean, anchor_std=anchor_std,
        partner_mean=partner_mean, partner_std=partner_std, anchor_conv_weight=anchor_conv_weight,
        partner_conv_weight=partner_conv_weight)
    _abi.require_cuda_rows(packed=packed)
    _abi.require_position(position, device)
    layers, batch, max_t, rdim = operand_cache.shape
    if packed.shape != (batch, layers * (384 + rdim)) or anchor_keys.shape != (layers, batch, max_t, 64) \
            or partner_anchor_cache.shape != (layers, batch, max_t, 128) \
            or anchor_raw_cache.shape != (layers, batch, max_t, 64) or anchor_mean.size(0) != layers:
        raise ValueError("caches must be [layers, B, T, width] and packed [B, layers * (384 + R)]")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_sparse_cache_append(
            _abi.ptr(packed), packed.stride(0), rdim, _abi.ptr(anchor_keys), _abi.ptr(partner_keys),
            _abi.ptr(operand_cache), _abi.ptr(partner_anchor_cache), _abi.ptr(anchor_raw_cache),
            _abi.ptr(partner_raw_cache), _abi.ptr(anchor_conv_cache), _abi.ptr(partner_conv_cache),
            _abi.ptr(anchor_mean), _abi.ptr(anchor_std), _abi.ptr(partner_mean), _abi.ptr(partner_std),
            _abi.ptr(anchor_conv_weight), _abi.ptr(partner_conv_weight), _abi.ptr(position), None,
            layers, batch, max_t, anchor_mean.size(2), int(block_size), _abi.code(packed),
            _abi.same_dtype("cache", anchor_keys, partner_keys, operand_cache, partner_anchor_cache,
                            anchor_raw_cache, partner_raw_cache, anchor_conv_cache, partner_conv_cache),
            _abi.same_dtype("block statistics", anchor_mean, anchor_std, partner_mean, partner_std),
            _abi.same_dtype("conv weight", anchor_conv_weight, partner_conv_weight),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@sparse_cache_append.register_fake
def _(packed, anchor_keys, partner_keys, operand_cache, partner_anchor_cache, anchor_raw_cache,
      partner_raw_cache, anchor_conv_cache, partner_conv_cache, anchor_mean, anchor_std,
      partner_mean, partner_std, anchor_conv_weight, partner_conv_weight, position, block_size):
    return None


@torch.library.custom_op("relation_lm::router_cache_prefill", mutates_args=_MUTATED,
                         device_types="cuda")
def router_cache_prefill(
    anchor_raw: Tensor,
    partner_raw: Tensor,
    anchor_raw_cache: Tensor,
    partner_raw_cache: Tensor,
    anchor_conv_cache: Tensor,
    partner_conv_cache: Tensor,
    anchor_mean: Tensor,
    anchor_std: Tensor,
    partner_mean: Tensor,
    partner_std: Tensor,
    anchor_conv_weight: Tensor,
    partner_conv_weight: Tensor,
    block_size: int,
) -> None:
    """Fill zero-initialised router caches and block statistics for a whole prefix
    ``anchor_raw, partner_raw [B, length, 64]`` in one launch (extension); the state equals that
    of ``length`` successive ``router_cache_update`` calls."""
    device = _abi.require_cuda_contiguous(
        anchor_raw_cache=anchor_raw_cache, partner_raw_cache=partner_raw_cache,
        anchor_conv_cache=anchor_conv_cache, partner_conv_cache=partner_conv_cache,
        anchor_mean=anchor_mean, anchor_std=anchor_std, partner_mean=partner_mean,
        partner_std=partner_std, anchor_conv_weight=anchor_conv_weight,
        partner_conv_weight=partner_conv_weight)
    for name, raw in (("anchor_raw", anchor_raw), ("partner_raw", partner_raw)):
        if raw.device != device or raw.dim() != 3 or raw.size(2) != 64 or raw.stride(2) != 1:
            raise ValueError(f"{name} must be a [B, length, 64] CUDA tensor with unit inner stride")
    batch, length = anchor_raw.size(0), anchor_raw.size(1)
    if partner_raw.shape != anchor_raw.shape:
        raise ValueError("anchor_raw and partner_raw must have the same shape")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_router_cache_prefill(
            _abi.ptr(anchor_raw), anchor_raw.stride(1), anchor_raw.stride(0), _abi.ptr(partner_raw),
            partner_raw.stride(1), partner_raw.stride(0), _abi.ptr(anchor_raw_cache),
            _abi.ptr(partner_raw_cache), _abi.ptr(anchor_conv_cache), _abi.ptr(partner_conv_cache),
            _abi.ptr(anchor_mean), _abi.ptr(anchor_std), _abi.ptr(partner_mean), _abi.ptr(partner_std),
            _abi.ptr(anchor_conv_weight), _abi.ptr(partner_conv_weight), length, batch,
            anchor_raw_cache.size(1), anchor_mean.size(1), int(block_size),
            _abi.same_dtype("raw key", anchor_raw, partner_raw),
            _abi.same_dtype("router cache", anchor_raw_cache, partner_raw_cache,
                            anchor_conv_cache, partner_conv_cache),
            _abi.same_dtype("block statistics", anchor_mean, anchor_std, partner_mean, partner_std),
            _abi.same_dtype("conv weight", anchor_conv_weight, partner_conv_weight),
            _abi.stream_ptr(device)))


@router_cache_prefill.register_fake
def _(anchor_raw, partner_raw, anchor_raw_cache, partner_raw_cache, anchor_conv_cache,
      partner_conv_cache, anchor_mean, anchor_std, partner_mean, partner_std,
      anchor_conv_weight, partner_conv_weight, block_size):
    return None


@torch.library.custom_op("relation_lm::packed_projection_append", mutates_args=_APPEND_MUTATED, device_types="cuda")
def packed_projection_append(
    x: Tensor,
    weight: Tensor,
    anchor_keys: Tensor,
    partner_keys: Tensor,
    operand_cache: Tensor,
    partner_anchor_cache: Tensor,
    anchor_raw_cache: Tensor,
    partner_raw_cache: Tensor,
    anchor_conv_cache: Tensor,
    partner_conv_cache: Tensor,
    anchor_mean: Tensor,
    anchor_std: Tensor,
    partner_mean: Tensor,
    partner_std: Tensor,
    anchor_conv_weight: Tensor,
    partner_conv_weight: Tensor,
    position: Tensor,
    block_size: int,
) -> Tensor:
    """The packed projection of one decode position for all layers with ``sparse_cache_append`` in its
    epilogue (extension; decode batches of at most 16 rows, ``d`` 256 or 512): one launch writes the
    token-cache rows and updates both router streams of every layer, each output element by the
    thread that computed it.  Returns the packed rows ``[B, layers * (384 + R)]``; the state equals
    ``sparse_cache_append(skinny_projection(x, weight), ...)`` bit for bit."""
    device = _abi.require_cuda_contiguous(
        weight=weight, anchor_keys=anchor_keys, partner_keys=partner_keys, operand_cache=operand_cache,
        partner_anchor_cache=partner_anchor_cache, anchor_raw_cache=anchor_raw_cache,
        partner_raw_cache=partner_raw_cache, anchor_conv_cache=anchor_conv_cache,
        partner_conv_cache=partner_conv_cache, anchor_mean=anchor_mean, anchor_std=anchor_std,
        partner_mean=partner_mean, partner_std=partner_std, anchor_conv_weight=anchor_conv_weight,
        partner_conv_weight=partner_conv_weight)
    _abi.require_cuda_rows(x=x)
    _abi.require_position(position, device)
    layers, batch, max_t, rdim = operand_cache.shape
    width = 384 + rdim
    if x.shape[0] != batch or weight.shape != (layers * width, x.shape[1]) or anchor_keys.shape != (layers, batch, max_t, 64) \
            or partner_anchor_cache.shape != (layers, batch, max_t, 128) or anchor_raw_cache.shape != (layers, batch, max_t, 64) \
            or anchor_mean.size(0) != layers or anchor_conv_weight.shape != (layers, 64, 3):
        raise ValueError("caches must be [layers, B, T, width], weight [layers * (384 + R), d], conv weights [layers, 64, 3]")
    if anchor_conv_weight.dtype != torch.float32 or partner_conv_weight.dtype != torch.float32:
        raise ValueError("conv weights must be float32")
    dtype = _abi.same_dtype("16-bit operand", x, weight, anchor_keys, partner_keys, operand_cache, partner_anchor_cache,
                            anchor_raw_cache, partner_raw_cache, anchor_conv_cache, partner_conv_cache, anchor_mean,
                            anchor_std, partner_mean, partner_std)
    packed = torch.empty((batch, layers * width), device=device, dtype=x.dtype)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_packed_projection_append(
            _abi.ptr(x), x.stride(0), _abi.ptr(weight), _abi.ptr(packed), rdim, _abi.ptr(anchor_keys),
            _abi.ptr(partner_keys), _abi.ptr(operand_cache), _abi.ptr(partner_anchor_cache),
            _abi.ptr(anchor_raw_cache), _abi.ptr(partner_raw_cache), _abi.ptr(anchor_conv_cache),
            _abi.ptr(partner_conv_cache), _abi.ptr(anchor_mean), _abi.ptr(anchor_std), _abi.ptr(partner_mean),
            _abi.ptr(partner_std), _abi.ptr(anchor_conv_weight), _abi.ptr(partner_conv_weight), _abi.ptr(position),
            layers, batch, x.size(1), max_t, anchor_mean.size(2), int(block_size), dtype,
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return packed


@packed_projection_append.register_fake
def _(x, weight, anchor_keys, partner_keys, operand_cache, partner_anchor_cache, anchor_raw_cache,
      partner_raw_cache, anchor_conv_cache, partner_conv_cache, anchor_mean, anchor_std, partner_mean,
      partner_std, anchor_conv_weight, partner_conv_weight, position, block_size):
    return x.new_empty((x.size(0), weight.size(0)))


def state_slide(tensors: list[Tensor], shifts: list[int], row_dim: int | list[int] = -2) -> None:
    """Slide position-indexed caches in place (extension; ``rlm_state_slide``): tensor ``k`` — contiguous,
    rows along ``row_dim`` (one value, or one per tensor: the position axis -2 of a cache ``[..., T, width]``,
    the block axis -3 of the router statistics ``[..., blocks, heads, width]``) — moves rows ``[shifts[k], rows)`` to the front and keeps its last
    ``shifts[k]`` rows as they were.  Up to 16 tensors per launch; longer lists take several launches.
    Not a registered operator: a decoder calls it between steps, outside its captured graph."""
    import ctypes

    if len(tensors) != len(shifts):
        raise ValueError("one shift per tensor")
    if not tensors:
        return
    device = tensors[0].device
    entries = []
    dims = list(row_dim) if isinstance(row_dim, (list, tuple)) else [row_dim] * len(tensors)
    if len(dims) != len(tensors):
        raise ValueError("one row_dim per tensor")
    for t, shift, axis in zip(tensors, shifts, dims):
        if t.numel() == 0:
            continue
        if not t.is_cuda or t.device != device or not t.is_contiguous():
            raise ValueError("state_slide takes contiguous CUDA tensors of one device")
        dim = int(axis) % t.dim()
        rows = t.size(dim)
        outer = 1
        for d in range(dim):
            outer *= t.size(d)
        inner = t.element_size()
        for d in range(dim + 1, t.dim()):
            inner *= t.size(d)
        if not 0 <= int(shift) < rows:
            raise ValueError("shift must be in [0, rows)")
        entries.append((t.data_ptr(), outer, rows, inner, int(shift)))
    for first in range(0, len(entries), 16):
        part = entries[first:first + 16]
        n = len(part)
        ptrs = (ctypes.c_void_p * n)(*[e[0] for e in part])
        cols = [(ctypes.c_int64 * n)(*[e[i] for e in part]) for i in (1, 2, 3, 4)]
        with _abi.device_guard(device):
            _abi.check(_abi.LIB.rlm_state_slide(ptrs, *cols, n, _abi.stream_ptr(device)))
