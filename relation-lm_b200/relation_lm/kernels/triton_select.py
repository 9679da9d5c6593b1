"""``relationlex::anchor_select`` and ``relationlex::partner_topk`` — the two-operator selectors.

The module keeps the reference project's import path
(``src/relation_lm/kernels/triton_select.py:255-346``) and operator namespace;
nothing here uses Triton.  Both operators are modes of the sm_100a kernel that
also serves ``relation_lm::relation_select_packed``.
"""
from __future__ import annotations

import torch
from torch import Tensor

from relation_lm.kernels import _abi


def _check_router(block_mean: Tensor, query: Tensor) -> None:
    if query.size(1) != 64 or block_mean.size(2) * block_mean.size(3) != 64 or block_mean.size(3) != 16:
        raise ValueError("this build supports gate width 64 with 4 router heads of width 16")


@torch.library.custom_op("relationlex::anchor_select", mutates_args=(), device_types="cuda")
def anchor_select(
    anchor_query: Tensor,
    anchor_keys: Tensor,
    router_query: Tensor,
    block_mean: Tensor,
    block_std: Tensor,
    gamma: Tensor,
    bias: Tensor,
    position: Tensor,
    local_window: int,
    top_blocks: int,
    strict_valid: bool,
) -> tuple[Tensor, Tensor]:
    """Exact top-1 anchor over the local window and the ``top_blocks`` best remote blocks."""
    device = _abi.require_cuda_contiguous(
        anchor_query=anchor_query, anchor_keys=anchor_keys, router_query=router_query,
        block_mean=block_mean, block_std=block_std, gamma=gamma, bias=bias)
    _check_router(block_mean, anchor_query)
    _abi.require_position(position, device)
    rows = anchor_query.size(0)
    out_index = torch.empty((rows,), device=device, dtype=torch.int32)
    out_score = torch.empty((rows,), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_anchor_select(
            _abi.ptr(anchor_query), _abi.ptr(anchor_keys), _abi.ptr(router_query),
            _abi.ptr(block_mean), _abi.ptr(block_std), _abi.ptr(gamma), _abi.ptr(bias),
            _abi.ptr(position), None, None, None, 0, _abi.ptr(out_index), _abi.ptr(out_score),
            rows, anchor_keys.size(0), anchor_keys.size(1), block_mean.size(1), bias.size(1),
            int(local_window), int(top_blocks), int(bool(strict_valid)),
            _abi.same_dtype("query", anchor_query, router_query), _abi.code(anchor_keys),
            _abi.same_dtype("block statistics", block_mean, block_std),
            _abi.same_dtype("gamma/bias", gamma, bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out_index, out_score


@anchor_select.register_fake
def _(anchor_query, anchor_keys, router_query, block_mean, block_std, gamma, bias, position,
      local_window, top_blocks, strict_valid):
    rows = anchor_query.size(0)
    return (anchor_query.new_empty((rows,), dtype=torch.int32),
            anchor_query.new_empty((rows,), dtype=torch.float32))


@torch.library.custom_op("relationlex::partner_topk", mutates_args=(), device_types="cuda")
def partner_topk(
    partner_query: Tensor,
    partner_keys: Tensor,
    router_query: Tensor,
    block_mean: Tensor,
    block_std: Tensor,
    gamma: Tensor,
    bias: Tensor,
    position: Tensor,
    anchor_index: Tensor,
    local_window: int,
    top_blocks: int,
    k_out: int,
    strict_valid: bool,
) -> tuple[Tensor, Tensor]:
    """Exact top-``k_out`` partners, the anchor excluded, for precomputed partner queries."""
    device = _abi.require_cuda_contiguous(
        partner_query=partner_query, partner_keys=partner_keys, router_query=router_query,
        block_mean=block_mean, block_std=block_std, gamma=gamma, bias=bias,
        anchor_index=anchor_index)
    _check_router(block_mean, partner_query)
    _abi.require_position(position, device)
    if anchor_index.dtype != torch.int32:
        raise ValueError("anchor_index must be int32")
    rows = partner_query.size(0)
    out_index = torch.empty((rows, k_out), device=device, dtype=torch.int32)
    out_score = torch.empty((rows, k_out), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_partner_topk(
            _abi.ptr(partner_query), _abi.ptr(partner_keys), _abi.ptr(router_query),
            _abi.ptr(block_mean), _abi.ptr(block_std), _abi.ptr(gamma), _abi.ptr(bias),
            _abi.ptr(position), None, None, _abi.ptr(anchor_index), None, 0, _abi.ptr(out_index),
            _abi.ptr(out_score), rows, partner_keys.size(0), partner_keys.size(1),
            block_mean.size(1), bias.size(1), int(local_window), int(top_blocks), int(k_out),
            int(bool(strict_valid)), _abi.same_dtype("query", partner_query, router_query),
            _abi.code(partner_keys), _abi.same_dtype("block statistics", block_mean, block_std),
            _abi.same_dtype("gamma/bias", gamma, bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out_index, out_score


@partner_topk.register_fake
def _(partner_query, partner_keys, router_query, block_mean, block_std, gamma, bias, position,
      anchor_index, local_window, top_blocks, k_out, strict_valid):
    rows = partner_query.size(0)
    return (partner_query.new_empty((rows, k_out), dtype=torch.int32),
            partner_query.new_empty((rows, k_out), dtype=torch.float32))


def _check_rows(rows: int, row_batch: Tensor, row_position: Tensor, exclude_index: Tensor) -> int:
    if row_batch.dtype != torch.int32 or row_position.dtype != torch.int32 or exclude_index.dtype != torch.int32:
        raise ValueError("row_batch, row_position and exclude_index must be int32")
    if row_batch.numel() != rows or row_position.numel() != rows:
        raise ValueError("row_batch and row_position need one entry per query row")
    if exclude_index.dim() != 2 or exclude_index.size(0) != rows or exclude_index.size(1) > 8:
        raise ValueError("exclude_index must be [N, E] with E <= 8")
    return exclude_index.size(1)


@torch.library.custom_op("relationlex::anchor_select_rows", mutates_args=(), device_types="cuda")
def anchor_select_rows(
    anchor_query: Tensor,
    anchor_keys: Tensor,
    router_query: Tensor,
    block_mean: Tensor,
    block_std: Tensor,
    gamma: Tensor,
    bias: Tensor,
    row_batch: Tensor,
    row_position: Tensor,
    exclude_index: Tensor,
    local_window: int,
    top_blocks: int,
    strict_valid: bool,
) -> tuple[Tensor, Tensor]:
    """Per-row ``anchor_select`` (extension): query row ``i`` selects in sequence ``row_batch[i]``
    at ``row_position[i]``; positions listed in ``exclude_index[i]`` (entries < 0 unused) are not
    candidates.  A row with no candidate left returns index 0 and score -inf."""
    device = _abi.require_cuda_contiguous(
        anchor_query=anchor_query, anchor_keys=anchor_keys, router_query=router_query,
        block_mean=block_mean, block_std=block_std, gamma=gamma, bias=bias, row_batch=row_batch,
        row_position=row_position, exclude_index=exclude_index)
    _check_router(block_mean, anchor_query)
    rows = anchor_query.size(0)
    n_excl = _check_rows(rows, row_batch, row_position, exclude_index)
    out_index = torch.empty((rows,), device=device, dtype=torch.int32)
    out_score = torch.empty((rows,), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_anchor_select(
            _abi.ptr(anchor_query), _abi.ptr(anchor_keys), _abi.ptr(router_query),
            _abi.ptr(block_mean), _abi.ptr(block_std), _abi.ptr(gamma), _abi.ptr(bias), None,
            _abi.ptr(row_batch), _abi.ptr(row_position), _abi.ptr(exclude_index) if n_excl else None,
            n_excl, _abi.ptr(out_index), _abi.ptr(out_score), rows, anchor_keys.size(0),
            anchor_keys.size(1), block_mean.size(1), bias.size(1), int(local_window), int(top_blocks),
            int(bool(strict_valid)), _abi.same_dtype("query", anchor_query, router_query),
            _abi.code(anchor_keys), _abi.same_dtype("block statistics", block_mean, block_std),
            _abi.same_dtype("gamma/bias", gamma, bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out_index, out_score


@anchor_select_rows.register_fake
def _(anchor_query, anchor_keys, router_query, block_mean, block_std, gamma, bias, row_batch,
      row_position, exclude_index, local_window, top_blocks, strict_valid):
    rows = anchor_query.size(0)
    return (anchor_query.new_empty((rows,), dtype=torch.int32),
            anchor_query.new_empty((rows,), dtype=torch.float32))


@torch.library.custom_op("relationlex::partner_topk_rows", mutates_args=(), device_types="cuda")
def partner_topk_rows(
    partner_query: Tensor,
    partner_keys: Tensor,
    router_query: Tensor,
    block_mean: Tensor,
    block_std: Tensor,
    gamma: Tensor,
    bias: Tensor,
    row_batch: Tensor,
    row_position: Tensor,
    anchor_index: Tensor,
    exclude_index: Tensor,
    local_window: int,
    top_blocks: int,
    k_out: int,
    strict_valid: bool,
) -> tuple[Tensor, Tensor]:
    """Per-row ``partner_topk`` (extension) with the anchor and every position of
    ``exclude_index[i]`` removed from the candidates."""
    device = _abi.require_cuda_contiguous(
        partner_query=partner_query, partner_keys=partner_keys, router_query=router_query,
        block_mean=block_mean, block_std=block_std, gamma=gamma, bias=bias, row_batch=row_batch,
        row_position=row_position, anchor_index=anchor_index, exclude_index=exclude_index)
    _check_router(block_mean, partner_query)
    rows = partner_query.size(0)
    n_excl = _check_rows(rows, row_batch, row_position, exclude_index)
    if anchor_index.dtype != torch.int32 or anchor_index.numel() != rows:
        raise ValueError("anchor_index must be int32 [N]")
    out_index = torch.empty((rows, k_out), device=device, dtype=torch.int32)
    out_score = torch.empty((rows, k_out), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_partner_topk(
            _abi.ptr(partner_query), _abi.ptr(partner_keys), _abi.ptr(router_query),
            _abi.ptr(block_mean), _abi.ptr(block_std), _abi.ptr(gamma), _abi.ptr(bias), None,
            _abi.ptr(row_batch), _abi.ptr(row_position), _abi.ptr(anchor_index),
            _abi.ptr(exclude_index) if n_excl else None, n_excl, _abi.ptr(out_index),
            _abi.ptr(out_score), rows, partner_keys.size(0), partner_keys.size(1),
            block_mean.size(1), bias.size(1), int(local_window), int(top_blocks), int(k_out),
            int(bool(strict_valid)), _abi.same_dtype("query", partner_query, router_query),
            _abi.code(partner_keys), _abi.same_dtype("block statistics", block_mean, block_std),
            _abi.same_dtype("gamma/bias", gamma, bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out_index, out_score


@partner_topk_rows.register_fake
def _(partner_query, partner_keys, router_query, block_mean, block_std, gamma, bias, row_batch,
      row_position, anchor_index, exclude_index, local_window, top_blocks, k_out, strict_valid):
    rows = partner_query.size(0)
    return (partner_query.new_empty((rows, k_out), dtype=torch.int32),
            partner_query.new_empty((rows, k_out), dtype=torch.float32))
