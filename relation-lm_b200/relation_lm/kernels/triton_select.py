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
            _abi.ptr(position), None, None, _abi.ptr(out_index), _abi.ptr(out_score),
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
            _abi.ptr(position), None, None, _abi.ptr(anchor_index), _abi.ptr(out_index),
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
