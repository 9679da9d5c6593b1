"""``relation_lm::relation_select_packed`` — fused routed anchor/partner selection.

Same operator name, schema and semantics as the reference project's
``src/relation_lm/kernels/relation_select.py:311-382`` (compatibility and
strict-valid remote-block rules included); the body is one launch of the
sm_100a kernel ``relation_select_kernel`` through the C ABI.
``relation_select_packed_rows`` is an additive extension for query rows that
carry their own sequence index and position (prefill).
"""
from __future__ import annotations

import torch
from torch import Tensor

from relation_lm.kernels import _abi


def _select(anchor_query, anchor_keys, anchor_router_query, anchor_block_mean, anchor_block_std,
            anchor_gamma, anchor_bias, partner_base, partner_anchor_cache, partner_keys,
            partner_block_mean, partner_block_std, partner_gamma, partner_bias, position,
            row_batch, row_position, local_window, top_blocks, k_out, strict_valid):
    _abi.require_cuda_rows(anchor_query=anchor_query, anchor_router_query=anchor_router_query,
                           partner_base=partner_base)
    device = _abi.require_cuda_contiguous(
        anchor_keys=anchor_keys,
        anchor_block_mean=anchor_block_mean, anchor_block_std=anchor_block_std,
        anchor_gamma=anchor_gamma, anchor_bias=anchor_bias,
        partner_anchor_cache=partner_anchor_cache, partner_keys=partner_keys,
        partner_block_mean=partner_block_mean, partner_block_std=partner_block_std,
        partner_gamma=partner_gamma, partner_bias=partner_bias, row_batch=row_batch,
        row_position=row_position)
    rows = anchor_query.size(0)
    n_seq, max_t = anchor_keys.size(0), anchor_keys.size(1)
    n_blocks = anchor_block_mean.size(1)
    if anchor_query.size(1) != 64 or anchor_block_mean.size(2) * anchor_block_mean.size(3) != 64 \
            or anchor_block_mean.size(3) != 16 or partner_base.size(1) != 128:
        raise ValueError("this build supports gate width 64 with 4 router heads of width 16")
    if position is not None:
        _abi.require_position(position, device)
    query_dtype = _abi.same_dtype("query", anchor_query, anchor_router_query, partner_base)
    key_dtype = _abi.same_dtype("key cache", anchor_keys, partner_keys, partner_anchor_cache)
    stats_dtype = _abi.same_dtype("block statistics", anchor_block_mean, anchor_block_std,
                                  partner_block_mean, partner_block_std)
    param_dtype = _abi.same_dtype("gamma/bias", anchor_gamma, anchor_bias, partner_gamma, partner_bias)
    out_anchor = torch.empty((rows,), device=device, dtype=torch.int32)
    out_anchor_score = torch.empty((rows,), device=device, dtype=torch.float32)
    out_partner = torch.empty((rows, k_out), device=device, dtype=torch.int32)
    out_partner_score = torch.empty((rows, k_out), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_select_packed(
            _abi.ptr(anchor_query), _abi.ptr(anchor_keys), _abi.ptr(anchor_router_query),
            _abi.ptr(anchor_block_mean), _abi.ptr(anchor_block_std), _abi.ptr(anchor_gamma),
            _abi.ptr(anchor_bias), _abi.ptr(partner_base), _abi.ptr(partner_anchor_cache),
            _abi.ptr(partner_keys), _abi.ptr(partner_block_mean), _abi.ptr(partner_block_std),
            _abi.ptr(partner_gamma), _abi.ptr(partner_bias), _abi.ptr(position),
            _abi.ptr(row_batch), _abi.ptr(row_position), _abi.ptr(out_anchor),
            _abi.ptr(out_anchor_score), _abi.ptr(out_partner), _abi.ptr(out_partner_score),
            anchor_query.stride(0), anchor_router_query.stride(0), partner_base.stride(0),
            rows, n_seq, max_t, n_blocks, anchor_bias.size(1), int(local_window), int(top_blocks),
            int(k_out), int(bool(strict_valid)), query_dtype, key_dtype, stats_dtype, param_dtype,
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out_anchor, out_anchor_score, out_partner, out_partner_score


@torch.library.custom_op("relation_lm::relation_select_packed", mutates_args=(),
                         device_types="cuda")
def relation_select_packed(
    anchor_query: Tensor,
    anchor_keys: Tensor,
    anchor_router_query: Tensor,
    anchor_block_mean: Tensor,
    anchor_block_std: Tensor,
    anchor_gamma: Tensor,
    anchor_bias: Tensor,
    partner_base: Tensor,
    partner_anchor_cache: Tensor,
    partner_keys: Tensor,
    partner_block_mean: Tensor,
    partner_block_std: Tensor,
    partner_gamma: Tensor,
    partner_bias: Tensor,
    position: Tensor,
    local_window: int,
    top_blocks: int,
    k_out: int,
    strict_valid: bool,
) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """Anchor index/score ``[B]`` and partner indices/scores ``[B, k_out]`` at ``position``."""
    return _select(anchor_query, anchor_keys, anchor_router_query, anchor_block_mean,
                   anchor_block_std, anchor_gamma, anchor_bias, partner_base,
                   partner_anchor_cache, partner_keys, partner_block_mean, partner_block_std,
                   partner_gamma, partner_bias, position, None, None, local_window, top_blocks,
                   k_out, strict_valid)


@relation_select_packed.register_fake
def _(anchor_query, anchor_keys, anchor_router_query, anchor_block_mean, anchor_block_std,
      anchor_gamma, anchor_bias, partner_base, partner_anchor_cache, partner_keys,
      partner_block_mean, partner_block_std, partner_gamma, partner_bias, position, local_window,
      top_blocks, k_out, strict_valid):
    rows = anchor_query.size(0)
    return (anchor_query.new_empty((rows,), dtype=torch.int32),
            anchor_query.new_empty((rows,), dtype=torch.float32),
            anchor_query.new_empty((rows, k_out), dtype=torch.int32),
            anchor_query.new_empty((rows, k_out), dtype=torch.float32))


@torch.library.custom_op("relation_lm::relation_select_packed_rows", mutates_args=(),
                         device_types="cuda")
def relation_select_packed_rows(
    anchor_query: Tensor,
    anchor_keys: Tensor,
    anchor_router_query: Tensor,
    anchor_block_mean: Tensor,
    anchor_block_std: Tensor,
    anchor_gamma: Tensor,
    anchor_bias: Tensor,
    partner_base: Tensor,
    partner_anchor_cache: Tensor,
    partner_keys: Tensor,
    partner_block_mean: Tensor,
    partner_block_std: Tensor,
    partner_gamma: Tensor,
    partner_bias: Tensor,
    row_batch: Tensor,
    row_position: Tensor,
    local_window: int,
    top_blocks: int,
    k_out: int,
    strict_valid: bool,
) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """Per-row form: query row ``i`` selects in sequence ``row_batch[i]`` at ``row_position[i]``.

    Row ``i`` equals ``relation_select_packed`` called with ``position = row_position[i]`` on
    that sequence, given block statistics that are final for every complete block.
    """
    if row_batch.dtype != torch.int32 or row_position.dtype != torch.int32:
        raise ValueError("row_batch and row_position must be int32")
    if row_batch.numel() != anchor_query.size(0) or row_position.numel() != anchor_query.size(0):
        raise ValueError("row_batch and row_position need one entry per query row")
    return _select(anchor_query, anchor_keys, anchor_router_query, anchor_block_mean,
                   anchor_block_std, anchor_gamma, anchor_bias, partner_base,
                   partner_anchor_cache, partner_keys, partner_block_mean, partner_block_std,
                   partner_gamma, partner_bias, None, row_batch, row_position, local_window,
                   top_blocks, k_out, strict_valid)


@relation_select_packed_rows.register_fake
def _(anchor_query, anchor_keys, anchor_router_query, anchor_block_mean, anchor_block_std,
      anchor_gamma, anchor_bias, partner_base, partner_anchor_cache, partner_keys,
      partner_block_mean, partner_block_std, partner_gamma, partner_bias, row_batch, row_position,
      local_window, top_blocks, k_out, strict_valid):
    rows = anchor_query.size(0)
    return (anchor_query.new_empty((rows,), dtype=torch.int32),
            anchor_query.new_empty((rows,), dtype=torch.float32),
            anchor_query.new_empty((rows, k_out), dtype=torch.int32),
            anchor_query.new_empty((rows, k_out), dtype=torch.float32))


@torch.library.custom_op("relation_lm::relation_select_packed_prefill", mutates_args=(), device_types="cuda")
def relation_select_packed_prefill(
    anchor_query: Tensor,
    anchor_keys: Tensor,
    anchor_router_query: Tensor,
    anchor_block_mean: Tensor,
    anchor_block_std: Tensor,
    anchor_gamma: Tensor,
    anchor_bias: Tensor,
    partner_base: Tensor,
    partner_anchor_cache: Tensor,
    partner_keys: Tensor,
    partner_block_mean: Tensor,
    partner_block_std: Tensor,
    partner_gamma: Tensor,
    partner_bias: Tensor,
    query_length: int,
    local_window: int,
    top_blocks: int,
    k_out: int,
    strict_valid: bool,
) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """Whole-sequence form (extension): the queries are rows ``b * query_length + t`` for every
    position ``t < query_length`` of every sequence ``b`` of caches ``[B, T, ...]``; row ``(b, t)``
    equals ``relation_select_packed`` at ``position = t`` on sequence ``b`` (given final block
    statistics), bit for bit.  A CTA serves a tile of consecutive positions: their shared block
    statistics and the union of their local windows are staged once, and every warp walks one
    query's chain at a time.  At most 512 candidates per query (window + remote blocks)."""
    _abi.require_cuda_rows(anchor_query=anchor_query, anchor_router_query=anchor_router_query,
                           partner_base=partner_base)
    device = _abi.require_cuda_contiguous(
        anchor_keys=anchor_keys, anchor_block_mean=anchor_block_mean, anchor_block_std=anchor_block_std,
        anchor_gamma=anchor_gamma, anchor_bias=anchor_bias, partner_anchor_cache=partner_anchor_cache,
        partner_keys=partner_keys, partner_block_mean=partner_block_mean, partner_block_std=partner_block_std,
        partner_gamma=partner_gamma, partner_bias=partner_bias)
    n_seq, max_t = anchor_keys.size(0), anchor_keys.size(1)
    rows = n_seq * int(query_length)
    if anchor_query.shape != (rows, 64) or anchor_router_query.shape != (rows, 64) or partner_base.shape != (rows, 128):
        raise ValueError("queries must hold one row per (sequence, position): [B * query_length, width]")
    if anchor_block_mean.size(2) * anchor_block_mean.size(3) != 64 or anchor_block_mean.size(3) != 16:
        raise ValueError("this build supports gate width 64 with 4 router heads of width 16")
    query_dtype = _abi.same_dtype("query", anchor_query, anchor_router_query, partner_base)
    key_dtype = _abi.same_dtype("key cache", anchor_keys, partner_keys, partner_anchor_cache)
    stats_dtype = _abi.same_dtype("block statistics", anchor_block_mean, anchor_block_std,
                                  partner_block_mean, partner_block_std)
    param_dtype = _abi.same_dtype("gamma/bias", anchor_gamma, anchor_bias, partner_gamma, partner_bias)
    out_anchor = torch.empty((rows,), device=device, dtype=torch.int32)
    out_anchor_score = torch.empty((rows,), device=device, dtype=torch.float32)
    out_partner = torch.empty((rows, k_out), device=device, dtype=torch.int32)
    out_partner_score = torch.empty((rows, k_out), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_select_packed_prefill(
            _abi.ptr(anchor_query), _abi.ptr(anchor_keys), _abi.ptr(anchor_router_query),
            _abi.ptr(anchor_block_mean), _abi.ptr(anchor_block_std), _abi.ptr(anchor_gamma),
            _abi.ptr(anchor_bias), _abi.ptr(partner_base), _abi.ptr(partner_anchor_cache),
            _abi.ptr(partner_keys), _abi.ptr(partner_block_mean), _abi.ptr(partner_block_std),
            _abi.ptr(partner_gamma), _abi.ptr(partner_bias), _abi.ptr(out_anchor), _abi.ptr(out_anchor_score),
            _abi.ptr(out_partner), _abi.ptr(out_partner_score), anchor_query.stride(0),
            anchor_router_query.stride(0), partner_base.stride(0), n_seq, int(query_length), max_t,
            anchor_block_mean.size(1), anchor_bias.size(1), int(local_window), int(top_blocks), int(k_out),
            int(bool(strict_valid)), query_dtype, key_dtype, stats_dtype, param_dtype,
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out_anchor, out_anchor_score, out_partner, out_partner_score


@relation_select_packed_prefill.register_fake
def _(anchor_query, anchor_keys, anchor_router_query, anchor_block_mean, anchor_block_std, anchor_gamma,
      anchor_bias, partner_base, partner_anchor_cache, partner_keys, partner_block_mean, partner_block_std,
      partner_gamma, partner_bias, query_length, local_window, top_blocks, k_out, strict_valid):
    rows = anchor_query.size(0)
    return (anchor_query.new_empty((rows,), dtype=torch.int32), anchor_query.new_empty((rows,), dtype=torch.float32),
            anchor_query.new_empty((rows, k_out), dtype=torch.int32),
            anchor_query.new_empty((rows, k_out), dtype=torch.float32))
