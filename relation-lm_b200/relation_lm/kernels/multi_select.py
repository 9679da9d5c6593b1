"""``relation_lm::relation_select_multi_rows`` / ``relation_select_multi_prefill`` — routed multi-anchor selection (extension).

The reference project's multi-anchor layer is dense: every slot scores all causal positions
(src/relation_lm/models/multi_relation_blocks.py:69-148).  This is its routed form, one launch
for all slots of every query row.  Its rules are the reference's, applied inside each slot's
routed candidate set (local window + that slot's best remote blocks):

* slot ``s`` is active for a query at position ``t`` iff ``s <= t``          (:82-84);
* slots choose their anchors one after another, a position taken by an earlier slot is barred
  (:86-93); an inactive slot reports anchor index 0                             (:94);
* partner selection of every slot bars the anchors of all active slots        (:133-139);
  an inactive slot has no partners                                            (:140-142);
* a partner slot is active iff its score is finite                            (:144-147).

With the window covering the whole history and no remote blocks the result equals the dense
block's selection (checked against outputs of the reference block itself).
"""
from __future__ import annotations

import torch
from torch import Tensor

from relation_lm.kernels import _abi


@torch.library.custom_op("relation_lm::relation_select_multi_rows", mutates_args=(), device_types="cuda")
def relation_select_multi_rows(
    anchor_query: Tensor,            # [N, S, 64]
    anchor_keys: Tensor,             # [S, B, T, 64]
    anchor_router_query: Tensor,     # [N, S, 64]
    anchor_block_mean: Tensor,       # [S, B, NB, 4, 16]
    anchor_block_std: Tensor,
    anchor_gamma: Tensor,            # [S, 4]
    anchor_bias: Tensor,             # [S, 4, buckets]
    partner_base: Tensor,            # [N, S, 128] query-side half of the factorised partner query
    partner_anchor_cache: Tensor,    # [S, B, T, 128] anchor-side half, cached per position
    partner_keys: Tensor,            # [S, B, T, 64]
    partner_block_mean: Tensor,
    partner_block_std: Tensor,
    partner_gamma: Tensor,
    partner_bias: Tensor,
    row_batch: Tensor,               # [N] int32
    row_position: Tensor,            # [N] int32
    local_window: int,
    top_blocks: int,
    partners_per_anchor: int,
    strict_valid: bool,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Returns ``(anchor_index [N,S] i32, anchor_score [N,S], anchor_active [N,S] bool,
    partner_index [N,S,K] i32, partner_score [N,S,K], partner_active [N,S,K] bool)``."""
    for name, query in (("anchor_query", anchor_query), ("anchor_router_query", anchor_router_query),
                        ("partner_base", partner_base)):
        if not query.is_cuda or query.dim() != 3 or query.stride(2) != 1 or query.stride(1) != query.size(2):
            raise ValueError(f"{name} must be a CUDA tensor [N, S, width] whose slots are contiguous inside a row "
                             "(the row stride is free: a column slice of one projection is fine)")
    device = _abi.require_cuda_contiguous(
        anchor_keys=anchor_keys,
        anchor_block_mean=anchor_block_mean, anchor_block_std=anchor_block_std, anchor_gamma=anchor_gamma,
        anchor_bias=anchor_bias, partner_anchor_cache=partner_anchor_cache,
        partner_keys=partner_keys, partner_block_mean=partner_block_mean, partner_block_std=partner_block_std,
        partner_gamma=partner_gamma, partner_bias=partner_bias, row_batch=row_batch, row_position=row_position)
    if anchor_query.dim() != 3 or anchor_query.size(2) != 64:
        raise ValueError("anchor_query must be [N, S, 64]")
    rows, slots = anchor_query.shape[0], anchor_query.shape[1]
    if slots > 8:
        raise ValueError("at most 8 anchor slots")
    if anchor_keys.dim() != 4 or anchor_keys.size(0) != slots or anchor_keys.size(3) != 64:
        raise ValueError("anchor_keys must be [S, B, T, 64]")
    _, batch, max_t, _ = anchor_keys.shape
    nb = anchor_block_mean.size(2)
    if anchor_router_query.shape != (rows, slots, 64) or partner_base.shape != (rows, slots, 128) \
            or partner_anchor_cache.shape != (slots, batch, max_t, 128) or partner_keys.shape != anchor_keys.shape \
            or anchor_block_mean.shape != (slots, batch, nb, 4, 16) or partner_block_mean.shape != anchor_block_mean.shape \
            or anchor_gamma.shape != (slots, 4) or anchor_bias.dim() != 3 or anchor_bias.shape[:2] != (slots, 4):
        raise ValueError("relation_select_multi_rows: inconsistent shapes")
    if row_batch.dtype != torch.int32 or row_position.dtype != torch.int32 \
            or row_batch.numel() != rows or row_position.numel() != rows:
        raise ValueError("row_batch and row_position must be int32 with one entry per query row")
    k = int(partners_per_anchor)
    anchor_index = torch.empty((rows, slots), dtype=torch.int32, device=device)
    anchor_score = torch.empty((rows, slots), dtype=torch.float32, device=device)
    anchor_active = torch.empty((rows, slots), dtype=torch.uint8, device=device)
    partner_index = torch.empty((rows, slots, k), dtype=torch.int32, device=device)
    partner_score = torch.empty((rows, slots, k), dtype=torch.float32, device=device)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_select_multi_rows(
            _abi.ptr(anchor_query), _abi.ptr(anchor_keys), _abi.ptr(anchor_router_query),
            _abi.ptr(anchor_block_mean), _abi.ptr(anchor_block_std), _abi.ptr(anchor_gamma), _abi.ptr(anchor_bias),
            _abi.ptr(partner_base), _abi.ptr(partner_anchor_cache), _abi.ptr(partner_keys),
            _abi.ptr(partner_block_mean), _abi.ptr(partner_block_std), _abi.ptr(partner_gamma),
            _abi.ptr(partner_bias), _abi.ptr(row_batch), _abi.ptr(row_position), _abi.ptr(anchor_index),
            _abi.ptr(anchor_score), _abi.ptr(anchor_active), _abi.ptr(partner_index), _abi.ptr(partner_score),
            anchor_query.stride(0), anchor_router_query.stride(0), partner_base.stride(0),
            rows, batch, slots, max_t, nb, anchor_bias.size(2), int(local_window), int(top_blocks), k,
            int(bool(strict_valid)),
            _abi.same_dtype("query", anchor_query, anchor_router_query, partner_base),
            _abi.same_dtype("key cache", anchor_keys, partner_keys, partner_anchor_cache),
            _abi.same_dtype("block statistics", anchor_block_mean, anchor_block_std, partner_block_mean, partner_block_std),
            _abi.same_dtype("router parameter", anchor_gamma, anchor_bias, partner_gamma, partner_bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return (anchor_index, anchor_score, anchor_active.bool(), partner_index, partner_score,
            torch.isfinite(partner_score))


@relation_select_multi_rows.register_fake
def _(anchor_query, anchor_keys, anchor_router_query, anchor_block_mean, anchor_block_std, anchor_gamma,
      anchor_bias, partner_base, partner_anchor_cache, partner_keys, partner_block_mean, partner_block_std,
      partner_gamma, partner_bias, row_batch, row_position, local_window, top_blocks, partners_per_anchor,
      strict_valid):
    rows, slots = anchor_query.size(0), anchor_query.size(1)
    k = partners_per_anchor
    f32 = torch.float32
    return (anchor_query.new_empty((rows, slots), dtype=torch.int32), anchor_query.new_empty((rows, slots), dtype=f32),
            anchor_query.new_empty((rows, slots), dtype=torch.bool),
            anchor_query.new_empty((rows, slots, k), dtype=torch.int32),
            anchor_query.new_empty((rows, slots, k), dtype=f32),
            anchor_query.new_empty((rows, slots, k), dtype=torch.bool))


@torch.library.custom_op("relation_lm::relation_select_multi_prefill", mutates_args=(), device_types="cuda")
def relation_select_multi_prefill(
    anchor_query: Tensor,            # [B * Tq, S, 64]
    anchor_keys: Tensor,             # [S, B, T, 64]
    anchor_router_query: Tensor,     # [B * Tq, S, 64]
    anchor_block_mean: Tensor,       # [S, B, NB, 4, 16]
    anchor_block_std: Tensor,
    anchor_gamma: Tensor,            # [S, 4]
    anchor_bias: Tensor,             # [S, 4, buckets]
    partner_base: Tensor,            # [B * Tq, S, 128]
    partner_anchor_cache: Tensor,    # [S, B, T, 128]
    partner_keys: Tensor,            # [S, B, T, 64]
    partner_block_mean: Tensor,
    partner_block_std: Tensor,
    partner_gamma: Tensor,
    partner_bias: Tensor,
    query_length: int,
    local_window: int,
    top_blocks: int,
    partners_per_anchor: int,
    strict_valid: bool,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Whole-sequence form of ``relation_select_multi_rows`` (bfloat16 tensors): query row
    ``b * query_length + t`` is position ``t`` of sequence ``b``; same results, bit for bit.  A CTA
    serves a tile of consecutive positions and stages each slot's block statistics and window union
    once per tile."""
    for name, query in (("anchor_query", anchor_query), ("anchor_router_query", anchor_router_query),
                        ("partner_base", partner_base)):
        if not query.is_cuda or query.dim() != 3 or query.stride(2) != 1 or query.stride(1) != query.size(2):
            raise ValueError(f"{name} must be a CUDA tensor [N, S, width] whose slots are contiguous inside a row")
    device = _abi.require_cuda_contiguous(
        anchor_keys=anchor_keys, anchor_block_mean=anchor_block_mean, anchor_block_std=anchor_block_std,
        anchor_gamma=anchor_gamma, anchor_bias=anchor_bias, partner_anchor_cache=partner_anchor_cache,
        partner_keys=partner_keys, partner_block_mean=partner_block_mean, partner_block_std=partner_block_std,
        partner_gamma=partner_gamma, partner_bias=partner_bias)
    rows, slots = anchor_query.shape[0], anchor_query.shape[1]
    if anchor_keys.dim() != 4 or anchor_keys.size(0) != slots or anchor_keys.size(3) != 64 or slots > 8:
        raise ValueError("anchor_keys must be [S, B, T, 64] with at most 8 slots")
    _, batch, max_t, _ = anchor_keys.shape
    nb = anchor_block_mean.size(2)
    tq = int(query_length)
    if rows != batch * tq or tq < 1 or tq > max_t:
        raise ValueError("the queries must be the positions 0 .. query_length - 1 of every sequence")
    if anchor_query.size(2) != 64 or anchor_router_query.shape != (rows, slots, 64) \
            or partner_base.shape != (rows, slots, 128) \
            or partner_anchor_cache.shape != (slots, batch, max_t, 128) or partner_keys.shape != anchor_keys.shape \
            or anchor_block_mean.shape != (slots, batch, nb, 4, 16) or partner_block_mean.shape != anchor_block_mean.shape \
            or anchor_gamma.shape != (slots, 4) or anchor_bias.dim() != 3 or anchor_bias.shape[:2] != (slots, 4):
        raise ValueError("relation_select_multi_prefill: inconsistent shapes")
    k = int(partners_per_anchor)
    anchor_index = torch.empty((rows, slots), dtype=torch.int32, device=device)
    anchor_score = torch.empty((rows, slots), dtype=torch.float32, device=device)
    anchor_active = torch.empty((rows, slots), dtype=torch.uint8, device=device)
    partner_index = torch.empty((rows, slots, k), dtype=torch.int32, device=device)
    partner_score = torch.empty((rows, slots, k), dtype=torch.float32, device=device)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_select_multi_prefill(
            _abi.ptr(anchor_query), _abi.ptr(anchor_keys), _abi.ptr(anchor_router_query),
            _abi.ptr(anchor_block_mean), _abi.ptr(anchor_block_std), _abi.ptr(anchor_gamma), _abi.ptr(anchor_bias),
            _abi.ptr(partner_base), _abi.ptr(partner_anchor_cache), _abi.ptr(partner_keys),
            _abi.ptr(partner_block_mean), _abi.ptr(partner_block_std), _abi.ptr(partner_gamma),
            _abi.ptr(partner_bias), _abi.ptr(anchor_index), _abi.ptr(anchor_score), _abi.ptr(anchor_active),
            _abi.ptr(partner_index), _abi.ptr(partner_score),
            anchor_query.stride(0), anchor_router_query.stride(0), partner_base.stride(0),
            tq, batch, slots, max_t, nb, anchor_bias.size(2), int(local_window), int(top_blocks), k,
            int(bool(strict_valid)),
            _abi.same_dtype("query", anchor_query, anchor_router_query, partner_base),
            _abi.same_dtype("key cache", anchor_keys, partner_keys, partner_anchor_cache),
            _abi.same_dtype("block statistics", anchor_block_mean, anchor_block_std, partner_block_mean, partner_block_std),
            _abi.same_dtype("router parameter", anchor_gamma, anchor_bias, partner_gamma, partner_bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return (anchor_index, anchor_score, anchor_active.bool(), partner_index, partner_score,
            torch.isfinite(partner_score))


@relation_select_multi_prefill.register_fake
def _(anchor_query, anchor_keys, anchor_router_query, anchor_block_mean, anchor_block_std, anchor_gamma,
      anchor_bias, partner_base, partner_anchor_cache, partner_keys, partner_block_mean, partner_block_std,
      partner_gamma, partner_bias, query_length, local_window, top_blocks, partners_per_anchor, strict_valid):
    rows, slots = anchor_query.size(0), anchor_query.size(1)
    k = partners_per_anchor
    f32 = torch.float32
    return (anchor_query.new_empty((rows, slots), dtype=torch.int32), anchor_query.new_empty((rows, slots), dtype=f32),
            anchor_query.new_empty((rows, slots), dtype=torch.bool),
            anchor_query.new_empty((rows, slots, k), dtype=torch.int32),
            anchor_query.new_empty((rows, slots, k), dtype=f32),
            anchor_query.new_empty((rows, slots, k), dtype=torch.bool))


@torch.library.custom_op("relation_lm::slot_mix_residual", mutates_args=("hidden",), device_types="cuda")
def slot_mix_residual(slot_context: Tensor, anchor_active: Tensor, slot_weight: Tensor, gate: Tensor,
                      hidden: Tensor) -> None:
    """Last step of a multi-anchor layer (extension; multi_relation_blocks.py:170-178 of the reference):
    ``hidden += gate * sum_s w[:, s] * slot_context[:, s]`` with ``w`` the slot weights
    (``slot_weight [S]``, the softmax of the learned logits) renormalised over each row's active
    slots.  ``slot_context [N, S, d]``, ``hidden [N, d]``, ``gate`` (one element): fp32;
    ``anchor_active [N, S]`` bool."""
    device = _abi.require_cuda_contiguous(slot_context=slot_context, anchor_active=anchor_active,
                                          slot_weight=slot_weight, gate=gate, hidden=hidden)
    rows, slots, dim = slot_context.shape
    if anchor_active.shape != (rows, slots) or slot_weight.numel() != slots or hidden.shape != (rows, dim) \
            or gate.numel() != 1:
        raise ValueError("slot_mix_residual: inconsistent shapes")
    if anchor_active.dtype not in (torch.bool, torch.uint8):
        raise ValueError("anchor_active must be bool")
    for name, t in (("slot_context", slot_context), ("slot_weight", slot_weight), ("gate", gate), ("hidden", hidden)):
        if t.dtype != torch.float32:
            raise ValueError(f"{name} must be float32")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_slot_mix_residual(
            _abi.ptr(slot_context), _abi.ptr(anchor_active.view(torch.uint8)), _abi.ptr(slot_weight), _abi.ptr(gate),
            _abi.ptr(hidden), rows, slots, dim, _abi.stream_ptr(device)))


@slot_mix_residual.register_fake
def _(slot_context, anchor_active, slot_weight, gate, hidden):
    return None
