"""Routed multi-anchor selection (extension).

The reference project's multi-anchor layer is dense: every slot scores all causal positions
(src/relation_lm/models/multi_relation_blocks.py:69-148).  This is its routed form, built from
the per-row selectors of this library.  Its rules are the reference's, applied inside each
slot's routed candidate set (local window + that slot's best remote blocks):

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

from relation_lm.kernels.triton_select import anchor_select_rows, partner_topk_rows


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
):
    """Returns ``(anchor_index [N,S] i32, anchor_score [N,S], anchor_active [N,S] bool,
    partner_index [N,S,K] i32, partner_score [N,S,K], partner_active [N,S,K] bool)``."""
    rows, slots = anchor_query.shape[0], anchor_query.shape[1]
    if slots > 8:
        raise ValueError("at most 8 anchor slots")
    device = anchor_query.device
    active = torch.arange(slots, device=device)[None, :] <= row_position[:, None]
    taken = torch.full((rows, slots), -1, dtype=torch.int32, device=device)
    anchor_index = torch.zeros((rows, slots), dtype=torch.int32, device=device)
    anchor_score = torch.full((rows, slots), -torch.inf, device=device)
    for s in range(slots):
        idx, score = anchor_select_rows(
            anchor_query[:, s].contiguous(), anchor_keys[s], anchor_router_query[:, s].contiguous(),
            anchor_block_mean[s], anchor_block_std[s], anchor_gamma[s], anchor_bias[s], row_batch,
            row_position, taken.clone(), local_window, top_blocks, strict_valid)
        live = active[:, s] & torch.isfinite(score)
        anchor_index[:, s] = torch.where(live, idx, torch.zeros_like(idx))
        anchor_score[:, s] = torch.where(live, score, torch.full_like(score, -torch.inf))
        taken[:, s] = torch.where(live, idx, torch.full_like(idx, -1))
        active[:, s] = live
    k = int(partners_per_anchor)
    partner_index = torch.zeros((rows, slots, k), dtype=torch.int32, device=device)
    partner_score = torch.full((rows, slots, k), -torch.inf, device=device)
    batch_index = row_batch.long()
    for s in range(slots):
        v = partner_base[:, s].float() + partner_anchor_cache[s][batch_index, anchor_index[:, s].long()].float()
        v = v.to(partner_base.dtype)
        idx, score = partner_topk_rows(
            v[:, :64].contiguous(), partner_keys[s], v[:, 64:].contiguous(), partner_block_mean[s],
            partner_block_std[s], partner_gamma[s], partner_bias[s], row_batch, row_position,
            taken[:, s].contiguous(), taken, local_window, top_blocks, k, strict_valid)
        live = active[:, s, None] & torch.isfinite(score)
        partner_index[:, s] = torch.where(live, idx, torch.zeros_like(idx))
        partner_score[:, s] = torch.where(live, score, torch.full_like(score, -torch.inf))
    return (anchor_index, anchor_score, active, partner_index, partner_score,
            torch.isfinite(partner_score))
