"""``relation_lm::relation_layer`` — a whole relation layer of a decode step in one launch (extension).

``relation_lm::relation_select_packed`` (src/relation_lm/kernels/relation_select.py:594-651 of the
reference) followed by the layer's relation tail (``relation_lm::relation_layer_tail`` of this
package: relation hidden states, second relation-MLP layer, norm-reduce, residual update, the next
LayerNorm and the next layer's query projection), inside the tail's thread-block cluster.  The
selection results are the separate operator's, bit for bit; they are returned as well.
"""
from __future__ import annotations

import torch
from torch import Tensor

from relation_lm.kernels import _abi


def relation_layer_supported(n_seq: int, k_out: int, relation_dim: int, hidden_dim: int, d_model: int,
                             n_query: int, dtype: torch.dtype, max_t: int, n_blocks: int, buckets: int,
                             local_window: int, top_blocks: int) -> bool:
    """Whether ``relation_layer`` serves these sizes on the current device (otherwise use
    ``relation_select_packed`` + ``relation_layer_tail``)."""
    if dtype not in (torch.bfloat16, torch.float16):
        return False
    return bool(_abi.LIB.rlm_relation_layer_supported(
        int(n_seq), int(k_out), int(relation_dim), int(hidden_dim), int(d_model), int(n_query),
        _abi.DTYPE_CODE[dtype], int(max_t), int(n_blocks), int(buckets), int(local_window), int(top_blocks)))


@torch.library.custom_op("relation_lm::relation_layer", mutates_args=("hidden", "normalized", "query"),
                         device_types="cuda")
def relation_layer(
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
    expanded_cache: Tensor,
    operand_cache: Tensor,
    product_weight: Tensor,
    second_weight: Tensor,
    second_bias: Tensor,
    norm_weight: Tensor,
    norm_bias: Tensor,
    norm_eps: float,
    hidden: Tensor,
    mix: Tensor,
    next_norm_weight: Tensor,
    next_norm_bias: Tensor,
    next_norm_eps: float,
    normalized: Tensor,
    query_weight: Tensor | None,
    query: Tensor | None,
) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """Selects at ``position`` (arguments of ``relation_select_packed``), then runs the relation tail
    on the selected rows (arguments of ``relation_layer_tail``).  Returns the selection: anchor
    index / score ``[B]``, partner indices / scores ``[B, k_out]``.  ``query`` may be the tensor the
    query arguments are slices of: a sequence's row is rewritten only after its selection."""
    _abi.require_cuda_rows(anchor_query=anchor_query, anchor_router_query=anchor_router_query,
                           partner_base=partner_base)
    device = _abi.require_cuda_contiguous(
        anchor_keys=anchor_keys, anchor_block_mean=anchor_block_mean, anchor_block_std=anchor_block_std,
        anchor_gamma=anchor_gamma, anchor_bias=anchor_bias, partner_anchor_cache=partner_anchor_cache,
        partner_keys=partner_keys, partner_block_mean=partner_block_mean, partner_block_std=partner_block_std,
        partner_gamma=partner_gamma, partner_bias=partner_bias,
        expanded_cache=expanded_cache, operand_cache=operand_cache, product_weight=product_weight,
        second_weight=second_weight, second_bias=second_bias, norm_weight=norm_weight, norm_bias=norm_bias,
        hidden=hidden, mix=mix, next_norm_weight=next_norm_weight, next_norm_bias=next_norm_bias,
        normalized=normalized, query_weight=query_weight, query=query)
    _abi.require_position(position, device)
    batch, max_t, rdim = operand_cache.shape
    hdim, dim = product_weight.size(0), second_weight.size(0)
    n_blocks = anchor_block_mean.size(1)
    if anchor_query.shape != (batch, 64) or anchor_router_query.shape != (batch, 64) \
            or partner_base.shape != (batch, 128) or anchor_keys.shape != (batch, max_t, 64) \
            or partner_keys.shape != anchor_keys.shape or partner_anchor_cache.shape != (batch, max_t, 128) \
            or anchor_block_mean.shape != (batch, n_blocks, 4, 16) \
            or any(t.shape != anchor_block_mean.shape for t in (anchor_block_std, partner_block_mean, partner_block_std)) \
            or anchor_bias.dim() != 2 or partner_bias.shape != anchor_bias.shape:
        raise ValueError("relation_layer: inconsistent selector shapes (gate width 64, 4 router heads of width 16)")
    if expanded_cache.shape != (batch, max_t, 2 * hdim) or product_weight.shape != (hdim, rdim) \
            or second_weight.shape != (dim, hdim) or second_bias.numel() != dim \
            or hidden.shape != (batch, dim) or normalized.shape != (batch, dim):
        raise ValueError("relation_layer: inconsistent tail shapes")
    for name, t in (("hidden", hidden), ("mix", mix), ("norm_weight", norm_weight), ("norm_bias", norm_bias),
                    ("next_norm_weight", next_norm_weight), ("next_norm_bias", next_norm_bias)):
        if t.dtype != torch.float32:
            raise ValueError(f"{name} must be float32")
    n_query = 0
    if query_weight is not None:
        if query is None or query_weight.dim() != 2 or query_weight.size(1) != dim \
                or query.shape != (batch, query_weight.size(0)):
            raise ValueError("query_weight [NQ, d] needs an output query [B, NQ]")
        n_query = query_weight.size(0)
    sixteen = [anchor_query, anchor_router_query, partner_base, anchor_keys, partner_keys, partner_anchor_cache,
               anchor_block_mean, anchor_block_std, partner_block_mean, partner_block_std,
               expanded_cache, operand_cache, product_weight, second_weight, second_bias, normalized]
    if query_weight is not None:
        sixteen += [query_weight, query]
    dtype = _abi.same_dtype("16-bit operand", *sixteen)
    param_dtype = _abi.same_dtype("gamma/bias", anchor_gamma, anchor_bias, partner_gamma, partner_bias)
    k_out = int(k_out)
    out_anchor = torch.empty((batch,), device=device, dtype=torch.int32)
    out_anchor_score = torch.empty((batch,), device=device, dtype=torch.float32)
    out_partner = torch.empty((batch, k_out), device=device, dtype=torch.int32)
    out_partner_score = torch.empty((batch, k_out), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_layer(
            _abi.ptr(anchor_query), _abi.ptr(anchor_keys), _abi.ptr(anchor_router_query),
            _abi.ptr(anchor_block_mean), _abi.ptr(anchor_block_std), _abi.ptr(anchor_gamma), _abi.ptr(anchor_bias),
            _abi.ptr(partner_base), _abi.ptr(partner_anchor_cache), _abi.ptr(partner_keys),
            _abi.ptr(partner_block_mean), _abi.ptr(partner_block_std), _abi.ptr(partner_gamma),
            _abi.ptr(partner_bias), _abi.ptr(position), _abi.ptr(out_anchor), _abi.ptr(out_anchor_score),
            _abi.ptr(out_partner), _abi.ptr(out_partner_score), anchor_query.stride(0),
            anchor_router_query.stride(0), partner_base.stride(0), n_blocks, anchor_bias.size(1),
            int(local_window), int(top_blocks), int(bool(strict_valid)), param_dtype,
            _abi.ptr(expanded_cache), _abi.ptr(operand_cache), _abi.ptr(product_weight), _abi.ptr(second_weight),
            _abi.ptr(second_bias), _abi.ptr(norm_weight), _abi.ptr(norm_bias), float(norm_eps), _abi.ptr(hidden),
            _abi.ptr(mix), _abi.ptr(next_norm_weight), _abi.ptr(next_norm_bias), float(next_norm_eps),
            _abi.ptr(normalized), _abi.ptr(query_weight), _abi.ptr(query), batch, k_out, max_t, rdim, hdim, dim,
            n_query, dtype, _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out_anchor, out_anchor_score, out_partner, out_partner_score


@relation_layer.register_fake
def _(anchor_query, anchor_keys, anchor_router_query, anchor_block_mean, anchor_block_std, anchor_gamma,
      anchor_bias, partner_base, partner_anchor_cache, partner_keys, partner_block_mean, partner_block_std,
      partner_gamma, partner_bias, position, local_window, top_blocks, k_out, strict_valid, expanded_cache,
      operand_cache, product_weight, second_weight, second_bias, norm_weight, norm_bias, norm_eps, hidden, mix,
      next_norm_weight, next_norm_bias, next_norm_eps, normalized, query_weight, query):
    rows = anchor_query.size(0)
    return (anchor_query.new_empty((rows,), dtype=torch.int32),
            anchor_query.new_empty((rows,), dtype=torch.float32),
            anchor_query.new_empty((rows, k_out), dtype=torch.int32),
            anchor_query.new_empty((rows, k_out), dtype=torch.float32))
