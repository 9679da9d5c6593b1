"""Relation-reduce tail: factorised first relation-MLP layer and fused norm + reduction.

Operator names, schemas and helper names follow the reference project's
``src/relation_lm/kernels/relation_reduce.py`` (``factor_relation_first_layer``
:23-57, ``recommended_relation_cache_mode`` :60-69, ``relation_hidden_cached``
:149-183, ``relation_hidden_cache_update`` :312-357, ``relation_norm_reduce``
:420-450).  The operators launch sm_100a kernels through the C ABI.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor

from relation_lm.kernels import _abi


@dataclass(frozen=True)
class FactorizedRelationWeights:
    """The first relation-MLP layer rewritten as per-token contributions."""

    anchor_weight: Tensor
    partner_weight: Tensor
    product_weight: Tensor
    first_bias: Tensor
    expanded_weight: Tensor
    expanded_bias: Tensor


def factor_relation_first_layer(first_weight: Tensor, first_bias: Tensor,
                                relation_dim: int) -> FactorizedRelationWeights:
    """Rewrite ``W [a, p, a*p, a-p] + b`` as ``(W_a+W_d) a + (W_p-W_d) p + W_m (a*p) + b``.

    ``expanded_weight`` stacks the anchor and partner matrices so one projection of a cached
    operand yields both of its contributions; ``expanded_bias`` carries ``b`` on the anchor half
    only, so the bias enters each relation exactly once.
    """
    relation_dim = int(relation_dim)
    if first_weight.dim() != 2 or first_bias.dim() != 1:
        raise ValueError("first_weight must be 2D and first_bias must be 1D")
    if first_weight.size(1) != 4 * relation_dim:
        raise ValueError("first_weight input dimension must equal 4 * relation_dim")
    w_a, w_p, w_m, w_d = first_weight.split(relation_dim, dim=1)
    anchor_weight = (w_a + w_d).contiguous()
    partner_weight = (w_p - w_d).contiguous()
    return FactorizedRelationWeights(
        anchor_weight=anchor_weight,
        partner_weight=partner_weight,
        product_weight=w_m.contiguous(),
        first_bias=first_bias.contiguous(),
        expanded_weight=torch.cat((anchor_weight, partner_weight), dim=0).contiguous(),
        expanded_bias=torch.cat((first_bias, torch.zeros_like(first_bias)), dim=0).contiguous(),
    )


def recommended_relation_cache_mode(batch_size: int) -> str:
    """``"fused_update"`` for a single sequence, ``"separate_update"`` for larger batches."""
    if batch_size < 1:
        raise ValueError("batch_size must be positive")
    return "fused_update" if batch_size == 1 else "separate_update"


def _check_indices(anchor_index: Tensor, partner_index: Tensor, rows: int) -> None:
    if anchor_index.dtype != torch.int32 or partner_index.dtype != torch.int32:
        raise ValueError("anchor_index and partner_index must be int32")
    if anchor_index.numel() != rows or partner_index.dim() != 2 or partner_index.size(0) != rows:
        raise ValueError("anchor_index must be [B] and partner_index [B, K]")


@torch.library.custom_op("relation_lm::relation_hidden_cached", mutates_args=(),
                         device_types="cuda")
def relation_hidden_cached(
    expanded_cache: Tensor,
    operand_cache: Tensor,
    anchor_index: Tensor,
    partner_index: Tensor,
    product_weight: Tensor,
) -> Tensor:
    """``gelu((o[p] * o[a]) W_m^T + E[a, :H] + E[p, H:])`` for every partner slot, ``[B, K, H]`` fp32."""
    device = _abi.require_cuda_contiguous(
        expanded_cache=expanded_cache, operand_cache=operand_cache, anchor_index=anchor_index,
        partner_index=partner_index, product_weight=product_weight)
    batch, max_t, rdim = operand_cache.shape
    hdim, k_out = product_weight.size(0), partner_index.size(1)
    _check_indices(anchor_index, partner_index, batch)
    if expanded_cache.shape != (batch, max_t, 2 * hdim) or product_weight.size(1) != rdim:
        raise ValueError("expanded_cache must be [B, T, 2H] and product_weight [H, R]")
    out = torch.empty((batch, k_out, hdim), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_hidden_cached(
            _abi.ptr(expanded_cache), _abi.ptr(operand_cache), _abi.ptr(anchor_index),
            _abi.ptr(partner_index), _abi.ptr(product_weight), None, _abi.ptr(out), batch, batch,
            max_t, rdim, hdim, k_out, _abi.same_dtype("cache", expanded_cache, operand_cache),
            _abi.code(product_weight), _abi.code(out), _abi.ptr(_abi.status_tensor(device)),
            _abi.stream_ptr(device)))
    return out


@relation_hidden_cached.register_fake
def _(expanded_cache, operand_cache, anchor_index, partner_index, product_weight):
    return operand_cache.new_empty(
        (operand_cache.size(0), partner_index.size(1), product_weight.size(0)), dtype=torch.float32)


@torch.library.custom_op("relation_lm::relation_hidden_cached_out", mutates_args=("out",),
                         device_types="cuda")
def relation_hidden_cached_out(
    out: Tensor,
    expanded_cache: Tensor,
    operand_cache: Tensor,
    anchor_index: Tensor,
    partner_index: Tensor,
    product_weight: Tensor,
) -> None:
    """``relation_hidden_cached`` writing into a caller-owned ``out [B, K, H]`` of any float dtype
    (extension: a 16-bit ``out`` feeds the second MLP layer without a cast)."""
    device = _abi.require_cuda_contiguous(
        out=out, expanded_cache=expanded_cache, operand_cache=operand_cache, anchor_index=anchor_index,
        partner_index=partner_index, product_weight=product_weight)
    batch, max_t, rdim = operand_cache.shape
    hdim, k_out = product_weight.size(0), partner_index.size(1)
    _check_indices(anchor_index, partner_index, batch)
    if expanded_cache.shape != (batch, max_t, 2 * hdim) or product_weight.size(1) != rdim \
            or out.shape != (batch, k_out, hdim):
        raise ValueError("expected expanded_cache [B, T, 2H], product_weight [H, R] and out [B, K, H]")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_hidden_cached(
            _abi.ptr(expanded_cache), _abi.ptr(operand_cache), _abi.ptr(anchor_index),
            _abi.ptr(partner_index), _abi.ptr(product_weight), None, _abi.ptr(out), batch, batch,
            max_t, rdim, hdim, k_out, _abi.same_dtype("cache", expanded_cache, operand_cache),
            _abi.code(product_weight), _abi.code(out), _abi.ptr(_abi.status_tensor(device)),
            _abi.stream_ptr(device)))


@relation_hidden_cached_out.register_fake
def _(out, expanded_cache, operand_cache, anchor_index, partner_index, product_weight):
    return None


@torch.library.custom_op("relation_lm::expanded_cache_append", mutates_args=("expanded_cache",),
                         device_types="cuda")
def expanded_cache_append(
    expanded_cache: Tensor,
    operand_cache: Tensor,
    anchor_weight: Tensor,
    partner_weight: Tensor,
    first_bias: Tensor,
    position: Tensor,
) -> None:
    """Expanded-cache rows of the current position for all layers of a stack in one launch
    (extension, tensor cores): ``expanded[l, :, t] = [W_a[l] o + b_1[l], W_p[l] o]`` with
    ``o = operand_cache[l, :, t]``.  Stacked 16-bit tensors: caches ``[L, B, T, .]``, weights
    ``[L, H, R]``, bias ``[L, H]``.  The per-layer kernels then use ``relation_hidden_cached``."""
    device = _abi.require_cuda_contiguous(
        expanded_cache=expanded_cache, operand_cache=operand_cache, anchor_weight=anchor_weight,
        partner_weight=partner_weight, first_bias=first_bias)
    _abi.require_position(position, device)
    if operand_cache.dim() != 4 or expanded_cache.dim() != 4 or anchor_weight.dim() != 3:
        raise ValueError("expected stacked tensors: caches [L, B, T, .], weights [L, H, R], bias [L, H]")
    layers, batch, max_t, rdim = operand_cache.shape
    hdim = anchor_weight.size(1)
    if expanded_cache.shape != (layers, batch, max_t, 2 * hdim) or anchor_weight.shape != (layers, hdim, rdim) \
            or partner_weight.shape != anchor_weight.shape or first_bias.shape != (layers, hdim):
        raise ValueError("expected expanded_cache [L, B, T, 2H], weights [L, H, R] and first_bias [L, H]")
    dtype = _abi.same_dtype("cache", expanded_cache, operand_cache)
    if len({anchor_weight.dtype, partner_weight.dtype, first_bias.dtype, expanded_cache.dtype}) != 1:
        raise ValueError("caches, weights and bias must share one 16-bit dtype")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_expanded_cache_append(
            _abi.ptr(expanded_cache), _abi.ptr(operand_cache), _abi.ptr(anchor_weight),
            _abi.ptr(partner_weight), _abi.ptr(first_bias), _abi.ptr(position), layers, batch, max_t,
            rdim, hdim, dtype, _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@expanded_cache_append.register_fake
def _(expanded_cache, operand_cache, anchor_weight, partner_weight, first_bias, position):
    return None


@torch.library.custom_op("relation_lm::expanded_cache_append_packed", mutates_args=("expanded_cache",),
                         device_types="cuda")
def expanded_cache_append_packed(
    expanded_cache: Tensor,
    packed: Tensor,
    anchor_weight: Tensor,
    partner_weight: Tensor,
    first_bias: Tensor,
    position: Tensor,
) -> None:
    """``expanded_cache_append`` with the operand rows of the position read from the packed projection
    rows ``packed [B, L * (384 + R)]`` (layout of ``sparse_cache_append``) instead of the operand cache:
    same results, no dependence on the state append, which it overlaps under programmatic launch.
    ``packed`` must not come from the launch right before this one on the stream."""
    device = _abi.require_cuda_contiguous(
        expanded_cache=expanded_cache, anchor_weight=anchor_weight, partner_weight=partner_weight,
        first_bias=first_bias)
    _abi.require_cuda_rows(packed=packed)
    _abi.require_position(position, device)
    if expanded_cache.dim() != 4 or anchor_weight.dim() != 3 or packed.dim() != 2:
        raise ValueError("expected expanded_cache [L, B, T, 2H], packed [B, L * (384 + R)], weights [L, H, R]")
    layers, batch, max_t, _ = expanded_cache.shape
    hdim, rdim = anchor_weight.size(1), anchor_weight.size(2)
    if expanded_cache.size(3) != 2 * hdim or anchor_weight.shape != (layers, hdim, rdim) \
            or partner_weight.shape != anchor_weight.shape or first_bias.shape != (layers, hdim) \
            or packed.shape != (batch, layers * (384 + rdim)):
        raise ValueError("expected expanded_cache [L, B, T, 2H], packed [B, L * (384 + R)], weights [L, H, R], bias [L, H]")
    if len({anchor_weight.dtype, partner_weight.dtype, first_bias.dtype, expanded_cache.dtype, packed.dtype}) != 1:
        raise ValueError("cache, packed rows, weights and bias must share one 16-bit dtype")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_expanded_cache_append_packed(
            _abi.ptr(expanded_cache), _abi.ptr(packed), packed.stride(0), 384 + rdim, 128, _abi.ptr(anchor_weight),
            _abi.ptr(partner_weight), _abi.ptr(first_bias), _abi.ptr(position), layers, batch, max_t, rdim, hdim,
            _abi.code(expanded_cache), _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@expanded_cache_append_packed.register_fake
def _(expanded_cache, packed, anchor_weight, partner_weight, first_bias, position):
    return None


@torch.library.custom_op("relation_lm::relation_hidden_cache_update",
                         mutates_args=("expanded_cache",), device_types="cuda")
def relation_hidden_cache_update(
    expanded_cache: Tensor,
    operand_cache: Tensor,
    anchor_index: Tensor,
    partner_index: Tensor,
    anchor_weight: Tensor,
    partner_weight: Tensor,
    product_weight: Tensor,
    first_bias: Tensor,
    position: Tensor,
) -> Tensor:
    """As ``relation_hidden_cached``, after computing and storing ``expanded_cache[:, position]``."""
    device = _abi.require_cuda_contiguous(
        expanded_cache=expanded_cache, operand_cache=operand_cache, anchor_index=anchor_index,
        partner_index=partner_index, anchor_weight=anchor_weight, partner_weight=partner_weight,
        product_weight=product_weight, first_bias=first_bias)
    _abi.require_position(position, device)
    batch, max_t, rdim = operand_cache.shape
    hdim, k_out = product_weight.size(0), partner_index.size(1)
    _check_indices(anchor_index, partner_index, batch)
    if expanded_cache.shape != (batch, max_t, 2 * hdim) or product_weight.size(1) != rdim \
            or anchor_weight.shape != product_weight.shape or partner_weight.shape != product_weight.shape \
            or first_bias.numel() != hdim:
        raise ValueError("expected expanded_cache [B, T, 2H], weights [H, R] and first_bias [H]")
    out = torch.empty((batch, k_out, hdim), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_hidden_cache_update(
            _abi.ptr(expanded_cache), _abi.ptr(operand_cache), _abi.ptr(anchor_index),
            _abi.ptr(partner_index), _abi.ptr(anchor_weight), _abi.ptr(partner_weight),
            _abi.ptr(product_weight), _abi.ptr(first_bias), _abi.ptr(position), _abi.ptr(out),
            batch, max_t, rdim, hdim, k_out,
            _abi.same_dtype("cache", expanded_cache, operand_cache),
            _abi.same_dtype("weight", anchor_weight, partner_weight, product_weight, first_bias),
            _abi.code(out), _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out


@relation_hidden_cache_update.register_fake
def _(expanded_cache, operand_cache, anchor_index, partner_index, anchor_weight, partner_weight,
      product_weight, first_bias, position):
    return operand_cache.new_empty(
        (operand_cache.size(0), partner_index.size(1), product_weight.size(0)), dtype=torch.float32)


@torch.library.custom_op("relation_lm::relation_norm_reduce", mutates_args=(),
                         device_types="cuda")
def relation_norm_reduce(
    raw: Tensor,
    partner_scores: Tensor,
    norm_weight: Tensor,
    norm_bias: Tensor,
    position: Tensor,
    norm_eps: float,
) -> Tensor:
    """LayerNorm of each partner's relation vector, softmax over the active partner slots
    (``k < clamp(ceil(log2(position + 2)), 1, K)`` and a finite score) and their weighted sum."""
    device = _abi.require_cuda_contiguous(raw=raw, partner_scores=partner_scores,
                                          norm_weight=norm_weight, norm_bias=norm_bias)
    _abi.require_position(position, device)
    batch, k_out, dim = raw.shape
    if partner_scores.shape != (batch, k_out) or partner_scores.dtype != torch.float32:
        raise ValueError("partner_scores must be float32 [B, K]")
    out = torch.empty((batch, dim), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_norm_reduce(
            _abi.ptr(raw), _abi.ptr(partner_scores), _abi.ptr(norm_weight), _abi.ptr(norm_bias),
            _abi.ptr(position), None, float(norm_eps), _abi.ptr(out), None, None, None, None, 0.0, None, 0, 1, 0, None,
            batch, k_out, dim,
            _abi.code(raw), _abi.same_dtype("norm parameter", norm_weight, norm_bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out


@relation_norm_reduce.register_fake
def _(raw, partner_scores, norm_weight, norm_bias, position, norm_eps):
    return raw.new_empty((raw.size(0), raw.size(2)), dtype=torch.float32)


def _hidden_update_into(out, expanded_cache, operand_cache, anchor_index, partner_index,
                        anchor_weight, partner_weight, product_weight, first_bias, position):
    device = _abi.require_cuda_contiguous(
        out=out, expanded_cache=expanded_cache, operand_cache=operand_cache,
        anchor_index=anchor_index, partner_index=partner_index, anchor_weight=anchor_weight,
        partner_weight=partner_weight, product_weight=product_weight, first_bias=first_bias)
    _abi.require_position(position, device)
    batch, max_t, rdim = operand_cache.shape
    hdim, k_out = product_weight.size(0), partner_index.size(1)
    _check_indices(anchor_index, partner_index, batch)
    if out.shape != (batch, k_out, hdim) or expanded_cache.shape != (batch, max_t, 2 * hdim):
        raise ValueError("expected out [B, K, H] and expanded_cache [B, T, 2H]")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_hidden_cache_update(
            _abi.ptr(expanded_cache), _abi.ptr(operand_cache), _abi.ptr(anchor_index),
            _abi.ptr(partner_index), _abi.ptr(anchor_weight), _abi.ptr(partner_weight),
            _abi.ptr(product_weight), _abi.ptr(first_bias), _abi.ptr(position), _abi.ptr(out),
            batch, max_t, rdim, hdim, k_out,
            _abi.same_dtype("cache", expanded_cache, operand_cache),
            _abi.same_dtype("weight", anchor_weight, partner_weight, product_weight, first_bias),
            _abi.code(out), _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@torch.library.custom_op("relation_lm::relation_hidden_cache_update_out",
                         mutates_args=("out", "expanded_cache"), device_types="cuda")
def relation_hidden_cache_update_out(
    out: Tensor,
    expanded_cache: Tensor,
    operand_cache: Tensor,
    anchor_index: Tensor,
    partner_index: Tensor,
    anchor_weight: Tensor,
    partner_weight: Tensor,
    product_weight: Tensor,
    first_bias: Tensor,
    position: Tensor,
) -> None:
    """``relation_hidden_cache_update`` writing into a caller-owned ``out [B, K, H]`` of any
    float dtype (extension: a 16-bit ``out`` feeds the second MLP layer without a cast)."""
    _hidden_update_into(out, expanded_cache, operand_cache, anchor_index, partner_index,
                        anchor_weight, partner_weight, product_weight, first_bias, position)


@relation_hidden_cache_update_out.register_fake
def _(out, expanded_cache, operand_cache, anchor_index, partner_index, anchor_weight,
      partner_weight, product_weight, first_bias, position):
    return None


@torch.library.custom_op("relation_lm::relation_norm_reduce_residual", mutates_args=("hidden",),
                         device_types="cuda")
def relation_norm_reduce_residual(
    raw: Tensor,
    partner_scores: Tensor,
    norm_weight: Tensor,
    norm_bias: Tensor,
    position: Tensor,
    norm_eps: float,
    hidden: Tensor,
    mix: Tensor,
) -> None:
    """``relation_norm_reduce`` fused with the layer's residual update (extension):
    ``hidden += mix * context`` in place, ``hidden [B, D]`` fp32, ``mix`` a 0-d fp32 tensor
    holding ``sigmoid(mix_logit)``."""
    device = _abi.require_cuda_contiguous(raw=raw, partner_scores=partner_scores,
                                          norm_weight=norm_weight, norm_bias=norm_bias,
                                          hidden=hidden, mix=mix)
    _abi.require_position(position, device)
    batch, k_out, dim = raw.shape
    if partner_scores.shape != (batch, k_out) or partner_scores.dtype != torch.float32:
        raise ValueError("partner_scores must be float32 [B, K]")
    if hidden.shape != (batch, dim) or hidden.dtype != torch.float32 or mix.dtype != torch.float32 \
            or mix.numel() != 1:
        raise ValueError("hidden must be float32 [B, D] and mix a one-element float32 tensor")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_norm_reduce(
            _abi.ptr(raw), _abi.ptr(partner_scores), _abi.ptr(norm_weight), _abi.ptr(norm_bias),
            _abi.ptr(position), None, float(norm_eps), None, _abi.ptr(hidden), _abi.ptr(mix),
            None, None, 0.0, None, 0, 1, 0, None, batch, k_out, dim, _abi.code(raw),
            _abi.same_dtype("norm parameter", norm_weight, norm_bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@relation_norm_reduce_residual.register_fake
def _(raw, partner_scores, norm_weight, norm_bias, position, norm_eps, hidden, mix):
    return None


@torch.library.custom_op("relation_lm::relation_norm_reduce_residual_norm_project",
                         mutates_args=("hidden", "normalized", "projected"), device_types="cuda")
def relation_norm_reduce_residual_norm_project(
    raw: Tensor,
    partner_scores: Tensor,
    norm_weight: Tensor,
    norm_bias: Tensor,
    position: Tensor,
    norm_eps: float,
    hidden: Tensor,
    mix: Tensor,
    next_norm_weight: Tensor,
    next_norm_bias: Tensor,
    next_norm_eps: float,
    normalized: Tensor,
    projection_weight: Tensor,
    projected: Tensor,
) -> None:
    """``relation_norm_reduce_residual_norm`` that also applies the next layer's query projection
    (extension, decode batches of a few rows): ``projected = normalized @ projection_weight.T`` with
    ``projection_weight [N, D]`` and ``projected [B, N]`` in the dtype of ``normalized``,
    ``N`` = 32, 64, ... 256 and ``D`` a multiple of 64.  One launch; a cluster of ``N / 32`` CTAs per row."""
    device = _abi.require_cuda_contiguous(raw=raw, partner_scores=partner_scores,
                                          norm_weight=norm_weight, norm_bias=norm_bias,
                                          hidden=hidden, mix=mix, next_norm_weight=next_norm_weight,
                                          next_norm_bias=next_norm_bias, normalized=normalized,
                                          projection_weight=projection_weight, projected=projected)
    _abi.require_position(position, device)
    batch, k_out, dim = raw.shape
    if partner_scores.shape != (batch, k_out) or partner_scores.dtype != torch.float32:
        raise ValueError("partner_scores must be float32 [B, K]")
    if hidden.shape != (batch, dim) or hidden.dtype != torch.float32 or mix.dtype != torch.float32 \
            or mix.numel() != 1:
        raise ValueError("hidden must be float32 [B, D] and mix a one-element float32 tensor")
    if normalized.shape != (batch, dim) or next_norm_weight.dtype != torch.float32 \
            or next_norm_bias.dtype != torch.float32 or next_norm_weight.numel() != dim:
        raise ValueError("normalized must be [B, D] and the next LayerNorm parameters float32 [D]")
    n_out = projection_weight.shape[0]
    if projection_weight.shape != (n_out, dim) or projected.shape != (batch, n_out) \
            or projection_weight.dtype != normalized.dtype or projected.dtype != normalized.dtype:
        raise ValueError("projection_weight must be [N, D] and projected [B, N] in the dtype of normalized")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_norm_reduce_project(
            _abi.ptr(raw), _abi.ptr(partner_scores), _abi.ptr(norm_weight), _abi.ptr(norm_bias),
            _abi.ptr(position), float(norm_eps), _abi.ptr(hidden), _abi.ptr(mix),
            _abi.ptr(next_norm_weight), _abi.ptr(next_norm_bias), float(next_norm_eps),
            _abi.ptr(normalized), _abi.ptr(projection_weight), _abi.ptr(projected), n_out,
            _abi.code(normalized), None, batch, k_out, dim, _abi.code(raw),
            _abi.same_dtype("norm parameter", norm_weight, norm_bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@relation_norm_reduce_residual_norm_project.register_fake
def _(raw, partner_scores, norm_weight, norm_bias, position, norm_eps, hidden, mix, next_norm_weight,
      next_norm_bias, next_norm_eps, normalized, projection_weight, projected):
    return None


@torch.library.custom_op("relation_lm::relation_norm_reduce_residual_norm",
                         mutates_args=("hidden", "normalized"), device_types="cuda")
def relation_norm_reduce_residual_norm(
    raw: Tensor,
    partner_scores: Tensor,
    norm_weight: Tensor,
    norm_bias: Tensor,
    position: Tensor,
    norm_eps: float,
    hidden: Tensor,
    mix: Tensor,
    next_norm_weight: Tensor,
    next_norm_bias: Tensor,
    next_norm_eps: float,
    normalized: Tensor,
) -> None:
    """``relation_norm_reduce_residual`` that also writes ``normalized = layer_norm(hidden)`` of
    the updated rows (extension): ``normalized [B, D]`` bfloat16 / float16 with the next layer's
    (or the output head's) fp32 LayerNorm parameters, ready for the next projection."""
    device = _abi.require_cuda_contiguous(raw=raw, partner_scores=partner_scores,
                                          norm_weight=norm_weight, norm_bias=norm_bias,
                                          hidden=hidden, mix=mix, next_norm_weight=next_norm_weight,
                                          next_norm_bias=next_norm_bias, normalized=normalized)
    _abi.require_position(position, device)
    batch, k_out, dim = raw.shape
    if partner_scores.shape != (batch, k_out) or partner_scores.dtype != torch.float32:
        raise ValueError("partner_scores must be float32 [B, K]")
    if hidden.shape != (batch, dim) or hidden.dtype != torch.float32 or mix.dtype != torch.float32 \
            or mix.numel() != 1:
        raise ValueError("hidden must be float32 [B, D] and mix a one-element float32 tensor")
    if normalized.shape != (batch, dim) or next_norm_weight.dtype != torch.float32 \
            or next_norm_bias.dtype != torch.float32 or next_norm_weight.numel() != dim:
        raise ValueError("normalized must be [B, D] and the next LayerNorm parameters float32 [D]")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_norm_reduce(
            _abi.ptr(raw), _abi.ptr(partner_scores), _abi.ptr(norm_weight), _abi.ptr(norm_bias),
            _abi.ptr(position), None, float(norm_eps), None, _abi.ptr(hidden), _abi.ptr(mix),
            _abi.ptr(next_norm_weight), _abi.ptr(next_norm_bias), float(next_norm_eps),
            _abi.ptr(normalized), _abi.code(normalized), 1, 0, None, batch, k_out, dim, _abi.code(raw),
            _abi.same_dtype("norm parameter", norm_weight, norm_bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@relation_norm_reduce_residual_norm.register_fake
def _(raw, partner_scores, norm_weight, norm_bias, position, norm_eps, hidden, mix, next_norm_weight,
      next_norm_bias, next_norm_eps, normalized):
    return None


@torch.library.custom_op("relation_lm::relation_norm_reduce_residual_norm_slices",
                         mutates_args=("hidden", "normalized"), device_types="cuda")
def relation_norm_reduce_residual_norm_slices(
    raw_slices: Tensor,
    raw_bias: Tensor,
    partner_scores: Tensor,
    norm_weight: Tensor,
    norm_bias: Tensor,
    position: Tensor,
    norm_eps: float,
    hidden: Tensor,
    mix: Tensor,
    next_norm_weight: Tensor,
    next_norm_bias: Tensor,
    next_norm_eps: float,
    normalized: Tensor,
) -> None:
    """``relation_norm_reduce_residual_norm`` whose partner rows arrive as the fp32 slices of a
    split-K projection, ``raw = raw_slices.sum(0) + raw_bias`` with ``raw_slices [S, B, K, D]`` and
    ``raw_bias [D]`` in the dtype of the LayerNorm parameters (extension)."""
    device = _abi.require_cuda_contiguous(raw_slices=raw_slices, raw_bias=raw_bias, partner_scores=partner_scores,
                                          norm_weight=norm_weight, norm_bias=norm_bias, hidden=hidden, mix=mix,
                                          next_norm_weight=next_norm_weight, next_norm_bias=next_norm_bias,
                                          normalized=normalized)
    _abi.require_position(position, device)
    if raw_slices.dim() != 4 or raw_slices.dtype != torch.float32:
        raise ValueError("raw_slices must be float32 [S, B, K, D]")
    splits, batch, k_out, dim = raw_slices.shape
    if partner_scores.shape != (batch, k_out) or partner_scores.dtype != torch.float32:
        raise ValueError("partner_scores must be float32 [B, K]")
    if hidden.shape != (batch, dim) or hidden.dtype != torch.float32 or mix.dtype != torch.float32 \
            or mix.numel() != 1:
        raise ValueError("hidden must be float32 [B, D] and mix a one-element float32 tensor")
    if normalized.shape != (batch, dim) or next_norm_weight.dtype != torch.float32 \
            or next_norm_bias.dtype != torch.float32 or next_norm_weight.numel() != dim or raw_bias.numel() != dim:
        raise ValueError("normalized must be [B, D], raw_bias [D] and the next LayerNorm parameters float32 [D]")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_norm_reduce(
            _abi.ptr(raw_slices), _abi.ptr(partner_scores), _abi.ptr(norm_weight), _abi.ptr(norm_bias),
            _abi.ptr(position), None, float(norm_eps), None, _abi.ptr(hidden), _abi.ptr(mix),
            _abi.ptr(next_norm_weight), _abi.ptr(next_norm_bias), float(next_norm_eps),
            _abi.ptr(normalized), _abi.code(normalized), splits, batch * k_out * dim, _abi.ptr(raw_bias),
            batch, k_out, dim, _abi.code(raw_slices),
            _abi.same_dtype("norm parameter", norm_weight, norm_bias, raw_bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@relation_norm_reduce_residual_norm_slices.register_fake
def _(raw_slices, raw_bias, partner_scores, norm_weight, norm_bias, position, norm_eps, hidden, mix,
      next_norm_weight, next_norm_bias, next_norm_eps, normalized):
    return None


_TAIL_SCRATCH: dict[tuple[int, int], Tensor] = {}


def _tail_scratch(device: torch.device, nbytes: int) -> Tensor:
    """Zero-initialised scratch of the fused tail, one buffer per (device, stream): launches on
    different streams may overlap on the GPU and must not share split-K sums.  Grown on demand
    and reused after; growing inside a stream capture is refused (the buffer would belong to the
    graph's private pool)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, int(torch.cuda.current_stream(device).cuda_stream))
    buf = _TAIL_SCRATCH.get(key)
    if buf is None or buf.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("relation_tail: call once with these sizes on this stream before capturing it "
                               "(the scratch buffer has to be allocated outside the capture)")
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _TAIL_SCRATCH[key] = buf
    return buf


@torch.library.custom_op("relation_lm::relation_tail", mutates_args=("hidden",), device_types="cuda")
def relation_tail(
    relation_hidden: Tensor,
    second_weight: Tensor,
    second_bias: Tensor,
    partner_scores: Tensor,
    norm_weight: Tensor,
    norm_bias: Tensor,
    position: Tensor,
    norm_eps: float,
    hidden: Tensor,
    mix: Tensor,
) -> None:
    """Second relation-MLP layer, ``relation_norm_reduce`` and the residual update in one launch
    (extension): ``hidden += mix * norm_reduce(relation_hidden @ W2.T + b2, scores)``.
    ``relation_hidden [B, K, H]``, ``second_weight [d, H]`` and ``second_bias [d]`` share
    bfloat16 or float16; ``hidden [B, d]`` and the norm parameters are fp32.  The split-K
    partial sums meet in a scratch buffer kept per device and stream, allocated at the first call
    on that stream (which must come before any capture of it) and left zero by every launch."""
    device = _abi.require_cuda_contiguous(
        relation_hidden=relation_hidden, second_weight=second_weight, second_bias=second_bias,
        partner_scores=partner_scores, norm_weight=norm_weight, norm_bias=norm_bias,
        hidden=hidden, mix=mix)
    _abi.require_position(position, device)
    batch, k_out, hdim = relation_hidden.shape
    dim = second_weight.size(0)
    if second_weight.shape != (dim, hdim) or second_bias.numel() != dim or hidden.shape != (batch, dim):
        raise ValueError("expected second_weight [d, H], second_bias [d] and hidden [B, d]")
    if partner_scores.shape != (batch, k_out) or partner_scores.dtype != torch.float32 \
            or hidden.dtype != torch.float32 or mix.dtype != torch.float32 \
            or norm_weight.dtype != torch.float32 or norm_bias.dtype != torch.float32:
        raise ValueError("scores, hidden, mix and the norm parameters must be float32")
    need = int(_abi.LIB.rlm_relation_tail_scratch_bytes(batch, k_out, dim))
    scratch = _tail_scratch(device, need)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_tail(
            _abi.ptr(relation_hidden), _abi.ptr(second_weight), _abi.ptr(second_bias),
            _abi.ptr(partner_scores), _abi.ptr(norm_weight), _abi.ptr(norm_bias), _abi.ptr(position),
            float(norm_eps), _abi.ptr(hidden), _abi.ptr(mix), None, _abi.ptr(scratch), scratch.numel(),
            batch, k_out, dim, hdim,
            _abi.same_dtype("relation MLP", relation_hidden, second_weight, second_bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@relation_tail.register_fake
def _(relation_hidden, second_weight, second_bias, partner_scores, norm_weight, norm_bias, position,
      norm_eps, hidden, mix):
    return None


@torch.library.custom_op("relation_lm::relation_hidden_cached_rows", mutates_args=(),
                         device_types="cuda")
def relation_hidden_cached_rows(
    expanded_cache: Tensor,
    operand_cache: Tensor,
    anchor_index: Tensor,
    partner_index: Tensor,
    product_weight: Tensor,
    row_batch: Tensor,
) -> Tensor:
    """Per-row form of ``relation_hidden_cached`` (extension, prefill): query row ``i`` gathers
    from sequence ``row_batch[i]`` of caches ``[B, T, ...]``; ``anchor_index [N]``,
    ``partner_index [N, K]``; returns ``[N, K, H]`` fp32."""
    device = _abi.require_cuda_contiguous(
        expanded_cache=expanded_cache, operand_cache=operand_cache, anchor_index=anchor_index,
        partner_index=partner_index, product_weight=product_weight, row_batch=row_batch)
    n_seq, max_t, rdim = operand_cache.shape
    rows, k_out = partner_index.shape
    hdim = product_weight.size(0)
    _check_indices(anchor_index, partner_index, rows)
    if row_batch.dtype != torch.int32 or row_batch.numel() != rows:
        raise ValueError("row_batch must be int32 with one entry per query row")
    if expanded_cache.shape != (n_seq, max_t, 2 * hdim) or product_weight.size(1) != rdim:
        raise ValueError("expanded_cache must be [B, T, 2H] and product_weight [H, R]")
    out = torch.empty((rows, k_out, hdim), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_hidden_cached(
            _abi.ptr(expanded_cache), _abi.ptr(operand_cache), _abi.ptr(anchor_index),
            _abi.ptr(partner_index), _abi.ptr(product_weight), _abi.ptr(row_batch), _abi.ptr(out),
            rows, n_seq, max_t, rdim, hdim, k_out,
            _abi.same_dtype("cache", expanded_cache, operand_cache), _abi.code(product_weight),
            _abi.code(out), _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out


@relation_hidden_cached_rows.register_fake
def _(expanded_cache, operand_cache, anchor_index, partner_index, product_weight, row_batch):
    return operand_cache.new_empty(
        (partner_index.size(0), partner_index.size(1), product_weight.size(0)), dtype=torch.float32)


@torch.library.custom_op("relation_lm::relation_hidden_cached_rows_out", mutates_args=("out",),
                         device_types="cuda")
def relation_hidden_cached_rows_out(
    out: Tensor,
    expanded_cache: Tensor,
    operand_cache: Tensor,
    anchor_index: Tensor,
    partner_index: Tensor,
    product_weight: Tensor,
    row_batch: Tensor,
) -> None:
    """``relation_hidden_cached_rows`` into a caller-owned ``out [N, K, H]`` of any float dtype: a
    prefill pass over thousands of rows keeps the hidden states in 16 bits (half the bytes of the
    fp32 form, and the dtype the second relation-MLP layer's tensor-core GEMM reads)."""
    device = _abi.require_cuda_contiguous(
        out=out, expanded_cache=expanded_cache, operand_cache=operand_cache, anchor_index=anchor_index,
        partner_index=partner_index, product_weight=product_weight, row_batch=row_batch)
    n_seq, max_t, rdim = operand_cache.shape
    rows, k_out = partner_index.shape
    hdim = product_weight.size(0)
    _check_indices(anchor_index, partner_index, rows)
    if row_batch.dtype != torch.int32 or row_batch.numel() != rows:
        raise ValueError("row_batch must be int32 with one entry per query row")
    if expanded_cache.shape != (n_seq, max_t, 2 * hdim) or product_weight.size(1) != rdim \
            or out.shape != (rows, k_out, hdim):
        raise ValueError("expanded_cache must be [B, T, 2H], product_weight [H, R] and out [N, K, H]")
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_hidden_cached(
            _abi.ptr(expanded_cache), _abi.ptr(operand_cache), _abi.ptr(anchor_index),
            _abi.ptr(partner_index), _abi.ptr(product_weight), _abi.ptr(row_batch), _abi.ptr(out),
            rows, n_seq, max_t, rdim, hdim, k_out,
            _abi.same_dtype("cache", expanded_cache, operand_cache), _abi.code(product_weight),
            _abi.code(out), _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@relation_hidden_cached_rows_out.register_fake
def _(out, expanded_cache, operand_cache, anchor_index, partner_index, product_weight, row_batch):
    return None


@torch.library.custom_op("relation_lm::relation_norm_reduce_rows", mutates_args=(),
                         device_types="cuda")
def relation_norm_reduce_rows(
    raw: Tensor,
    partner_scores: Tensor,
    norm_weight: Tensor,
    norm_bias: Tensor,
    row_position: Tensor,
    norm_eps: float,
) -> Tensor:
    """Per-row form of ``relation_norm_reduce`` (extension, prefill): row ``i`` uses the active-K
    limit of position ``row_position[i]``."""
    device = _abi.require_cuda_contiguous(raw=raw, partner_scores=partner_scores,
                                          norm_weight=norm_weight, norm_bias=norm_bias,
                                          row_position=row_position)
    rows, k_out, dim = raw.shape
    if partner_scores.shape != (rows, k_out) or partner_scores.dtype != torch.float32:
        raise ValueError("partner_scores must be float32 [N, K]")
    if row_position.dtype != torch.int32 or row_position.numel() != rows:
        raise ValueError("row_position must be int32 with one entry per row")
    out = torch.empty((rows, dim), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_norm_reduce(
            _abi.ptr(raw), _abi.ptr(partner_scores), _abi.ptr(norm_weight), _abi.ptr(norm_bias),
            None, _abi.ptr(row_position), float(norm_eps), _abi.ptr(out), None, None, None, None, 0.0,
            None, 0, 1, 0, None, rows, k_out,
            dim, _abi.code(raw), _abi.same_dtype("norm parameter", norm_weight, norm_bias),
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out


@relation_norm_reduce_rows.register_fake
def _(raw, partner_scores, norm_weight, norm_bias, row_position, norm_eps):
    return raw.new_empty((raw.size(0), raw.size(2)), dtype=torch.float32)


def relation_layer_tail_supported(n_seq: int, k_out: int, relation_dim: int, hidden_dim: int, d_model: int,
                                  n_query: int, dtype: torch.dtype) -> bool:
    """Whether ``relation_layer_tail`` serves these sizes on the current device."""
    if dtype not in (torch.bfloat16, torch.float16):
        return False
    return bool(_abi.LIB.rlm_relation_layer_tail_supported(int(n_seq), int(k_out), int(relation_dim),
                                                           int(hidden_dim), int(d_model), int(n_query),
                                                           _abi.DTYPE_CODE[dtype]))


@torch.library.custom_op("relation_lm::relation_layer_tail", mutates_args=("hidden", "normalized", "query"),
                         device_types="cuda")
def relation_layer_tail(
    expanded_cache: Tensor,
    operand_cache: Tensor,
    anchor_index: Tensor,
    partner_index: Tensor,
    partner_scores: Tensor,
    product_weight: Tensor,
    second_weight: Tensor,
    second_bias: Tensor,
    norm_weight: Tensor,
    norm_bias: Tensor,
    position: Tensor,
    norm_eps: float,
    hidden: Tensor,
    mix: Tensor,
    next_norm_weight: Tensor,
    next_norm_bias: Tensor,
    next_norm_eps: float,
    normalized: Tensor,
    query_weight: Tensor | None,
    query: Tensor | None,
) -> None:
    """One launch for a layer's whole relation tail (extension; decode batches of a few sequences):
    ``relation_hidden_cached`` -> second relation-MLP layer -> ``relation_norm_reduce`` ->
    ``hidden += mix * context`` -> ``normalized = LayerNorm(hidden)`` (16-bit) and, when
    ``query_weight [NQ, d]`` is given, ``query = normalized @ query_weight.T``.  The relation hidden
    states never reach device memory and no library GEMM is called.  Caches and weights share
    bfloat16 or float16; ``hidden [B, d]`` and all LayerNorm parameters are fp32."""
    device = _abi.require_cuda_contiguous(
        expanded_cache=expanded_cache, operand_cache=operand_cache, anchor_index=anchor_index,
        partner_index=partner_index, partner_scores=partner_scores, product_weight=product_weight,
        second_weight=second_weight, second_bias=second_bias, norm_weight=norm_weight, norm_bias=norm_bias,
        hidden=hidden, mix=mix, next_norm_weight=next_norm_weight, next_norm_bias=next_norm_bias,
        normalized=normalized, query_weight=query_weight, query=query)
    _abi.require_position(position, device)
    batch, max_t, rdim = operand_cache.shape
    hdim, dim = product_weight.size(0), second_weight.size(0)
    k_out = partner_index.size(1)
    if expanded_cache.shape != (batch, max_t, 2 * hdim) or product_weight.shape != (hdim, rdim) \
            or second_weight.shape != (dim, hdim) or second_bias.numel() != dim \
            or anchor_index.shape != (batch,) or partner_index.shape != (batch, k_out) \
            or partner_scores.shape != (batch, k_out) or hidden.shape != (batch, dim) \
            or normalized.shape != (batch, dim):
        raise ValueError("relation_layer_tail: inconsistent shapes")
    if anchor_index.dtype != torch.int32 or partner_index.dtype != torch.int32:
        raise ValueError("index tensors must be int32")
    for name, t in (("partner_scores", partner_scores), ("hidden", hidden), ("mix", mix),
                    ("norm_weight", norm_weight), ("norm_bias", norm_bias),
                    ("next_norm_weight", next_norm_weight), ("next_norm_bias", next_norm_bias)):
        if t.dtype != torch.float32:
            raise ValueError(f"{name} must be float32")
    n_query = 0
    if query_weight is not None:
        if query is None or query_weight.dim() != 2 or query_weight.size(1) != dim \
                or query.shape != (batch, query_weight.size(0)):
            raise ValueError("query_weight [NQ, d] needs an output query [B, NQ]")
        n_query = query_weight.size(0)
    sixteen = [expanded_cache, operand_cache, product_weight, second_weight, second_bias, normalized]
    if query_weight is not None:
        sixteen += [query_weight, query]
    dtype = _abi.same_dtype("16-bit operand", *sixteen)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_relation_layer_tail(
            _abi.ptr(expanded_cache), _abi.ptr(operand_cache), _abi.ptr(anchor_index), _abi.ptr(partner_index),
            _abi.ptr(partner_scores), _abi.ptr(product_weight), _abi.ptr(second_weight), _abi.ptr(second_bias),
            _abi.ptr(norm_weight), _abi.ptr(norm_bias), _abi.ptr(position), float(norm_eps), _abi.ptr(hidden),
            _abi.ptr(mix), _abi.ptr(next_norm_weight), _abi.ptr(next_norm_bias), float(next_norm_eps),
            _abi.ptr(normalized), _abi.ptr(query_weight), _abi.ptr(query), batch, k_out, max_t, rdim, hdim,
            dim, n_query, dtype, _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))


@relation_layer_tail.register_fake
def _(expanded_cache, operand_cache, anchor_index, partner_index, partner_scores, product_weight,
      second_weight, second_bias, norm_weight, norm_bias, position, norm_eps, hidden, mix,
      next_norm_weight, next_norm_bias, next_norm_eps, normalized, query_weight, query):
    return None
