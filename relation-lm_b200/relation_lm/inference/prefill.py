"""Routed relation layers over whole sequences (prefill): every position of every sequence is a
query row, all in one pass.

The reference project's kernels serve one position per launch
(src/relation_lm/kernels/relation_select.py:50-51 reads one scalar position); its whole-sequence
code is dense (src/relation_lm/models/stacked_relation.py:65-136).  This module is the routed
whole-sequence form: the per-row operators of this library (``*_rows``) applied to all
``B * T`` rows, with the state a decode loop would have built position by position produced in
bulk first:

* ``build_state``: one packed projection of the memory stream for all positions
  (src/relation_lm/inference/packed_cache.py:52-57), split into the four token caches;
  ``router_cache_prefill`` (conv + block statistics of both router streams, equal to ``T``
  successive ``router_cache_update`` calls); the expanded cache ``[W_a o + b, W_p o]`` of the
  factorised first relation-MLP layer (src/relation_lm/kernels/relation_reduce.py:42-49).
* ``forward``: LayerNorm -> 256-wide query projection -> ``relation_select_packed_rows`` ->
  ``relation_hidden_cached_rows`` (16-bit) -> second relation-MLP layer (tensor-core projection) ->
  ``relation_norm_reduce_rows`` -> ``hidden + sigmoid(mix) * context``.

Row ``(b, t)`` sees exactly what the decode step at position ``t`` of sequence ``b`` sees: block
statistics of complete blocks only and candidates at positions ``<= t``.
"""
from __future__ import annotations

import torch
from torch import Tensor

from relation_lm.inference.routed_model import RoutedRelationLM
from relation_lm.kernels.packed_projection import layer_norm_cast, packed_projection
from relation_lm.kernels.relation_reduce import relation_hidden_cached_rows_out, relation_norm_reduce_rows
from relation_lm.kernels.relation_select import relation_select_packed_prefill, relation_select_packed_rows
from relation_lm.kernels.router_cache import router_cache_prefill


class RoutedPrefillLayer:
    """Layer ``layer`` of a ``RoutedRelationLM`` applied to whole sequences ``[B, T, d]``."""

    def __init__(self, model: RoutedRelationLM, layer: int = 0, device="cuda",
                 dtype: torch.dtype = torch.bfloat16, tiled_select: bool = True) -> None:
        self.tiled_select = bool(tiled_select)
        if dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("the prefill path runs its projections on the tensor cores: bfloat16 or float16")
        self.config, self.layer, self.device, self.dtype = model.config, int(layer), torch.device(device), dtype
        w = model.decode_weights(self.device, dtype)
        cfg, l = self.config, self.layer
        width = cfg.packed_width
        self.w = {
            "memory_norm_w": w["memory_norm_w"], "memory_norm_b": w["memory_norm_b"],
            "input_norm_w": w["input_norm_w"][l], "input_norm_b": w["input_norm_b"][l],
            "w_packed": w["w_packed"][l * width:(l + 1) * width].contiguous(),
            "w_query": w["w_query"][l],
            "w_expand": torch.cat((w["anchor_weight"][l], w["partner_weight"][l]), 0).contiguous(),
            "b_expand": torch.cat((w["first_bias"][l].float(), torch.zeros(cfg.hidden_dim, device=self.device))),
            "product_weight": w["product_weight"][l], "w2": w["w2"][l], "b2": w["b2"][l].float().contiguous(),
            "relation_norm_w": w["relation_norm_w"][l], "relation_norm_b": w["relation_norm_b"][l],
            "mix": w["mix"][l],
            "anchor_gamma": w["anchor_gamma"][l], "anchor_bias": w["anchor_bias"][l],
            "partner_gamma": w["partner_gamma"][l], "partner_bias": w["partner_bias"][l],
            "anchor_conv_weight": w["anchor_conv_weight"][l], "partner_conv_weight": w["partner_conv_weight"][l],
        }

    def rows(self, batch: int, length: int) -> tuple[Tensor, Tensor]:
        """``(row_batch, row_position)`` of all ``batch * length`` query rows, sequence-major."""
        rb = torch.arange(batch, device=self.device, dtype=torch.int32).repeat_interleave(length)
        rp = torch.arange(length, device=self.device, dtype=torch.int32).repeat(batch)
        return rb, rp

    def build_state(self, x: Tensor) -> dict[str, Tensor]:
        """Caches and block statistics of sequences whose embedded inputs are ``x [B, T, d]`` (fp32)."""
        cfg, w = self.config, self.w
        B, T, d = x.shape
        if T != cfg.max_context:
            raise ValueError("the sequences must fill the configured context")
        R, H, nb = cfg.relation_dim, cfg.hidden_dim, T // cfg.block_size
        memory = torch.empty(B * T, d, device=self.device, dtype=self.dtype)
        layer_norm_cast(x.view(B * T, d), w["memory_norm_w"], w["memory_norm_b"], cfg.norm_eps, memory)
        packed = packed_projection(memory, w["w_packed"]).view(B, T, cfg.packed_width)
        state = {
            "anchor_keys": packed[..., 0:64].contiguous(), "partner_keys": packed[..., 64:128].contiguous(),
            "operand_cache": packed[..., 128:128 + R].contiguous(),
            "partner_anchor_cache": packed[..., 128 + R:256 + R].contiguous(),
        }
        zeros = lambda *s: torch.zeros(*s, device=self.device, dtype=self.dtype)  # noqa: E731
        names = ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache")
        for n in names:
            state[n] = zeros(B, T, 64)
        for n in ("anchor_mean", "anchor_std", "partner_mean", "partner_std"):
            state[n] = zeros(B, nb, 4, 16)
        router_cache_prefill(packed[..., 256 + R:320 + R], packed[..., 320 + R:384 + R],
                             *[state[n] for n in names], state["anchor_mean"], state["anchor_std"],
                             state["partner_mean"], state["partner_std"], w["anchor_conv_weight"],
                             w["partner_conv_weight"], cfg.block_size)
        state["expanded_cache"] = packed_projection(state["operand_cache"].view(B * T, R), w["w_expand"],
                                                    w["b_expand"]).view(B, T, 2 * H)
        state["packed"] = packed
        return state

    def forward(self, x: Tensor, state: dict[str, Tensor], keep: dict | None = None) -> Tensor:
        """The layer's output ``[B, T, d]`` (fp32) for residual inputs ``x [B, T, d]`` (fp32).  With a
        dict in ``keep`` the intermediates (queries, selections, hidden states, second-layer
        output, context) are left there for a checker."""
        cfg, w = self.config, self.w
        B, T, d = x.shape
        N, K, H = B * T, cfg.k_max, cfg.hidden_dim
        rb, rp = self.rows(B, T)
        normalized = torch.empty(N, d, device=self.device, dtype=self.dtype)
        layer_norm_cast(x.view(N, d), w["input_norm_w"], w["input_norm_b"], cfg.norm_eps, normalized)
        q = packed_projection(normalized, w["w_query"])
        select_args = (q[:, 0:64], state["anchor_keys"], q[:, 64:128], state["anchor_mean"], state["anchor_std"],
                       w["anchor_gamma"], w["anchor_bias"], q[:, 128:256], state["partner_anchor_cache"],
                       state["partner_keys"], state["partner_mean"], state["partner_std"], w["partner_gamma"],
                       w["partner_bias"])
        selected = None
        if self.tiled_select and cfg.local_window + cfg.top_blocks * cfg.block_size <= 512:
            # all positions of every sequence: tiles of consecutive positions share their staging
            try:
                selected = relation_select_packed_prefill(*select_args, T, cfg.local_window, cfg.top_blocks, K,
                                                          cfg.strict_valid)
            except (ValueError, RuntimeError) as error:
                if "shared memory" not in str(error):       # only "the tile's staging does not fit" falls back
                    raise
                self.tiled_select = False                   # rejected before anything was launched
        if selected is None:
            selected = relation_select_packed_rows(*select_args, rb, rp, cfg.local_window, cfg.top_blocks, K,
                                                   cfg.strict_valid)
        anchor, anchor_score, partner, partner_score = selected
        hidden_rel = torch.empty(N, K, H, device=self.device, dtype=self.dtype)
        relation_hidden_cached_rows_out(hidden_rel, state["expanded_cache"], state["operand_cache"], anchor,
                                        partner, w["product_weight"], rb)
        raw = packed_projection(hidden_rel.view(N * K, H), w["w2"], w["b2"]).view(N, K, d)
        context = relation_norm_reduce_rows(raw, partner_score, w["relation_norm_w"], w["relation_norm_b"], rp,
                                            cfg.norm_eps)
        out = torch.addcmul(x.view(N, d), context, w["mix"]).view(B, T, d)
        if keep is not None:
            keep.update(query=q, anchor=anchor, anchor_score=anchor_score, partner=partner,
                        partner_score=partner_score, hidden=hidden_rel, raw=raw, context=context,
                        row_batch=rb, row_position=rp)
        return out
