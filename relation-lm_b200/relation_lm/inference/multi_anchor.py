"""Routed multi-anchor relation layers: parameters and the whole-sequence (prefill) pass.

The reference project's ``MultiAnchorRelationBlock`` / ``RelationBlockStack``
(src/relation_lm/models/multi_relation_blocks.py:21-207) are dense: every anchor slot scores
all causal positions.  This module keeps the reference's parameters (same names and shapes, so
a state dict moves between the two) and adds one block router per slot (names as the
reference's ``DistilledBlockRouter``, src/relation_lm/routing/block_router.py:21-48); the pass
below is the routed form of the reference's ``forward`` for all positions at once:

1. per block, memory side (``build_state``): one packed projection of ``memory`` for all slots
   — per slot anchor key | partner key | anchor half of the partner query (exact 64 + router 64)
   | anchor router key | partner router key, then the shared operand — split into per-slot
   caches; ``router_cache_prefill`` per slot and stream; the expanded cache of the factorised
   first relation-MLP layer;
2. query side (``forward``): LayerNorm -> one projection for all slots' queries ->
   ``relation_select_multi_rows`` (distinct anchors, anchors barred from every partner set) ->
   relation hidden rows for the ``S * K`` (anchor, partner) pairs of every query -> second
   relation-MLP layer -> per-slot LayerNorm + softmax over the finite partner scores (no
   active-K limit: multi_relation_blocks.py:164-168) -> slot mixing and the gated residual.

With a window that covers the whole history and no remote blocks the pass reproduces the dense
reference block (pinned by golden outputs of the reference stack itself).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import Tensor, nn


@dataclass
class MultiAnchorConfig:
    d_model: int = 512
    gate_dim: int = 64
    relation_dim: int = 128
    ff_mult: int = 4
    anchors_per_block: int = 4
    partners_per_anchor: int = 4
    depth: int = 4
    max_context: int = 2048
    block_size: int = 32
    local_window: int = 64
    top_blocks: int = 3
    strict_valid: bool = False
    router_heads: int = 4
    router_head_dim: int = 16
    relative_buckets: int = 16
    norm_eps: float = 1.0e-5

    @property
    def hidden_dim(self) -> int:
        return self.ff_mult * self.d_model

    @property
    def slot_width(self) -> int:
        """Packed memory-side columns of one slot: anchor key 64 | partner key 64 | partner-anchor 128
        | anchor router key 64 | partner router key 64."""
        return 384


class SlotRouterParameters(nn.Module):
    """One block router per anchor slot (leading slot dimension on the small tables)."""

    def __init__(self, cfg: MultiAnchorConfig) -> None:
        super().__init__()
        s, d, width = cfg.anchors_per_block, cfg.d_model, cfg.router_heads * cfg.router_head_dim
        self.anchor_q = nn.Linear(d, s * width, bias=False)
        self.anchor_k = nn.Linear(d, s * width, bias=False)
        self.partner_q = nn.ModuleList(nn.Linear(2 * d, width, bias=False) for _ in range(s))
        self.partner_k = nn.Linear(d, s * width, bias=False)
        self.anchor_gamma = nn.Parameter(torch.zeros(s, cfg.router_heads))
        self.partner_gamma = nn.Parameter(torch.zeros(s, cfg.router_heads))
        self.anchor_bias = nn.Parameter(torch.zeros(s, cfg.router_heads, cfg.relative_buckets))
        self.partner_bias = nn.Parameter(torch.zeros(s, cfg.router_heads, cfg.relative_buckets))
        self.anchor_conv_weight = nn.Parameter(torch.zeros(s, width, 3))
        self.partner_conv_weight = nn.Parameter(torch.zeros(s, width, 3))


class MultiAnchorLayerParameters(nn.Module):
    """Parameters of one multi-anchor layer (names as the reference's ``MultiAnchorRelationBlock``)."""

    def __init__(self, cfg: MultiAnchorConfig) -> None:
        super().__init__()
        h, d, g, r = cfg.anchors_per_block, cfg.d_model, cfg.gate_dim, cfg.relation_dim
        self.input_norm = nn.LayerNorm(d, eps=cfg.norm_eps)
        self.anchor_query = nn.Linear(d, h * g, bias=False)
        self.anchor_key = nn.Linear(d, h * g, bias=False)
        self.partner_query = nn.ModuleList(nn.Linear(2 * d, g, bias=False) for _ in range(h))
        self.partner_key = nn.Linear(d, h * g, bias=False)
        self.operand = nn.Linear(d, r, bias=False)
        self.relation_mlp = nn.Sequential(
            nn.Linear(4 * r, cfg.hidden_dim), nn.GELU(), nn.Linear(cfg.hidden_dim, d), nn.LayerNorm(d, eps=cfg.norm_eps))
        self.slot_mix_logits = nn.Parameter(torch.zeros(h))
        self.residual_gate = nn.Parameter(torch.tensor(-1.5))
        self.router = SlotRouterParameters(cfg)


class MultiAnchorRoutedStack(nn.Module):
    """``depth`` multi-anchor layers over one shared memory stream and a final LayerNorm
    (the reference's ``RelationBlockStack``)."""

    def __init__(self, cfg: MultiAnchorConfig, seed: int = 0) -> None:
        super().__init__()
        if cfg.gate_dim != 64 or cfg.router_heads * cfg.router_head_dim != 64:
            raise ValueError("the selection kernels are built for gate width 64 and a 4 x 16 router")
        if cfg.anchors_per_block > 8:
            raise ValueError("at most 8 anchor slots")
        if cfg.max_context % cfg.block_size != 0:
            raise ValueError("max_context must be a multiple of block_size")
        self.config = cfg
        self.blocks = nn.ModuleList(MultiAnchorLayerParameters(cfg) for _ in range(cfg.depth))
        self.final_norm = nn.LayerNorm(cfg.d_model, eps=cfg.norm_eps)
        self.reset_parameters(seed)

    def reset_parameters(self, seed: int) -> None:
        """Seeded random init: Xavier-uniform matrices, N(0, 0.1^2) conv taps, N(0, 1) router gamma /
        bias tables and slot logits, small random biases and LayerNorm affines."""
        g = torch.Generator(device="cpu").manual_seed(int(seed))
        with torch.no_grad():
            for name, p in self.named_parameters():
                if name.endswith("conv_weight"):
                    p.copy_(torch.randn(p.shape, generator=g) * 0.1)
                elif name.endswith("gamma") or name.endswith("anchor_bias") or name.endswith("partner_bias") \
                        or name.endswith("slot_mix_logits"):
                    p.copy_(torch.randn(p.shape, generator=g))
                elif name.endswith("residual_gate"):
                    p.fill_(-1.5)
                elif p.dim() == 2:
                    bound = math.sqrt(6.0 / (p.size(0) + p.size(1)))
                    p.copy_((torch.rand(p.shape, generator=g) * 2 - 1) * bound)
                elif "norm" in name or name.endswith("relation_mlp.3.weight") or name.endswith("relation_mlp.3.bias"):
                    base = 1.0 if name.endswith("weight") else 0.0
                    p.copy_(base + torch.randn(p.shape, generator=g) * 0.05)
                else:
                    p.copy_(torch.randn(p.shape, generator=g) * 0.02)

    def layer_weights(self, layer: int, device, dtype) -> dict[str, Tensor]:
        """One layer's parameters in the layout the routed pass consumes (see the module docstring)."""
        cfg, block = self.config, self.blocks[layer]
        d, s_count, g = cfg.d_model, cfg.anchors_per_block, cfg.gate_dim
        r = block.router
        memory_rows, query_anchor, query_router, query_partner = [], [], [], []
        for s in range(s_count):
            rows = slice(s * g, (s + 1) * g)
            partner_anchor = torch.cat((block.partner_query[s].weight[:, d:], r.partner_q[s].weight[:, d:]), 0)
            memory_rows += [block.anchor_key.weight[rows], block.partner_key.weight[rows], partner_anchor,
                            r.anchor_k.weight[rows], r.partner_k.weight[rows]]
            query_anchor.append(block.anchor_query.weight[rows])
            query_router.append(r.anchor_q.weight[rows])
            query_partner.append(torch.cat((block.partner_query[s].weight[:, :d], r.partner_q[s].weight[:, :d]), 0))
        memory_rows.append(block.operand.weight)
        first = block.relation_mlp[0]
        a_raw, p_raw, product, diff = first.weight.split(cfg.relation_dim, dim=1)
        f32 = torch.float32

        def put(t, dt=dtype):
            return t.detach().to(device=device, dtype=dt).contiguous()

        return {
            "input_norm_w": put(block.input_norm.weight, f32), "input_norm_b": put(block.input_norm.bias, f32),
            # [S * 384 + R, d]
            "w_memory": put(torch.cat(memory_rows, 0)),
            # [S * 64 | S * 64 | S * 128, d]: all anchor queries, all anchor router queries, all partner bases
            "w_query": put(torch.cat(query_anchor + query_router + query_partner, 0)),
            "w_expand": put(torch.cat((a_raw + diff, p_raw - diff), 0)),
            "b_expand": put(torch.cat((first.bias, torch.zeros_like(first.bias))), f32),
            "product_weight": put(product), "w2": put(block.relation_mlp[2].weight),
            "b2": put(block.relation_mlp[2].bias, f32),
            "relation_norm_w": put(block.relation_mlp[3].weight, f32),
            "relation_norm_b": put(block.relation_mlp[3].bias, f32),
            "slot_weight": put(block.slot_mix_logits.softmax(0), f32),
            "gate": put(torch.sigmoid(block.residual_gate), f32),
            "anchor_gamma": put(r.anchor_gamma, f32), "anchor_bias": put(r.anchor_bias, f32),
            "partner_gamma": put(r.partner_gamma, f32), "partner_bias": put(r.partner_bias, f32),
            "anchor_conv_weight": put(r.anchor_conv_weight, f32), "partner_conv_weight": put(r.partner_conv_weight, f32),
        }


class MultiAnchorPrefill:
    """The routed pass of a ``MultiAnchorRoutedStack`` over whole sequences on one GPU."""

    def __init__(self, stack: MultiAnchorRoutedStack, device="cuda", dtype: torch.dtype = torch.bfloat16,
                 tiled_select: bool = True) -> None:
        if dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("the routed pass runs its projections on the tensor cores: bfloat16 or float16")
        self.config, self.device, self.dtype = stack.config, torch.device(device), dtype
        self.tiled_select = bool(tiled_select)           # whole-sequence selector (bfloat16) instead of the per-row one
        self.layers = [stack.layer_weights(l, self.device, dtype) for l in range(stack.config.depth)]
        self.final_norm_w = stack.final_norm.weight.detach().to(self.device, torch.float32)
        self.final_norm_b = stack.final_norm.bias.detach().to(self.device, torch.float32)

    def rows(self, batch: int, length: int) -> tuple[Tensor, Tensor]:
        rb = torch.arange(batch, device=self.device, dtype=torch.int32).repeat_interleave(length)
        rp = torch.arange(length, device=self.device, dtype=torch.int32).repeat(batch)
        return rb, rp

    def build_state(self, layer: int, memory: Tensor) -> dict[str, Tensor]:
        """Per-slot caches and block statistics of layer ``layer`` for ``memory [B, T, d]`` (16-bit)."""
        from relation_lm.kernels.packed_projection import packed_projection
        from relation_lm.kernels.router_cache import router_cache_prefill

        cfg, w = self.config, self.layers[layer]
        B, T, d = memory.shape
        S, R, H, nb = cfg.anchors_per_block, cfg.relation_dim, cfg.hidden_dim, T // cfg.block_size
        packed = packed_projection(memory.reshape(B * T, d), w["w_memory"]).view(B, T, S * 384 + R)
        slots = packed[..., :S * 384].view(B, T, S, 384)

        def per_slot(lo, hi):
            return slots[..., lo:hi].permute(2, 0, 1, 3).contiguous()          # [S, B, T, width]

        state = {"anchor_keys": per_slot(0, 64), "partner_keys": per_slot(64, 128),
                 "partner_anchor_cache": per_slot(128, 256),
                 "operand_cache": packed[..., S * 384:].contiguous(), "packed": packed}
        zeros = lambda *shape: torch.zeros(*shape, device=self.device, dtype=self.dtype)  # noqa: E731
        for n in ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache"):
            state[n] = zeros(S, B, T, 64)
        for n in ("anchor_mean", "anchor_std", "partner_mean", "partner_std"):
            state[n] = zeros(S, B, nb, 4, 16)
        for s in range(S):
            router_cache_prefill(slots[:, :, s, 256:320], slots[:, :, s, 320:384], state["anchor_raw_cache"][s],
                                 state["partner_raw_cache"][s], state["anchor_conv_cache"][s],
                                 state["partner_conv_cache"][s], state["anchor_mean"][s], state["anchor_std"][s],
                                 state["partner_mean"][s], state["partner_std"][s], w["anchor_conv_weight"][s],
                                 w["partner_conv_weight"][s], cfg.block_size)
        state["expanded_cache"] = packed_projection(state["operand_cache"].view(B * T, R), w["w_expand"],
                                                    w["b_expand"]).view(B, T, 2 * H)
        return state

    def forward_layer(self, layer: int, hidden: Tensor, state: dict[str, Tensor], keep: dict | None = None) -> Tensor:
        """Updates the residual stream ``hidden [B, T, d]`` (fp32) in place and returns it."""
        from relation_lm.kernels.multi_select import (relation_select_multi_prefill, relation_select_multi_rows,
                                                      slot_mix_residual)
        from relation_lm.kernels.packed_projection import layer_norm_cast, packed_projection
        from relation_lm.kernels.relation_reduce import relation_hidden_cached_rows_out, relation_norm_reduce_rows

        cfg, w = self.config, self.layers[layer]
        B, T, d = hidden.shape
        N, S, K, H = B * T, cfg.anchors_per_block, cfg.partners_per_anchor, cfg.hidden_dim
        rb, rp = self.rows(B, T)
        normalized = torch.empty(N, d, device=self.device, dtype=self.dtype)
        layer_norm_cast(hidden.view(N, d), w["input_norm_w"], w["input_norm_b"], cfg.norm_eps, normalized)
        q = packed_projection(normalized, w["w_query"])                          # [N, S * 256]
        anchor_query = q[:, :S * 64].unflatten(1, (S, 64))                       # column slices of one projection
        anchor_router_query = q[:, S * 64:S * 128].unflatten(1, (S, 64))
        partner_base = q[:, S * 128:].unflatten(1, (S, 128))
        select_args = (anchor_query, state["anchor_keys"], anchor_router_query, state["anchor_mean"], state["anchor_std"],
                       w["anchor_gamma"], w["anchor_bias"], partner_base, state["partner_anchor_cache"],
                       state["partner_keys"], state["partner_mean"], state["partner_std"], w["partner_gamma"],
                       w["partner_bias"])
        tiled = (self.tiled_select and self.dtype == torch.bfloat16
                 and cfg.local_window + cfg.top_blocks * cfg.block_size <= 512)
        selected = None
        if tiled:
            # whole sequences: tiles of consecutive positions share the staged statistics and windows
            try:
                selected = relation_select_multi_prefill(*select_args, T, cfg.local_window, cfg.top_blocks, K,
                                                         cfg.strict_valid)
            except (ValueError, RuntimeError) as error:
                if "shared memory" not in str(error):       # only "the tile's staging does not fit" falls back
                    raise
                self.tiled_select = False                   # rejected before anything was launched
        if selected is None:
            selected = relation_select_multi_rows(*select_args, rb, rp, cfg.local_window, cfg.top_blocks, K,
                                                  cfg.strict_valid)
        anchor, anchor_score, anchor_active, partner, partner_score, partner_active = selected
        pair_rows = rb.repeat_interleave(S)
        hidden_rel = torch.empty(N * S, K, H, device=self.device, dtype=self.dtype)
        relation_hidden_cached_rows_out(hidden_rel, state["expanded_cache"], state["operand_cache"],
                                        anchor.view(N * S), partner.view(N * S, K), w["product_weight"], pair_rows)
        raw = packed_projection(hidden_rel.view(N * S * K, H), w["w2"], w["b2"]).view(N * S, K, d)
        # softmax over the finite partner scores of a slot, no active-K limit: a position far enough out
        no_limit = torch.full((N * S,), (1 << 30) - 2, device=self.device, dtype=torch.int32)
        slot_context = relation_norm_reduce_rows(raw, partner_score.view(N * S, K), w["relation_norm_w"],
                                                 w["relation_norm_b"], no_limit, cfg.norm_eps).view(N, S, d)
        slot_mix_residual(slot_context, anchor_active, w["slot_weight"], w["gate"], hidden.view(N, d))
        if keep is not None:
            keep.update(query=q, anchor=anchor, anchor_score=anchor_score, anchor_active=anchor_active,
                        partner=partner, partner_score=partner_score, partner_active=partner_active,
                        hidden_rel=hidden_rel, raw=raw, slot_context=slot_context, row_batch=rb, row_position=rp)
        return hidden

    def forward(self, hidden: Tensor, memory: Tensor, keep: list | None = None) -> Tensor:
        """The stack's output ``[B, T, d]`` (fp32): ``depth`` layers on a copy of ``hidden`` with one
        shared ``memory`` (16-bit), then the final LayerNorm."""
        current = hidden.clone()
        for l in range(self.config.depth):
            state = self.build_state(l, memory)
            kept = {} if keep is not None else None
            self.forward_layer(l, current, state, kept)
            if keep is not None:
                kept["state"] = state
                keep.append(kept)
        return torch.nn.functional.layer_norm(current, (current.size(-1),), self.final_norm_w, self.final_norm_b,
                                              self.config.norm_eps)
