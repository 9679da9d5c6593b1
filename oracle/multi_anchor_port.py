"""CPU port of the routed multi-anchor layer pass — TEST INFRASTRUCTURE only.

Mirrors ``relation_lm.inference.multi_anchor.MultiAnchorPrefill`` operator for operator with the
CPU oracle (``relation_oracle.c``) in place of every CUDA kernel and fp32 torch matmuls in place of
the GPU GEMMs; values the GPU path stores in a 16-bit tensor are rounded to that dtype here too.
The selection composes ``oracle.anchor_select`` / ``oracle.partner_topk`` with exclusion lists
under the rules of the reference's dense block (src/relation_lm/models/multi_relation_blocks.py:69-148).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

import oracle


class OracleMultiAnchor:
    def __init__(self, stack, dtype: torch.dtype = torch.float32) -> None:
        self.config, self.dtype = stack.config, dtype
        self.layers = [{k: v.float() for k, v in stack.layer_weights(l, "cpu", dtype).items()}
                       for l in range(stack.config.depth)]
        self.final_norm_w = stack.final_norm.weight.detach().float()
        self.final_norm_b = stack.final_norm.bias.detach().float()

    def _round(self, x):
        return x if self.dtype == torch.float32 else x.to(self.dtype).float()

    def build_state(self, layer: int, memory: torch.Tensor, packed: torch.Tensor | None = None) -> dict:
        """State of layer ``layer``; with ``packed`` (the memory-side projection as another implementation
        computed it, ``[B, T, S * 384 + R]``) everything downstream of that projection is derived from it."""
        cfg, w = self.config, self.layers[layer]
        B, T, d = memory.shape
        S, R, nb = cfg.anchors_per_block, cfg.relation_dim, T // cfg.block_size
        if packed is None:
            packed = self._round(memory.reshape(B * T, d).float() @ w["w_memory"].T).view(B, T, S * 384 + R)
        packed = packed.float()
        slots = packed[..., :S * 384].view(B, T, S, 384)
        per_slot = lambda lo, hi: slots[..., lo:hi].permute(2, 0, 1, 3).contiguous()  # noqa: E731
        state = {"anchor_keys": per_slot(0, 64), "partner_keys": per_slot(64, 128),
                 "partner_anchor_cache": per_slot(128, 256), "operand_cache": packed[..., S * 384:].contiguous()}
        names = ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache")
        for n in names:
            state[n] = torch.zeros(S, B, T, 64)
        for n in ("anchor_mean", "anchor_std", "partner_mean", "partner_std"):
            state[n] = torch.zeros(S, B, nb, 4, 16)
        if cfg.top_blocks > 0:                                   # block statistics only matter with remote blocks
            for s in range(S):
                for t in range(T):
                    oracle.router_cache_update(
                        slots[:, t, s, 256:320], slots[:, t, s, 320:384], *[state[n][s] for n in names],
                        state["anchor_mean"][s], state["anchor_std"][s], state["partner_mean"][s],
                        state["partner_std"][s], w["anchor_conv_weight"][s], w["partner_conv_weight"][s], t,
                        cfg.block_size, inplace=True, cache_dtype=self.dtype, stats_dtype=self.dtype)
        state["expanded_cache"] = self._round(state["operand_cache"].view(B * T, R) @ w["w_expand"].T
                                              + w["b_expand"]).view(B, T, -1)
        return state

    def select(self, layer: int, q: torch.Tensor, state: dict, row_batch, row_pos):
        """The routed multi-anchor selection of query rows ``q [N, S * 256]`` from oracle calls."""
        cfg, w = self.config, self.layers[layer]
        S, K, L, top = cfg.anchors_per_block, cfg.partners_per_anchor, cfg.local_window, cfg.top_blocks
        N = q.size(0)
        aq = q[:, :S * 64].reshape(N, S, 64)
        arq = q[:, S * 64:S * 128].reshape(N, S, 64)
        pb = q[:, S * 128:].reshape(N, S, 128)
        active = torch.arange(S)[None, :] <= row_pos[:, None]
        taken = torch.full((N, S), -1, dtype=torch.int32)
        anchors = torch.zeros(N, S, dtype=torch.int32)
        for s in range(S):
            idx, score = oracle.anchor_select(aq[:, s], state["anchor_keys"][s], arq[:, s], state["anchor_mean"][s],
                                              state["anchor_std"][s], w["anchor_gamma"][s], w["anchor_bias"][s], 0, L,
                                              top, cfg.strict_valid, row_batch=row_batch, row_pos=row_pos,
                                              exclude_index=taken.clone())
            live = active[:, s] & torch.isfinite(score)
            anchors[:, s] = torch.where(live, idx, torch.zeros_like(idx))
            taken[:, s] = torch.where(live, idx, torch.full_like(idx, -1))
            active[:, s] = live
        partners = torch.zeros(N, S, K, dtype=torch.int32)
        scores = torch.full((N, S, K), -torch.inf)
        for s in range(S):
            v = pb[:, s].float() + state["partner_anchor_cache"][s][row_batch.long(), anchors[:, s].long()].float()
            idx, score = oracle.partner_topk(v[:, :64], state["partner_keys"][s], v[:, 64:], state["partner_mean"][s],
                                             state["partner_std"][s], w["partner_gamma"][s], w["partner_bias"][s], 0,
                                             taken[:, s], L, top, K, cfg.strict_valid, row_batch=row_batch,
                                             row_pos=row_pos, exclude_index=taken)
            live = active[:, s, None] & torch.isfinite(score)
            partners[:, s] = torch.where(live, idx, torch.zeros_like(idx))
            scores[:, s] = torch.where(live, score, torch.full_like(score, -torch.inf))
        return anchors, active, partners, scores

    def forward_layer(self, layer: int, hidden: torch.Tensor, state: dict, keep: dict | None = None):
        cfg, w = self.config, self.layers[layer]
        B, T, d = hidden.shape
        N, S, K = B * T, cfg.anchors_per_block, cfg.partners_per_anchor
        row_batch = torch.arange(B, dtype=torch.int32).repeat_interleave(T)
        row_pos = torch.arange(T, dtype=torch.int32).repeat(B)
        normalized = self._round(F.layer_norm(hidden.view(N, d), (d,), w["input_norm_w"], w["input_norm_b"], cfg.norm_eps))
        q = self._round(normalized @ w["w_query"].T)
        anchors, active, partners, scores = self.select(layer, q, state, row_batch, row_pos)
        pair_rows = row_batch.repeat_interleave(S)
        hidden_rel, _ = oracle.relation_hidden(state["expanded_cache"], state["operand_cache"], anchors.view(N * S),
                                               partners.view(N * S, K), w["product_weight"], row_batch=pair_rows,
                                               row_pos=row_pos.repeat_interleave(S))
        raw = self._round(self._round(hidden_rel) @ w["w2"].T + w["b2"])
        no_limit = torch.full((N * S,), (1 << 30) - 2, dtype=torch.int32)
        slot_context = oracle.relation_norm_reduce(raw, scores.view(N * S, K), w["relation_norm_w"],
                                                   w["relation_norm_b"], 0, cfg.norm_eps, row_pos=no_limit).view(N, S, d)
        weight = w["slot_weight"][None, :] * active
        weight = weight / weight.sum(-1, keepdim=True).clamp_min(1.0e-9)
        context = (slot_context * weight[..., None]).sum(1)
        out = hidden + (w["gate"] * context).view(B, T, d)
        if keep is not None:
            keep.update(anchor=anchors, anchor_active=active, partner=partners, partner_score=scores,
                        slot_context=slot_context, context=context)
        return out

    def forward(self, hidden: torch.Tensor, memory: torch.Tensor, keep: list | None = None) -> torch.Tensor:
        current = hidden
        for l in range(self.config.depth):
            state = self.build_state(l, memory)
            kept = {} if keep is not None else None
            current = self.forward_layer(l, current, state, kept)
            if keep is not None:
                keep.append(kept)
        return F.layer_norm(current, (current.size(-1),), self.final_norm_w, self.final_norm_b, self.config.norm_eps)
