"""CPU port of one stateful decode step — TEST INFRASTRUCTURE and timed CPU baseline only.

Mirrors ``relation_lm.inference.stateful_decode.StatefulDecoder.step`` operator for operator,
with the CPU oracle (``relation_oracle.c``) in place of every CUDA kernel and fp32 torch CPU
matmuls in place of the GPU GEMMs.  Values that the GPU path stores in a lower-precision
tensor (weights, caches, GEMM outputs) are rounded to that dtype here too, so the two paths
see the same operands up to GEMM accumulation order.  State lives in fp32 tensors.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

import oracle


class OracleDecoder:
    def __init__(self, model, batch: int, dtype: torch.dtype = torch.float32) -> None:
        cfg = model.config
        self.config, self.batch, self.dtype = cfg, int(batch), dtype
        self.w = {k: v.float() for k, v in model.decode_weights("cpu", dtype).items()}
        self.input_scale = float(model.input_scale)
        L, B, T, R, H = cfg.layers, self.batch, cfg.max_context, cfg.relation_dim, cfg.hidden_dim
        nb = T // cfg.block_size
        z = lambda *s: torch.zeros(*s)  # noqa: E731
        self.anchor_keys, self.partner_keys = z(L, B, T, 64), z(L, B, T, 64)
        self.operand_cache, self.partner_anchor_cache = z(L, B, T, R), z(L, B, T, 128)
        self.expanded_cache = z(L, B, T, 2 * H)
        self.router_caches = [z(L, B, T, 64) for _ in range(4)]
        self.router_stats = [z(L, B, nb, 4, 16) for _ in range(4)]
        self.position = 0
        self.last_selection = []
        self.scored = [0, 0]

    def _round(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.dtype == torch.float32 else x.to(self.dtype).float()

    def slide(self, blocks: int = 1) -> None:
        """``StatefulDecoder.slide``: the oldest ``blocks`` router blocks leave, every later row (and
        block statistic) moves to the front, the last rows keep their content, the position drops."""
        rows = blocks * self.config.block_size
        for c in (self.anchor_keys, self.partner_keys, self.operand_cache, self.partner_anchor_cache,
                  self.expanded_cache, *self.router_caches):
            c[:, :, :c.size(2) - rows] = c[:, :, rows:].clone()
        for s in self.router_stats:
            s[:, :, :s.size(2) - blocks] = s[:, :, blocks:].clone()
        self.position -= rows

    def step(self, tokens: torch.Tensor, boundaries: torch.Tensor):
        cfg, w, t = self.config, self.w, self.position
        R = cfg.relation_dim
        x = (self._round(w["token_embedding"][tokens] + w["boundary_embedding"][boundaries])) \
            * self.input_scale + w["position_embedding"][t]
        memory = self._round(F.layer_norm(x, (cfg.d_model,), w["memory_norm_w"], w["memory_norm_b"], cfg.norm_eps))
        hidden = x
        packed = self._round(memory @ w["w_packed"].T)
        width = 384 + R
        self.last_selection = []
        for l in range(cfg.layers):
            p = packed[:, l * width:(l + 1) * width]
            self.anchor_keys[l, :, t] = p[:, 0:64]
            self.partner_keys[l, :, t] = p[:, 64:128]
            self.operand_cache[l, :, t] = p[:, 128:128 + R]
            self.partner_anchor_cache[l, :, t] = p[:, 128 + R:256 + R]
            oracle.router_cache_update(
                p[:, 256 + R:320 + R], p[:, 320 + R:384 + R], *[c[l] for c in self.router_caches],
                *[s[l] for s in self.router_stats], w["anchor_conv_weight"][l],
                w["partner_conv_weight"][l], t, cfg.block_size, inplace=True,
                cache_dtype=self.dtype, stats_dtype=self.dtype)
        for l in range(cfg.layers):
            normalized = self._round(F.layer_norm(hidden, (cfg.d_model,), w["input_norm_w"][l],
                                                  w["input_norm_b"][l], cfg.norm_eps))
            q = self._round(normalized @ w["w_query"][l].T)
            anchor, _, partner, partner_score, scored = oracle.relation_select(
                q[:, 0:64], self.anchor_keys[l], q[:, 64:128], self.router_stats[0][l],
                self.router_stats[1][l], w["anchor_gamma"][l], w["anchor_bias"][l], q[:, 128:256],
                self.partner_anchor_cache[l], self.partner_keys[l], self.router_stats[2][l],
                self.router_stats[3][l], w["partner_gamma"][l], w["partner_bias"][l], t,
                cfg.local_window, cfg.top_blocks, cfg.k_max, cfg.strict_valid)
            self.scored[0] += scored[0]
            self.scored[1] += scored[1]
            relation_hidden, _ = oracle.relation_hidden(
                self.expanded_cache[l], self.operand_cache[l], anchor, partner, w["product_weight"][l],
                w["anchor_weight"][l], w["partner_weight"][l], w["first_bias"][l], position=t,
                inplace=True, cache_dtype=self.dtype)
            raw = self._round(self._round(relation_hidden) @ w["w2"][l].T + w["b2"][l])
            context = oracle.relation_norm_reduce(raw, partner_score, w["relation_norm_w"][l],
                                                  w["relation_norm_b"][l], t, cfg.norm_eps)
            hidden = hidden + w["mix"][l] * context
            self.last_selection.append((anchor, partner))
        final = self._round(F.layer_norm(hidden, (cfg.d_model,), w["final_norm_w"], w["final_norm_b"], cfg.norm_eps))
        self.last_final = final
        token_logits = final @ w["token_embedding"].T
        boundary_logits = final @ w["boundary_w"].T + w["boundary_b"]
        self.position += 1
        return token_logits, boundary_logits
