"""Stateful sparse decode: one new position per call, all history in caches.

The step is the composition the reference's decode operators were written for (its own
driver is not public; the order follows docs/architecture.md:26-40 and
docs/benchmarks.md:87-113 of the reference project):

1. embed the new token, ``memory = LayerNorm(x)``; one packed projection of ``memory`` for
   every layer (packed_cache.py:52-57) followed by ``sparse_cache_append`` (token-cache rows
   + ``router_cache_update`` of all layers, one launch);
2. per layer: ``LayerNorm(hidden)`` -> one 256-wide query-side projection ->
   ``relation_select_packed`` -> ``relation_hidden_cache_update`` -> second relation-MLP layer
   -> ``relation_norm_reduce`` -> ``hidden += sigmoid(mix) * context``;
3. final LayerNorm, tied token head, boundary head.

Every state tensor is allocated once and mutated in place; ``position`` lives on the device
and is advanced there, so a captured CUDA graph of ``step`` replays for successive positions.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from relation_lm.inference.routed_model import RoutedRelationLM
from relation_lm.kernels import _abi
from relation_lm.kernels.packed_projection import (decode_embed_norm, decode_front, decode_front_supported,
                                                    greedy_token, l2_prefetch, layer_norm_cast,
                                                    mapped_host_view, packed_projection, packed_projection_slices,
                                                    skinny_argmax_scratch_bytes, skinny_projection,
                                                    skinny_projection_greedy, skinny_projection_greedy_into,
                                                    skinny_projection_supported)
from relation_lm.kernels.relation_reduce import (expanded_cache_append, expanded_cache_append_packed,
                                                 relation_hidden_cache_update,
                                                 relation_layer_tail, relation_layer_tail_supported,
                                                 relation_hidden_cached_out,
                                                 relation_hidden_cache_update_out,
                                                 relation_norm_reduce_residual_norm,
                                                 relation_norm_reduce_residual_norm_project,
                                                 relation_norm_reduce_residual_norm_slices,
                                                 relation_norm_reduce,
                                                 relation_norm_reduce_residual, relation_tail)
from relation_lm.kernels.relation_select import relation_select_packed
from relation_lm.kernels.relation_layer import relation_layer, relation_layer_supported
from relation_lm.kernels.router_cache import packed_projection_append, sparse_cache_append, state_slide


class StatefulDecoder:
    def __init__(self, model: RoutedRelationLM, batch: int, device="cuda",
                 dtype: torch.dtype = torch.bfloat16, fused_tail: bool = False,
                 programmatic_launch: bool = True, second_layer_split: bool = False,
                 fused_query: bool | None = None, layer_tail: bool | None = None,
                 skinny: bool | None = None, append_in_projection: bool | None = None,
                 whole_layer: bool | None = None, fused_front: bool | None = None,
                 prefetch: bool | None = None) -> None:
        cfg = model.config
        self.programmatic_launch = bool(programmatic_launch)
        self.config, self.batch, self.device, self.dtype = cfg, int(batch), torch.device(device), dtype
        self.w = model.decode_weights(self.device, dtype)
        self.input_scale = float(model.input_scale)
        L, B, T, R, H = cfg.layers, self.batch, cfg.max_context, cfg.relation_dim, cfg.hidden_dim
        nb = T // cfg.block_size

        def zeros(*shape, dt=dtype):
            return torch.zeros(*shape, device=self.device, dtype=dt)

        self.anchor_keys = zeros(L, B, T, 64)
        self.partner_keys = zeros(L, B, T, 64)
        self.operand_cache = zeros(L, B, T, R)
        self.partner_anchor_cache = zeros(L, B, T, 128)
        self.expanded_cache = zeros(L, B, T, 2 * H)
        self.router_caches = [zeros(L, B, T, 64) for _ in range(4)]   # raw a, raw p, conv a, conv p
        self.router_stats = [zeros(L, B, nb, 4, 16) for _ in range(4)]  # mean a, std a, mean p, std p
        self.position = torch.zeros((), device=self.device, dtype=torch.int64)
        self.last_selection: list[tuple[Tensor, Tensor]] = []
        # When set to a list, the fused step appends one dict of cloned intermediates per layer
        # (and one for the embedding / append stage), so that a checker can feed every kernel's own
        # inputs to an independent implementation.  Not for captured graphs.
        self.trace: list[dict[str, Tensor]] | None = None
        self.last_final: Tensor | None = None           # final LayerNorm output of the last step
        self._graph = None
        # Low-precision decode batches take the fused path: LayerNorm folded into the tcgen05
        # projections, 16-bit relation hidden states, residual update inside norm-reduce.
        self.fused = (dtype in (torch.bfloat16, torch.float16)
                      and cfg.d_model % 64 == 0 and cfg.d_model <= 1024)
        # The single-launch tail (second MLP layer + norm-reduce + residual) is optional: at
        # decode batch sizes its one-CTA finalisation costs more than the launch it saves.
        self.fused_tail = fused_tail and self.fused and 128 % cfg.k_max == 0 and cfg.k_max <= 32
        # One tensor-core launch expands the position's operand rows of all layers (shapes permitting).
        self.stacked_expand = self.fused and R % 64 == 0 and H % 128 == 0
        # Second relation-MLP layer: cuBLAS (F.linear) by default.  Optionally, with at most one row
        # tile (B * K <= 128), the library's GEMM splits the reduction over the hidden width across
        # several CTAs and norm-reduce sums the slices: no library call in the step, a few percent slower.
        self.second_layer_splits = 1
        if self.fused and second_layer_split and B * cfg.k_max <= 128 and H % 64 == 0 and cfg.d_model % 32 == 0:
            blocks = H // 64
            self.second_layer_splits = next((s for s in (4, 2) if blocks % s == 0 and blocks // s >= 2), 1)
        if self.second_layer_splits > 1:
            self.b2_f32 = self.w["b2"].float().contiguous()                    # [L, d], dtype of the norm parameters
        # Next layer's query projection inside norm-reduce (a cluster of CTAs per row): one launch
        # fewer per layer for batches of a few rows; larger batches keep the tensor-core projection.
        n_query = self.w["w_query"].shape[1]
        can_fuse_query = (self.fused and not self.fused_tail and self.second_layer_splits == 1
                          and n_query % 32 == 0 and n_query <= 256)
        self.fused_query = can_fuse_query and (B <= 32 if fused_query is None else bool(fused_query))
        # The whole relation tail of a layer (relation hidden, second MLP layer, norm-reduce, residual,
        # next LayerNorm, next query projection) as ONE cluster launch with the hidden states on chip:
        # two launches per layer and no library GEMM in the step, for small batches of d <= 512.
        can_tail = (self.fused and not self.fused_tail and self.second_layer_splits == 1 and self.stacked_expand
                    and B <= 64 and relation_layer_tail_supported(B, cfg.k_max, R, H, cfg.d_model, n_query, dtype))
        self.layer_tail = can_tail if layer_tail is None else (bool(layer_tail) and can_tail)
        if self.layer_tail:
            self.fused_query = False
        if self.fused_query or self.layer_tail:
            self.query = zeros(B, n_query)
        # ... and the selector can run in front of the tail inside the same cluster: one launch per layer.
        # Off by default: with the step's working set cold in L2 it measured 3-5 % slower than the two
        # launches (equal when warm), whose selector overlaps the tail's weight loads just as well.
        can_whole = self.layer_tail and relation_layer_supported(
            B, cfg.k_max, R, H, cfg.d_model, n_query, dtype, T, nb, self.w["anchor_bias"].shape[-1],
            cfg.local_window, cfg.top_blocks)
        self.whole_layer = bool(whole_layer) and can_whole
        # Projections of a handful of rows stream their weights through the CUDA cores (no tensor-memory
        # set-up); the head's launch then also takes the greedy arg-max and the position increment.
        can_skinny = self.fused and skinny_projection_supported(B, cfg.d_model, dtype)
        self.skinny = can_skinny if skinny is None else (bool(skinny) and can_skinny)
        # ... and the packed projection can take the cache append and router update into its epilogue
        # (one launch fewer; off by default: the channels' serial statistics in the epilogue cost more
        # than the separate, fully parallel append launch that overlaps its neighbours)
        self.append_in_projection = bool(append_in_projection) and self.skinny
        # ... and the step's front (embedding, two LayerNorms, packed projection, layer 0's query projection)
        # is one launch of the same kind over the two weight matrices stacked: three launches fewer
        can_front = (self.skinny and not self.append_in_projection and (self.fused_query or self.layer_tail)
                     and decode_front_supported(B, cfg.d_model, self.w["w_packed"].shape[0], dtype))
        self.fused_front = can_front if fused_front is None else (bool(fused_front) and can_front)
        if self.fused_front:
            self.front_weight = torch.cat((self.w["w_packed"], self.w["w_query"][0]), 0).contiguous()
        # A step of a small batch is a chain of dependent launches on a fraction of the SMs; when it
        # starts with a cold L2 every one of them first waits for its weights and caches to come from
        # DRAM.  One launch on a side stream at the head of the step can ask for all of them at once.
        # Off by default: measured 3-5 us SLOWER per step (cold and warm) than letting every kernel
        # fetch its own data under programmatic launch; the fork and join cost more than they hide.
        self.prefetch = bool(prefetch) and self.fused
        self._side_stream = torch.cuda.Stream(self.device) if self.prefetch else None
        self._project = skinny_projection if self.skinny else packed_projection
        if self.skinny:
            self.argmax_scratch = torch.zeros(skinny_argmax_scratch_bytes(), device=self.device, dtype=torch.uint8)
        if self.fused:
            self.relation_hidden = zeros(B, cfg.k_max, H)
            self.normalized = zeros(B, cfg.d_model)             # LayerNorm'd input of the next projection
            self.memory_normalized = zeros(B, cfg.d_model)      # memory-norm'd input of the packed projection
            self.head_weight = torch.cat((self.w["token_embedding"], self.w["boundary_w"]), 0).contiguous()
            pad = (-self.head_weight.size(0)) % 128        # whole 128-column tiles for the projection kernel
            if pad:
                self.head_weight = torch.cat((self.head_weight, zeros(pad, cfg.d_model)), 0).contiguous()
            # the boundary head's bias rides in the projection's epilogue (token columns: zero)
            self.head_bias = torch.zeros(self.head_weight.size(0), device=self.device, dtype=torch.float32)
            self.head_bias[cfg.vocab_size:cfg.vocab_size + cfg.boundary_vocab_size] = self.w["boundary_b"].float()

    # ------------------------------------------------------------------ state
    def reset(self) -> None:
        for t in (self.anchor_keys, self.partner_keys, self.operand_cache, self.partner_anchor_cache,
                  self.expanded_cache, *self.router_caches, *self.router_stats):
            t.zero_()
        self.position.zero_()

    def slide(self, blocks: int = 1) -> None:
        """Drop the oldest ``blocks`` router blocks of every sequence and lower the position by as
        many rows (``relation_lm.kernels.router_cache.state_slide``): how a decoder goes on once its
        position has reached ``max_context``.  Afterwards position ``p`` of the state is what position
        ``p + blocks * block_size`` was — keys, operands, expanded rows, router caches and the
        statistics of every block, none of them recomputed — so later steps choose among the rows a
        ring buffer of ``max_context`` rows would still hold, and count positions (the position
        embedding, the ``ceil(log2(t + 2))`` partner limit) from the oldest row kept.  One launch for
        the caches and statistics and one for the position, on the current stream, between steps
        (outside the captured graph, whose buffers it leaves where they are)."""
        cfg = self.config
        blocks = int(blocks)
        if not 0 < blocks < cfg.max_context // cfg.block_size:
            raise ValueError("slide by at least one block and fewer than the context holds")
        rows = blocks * cfg.block_size
        caches = [self.anchor_keys, self.partner_keys, self.operand_cache, self.partner_anchor_cache,
                  self.expanded_cache, *self.router_caches]
        state_slide(caches + list(self.router_stats), [rows] * len(caches) + [blocks] * 4,
                    row_dim=[-2] * len(caches) + [-3] * 4)
        self.position.sub_(rows)

    def state_bytes(self) -> int:
        tensors = (self.anchor_keys, self.partner_keys, self.operand_cache, self.partner_anchor_cache,
                   self.expanded_cache, *self.router_caches, *self.router_stats)
        return sum(t.numel() * t.element_size() for t in tensors)

    # ------------------------------------------------------------------ one position
    def step(self, tokens: Tensor, boundaries: Tensor, keep_selection: bool = False):
        """Consume one token per sequence at the current position; returns (token logits
        ``[B, V]``, boundary logits ``[B, Vb]``) and advances the position."""
        if self.fused:
            # The fused step keeps the selector's rule for programmatic launch: the caches are
            # written by the append, two launches before the first selector.
            previous = _abi.set_programmatic_launch(self.programmatic_launch)
            try:
                return self._step_fused(tokens, boundaries, keep_selection)
            finally:
                _abi.set_programmatic_launch(previous)
        return self._step_unfused(tokens, boundaries, keep_selection)

    def step_greedy(self, tokens: Tensor, boundaries: Tensor, chosen_out: Tensor | None = None) -> Tensor:
        """One step followed by the greedy choice: returns the next token ids ``[B]`` (int64) and
        advances the position.  On the fused path the arg-max and the position increment are one
        launch of the library; with ``chosen_out`` (int64 ``[B]``, skinny fused path only) the choice is
        written there — a device view of pinned host memory included."""
        if chosen_out is not None and not (self.fused and self.skinny):
            raise ValueError("chosen_out needs the fused path with the head projection's greedy launch")
        if not self.fused:
            token_logits, _ = self.step(tokens, boundaries)
            return token_logits.argmax(-1)
        previous = _abi.set_programmatic_launch(self.programmatic_launch)
        try:
            if self.skinny:
                return self._step_fused(tokens, boundaries, False, advance=False, greedy=True, chosen_out=chosen_out)
            self._step_fused(tokens, boundaries, False, advance=False)
            return greedy_token(self.last_logits, self.config.vocab_size, self.position)
        finally:
            _abi.set_programmatic_launch(previous)

    def _step_unfused(self, tokens: Tensor, boundaries: Tensor, keep_selection: bool):
        cfg, w = self.config, self.w
        pos = self.position
        x = (F.embedding(tokens, w["token_embedding"]) + F.embedding(boundaries, w["boundary_embedding"])).float()
        x = x * self.input_scale + w["position_embedding"].index_select(0, pos.view(1))
        memory = F.layer_norm(x, (cfg.d_model,), w["memory_norm_w"], w["memory_norm_b"], cfg.norm_eps).to(self.dtype)
        hidden = x
        packed = F.linear(memory, w["w_packed"])                      # [B, layers * 512]
        sparse_cache_append(packed, self.anchor_keys, self.partner_keys, self.operand_cache,
                            self.partner_anchor_cache, *self.router_caches, *self.router_stats,
                            w["anchor_conv_weight"], w["partner_conv_weight"], pos, cfg.block_size)
        if keep_selection:
            self.last_selection = []
        B, K = self.batch, cfg.k_max
        for l in range(cfg.layers):
            normalized = F.layer_norm(hidden, (cfg.d_model,), w["input_norm_w"][l], w["input_norm_b"][l],
                                      cfg.norm_eps).to(self.dtype)
            q = F.linear(normalized, w["w_query"][l])                 # [B, 256]
            anchor, _, partner, partner_score = relation_select_packed(
                q[:, 0:64], self.anchor_keys[l], q[:, 64:128], self.router_stats[0][l],
                self.router_stats[1][l], w["anchor_gamma"][l], w["anchor_bias"][l], q[:, 128:256],
                self.partner_anchor_cache[l], self.partner_keys[l], self.router_stats[2][l],
                self.router_stats[3][l], w["partner_gamma"][l], w["partner_bias"][l], pos,
                cfg.local_window, cfg.top_blocks, K, cfg.strict_valid)
            relation_hidden = relation_hidden_cache_update(
                self.expanded_cache[l], self.operand_cache[l], anchor, partner, w["anchor_weight"][l],
                w["partner_weight"][l], w["product_weight"][l], w["first_bias"][l], pos)
            raw = F.linear(relation_hidden.to(self.dtype), w["w2"][l], w["b2"][l])      # [B, K, d]
            context = relation_norm_reduce(raw, partner_score, w["relation_norm_w"][l],
                                           w["relation_norm_b"][l], pos, cfg.norm_eps)
            hidden = torch.addcmul(hidden, context, w["mix"][l])
            if keep_selection:
                self.last_selection.append((anchor, partner))
        final = F.layer_norm(hidden, (cfg.d_model,), w["final_norm_w"], w["final_norm_b"], cfg.norm_eps).to(self.dtype)
        self.last_final = final
        token_logits = F.linear(final, w["token_embedding"])
        boundary_logits = F.linear(final, w["boundary_w"], w["boundary_b"])
        pos.add_(1)
        return token_logits, boundary_logits

    def _step_fused(self, tokens: Tensor, boundaries: Tensor, keep_selection: bool, advance: bool = True,
                    greedy: bool = False, chosen_out: Tensor | None = None):
        """The same step with the elementwise glue folded into the library's kernels:
        1 launch per layer where the selector fits in front of the single-launch relation tail, 2
        (select, tail) where only the tail applies, otherwise up to 5
        (query projection, select, relation hidden, second MLP layer GEMM, norm-reduce + residual +
        next LayerNorm).  Every LayerNorm is
        computed by the kernel that produces its input (the embedding, the residual update) and
        handed on as a 16-bit matrix, so the projections are plain tensor-core GEMMs."""
        cfg, w = self.config, self.w
        pos = self.position
        tokens, boundaries = tokens.contiguous(), boundaries.contiguous()
        if self.prefetch:
            main = torch.cuda.current_stream(self.device)
            self._side_stream.wait_stream(main)
            with torch.cuda.stream(self._side_stream):
                # in the order the step reads them
                l2_prefetch([w["anchor_weight"], w["partner_weight"], self.anchor_keys, self.partner_keys,
                             *self.router_stats, self.partner_anchor_cache, w["product_weight"], w["w2"],
                             self.operand_cache, w["w_query"], self.head_weight])
        if self.fused_front:
            hidden, packed = decode_front(tokens, boundaries, w["token_embedding"], w["boundary_embedding"],
                                          w["position_embedding"], pos, self.input_scale, w["memory_norm_w"],
                                          w["memory_norm_b"], w["input_norm_w"][0], w["input_norm_b"][0], cfg.norm_eps,
                                          self.front_weight, w["w_packed"].shape[0], self.memory_normalized,
                                          self.normalized, self.query)
        else:
            hidden = decode_embed_norm(tokens, boundaries, w["token_embedding"], w["boundary_embedding"],
                                       w["position_embedding"], pos, self.input_scale,
                                       w["memory_norm_w"], w["memory_norm_b"], self.memory_normalized,
                                       w["input_norm_w"][0], w["input_norm_b"][0], self.normalized, cfg.norm_eps)
        if self.fused_front:
            sparse_cache_append(packed, self.anchor_keys, self.partner_keys, self.operand_cache,
                                self.partner_anchor_cache, *self.router_caches, *self.router_stats,
                                w["anchor_conv_weight"], w["partner_conv_weight"], pos, cfg.block_size)
        elif self.append_in_projection:
            # the packed projection's epilogue writes the token caches and updates the router state
            packed = packed_projection_append(self.memory_normalized, w["w_packed"], self.anchor_keys,
                                              self.partner_keys, self.operand_cache, self.partner_anchor_cache,
                                              *self.router_caches, *self.router_stats, w["anchor_conv_weight"],
                                              w["partner_conv_weight"], pos, cfg.block_size)
        else:
            packed = self._project(self.memory_normalized, w["w_packed"])
            sparse_cache_append(packed, self.anchor_keys, self.partner_keys, self.operand_cache,
                                self.partner_anchor_cache, *self.router_caches, *self.router_stats,
                                w["anchor_conv_weight"], w["partner_conv_weight"], pos, cfg.block_size)
        if self.stacked_expand and self.fused_front:
            # every layer's operand row of this position is known: expand them all at once, straight from
            # the packed rows (written two launches back), so that this launch overlaps the append
            expanded_cache_append_packed(self.expanded_cache, packed, w["anchor_weight"], w["partner_weight"],
                                         w["first_bias"], pos)
        elif self.stacked_expand:
            expanded_cache_append(self.expanded_cache, self.operand_cache, w["anchor_weight"],
                                  w["partner_weight"], w["first_bias"], pos)
        if keep_selection:
            self.last_selection = []
        trace = self.trace
        if trace is not None:
            trace.append({"stage": "append", "embedded": hidden.clone(), "packed": packed.clone(),
                          "memory_normalized": self.memory_normalized.clone(),
                          "normalized": self.normalized.clone()})
        K = cfg.k_max
        for l in range(cfg.layers):
            # layer 0 projects the embedding's normalised rows; later layers find their queries
            # written by the previous layer's norm-reduce when that fusion is on
            q = self.query if ((self.fused_query or self.layer_tail) and (l > 0 or self.fused_front)) \
                else self._project(self.normalized, w["w_query"][l])
            last = l + 1 == cfg.layers
            next_w = w["final_norm_w"] if last else w["input_norm_w"][l + 1]
            next_b = w["final_norm_b"] if last else w["input_norm_b"][l + 1]
            if self.whole_layer:
                if trace is not None:
                    entry = {"stage": "layer", "layer": l, "query": q.clone(), "hidden_before": hidden.clone()}
                    trace.append(entry)
                anchor, _, partner, partner_score = relation_layer(
                    q[:, 0:64], self.anchor_keys[l], q[:, 64:128], self.router_stats[0][l],
                    self.router_stats[1][l], w["anchor_gamma"][l], w["anchor_bias"][l], q[:, 128:256],
                    self.partner_anchor_cache[l], self.partner_keys[l], self.router_stats[2][l],
                    self.router_stats[3][l], w["partner_gamma"][l], w["partner_bias"][l], pos,
                    cfg.local_window, cfg.top_blocks, K, cfg.strict_valid,
                    self.expanded_cache[l], self.operand_cache[l], w["product_weight"][l], w["w2"][l], w["b2"][l],
                    w["relation_norm_w"][l], w["relation_norm_b"][l], cfg.norm_eps, hidden, w["mix"][l], next_w,
                    next_b, cfg.norm_eps, self.normalized, None if last else w["w_query"][l + 1],
                    None if last else self.query)
                if trace is not None:
                    entry.update(anchor=anchor.clone(), partner=partner.clone(), partner_score=partner_score.clone(),
                                 hidden_after=hidden.clone(), next_normalized=self.normalized.clone())
                    if not last:
                        entry["next_query"] = self.query.clone()
                if keep_selection:
                    self.last_selection.append((anchor, partner))
                continue
            anchor, _, partner, partner_score = relation_select_packed(
                q[:, 0:64], self.anchor_keys[l], q[:, 64:128], self.router_stats[0][l],
                self.router_stats[1][l], w["anchor_gamma"][l], w["anchor_bias"][l], q[:, 128:256],
                self.partner_anchor_cache[l], self.partner_keys[l], self.router_stats[2][l],
                self.router_stats[3][l], w["partner_gamma"][l], w["partner_bias"][l], pos,
                cfg.local_window, cfg.top_blocks, K, cfg.strict_valid)
            if trace is not None:
                entry = {"stage": "layer", "layer": l, "query": q.clone(), "anchor": anchor.clone(),
                         "partner": partner.clone(), "partner_score": partner_score.clone(),
                         "hidden_before": hidden.clone()}
                trace.append(entry)
            if self.layer_tail:
                relation_layer_tail(self.expanded_cache[l], self.operand_cache[l], anchor, partner, partner_score,
                                    w["product_weight"][l], w["w2"][l], w["b2"][l], w["relation_norm_w"][l],
                                    w["relation_norm_b"][l], pos, cfg.norm_eps, hidden, w["mix"][l], next_w, next_b,
                                    cfg.norm_eps, self.normalized, None if last else w["w_query"][l + 1],
                                    None if last else self.query)
                if trace is not None:
                    entry.update(hidden_after=hidden.clone(), next_normalized=self.normalized.clone())
                    if not last:
                        entry["next_query"] = self.query.clone()
                if keep_selection:
                    self.last_selection.append((anchor, partner))
                continue
            if self.stacked_expand:
                relation_hidden_cached_out(self.relation_hidden, self.expanded_cache[l], self.operand_cache[l],
                                           anchor, partner, w["product_weight"][l])
            else:
                relation_hidden_cache_update_out(
                    self.relation_hidden, self.expanded_cache[l], self.operand_cache[l], anchor, partner,
                    w["anchor_weight"][l], w["partner_weight"][l], w["product_weight"][l],
                    w["first_bias"][l], pos)
            if self.fused_tail:
                relation_tail(self.relation_hidden, w["w2"][l], w["b2"][l], partner_score,
                              w["relation_norm_w"][l], w["relation_norm_b"][l], pos, cfg.norm_eps,
                              hidden, w["mix"][l])
                layer_norm_cast(hidden, next_w, next_b, cfg.norm_eps, self.normalized)
            elif self.second_layer_splits > 1:
                # few rows, long reduction: split-K tensor-core GEMM, its fp32 slices summed by norm-reduce
                slices = packed_projection_slices(self.relation_hidden.view(-1, self.relation_hidden.size(-1)),
                                                  w["w2"][l], self.second_layer_splits)
                relation_norm_reduce_residual_norm_slices(
                    slices.view(self.second_layer_splits, -1, K, cfg.d_model), self.b2_f32[l], partner_score,
                    w["relation_norm_w"][l], w["relation_norm_b"][l], pos, cfg.norm_eps, hidden, w["mix"][l],
                    next_w, next_b, cfg.norm_eps, self.normalized)
            else:
                raw = F.linear(self.relation_hidden, w["w2"][l], w["b2"][l])            # [B, K, d]
                if trace is not None:
                    entry["raw"] = raw.clone()
                if self.fused_query and not last:
                    relation_norm_reduce_residual_norm_project(
                        raw, partner_score, w["relation_norm_w"][l], w["relation_norm_b"][l], pos, cfg.norm_eps,
                        hidden, w["mix"][l], next_w, next_b, cfg.norm_eps, self.normalized,
                        w["w_query"][l + 1], self.query)
                else:
                    relation_norm_reduce_residual_norm(raw, partner_score, w["relation_norm_w"][l],
                                                       w["relation_norm_b"][l], pos, cfg.norm_eps, hidden,
                                                       w["mix"][l], next_w, next_b, cfg.norm_eps, self.normalized)
            if trace is not None:
                entry.update(relation_hidden=self.relation_hidden.clone(), hidden_after=hidden.clone(),
                             next_normalized=self.normalized.clone())
                if self.fused_query and not last:
                    entry["next_query"] = self.query.clone()
            if keep_selection:
                self.last_selection.append((anchor, partner))
        self.last_final = self.normalized
        if greedy:
            # head projection + greedy arg-max + position increment in one launch
            if chosen_out is not None:
                chosen = chosen_out
                logits = skinny_projection_greedy_into(self.normalized, self.head_weight, self.head_bias,
                                                       cfg.vocab_size, self.argmax_scratch, pos, chosen_out)
            else:
                logits, chosen = skinny_projection_greedy(self.normalized, self.head_weight, self.head_bias,
                                                          cfg.vocab_size, self.argmax_scratch, pos)
            self.last_logits = logits
            if self.prefetch:
                main.wait_stream(self._side_stream)      # join the side branch (long finished) at the step's end
            return chosen
        logits = self._project(self.normalized, self.head_weight, self.head_bias)
        if self.prefetch:
            main.wait_stream(self._side_stream)
        self.last_logits = logits                        # [B, padded vocab + boundary vocab]
        token_logits = logits[:, :cfg.vocab_size]
        boundary_logits = logits[:, cfg.vocab_size:cfg.vocab_size + cfg.boundary_vocab_size]
        if advance:
            pos.add_(1)
        return token_logits, boundary_logits

    # ------------------------------------------------------------------ CUDA graph
    def capture(self) -> None:
        """Capture one ``step`` into a CUDA graph with static input / output buffers.  State and
        position are left exactly as they were."""
        B = self.batch
        self.static_tokens = torch.zeros(B, device=self.device, dtype=torch.int64)
        self.static_boundaries = torch.zeros(B, device=self.device, dtype=torch.int64)
        saved = int(self.position.item())
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(2):                                   # warm-up outside capture
                self.step_greedy(self.static_tokens, self.static_boundaries)
                self.position.fill_(saved)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                if self.fused:
                    self.static_next = self.step_greedy(self.static_tokens, self.static_boundaries)
                    V, Vb = self.config.vocab_size, self.config.boundary_vocab_size
                    self.static_token_logits = self.last_logits[:, :V]
                    self.static_boundary_logits = self.last_logits[:, V:V + Vb]
                else:
                    self.static_token_logits, self.static_boundary_logits = self.step(
                        self.static_tokens, self.static_boundaries)
                    self.static_next = self.static_token_logits.argmax(-1)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self.position.fill_(saved)
        self._graph = graph

    def replay(self) -> None:
        self._graph.replay()

    def capture_host_io(self, mapped: bool | None = None) -> None:
        """Capture the greedy step together with its host transfers, so that a serving loop pays one
        graph launch and one stream synchronisation per position (``step_host``): it writes the token
        and boundary ids into the pinned tensors ``host_tokens`` / ``host_boundaries`` ``[B]`` (int64; the
        two rows of ``host_ids``, copied to the device by one node at the head of the graph) and finds the
        chosen tokens in the pinned ``host_next``.  ``mapped`` (default: whenever the head projection's
        greedy launch applies): the head kernel writes the choices into the pinned memory itself, through
        a device view of ``host_next``, instead of a copy node at the tail of the graph.  (Reading the ids
        through such a view was measured too: it puts a host-memory round trip at the start of the step's
        dependency chain and is 10-20 us slower than the copy.)  State and position are left exactly as
        they were."""
        B = self.batch
        self.host_ids = torch.zeros(2, B, dtype=torch.int64).pin_memory()
        self.host_tokens, self.host_boundaries = self.host_ids[0], self.host_ids[1]
        self.host_next = torch.zeros(B, dtype=torch.int64).pin_memory()
        can_map = self.fused and self.skinny
        mapped = can_map if mapped is None else (bool(mapped) and can_map)
        ids = torch.zeros(2, B, device=self.device, dtype=torch.int64)
        tokens, boundaries = ids[0], ids[1]
        chosen_view = None
        if mapped:
            try:
                chosen_view = mapped_host_view(self.host_next, self.device)
            except (RuntimeError, TypeError, ValueError):      # no device view of pinned memory here: copy node
                mapped = False
        saved = int(self.position.item())
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(2):                                   # warm-up outside capture
                self.step_greedy(tokens, boundaries, chosen_view)
                self.position.fill_(saved)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                ids.copy_(self.host_ids, non_blocking=True)
                chosen = self.step_greedy(tokens, boundaries, chosen_view)
                if not mapped:
                    self.host_next.copy_(chosen, non_blocking=True)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self.position.fill_(saved)
        self.host_io_mapped = mapped
        self._host_graph, self._host_graph_buffers = graph, (ids, chosen)

    def step_host(self) -> Tensor:
        """One position through the graph of ``capture_host_io``: reads ``host_tokens`` /
        ``host_boundaries``, returns ``host_next`` (valid on return: the stream is synchronised)."""
        self._host_graph.replay()
        torch.cuda.current_stream(self.device).synchronize()
        return self.host_next
