"""Whole-sequence (prefill) relation layer at the long-context configuration itself: batch 8,
context 4096, d_model 512, block 64, window 128, 4 remote blocks, K = 8, bf16, hidden states
N(0, 1) with 5 % of the positions scaled by 4 (seeded).

All 32 768 query rows run on the GPU; a seeded sample of rows (every early and block-edge position
of two sequences plus 2 000 random rows) is checked against the CPU oracle, each kernel on the
GPU path's own inputs:

* the state built in bulk (router caches, block statistics) equals ``T`` successive oracle updates,
  bit for bit, for every sequence; the token caches equal the packed projection's slices;
* selected anchor / partner indices and scores of the sampled rows: bit-exact;
* relation hidden states, second-layer output: within 1e-2 of the row's largest magnitude;
  reduced context (fp32 arithmetic on identical inputs): 1e-4;
* size-independent properties over ALL rows: causality, anchor never among the partners, partners
  distinct, scores sorted, empty slots carry the sentinel index.
"""
from __future__ import annotations

import pytest
import torch

import oracle
from gpu_util import assert_rel_close, assert_scores_equal, assert_status_clear

pytestmark = pytest.mark.gpu

ROUTER_STATE = ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache",
                "anchor_mean", "anchor_std", "partner_mean", "partner_std")


def long_context_inputs(batch=8, length=4096, d_model=512, seed=1003):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(batch, length, d_model, generator=g)
    strong = torch.rand(batch, length, generator=g) < 0.05
    return torch.where(strong[..., None], x * 4.0, x)


def _layer(T=4096, **kw):
    from relation_lm.inference.prefill import RoutedPrefillLayer
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM

    cfg = RoutedRelationConfig(vocab_size=64, boundary_vocab_size=8, d_model=512, layers=1, max_context=T,
                               block_size=64, local_window=128, top_blocks=4, k_max=8, **kw)
    return RoutedPrefillLayer(RoutedRelationLM(cfg, seed=1003), 0, "cuda", torch.bfloat16)


def test_long_context_prefill_layer_matches_oracle_on_sampled_rows():
    layer = _layer()
    cfg, w = layer.config, layer.w
    B, T, d, K, R = 8, cfg.max_context, cfg.d_model, cfg.k_max, cfg.relation_dim
    x = long_context_inputs(B, T, d).cuda()
    state = layer.build_state(x)
    keep: dict = {}
    out = layer.forward(x, state, keep)
    torch.cuda.synchronize()
    assert_status_clear()
    wc = {k: v.float().cpu() for k, v in w.items()}
    packed = state["packed"].float().cpu()

    # ---- state: token caches are slices of the packed projection; router state == T oracle updates
    for name, lo, hi in (("anchor_keys", 0, 64), ("partner_keys", 64, 128), ("operand_cache", 128, 128 + R),
                         ("partner_anchor_cache", 128 + R, 256 + R)):
        assert torch.equal(state[name].float().cpu(), packed[..., lo:hi]), name
    host = [torch.zeros(B, T, 64) for _ in range(4)] + [torch.zeros(B, T // cfg.block_size, 4, 16) for _ in range(4)]
    for t in range(T):
        oracle.router_cache_update(packed[:, t, 256 + R:320 + R], packed[:, t, 320 + R:384 + R], *host,
                                   wc["anchor_conv_weight"], wc["partner_conv_weight"], t, cfg.block_size,
                                   inplace=True, cache_dtype=torch.bfloat16, stats_dtype=torch.bfloat16)
    for name, want in zip(ROUTER_STATE, host):
        assert torch.equal(state[name].float().cpu(), want), name
    o = state["operand_cache"].float().cpu()
    want_expanded = o @ wc["w_expand"].T + wc["b_expand"]
    assert_rel_close(state["expanded_cache"], want_expanded, 1e-2, "expanded cache")

    # ---- properties over all rows
    rb, rp = keep["row_batch"].cpu().long(), keep["row_position"].cpu().long()
    anchor, partner, score = keep["anchor"].cpu().long(), keep["partner"].cpu().long(), keep["partner_score"].cpu()
    valid = score > -torch.inf
    assert bool((anchor <= rp).all()) and bool((anchor >= 0).all())
    assert bool((partner[valid] <= rp[:, None].expand_as(partner)[valid]).all())
    assert not bool((partner == anchor[:, None])[valid].any())
    assert bool((score[:, :-1] >= score[:, 1:]).all())
    sentinel = (rp - cfg.local_window + 1)[:, None].expand_as(partner)
    assert torch.equal(partner[~valid], sentinel[~valid])
    sorted_partners = torch.where(valid, partner, torch.arange(-K, 0)[None, :] - 10).sort(-1).values
    assert bool((sorted_partners[:, 1:] != sorted_partners[:, :-1]).all())
    # every row with at least K + 1 causal candidates has K partners
    assert bool(valid[rp >= K].all())

    # ---- sampled rows against the oracle
    g = torch.Generator().manual_seed(77)
    edges = torch.tensor([0, 1, 2, 7, 8, 9, 62, 63, 64, 65, 126, 127, 128, 129, 191, 192, 255, 256, 383, 384,
                          2047, 2048, 4094, 4095])
    rows = torch.cat([edges, T + edges, torch.randint(0, B * T, (2000,), generator=g)]).unique()
    q = keep["query"].cpu()[rows]
    caches = {n: state[n].cpu() for n in ("anchor_keys", "partner_keys", "partner_anchor_cache",
                                           "anchor_mean", "anchor_std", "partner_mean", "partner_std")}
    row_batch, row_pos = rb[rows].int(), rp[rows].int()
    wa, _, wp, ws, _ = oracle.relation_select(
        q[:, 0:64], caches["anchor_keys"], q[:, 64:128], caches["anchor_mean"], caches["anchor_std"],
        wc["anchor_gamma"], wc["anchor_bias"], q[:, 128:256], caches["partner_anchor_cache"], caches["partner_keys"],
        caches["partner_mean"], caches["partner_std"], wc["partner_gamma"], wc["partner_bias"], 0,
        cfg.local_window, cfg.top_blocks, K, cfg.strict_valid, row_batch=row_batch, row_pos=row_pos)
    assert torch.equal(keep["anchor"].cpu()[rows], wa)
    assert torch.equal(keep["partner"].cpu()[rows], wp)
    assert_scores_equal(keep["partner_score"][rows.cuda()], ws)
    # relation hidden on the gathered rows (compacted caches: row 0 the anchor, rows 1..K the partners)
    idx = torch.cat((wa[:, None], wp), 1).long().clamp(0, T - 1)
    seq = row_batch.long()[:, None]
    small_expanded = state["expanded_cache"].cpu()[seq, idx]
    small_operand = state["operand_cache"].cpu()[seq, idx]
    n = rows.numel()
    want_hidden, _ = oracle.relation_hidden(small_expanded, small_operand, torch.zeros(n, dtype=torch.int32),
                                            torch.arange(1, K + 1, dtype=torch.int32).repeat(n, 1),
                                            wc["product_weight"])
    ok = ws > -torch.inf
    got_hidden = keep["hidden"][rows.cuda()].cpu()
    assert_rel_close(got_hidden[ok], want_hidden[ok], 1e-2, "relation hidden")
    got_raw = keep["raw"][rows.cuda()].cpu()
    assert_rel_close(got_raw[ok], (oracle.linear(got_hidden, wc["w2"]) + wc["b2"])[ok], 1e-2, "second layer")
    want_ctx = oracle.relation_norm_reduce(got_raw, ws, wc["relation_norm_w"], wc["relation_norm_b"], 0,
                                           cfg.norm_eps, row_pos=row_pos)
    assert_rel_close(keep["context"][rows.cuda()], want_ctx, 1e-4, "context")
    want_out = x.view(B * T, d)[rows.cuda()].cpu() + wc["mix"] * want_ctx
    assert_rel_close(out.view(B * T, d)[rows.cuda()], want_out, 1e-4, "layer output")
