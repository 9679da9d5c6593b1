"""Routed multi-anchor selection on the GPU: the exclusion rules against the reference's dense
multi-anchor block (golden fixture), and the routed composition against the same composition
built from the oracle (indices bit-exact)."""
from __future__ import annotations

import pytest
import torch

import oracle
from gpu_util import assert_status_clear
from test_oracle_golden import multi_anchor_dense_check

pytestmark = pytest.mark.gpu


def test_exclusion_rules_match_the_dense_reference_block(golden):
    from relation_lm.kernels.triton_select import anchor_select_rows, partner_topk_rows

    ref = golden["multi_anchor_dense"]["outputs"]

    def anchor_rows(aq, ak, rq, mean, std, gamma, bias, rb, rp, excl, L, top, strict):
        idx, score = anchor_select_rows(aq.cuda(), ak.cuda(), rq.cuda(), mean.cuda(), std.cuda(), gamma.cuda(),
                                        bias.cuda(), rb.cuda(), rp.cuda(), excl.cuda(), L, top, strict)
        return idx.cpu(), score.cpu()

    def partner_rows(pq, pk, rq, mean, std, gamma, bias, rb, rp, anchor, excl, L, top, K, strict):
        idx, score = partner_topk_rows(pq.cuda(), pk.cuda(), rq.cuda(), mean.cuda(), std.cuda(), gamma.cuda(),
                                       bias.cuda(), rb.cuda(), rp.cuda(), anchor.cuda(), excl.cuda(), L, top, K, strict)
        return idx.cpu(), score.cpu()

    multi_anchor_dense_check(ref, anchor_rows, partner_rows)
    assert_status_clear()


@pytest.mark.parametrize("strict", [False, True])
def test_routed_multi_anchor_matches_oracle_composition(strict):
    """Multi-anchor shape scaled down: 4 slots x 4 partners, block 32, window 64, 3 remote
    blocks, bf16 caches; every position of 2 sequences of 256."""
    from relation_lm.kernels.multi_select import relation_select_multi_rows

    S, B, T, NB, L, top, K = 4, 2, 256, 8, 64, 3, 4
    g = torch.Generator().manual_seed(4404)
    N = B * T
    dt = torch.bfloat16
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    x = {"aq": rn(N, S, 64).to(dt), "ak": rn(S, B, T, 64).to(dt), "arq": rn(N, S, 64).to(dt),
         "am": rn(S, B, NB, 4, 16).to(dt), "as": rn(S, B, NB, 4, 16).abs().to(dt),
         "ag": rn(S, 4), "ab": rn(S, 4, 16), "pb": rn(N, S, 128).to(dt),
         "pac": rn(S, B, T, 128).to(dt), "pk": rn(S, B, T, 64).to(dt), "pm": rn(S, B, NB, 4, 16).to(dt),
         "ps": rn(S, B, NB, 4, 16).abs().to(dt), "pg": rn(S, 4), "pbias": rn(S, 4, 16)}
    row_batch = torch.arange(B, dtype=torch.int32).repeat_interleave(T)
    row_pos = torch.arange(T, dtype=torch.int32).repeat(B)
    d = {k: v.cuda() for k, v in x.items()}
    got = relation_select_multi_rows(d["aq"], d["ak"], d["arq"], d["am"], d["as"], d["ag"], d["ab"], d["pb"],
                                     d["pac"], d["pk"], d["pm"], d["ps"], d["pg"], d["pbias"],
                                     row_batch.cuda(), row_pos.cuda(), L, top, K, strict)
    # the same composition from oracle calls
    active = torch.arange(S)[None, :] <= row_pos[:, None]
    taken = torch.full((N, S), -1, dtype=torch.int32)
    anchors = torch.zeros(N, S, dtype=torch.int32)
    for s in range(S):
        idx, score = oracle.anchor_select(x["aq"][:, s], x["ak"][s], x["arq"][:, s], x["am"][s], x["as"][s],
                                          x["ag"][s], x["ab"][s], 0, L, top, strict, row_batch=row_batch,
                                          row_pos=row_pos, exclude_index=taken.clone())
        live = active[:, s] & torch.isfinite(score)
        anchors[:, s] = torch.where(live, idx, torch.zeros_like(idx))
        taken[:, s] = torch.where(live, idx, torch.full_like(idx, -1))
        active[:, s] = live
    assert torch.equal(got[0].cpu(), anchors)
    assert torch.equal(got[2].cpu(), active)
    for s in range(S):
        # the kernel adds the anchor's cached row to the query-side base in fp32, like the packed selector
        v = x["pb"][:, s].float() + x["pac"][s][row_batch.long(), anchors[:, s].long()].float()
        idx, score = oracle.partner_topk(v[:, :64], x["pk"][s], v[:, 64:], x["pm"][s], x["ps"][s], x["pg"][s],
                                         x["pbias"][s], 0, taken[:, s], L, top, K, strict, row_batch=row_batch,
                                         row_pos=row_pos, exclude_index=taken)
        live = active[:, s, None] & torch.isfinite(score)
        assert torch.equal(got[5].cpu()[:, s], live), s
        assert torch.equal(got[3].cpu()[:, s][live], idx[live]), s
        assert torch.equal(got[4].cpu()[:, s][live], score[live]), s
    # invariants of the reference's own multi-anchor test (tests/test_multi_relation_blocks.py:34-42)
    a, act, p, pact = got[0].cpu(), got[2].cpu(), got[3].cpu(), got[5].cpu()
    for r in range(0, N, 7):
        chosen = a[r][act[r]]
        assert chosen.unique().numel() == chosen.numel() and torch.all(chosen <= row_pos[r])
        partners = p[r][pact[r]]
        assert torch.all(partners <= row_pos[r])
        assert not set(partners.tolist()) & set(chosen.tolist())
    assert_status_clear()


def _check_layer_against_port(runner, port, layer, kept, rows, hidden_before, hidden_after):
    """One layer of the GPU pass, kernel by kernel on the GPU's own inputs, for the query rows `rows`."""
    from gpu_util import assert_rel_close, assert_scores_equal

    cfg = runner.config
    S, K, d = cfg.anchors_per_block, cfg.partners_per_anchor, cfg.d_model
    state = {k: v.float().cpu() for k, v in kept["state"].items() if k != "packed"}
    row_batch, row_pos = kept["row_batch"].cpu()[rows], kept["row_position"].cpu()[rows]
    q = kept["query"].cpu()[rows]
    anchors, active, partners, scores = port.select(layer, q, state, row_batch, row_pos)
    assert torch.equal(kept["anchor"].cpu()[rows], anchors)
    assert torch.equal(kept["anchor_active"].cpu()[rows], active)
    assert torch.equal(kept["partner"].cpu()[rows], partners)
    assert_scores_equal(kept["partner_score"][rows.cuda()], scores)
    w = port.layers[layer]
    n = rows.numel()
    pair_index = (rows[:, None] * S + torch.arange(S)[None, :]).reshape(-1)            # rows of the [N * S, ...] tensors
    pair_rows = row_batch.repeat_interleave(S)
    want_hidden, _ = oracle.relation_hidden(state["expanded_cache"], state["operand_cache"], anchors.view(n * S),
                                            partners.view(n * S, K), w["product_weight"], row_batch=pair_rows,
                                            row_pos=row_pos.repeat_interleave(S))
    live = scores.view(n * S, K) > -torch.inf
    got_hidden = kept["hidden_rel"][pair_index.cuda()].cpu()
    assert_rel_close(got_hidden[live], want_hidden[live], 1e-2, "relation hidden")
    got_raw = kept["raw"][pair_index.cuda()].cpu()
    assert_rel_close(got_raw[live], (oracle.linear(got_hidden, w["w2"]) + w["b2"])[live], 1e-2, "second layer")
    no_limit = torch.full((n * S,), (1 << 30) - 2, dtype=torch.int32)
    want_ctx = oracle.relation_norm_reduce(got_raw, scores.view(n * S, K), w["relation_norm_w"], w["relation_norm_b"],
                                           0, cfg.norm_eps, row_pos=no_limit).view(n, S, d)
    assert_rel_close(kept["slot_context"][rows.cuda()], want_ctx, 1e-4, "slot context")
    weight = w["slot_weight"][None, :] * active
    weight = weight / weight.sum(-1, keepdim=True).clamp_min(1.0e-9)
    want_after = hidden_before[rows] + w["gate"] * (want_ctx * weight[..., None]).sum(1)
    assert_rel_close(hidden_after[rows], want_after, 1e-4, "residual")


def test_routed_multi_anchor_stack_matches_cpu_port():
    """Depth-2 routed multi-anchor stack (4 slots x 4 partners, block 32, window 64, 3 remote blocks,
    bf16) on 2 sequences of 256: state bit-equal to the port's, every kernel of every layer
    against the port on the GPU pass's own inputs, all rows."""
    from oracle.multi_anchor_port import OracleMultiAnchor
    from relation_lm.inference.multi_anchor import MultiAnchorConfig, MultiAnchorPrefill, MultiAnchorRoutedStack

    cfg = MultiAnchorConfig(d_model=128, depth=2, max_context=256, block_size=32, local_window=64, top_blocks=3)
    stack = MultiAnchorRoutedStack(cfg, seed=4405)
    runner = MultiAnchorPrefill(stack, "cuda", torch.bfloat16)
    port = OracleMultiAnchor(stack, torch.bfloat16)
    g = torch.Generator().manual_seed(4406)
    B, T, d = 2, cfg.max_context, cfg.d_model
    hidden = torch.randn(B, T, d, generator=g)
    memory = torch.randn(B, T, d, generator=g).bfloat16()
    rows = torch.arange(B * T)
    current = hidden.cuda()
    for layer in range(cfg.depth):
        state = runner.build_state(layer, memory.cuda())
        from gpu_util import assert_rel_close
        want_packed = oracle.linear(memory.view(B * T, d), port.layers[layer]["w_memory"]).view(B, T, -1)
        assert_rel_close(state["packed"], want_packed, 1e-2, "memory-side projection")
        # everything downstream of that projection, from the GPU's own projection: bit for bit
        want_state = port.build_state(layer, memory.float(), packed=state["packed"].cpu())
        for name, want in want_state.items():
            if name == "expanded_cache":
                assert_rel_close(state[name], want, 1e-2, name)
            else:
                assert torch.equal(state[name].float().cpu(), want), (layer, name)
        before = current.clone()
        kept = {"state": state}
        runner.forward_layer(layer, current, state, kept)
        _check_layer_against_port(runner, port, layer, kept, rows, before.view(B * T, d).cpu(),
                                  current.view(B * T, d).cpu())
    assert_status_clear()


def test_multi_anchor_stack_configuration_at_full_shape():
    """The multi-anchor configuration itself — depth 4, batch 16, context 2048, d_model 512, 4 anchors
    x 4 partners, block 32, 3 remote blocks, bf16, N(0, 1) inputs: size-independent properties on all
    32 768 rows of every layer (distinct causal anchors, no anchor in any partner set, activity
    rules), and 1 500 sampled rows of the first and last layer against the port."""
    from oracle.multi_anchor_port import OracleMultiAnchor
    from relation_lm.inference.multi_anchor import MultiAnchorConfig, MultiAnchorPrefill, MultiAnchorRoutedStack

    cfg = MultiAnchorConfig()
    assert (cfg.depth, cfg.max_context, cfg.d_model, cfg.anchors_per_block, cfg.partners_per_anchor,
            cfg.block_size, cfg.top_blocks) == (4, 2048, 512, 4, 4, 32, 3)
    stack = MultiAnchorRoutedStack(cfg, seed=1004)
    runner = MultiAnchorPrefill(stack, "cuda", torch.bfloat16)
    port = OracleMultiAnchor(stack, torch.bfloat16)
    g = torch.Generator().manual_seed(1004)
    B, T, d, S = 16, cfg.max_context, cfg.d_model, cfg.anchors_per_block
    hidden = torch.randn(B, T, d, generator=g).cuda()
    memory = torch.randn(B, T, d, generator=g).bfloat16().cuda()
    sample = torch.randint(0, B * T, (1500,), generator=g).unique()
    current = hidden.clone()
    for layer in range(cfg.depth):
        state = runner.build_state(layer, memory)
        before = current.clone()
        kept = {"state": state}
        runner.forward_layer(layer, current, state, kept)
        anchor, active = kept["anchor"].cpu().long(), kept["anchor_active"].cpu()
        partner, pactive = kept["partner"].cpu().long(), kept["partner_active"].cpu()
        rp = kept["row_position"].cpu().long()
        assert torch.equal(active, torch.arange(S)[None, :] <= rp[:, None])           # slot s active iff s <= t
        assert bool((anchor <= rp[:, None]).all()) and bool((anchor[~active] == 0).all())
        masked = torch.where(active, anchor, -1 - torch.arange(S)[None, :])            # inactive slots: unique dummies
        ordered = masked.sort(-1).values
        assert bool((ordered[:, 1:] != ordered[:, :-1]).all())                         # distinct anchors
        assert bool((partner <= rp[:, None, None]).all())
        clash = (partner[:, :, :, None] == masked[:, None, None, :]) & pactive[..., None]
        assert not bool(clash.any())                                                   # no anchor in any partner set
        assert not bool(pactive[~active].any())
        if layer in (0, cfg.depth - 1):
            _check_layer_against_port(runner, port, layer, kept, sample, before.view(B * T, d).cpu(),
                                      current.view(B * T, d).cpu())
        del kept, state
    assert torch.isfinite(current).all()
    assert_status_clear()


@pytest.mark.parametrize("S,B,T,NB,L,top,K,Tq,strict", [
    (4, 2, 2048, 64, 64, 3, 4, 2048, True),      # the multi-anchor configuration's shape (block 32, 160 candidates)
    (4, 3, 256, 8, 64, 3, 4, 256, False),
    (3, 2, 512, 8, 128, 2, 8, 300, True),        # block 64, 256 candidates, queries over a prefix only, ragged last tile
    (8, 1, 192, 12, 16, 1, 2, 192, False),       # eight slots, block 16 (remote passes span blocks)
    (2, 2, 128, 4, 128, 0, 4, 128, True),        # no remote blocks: the window is the whole history
    (2, 1, 4096, 128, 128, 4, 8, 600, True),     # 128 blocks of statistics: tiles of 8 warps instead of 16
])
def test_whole_sequence_multi_anchor_selector_equals_the_per_row_selector(S, B, T, NB, L, top, K, Tq, strict):
    """The tiled whole-sequence form against the per-row multi-anchor kernel on the same rows: anchors,
    anchor scores, activity flags, partner indices and scores, all bit for bit (and therefore the
    oracle composition the per-row kernel is pinned to)."""
    from relation_lm.kernels.multi_select import relation_select_multi_prefill, relation_select_multi_rows

    g = torch.Generator().manual_seed(4500 + S + T)
    N = B * Tq
    dt = torch.bfloat16
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    x = [rn(N, S, 64).to(dt), rn(S, B, T, 64).to(dt), rn(N, S, 64).to(dt), rn(S, B, NB, 4, 16).to(dt),
         rn(S, B, NB, 4, 16).abs().to(dt), rn(S, 4), rn(S, 4, 16), rn(N, S, 128).to(dt), rn(S, B, T, 128).to(dt),
         rn(S, B, T, 64).to(dt), rn(S, B, NB, 4, 16).to(dt), rn(S, B, NB, 4, 16).abs().to(dt), rn(S, 4), rn(S, 4, 16)]
    # some exact duplicates among the keys of slot 0: ties between positions, and between slots' choices
    x[1][0, :, 5::17] = x[1][0, :, 4:5]
    x[9][0, :, 3::11] = x[9][0, :, 2:3]
    d = [v.cuda() for v in x]
    row_batch = torch.arange(B, dtype=torch.int32).repeat_interleave(Tq).cuda()
    row_pos = torch.arange(Tq, dtype=torch.int32).repeat(B).cuda()
    want = relation_select_multi_rows(*d, row_batch, row_pos, L, top, K, strict)
    got = relation_select_multi_prefill(*d, Tq, L, top, K, strict)
    names = ("anchor", "anchor score", "anchor active", "partner", "partner score", "partner active")
    for name, a, b in zip(names, got, want):
        if a.dtype == torch.float32:
            assert torch.equal(a.view(torch.int32), b.view(torch.int32)), name
        else:
            assert torch.equal(a, b), name
    assert bool(got[2].any()) and bool(got[5].any())
    assert_status_clear()
