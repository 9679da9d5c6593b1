"""The benchmarked decode step, at the benchmarked configuration, against the CPU oracle.

6 relation layers, d_model 512, context 512, block 32, window 64, 2 remote blocks, K = 8,
bf16, batch 8 — the fused step that ``bench.py`` times (LayerNorm-fused projections, stacked
cache / expanded-cache appends, selector, relation hidden, second MLP layer, norm-reduce with
residual, next LayerNorm and next query projection).  The check is teacher-forced: at every
checked position each kernel's OWN 16-bit inputs, as the GPU step produced them, go to the
oracle's version of that kernel.

* selected anchor / partner indices and their scores: bit-exact, every layer;
* router caches, block statistics and the token-cache rows: bit-equal to the oracle's update;
* relation hidden, second-layer output, residual stream, normalised rows, query rows, logits:
  within 1e-2 of the row's largest magnitude (fp32 results from identical inputs: 1e-4).

Checked positions: the first two block boundaries and the last 72 positions (two more
boundaries, the published protocol's generated span).
"""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

import oracle
from gpu_util import assert_rel_close, assert_scores_equal, assert_status_clear

pytestmark = pytest.mark.gpu

ROUTER_STATE = ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache",
                "anchor_mean", "anchor_std", "partner_mean", "partner_std")


def _zipf(batch, length, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    weights = torch.arange(1, vocab + 1, dtype=torch.float64).pow(-1.1)
    return torch.multinomial(weights / weights.sum(), batch * length, replacement=True,
                             generator=g).view(batch, length)


def _router_state(dec):
    return [t.float().cpu() for t in (*dec.router_caches, *dec.router_stats)]


def _check_position(dec, wc, t, tokens_t, bounds_t, before, trace):
    cfg = dec.config
    R, H, K, d, bs = cfg.relation_dim, cfg.hidden_dim, cfg.k_max, cfg.d_model, cfg.block_size
    width = 384 + R
    head = trace[0]
    assert head["stage"] == "append"
    embedded = (wc["token_embedding"][tokens_t] + wc["boundary_embedding"][bounds_t]) * dec.input_scale \
        + wc["position_embedding"][t]
    assert_rel_close(head["embedded"], embedded, 1e-2, "embedding")
    x = head["embedded"].cpu()
    assert_rel_close(head["memory_normalized"],
                     F.layer_norm(x, (d,), wc["memory_norm_w"], wc["memory_norm_b"], cfg.norm_eps), 1e-2, "memory norm")
    assert_rel_close(head["normalized"],
                     F.layer_norm(x, (d,), wc["input_norm_w"][0], wc["input_norm_b"][0], cfg.norm_eps), 1e-2, "input norm 0")
    packed = head["packed"].cpu()
    assert_rel_close(packed, oracle.linear(head["memory_normalized"].cpu(), wc["w_packed"]), 1e-2, "packed projection")
    after = _router_state(dec)
    layers = [e for e in trace if e["stage"] == "layer"]
    assert len(layers) == cfg.layers
    for l, e in enumerate(layers):
        p = packed[:, l * width:(l + 1) * width].float()
        # token-cache rows and the router update of this layer: bit for bit
        for cache, lo, hi in ((dec.anchor_keys, 0, 64), (dec.partner_keys, 64, 128),
                              (dec.operand_cache, 128, 128 + R), (dec.partner_anchor_cache, 128 + R, 256 + R)):
            assert torch.equal(cache[l, :, t].float().cpu(), p[:, lo:hi]), (t, l, lo)
        _, want_state = oracle.router_cache_update(
            p[:, 256 + R:320 + R], p[:, 320 + R:384 + R], *[s[l] for s in before],
            wc["anchor_conv_weight"][l], wc["partner_conv_weight"][l], t, bs,
            cache_dtype=torch.bfloat16, stats_dtype=torch.bfloat16)
        for name, mine in zip(ROUTER_STATE, after):
            assert torch.equal(mine[l], want_state[name]), (t, l, name)
        # expanded-cache row of this position
        o_t = dec.operand_cache[l, :, t].float().cpu()
        want_row = torch.cat((o_t @ wc["anchor_weight"][l].T + wc["first_bias"][l], o_t @ wc["partner_weight"][l].T), -1)
        assert_rel_close(dec.expanded_cache[l, :, t], want_row, 1e-2, f"expanded row t={t} l={l}")
        # selection: the GPU's own query rows and caches through the oracle
        q = e["query"].cpu()
        anchor, anchor_score, partner, partner_score, _ = oracle.relation_select(
            q[:, 0:64], dec.anchor_keys[l].cpu(), q[:, 64:128], after[4][l], after[5][l],
            wc["anchor_gamma"][l], wc["anchor_bias"][l], q[:, 128:256], dec.partner_anchor_cache[l].cpu(),
            dec.partner_keys[l].cpu(), after[6][l], after[7][l], wc["partner_gamma"][l], wc["partner_bias"][l],
            t, cfg.local_window, cfg.top_blocks, K, cfg.strict_valid)
        assert torch.equal(e["anchor"].cpu(), anchor), (t, l)
        assert torch.equal(e["partner"].cpu(), partner), (t, l)
        assert_scores_equal(e["partner_score"], partner_score)
        # relation hidden on the gathered rows (compacted caches: row 0 the anchor, rows 1..K the partners)
        idx = torch.cat((e["anchor"][:, None], e["partner"]), 1).long().clamp(0, cfg.max_context - 1)
        rows = torch.arange(dec.batch, device=idx.device)[:, None]
        small_expanded = dec.expanded_cache[l][rows, idx].cpu()
        small_operand = dec.operand_cache[l][rows, idx].cpu()
        local_anchor = torch.zeros(dec.batch, dtype=torch.int32)
        local_partner = torch.arange(1, K + 1, dtype=torch.int32).repeat(dec.batch, 1)
        want_hidden, _ = oracle.relation_hidden(small_expanded, small_operand, local_anchor, local_partner,
                                                wc["product_weight"][l])
        valid = partner_score > -torch.inf
        if "raw" in e:
            assert_rel_close(e["relation_hidden"].cpu()[valid], want_hidden[valid], 1e-2, f"relation hidden t={t} l={l}")
            # second relation-MLP layer on the GPU's own hidden states
            want_raw = oracle.linear(e["relation_hidden"].cpu(), wc["w2"][l]) + wc["b2"][l]
            assert_rel_close(e["raw"].cpu()[valid], want_raw[valid], 1e-2, f"second layer t={t} l={l}")
            # norm-reduce + residual on the GPU's own second-layer output
            context = oracle.relation_norm_reduce(e["raw"].cpu(), partner_score, wc["relation_norm_w"][l],
                                                  wc["relation_norm_b"][l], t, cfg.norm_eps)
            want_after = e["hidden_before"].cpu() + wc["mix"][l] * context
            assert_rel_close(e["hidden_after"], want_after, 1e-4, f"residual t={t} l={l}")
        else:
            # single-launch tail: hidden states (rounded to 16 bits, as the kernel hands them to its second
            # GEMM) and the fp32 second-layer output stay on chip; the oracle composes the same steps
            want_raw = oracle.linear(want_hidden.bfloat16(), wc["w2"][l]) + wc["b2"][l]
            context = oracle.relation_norm_reduce(want_raw, partner_score, wc["relation_norm_w"][l],
                                                  wc["relation_norm_b"][l], t, cfg.norm_eps)
            want_after = e["hidden_before"].cpu() + wc["mix"][l] * context
            assert_rel_close(e["hidden_after"], want_after, 1e-2, f"residual t={t} l={l}")
        last = l + 1 == cfg.layers
        nw = wc["final_norm_w"] if last else wc["input_norm_w"][l + 1]
        nb = wc["final_norm_b"] if last else wc["input_norm_b"][l + 1]
        assert_rel_close(e["next_normalized"], F.layer_norm(e["hidden_after"].cpu(), (d,), nw, nb, cfg.norm_eps),
                         1e-2, f"next norm t={t} l={l}")
        if not last:
            want_q = oracle.linear(e["next_normalized"].cpu(), wc["w_query"][l + 1])
            assert_rel_close(layers[l + 1]["query"], want_q, 1e-2, f"query t={t} l={l + 1}")
        else:
            head_w = dec.head_weight.float().cpu()
            want_logits = oracle.linear(e["next_normalized"].cpu(), head_w) + dec.head_bias.cpu()
            assert_rel_close(dec.last_logits, want_logits, 1e-2, f"logits t={t}")
    want_q0 = oracle.linear(head["normalized"].cpu(), wc["w_query"][0])
    assert_rel_close(layers[0]["query"], want_q0, 1e-2, f"query t={t} l=0")


@pytest.mark.parametrize("mode", ["whole_layer", "layer_tail", "layer_tail_separate_front", "separate"])
def test_fused_bf16_step_of_the_ctx512_decode_configuration_is_pinned_per_kernel(mode):
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM
    from relation_lm.inference.stateful_decode import StatefulDecoder

    cfg = RoutedRelationConfig()                     # 6 layers, d 512, ctx 512, block 32, window 64, top 2, K 8
    assert (cfg.layers, cfg.d_model, cfg.max_context, cfg.block_size, cfg.local_window) == (6, 512, 512, 32, 64)
    model = RoutedRelationLM(cfg, seed=1002)
    B, T = 8, cfg.max_context
    layer_tail = mode != "separate"
    dec = StatefulDecoder(model, B, "cuda", torch.bfloat16, layer_tail=layer_tail, whole_layer=mode == "whole_layer",
                          fused_front=mode != "layer_tail_separate_front")
    if layer_tail and not dec.layer_tail:
        pytest.skip("clusters of 16 CTAs are not available on this device")
    assert dec.whole_layer == (mode == "whole_layer")
    assert dec.fused_front == (mode != "layer_tail_separate_front")
    assert dec.fused and dec.stacked_expand and not dec.fused_tail and dec.layer_tail == layer_tail
    assert dec.fused_query != layer_tail
    wc = {k: v.float().cpu() for k, v in dec.w.items()}
    tokens = _zipf(B, T, cfg.vocab_size, 1002)
    bounds = torch.randint(0, cfg.boundary_vocab_size, (B, T), generator=torch.Generator().manual_seed(1079))
    checked = {0, 1, 2, 31, 32, 33, 63, 64, 65} | set(range(T - 72, T) if layer_tail else range(T - 40, T))
    tok_dev, bnd_dev = tokens.cuda(), bounds.cuda()
    for t in range(T):
        if t in checked:
            before = _router_state(dec)
            dec.trace = []
            dec.step(tok_dev[:, t], bnd_dev[:, t])
            trace, dec.trace = dec.trace, None
            _check_position(dec, wc, t, tokens[:, t], bounds[:, t], before, trace)
        else:
            dec.step(tok_dev[:, t], bnd_dev[:, t])
    assert int(dec.position.item()) == T
    assert_status_clear()


@pytest.mark.parametrize("position", [0, 1, 31, 32, 511])
def test_stacked_cache_append_bf16_matches_per_layer_oracle_updates(position):
    """``sparse_cache_append`` as the decoder calls it (all layers in one launch, bf16 caches and
    statistics, fp32 conv weights): token-cache rows equal the packed slices and all eight
    router tensors of every layer equal the oracle's single-layer update, bit for bit; rows other
    than ``position`` and blocks other than its block are untouched."""
    from relation_lm.kernels.router_cache import sparse_cache_append

    layers, B, T, bs, R = 6, 8, 512, 32, 128
    nb, width = T // bs, 384 + R
    g = torch.Generator().manual_seed(7100 + position)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    packed = rn(B, layers * width).bfloat16()
    token_caches = [torch.zeros(layers, B, T, w_, dtype=torch.bfloat16) for w_ in (64, 64, R, 128)]
    router = []
    for _ in range(4):
        c = torch.zeros(layers, B, T, 64)
        c[:, :, :position] = rn(layers, B, position, 64)
        c[:, :, position:] = rn(layers, B, T - position, 64) * 0.5      # stale rows beyond the position
        router.append(c.bfloat16())
    stats = [rn(layers, B, nb, 4, 16).bfloat16() for _ in range(4)]
    conv_a, conv_p = rn(layers, 64, 3) * 0.1, rn(layers, 64, 3) * 0.1
    dev_tok = [c.cuda() for c in token_caches]
    dev_router = [c.cuda() for c in router]
    dev_stats = [c.cuda() for c in stats]
    sparse_cache_append(packed.cuda(), *dev_tok, *dev_router, *dev_stats, conv_a.cuda(), conv_p.cuda(),
                        torch.tensor(position, device="cuda"), bs)
    for l in range(layers):
        p = packed[:, l * width:(l + 1) * width]
        for cache, lo, hi in zip(dev_tok, (0, 64, 128, 128 + R), (64, 128, 128 + R, 256 + R)):
            got = cache[l].cpu()
            assert torch.equal(got[:, position], p[:, lo:hi])
            got[:, position] = 0
            assert not got.any()
        _, want = oracle.router_cache_update(
            p[:, 256 + R:320 + R], p[:, 320 + R:384 + R], *[c[l] for c in router], *[s[l] for s in stats],
            conv_a[l], conv_p[l], position, bs)
        for name, mine in zip(ROUTER_STATE, dev_router + dev_stats):
            assert torch.equal(mine[l].float().cpu(), want[name]), (l, name)
    assert_status_clear()
