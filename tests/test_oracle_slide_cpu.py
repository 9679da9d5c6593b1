"""The CPU port's sliding state (``OracleDecoder.slide``), the checker of the GPU decoder's
``slide``: what moves where, and that decoding goes on past ``max_context``."""
from __future__ import annotations

import pytest
import torch


def test_port_slides_and_goes_on():
    pytest.importorskip("oracle")
    from oracle.decode_port import OracleDecoder
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM

    cfg = RoutedRelationConfig(vocab_size=300, boundary_vocab_size=8, d_model=128, layers=2, max_context=48,
                               block_size=8, local_window=16, top_blocks=2)
    model = RoutedRelationLM(cfg, seed=4)
    B, T, bs = 2, cfg.max_context, cfg.block_size
    port = OracleDecoder(model, B, torch.float32)
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, 300, (B, T + 20), generator=g)
    bounds = torch.randint(0, 8, (B, T + 20), generator=g)
    for t in range(T):
        port.step(tokens[:, t], bounds[:, t])
    with pytest.raises(IndexError):                       # the context is full: no row, no position left
        port.step(tokens[:, T], bounds[:, T])
    caches = [port.anchor_keys, port.operand_cache, port.expanded_cache, port.router_caches[2]]
    before = [c.clone() for c in caches]
    stats_before = port.router_stats[1].clone()
    port.slide(2)
    assert port.position == T - 2 * bs
    for now, old in zip(caches, before):
        assert torch.equal(now[:, :, :T - 2 * bs], old[:, :, 2 * bs:])
        assert torch.equal(now[:, :, T - 2 * bs:], old[:, :, T - 2 * bs:])        # stale rows stay
    assert torch.equal(port.router_stats[1][:, :, :T // bs - 2], stats_before[:, :, 2:])
    for t in range(T, T + 20):
        if port.position == T:
            port.slide(1)
        logits, _ = port.step(tokens[:, t], bounds[:, t])
        assert torch.isfinite(logits).all()
        for anchor, partner in port.last_selection:
            assert int(anchor.max()) < port.position and int(partner.max()) < port.position
