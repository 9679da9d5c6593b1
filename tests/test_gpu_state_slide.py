"""Sliding decode state: ``state_slide`` against plain tensor slicing (bit-exact), and a decoder that
goes on past ``max_context`` against the CPU port doing the same with slices.

The reference has no code for contexts beyond its cache length (docs/roadmap.md:8 of the reference
lists "persistent ring-buffer state" as open), so the decode comparison is between this package's
decoder and its CPU port (oracle kernels, state moved with ``c[:, :, :T - s] = c[:, :, s:]``).
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from gpu_util import assert_status_clear

pytestmark = pytest.mark.gpu


def _reference(t: torch.Tensor, shift: int, dim: int) -> torch.Tensor:
    out = t.clone()
    rows = t.size(dim)
    keep = out.narrow(dim, 0, rows - shift)
    keep.copy_(t.narrow(dim, shift, rows - shift))
    return out


@pytest.mark.parametrize("shift", [1, 7, 16, 17, 47])
def test_state_slide_equals_slicing(shift):
    from relation_lm.kernels.router_cache import state_slide

    g = torch.Generator().manual_seed(100 + shift)
    caches = [torch.randn(3, 5, 64, 64, generator=g).to(torch.bfloat16).cuda(),          # 128-byte rows
              torch.randn(2, 2, 48, 192, generator=g).cuda(),                            # fp32, 768-byte rows
              torch.randn(1, 1, 200, 8, generator=g).to(torch.float16).cuda(),           # 16-byte rows
              torch.randn(4, 1, 64, 4104, generator=g).to(torch.bfloat16).cuda()]        # wide rows, many columns
    stats = torch.randn(2, 3, 64, 4, 16, generator=g).to(torch.bfloat16).cuda()          # rows are blocks
    before = [c.clone() for c in caches] + [stats.clone()]
    state_slide(caches + [stats], [shift] * 5, row_dim=[-2] * 4 + [-3])
    for mine, start, dim in zip(caches + [stats], before, [2, 2, 2, 2, 2]):
        assert torch.equal(mine, _reference(start, shift, dim)), (tuple(mine.shape), shift)
    assert_status_clear()


def test_state_slide_many_tensors_and_no_ops():
    from relation_lm.kernels.router_cache import state_slide

    g = torch.Generator().manual_seed(7)
    tensors = [torch.randn(2, 24 + k, 16, generator=g).cuda() for k in range(20)]      # more than one launch
    before = [t.clone() for t in tensors]
    shifts = [k % 5 for k in range(20)]                                                   # zeros among them
    state_slide(tensors, shifts)
    for mine, start, shift in zip(tensors, before, shifts):
        assert torch.equal(mine, _reference(start, shift, 1))
    state_slide([], [])
    empty = torch.zeros(0, 8, 16, device="cuda")
    state_slide([empty], [3])
    assert_status_clear()


def test_state_slide_rejects_bad_arguments():
    from relation_lm.kernels import _abi
    from relation_lm.kernels.router_cache import state_slide

    t = torch.zeros(2, 8, 16, device="cuda")
    with pytest.raises(ValueError):
        state_slide([t], [8])
    with pytest.raises(ValueError):
        state_slide([t.transpose(0, 1)], [1])
    narrow = torch.zeros(2, 8, 2, device="cuda")                                         # 8-byte rows
    with pytest.raises(ValueError, match="16 bytes"):
        state_slide([narrow], [1])
    # the C entry itself: shift == rows, and more than 16 tensors
    one = lambda *v: (ctypes.c_int64 * len(v))(*v)  # noqa: E731
    ptr = (ctypes.c_void_p * 1)(t.data_ptr())
    assert _abi.LIB.rlm_state_slide(ptr, one(2), one(8), one(64), one(8), 1, None) == -2     # RLM_ERR_SHAPE
    assert _abi.LIB.rlm_state_slide(ptr, one(2), one(8), one(64), one(1), 17, None) == -2
    assert _abi.LIB.rlm_state_slide(None, one(2), one(8), one(64), one(1), 1, None) == -1    # RLM_ERR_NULL
    assert torch.count_nonzero(t) == 0


def _small_model(seed=3, **kw):
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM

    cfg = RoutedRelationConfig(vocab_size=500, boundary_vocab_size=16, d_model=128, layers=3,
                               max_context=96, block_size=8, local_window=16, top_blocks=2, **kw)
    return RoutedRelationLM(cfg, seed=seed)


@pytest.mark.parametrize("blocks", [1, 3])
def test_fp32_decode_beyond_context_matches_cpu_port(blocks):
    """250 positions through a 96-row state: whenever the context is full both sides slide by
    ``blocks`` router blocks.  Selections identical at every layer and position, logits to 2e-3, the
    whole state (stale rows included) to 2e-5."""
    from oracle.decode_port import OracleDecoder
    from relation_lm.inference.stateful_decode import StatefulDecoder

    model = _small_model(seed=17)
    T = model.config.max_context
    B, steps = 2, 250
    gpu = StatefulDecoder(model, B, "cuda", torch.float32)
    cpu = OracleDecoder(model, B, torch.float32)
    g = torch.Generator().manual_seed(21)
    tokens = torch.randint(0, 500, (B, steps), generator=g)
    bounds = torch.randint(0, 16, (B, steps), generator=g)
    slides = 0
    for t in range(steps):
        if cpu.position == T:
            gpu.slide(blocks)
            cpu.slide(blocks)
            slides += 1
            assert int(gpu.position.item()) == cpu.position == T - blocks * model.config.block_size
        tl, bl = gpu.step(tokens[:, t].cuda(), bounds[:, t].cuda(), keep_selection=True)
        ctl, cbl = cpu.step(tokens[:, t], bounds[:, t])
        for layer, ((ga, gp), (ca, cp)) in enumerate(zip(gpu.last_selection, cpu.last_selection)):
            assert torch.equal(ga.cpu(), ca), (t, layer)
            assert torch.equal(gp.cpu(), cp), (t, layer)
        assert torch.allclose(tl.cpu(), ctl, atol=2e-3, rtol=1e-4), (t, (tl.cpu() - ctl).abs().max())
        assert torch.allclose(bl.cpu(), cbl, atol=2e-3, rtol=1e-4)
    assert slides == {1: 20, 3: 7}[blocks]
    for name in ("anchor_keys", "partner_keys", "operand_cache", "partner_anchor_cache", "expanded_cache"):
        assert torch.allclose(getattr(gpu, name).cpu(), getattr(cpu, name), atol=2e-5, rtol=1e-5), name
    for mine, theirs in zip(gpu.router_caches + gpu.router_stats, cpu.router_caches + cpu.router_stats):
        assert torch.allclose(mine.cpu(), theirs, atol=2e-5, rtol=1e-5)
    assert_status_clear()


def test_graphed_bf16_decode_slides_between_replays():
    """The captured bf16 step (the benchmarked path) with slides between replays: bit-equal to the
    eager decoder doing the same, and tracking the CPU port (bf16 rounding on both sides)."""
    from oracle.decode_port import OracleDecoder
    from relation_lm.inference.stateful_decode import StatefulDecoder

    model = _small_model(seed=19)
    T, bs = model.config.max_context, model.config.block_size
    B, steps = 2, 160
    g = torch.Generator().manual_seed(22)
    tokens = torch.randint(0, 500, (B, steps), generator=g)
    bounds = torch.randint(0, 16, (B, steps), generator=g)
    eager = StatefulDecoder(model, B, "cuda", torch.bfloat16)
    graphed = StatefulDecoder(model, B, "cuda", torch.bfloat16)
    graphed.capture()
    cpu = OracleDecoder(model, B, torch.bfloat16)
    position = 0
    for t in range(steps):
        if position == T:
            eager.slide(2)
            graphed.slide(2)
            cpu.slide(2)
            position -= 2 * bs
        tl, _ = eager.step(tokens[:, t].cuda(), bounds[:, t].cuda())
        graphed.static_tokens.copy_(tokens[:, t])
        graphed.static_boundaries.copy_(bounds[:, t])
        graphed.replay()
        ctl, _ = cpu.step(tokens[:, t], bounds[:, t])
        position += 1
        assert torch.equal(tl, graphed.static_token_logits), t
        cos = torch.nn.functional.cosine_similarity(tl.float().cpu().flatten(), ctl.flatten(), dim=0)
        assert cos > 0.98, (t, float(cos))
    assert int(graphed.position.item()) == position
    assert torch.equal(eager.expanded_cache, graphed.expanded_cache)
    assert torch.equal(eager.router_stats[1], graphed.router_stats[1])
    assert_status_clear()
