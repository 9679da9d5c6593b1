"""The stateful decode step on the GPU vs its CPU port (oracle kernels + fp32 matmuls).

fp32 model: selected indices must be identical at every layer and position and logits agree
to 2e-3 (the two paths differ only in GEMM accumulation order).  bf16 model: GEMM outputs are
rounded to bf16 on both sides, so rare near-tie selections may differ; reduced states must
stay within 1e-2 relative where the selections agree.
"""
from __future__ import annotations

import pytest
import torch

from gpu_util import assert_status_clear

pytestmark = pytest.mark.gpu


def _small_model(seed=3, **kw):
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM

    cfg = RoutedRelationConfig(vocab_size=500, boundary_vocab_size=16, d_model=128, layers=3,
                               max_context=96, block_size=8, local_window=16, top_blocks=2, **kw)
    return RoutedRelationLM(cfg, seed=seed)


@pytest.mark.parametrize("strict", [False, True])
def test_fp32_decode_matches_cpu_port(strict):
    from oracle.decode_port import OracleDecoder
    from relation_lm.inference.stateful_decode import StatefulDecoder

    model = _small_model(strict_valid=strict)
    B, steps = 3, 96
    gpu = StatefulDecoder(model, B, "cuda", torch.float32)
    cpu = OracleDecoder(model, B, torch.float32)
    g = torch.Generator().manual_seed(11)
    tokens = torch.randint(0, 500, (B, steps), generator=g)
    bounds = torch.randint(0, 16, (B, steps), generator=g)
    for t in range(steps):
        tl, bl = gpu.step(tokens[:, t].cuda(), bounds[:, t].cuda(), keep_selection=True)
        ctl, cbl = cpu.step(tokens[:, t], bounds[:, t])
        for layer, ((ga, gp), (ca, cp)) in enumerate(zip(gpu.last_selection, cpu.last_selection)):
            assert torch.equal(ga.cpu(), ca), (t, layer)
            assert torch.equal(gp.cpu(), cp), (t, layer)
        assert torch.allclose(tl.cpu(), ctl, atol=2e-3, rtol=1e-4), (t, (tl.cpu() - ctl).abs().max())
        assert torch.allclose(bl.cpu(), cbl, atol=2e-3, rtol=1e-4)
    for name in ("anchor_keys", "partner_keys", "operand_cache", "partner_anchor_cache", "expanded_cache"):
        assert torch.allclose(getattr(gpu, name).cpu(), getattr(cpu, name), atol=2e-5, rtol=1e-5), name
    for mine, theirs in zip(gpu.router_caches + gpu.router_stats, cpu.router_caches + cpu.router_stats):
        assert torch.allclose(mine.cpu(), theirs, atol=2e-5, rtol=1e-5)
    assert_status_clear()


def test_graph_replay_equals_eager_steps():
    from relation_lm.inference.stateful_decode import StatefulDecoder

    model = _small_model(seed=5)
    B, steps = 2, 40
    g = torch.Generator().manual_seed(12)
    tokens = torch.randint(0, 500, (B, steps), generator=g).cuda()
    bounds = torch.randint(0, 16, (B, steps), generator=g).cuda()
    eager = StatefulDecoder(model, B, "cuda", torch.bfloat16)
    graphed = StatefulDecoder(model, B, "cuda", torch.bfloat16)
    graphed.capture()
    for t in range(steps):
        tl, _ = eager.step(tokens[:, t], bounds[:, t])
        graphed.static_tokens.copy_(tokens[:, t])
        graphed.static_boundaries.copy_(bounds[:, t])
        graphed.replay()
        assert torch.equal(tl, graphed.static_token_logits), t
    assert int(graphed.position.item()) == steps
    assert torch.equal(eager.expanded_cache, graphed.expanded_cache)
    assert_status_clear()


def test_bf16_decode_tracks_cpu_port():
    from oracle.decode_port import OracleDecoder
    from relation_lm.inference.stateful_decode import StatefulDecoder

    model = _small_model(seed=9)
    B, steps = 4, 64
    gpu = StatefulDecoder(model, B, "cuda", torch.bfloat16)
    cpu = OracleDecoder(model, B, torch.bfloat16)
    g = torch.Generator().manual_seed(13)
    tokens = torch.randint(0, 500, (B, steps), generator=g)
    bounds = torch.randint(0, 16, (B, steps), generator=g)
    same = total = 0
    for t in range(steps):
        tl, _ = gpu.step(tokens[:, t].cuda(), bounds[:, t].cuda(), keep_selection=True)
        ctl, _ = cpu.step(tokens[:, t], bounds[:, t])
        (ga, gp), (ca, cp) = gpu.last_selection[0], cpu.last_selection[0]
        same += int((ga.cpu() == ca).sum()) + int((gp.cpu() == cp).sum())
        total += ga.numel() + gp.numel()
        assert torch.isfinite(tl).all()
        cos = torch.nn.functional.cosine_similarity(tl.float().cpu().flatten(), ctl.flatten(), dim=0)
        assert cos > 0.98, (t, float(cos))
    assert same / total > 0.97, same / total
    assert_status_clear()


def test_fused_tail_decode_tracks_default_path():
    """The single-launch tail sums its split-K partials with atomics (order not fixed), so the
    decode is compared by tolerance with the default path."""
    from relation_lm.inference.stateful_decode import StatefulDecoder

    model = _small_model(seed=21)
    B, steps = 2, 24
    g = torch.Generator().manual_seed(14)
    tokens = torch.randint(0, 500, (B, steps), generator=g).cuda()
    bounds = torch.randint(0, 16, (B, steps), generator=g).cuda()
    plain = StatefulDecoder(model, B, "cuda", torch.bfloat16, layer_tail=False)
    fused = StatefulDecoder(model, B, "cuda", torch.bfloat16, fused_tail=True)
    assert fused.fused_tail
    for t in range(steps):
        a, _ = plain.step(tokens[:, t], bounds[:, t])
        b, _ = fused.step(tokens[:, t], bounds[:, t])
        cos = torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0)
        assert cos > 0.995, (t, float(cos))
    assert_status_clear()


def test_programmatic_launch_does_not_change_results():
    """The fused bf16 step with and without programmatic dependent launch (kernels starting
    their set-up and the selector its cache prefetch while the previous kernel still runs):
    bit-identical logits, selections and state, eagerly and through the captured graph."""
    from relation_lm.inference.stateful_decode import StatefulDecoder

    model = _small_model(seed=9)
    B, steps = 4, 48
    g = torch.Generator().manual_seed(21)
    tokens = torch.randint(0, 500, (B, steps), generator=g).cuda()
    bounds = torch.randint(0, 16, (B, steps), generator=g).cuda()
    plain = StatefulDecoder(model, B, "cuda", torch.bfloat16, programmatic_launch=False)
    early = StatefulDecoder(model, B, "cuda", torch.bfloat16, programmatic_launch=True)
    assert plain.fused and early.fused
    for t in range(steps // 2):
        a = plain.step(tokens[:, t], bounds[:, t], keep_selection=True)
        b = early.step(tokens[:, t], bounds[:, t], keep_selection=True)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), t
        for (pa, pp), (ea, ep) in zip(plain.last_selection, early.last_selection):
            assert torch.equal(pa, ea) and torch.equal(pp, ep), t
    early.capture()
    for t in range(steps // 2, steps):
        a = plain.step(tokens[:, t], bounds[:, t])
        early.static_tokens.copy_(tokens[:, t])
        early.static_boundaries.copy_(bounds[:, t])
        early.replay()
        assert torch.equal(a[0], early.static_token_logits), t
    for name in ("anchor_keys", "partner_keys", "operand_cache", "partner_anchor_cache", "expanded_cache"):
        assert torch.equal(getattr(plain, name), getattr(early, name)), name
    assert_status_clear()


def test_split_k_second_layer_decode_tracks_default_path():
    """The optional all-library step (second relation-MLP layer as a split-K GEMM summed inside
    norm-reduce) against the default step (cuBLAS): same selections, logits within bf16 noise."""
    from relation_lm.inference.stateful_decode import StatefulDecoder

    model = _small_model(seed=13)
    B, steps = 4, 24
    g = torch.Generator().manual_seed(23)
    tokens = torch.randint(0, 500, (B, steps), generator=g).cuda()
    bounds = torch.randint(0, 16, (B, steps), generator=g).cuda()
    plain = StatefulDecoder(model, B, "cuda", torch.bfloat16, layer_tail=False)
    split = StatefulDecoder(model, B, "cuda", torch.bfloat16, second_layer_split=True)
    assert split.second_layer_splits > 1 and plain.second_layer_splits == 1
    agree = 0
    for t in range(steps):
        a = plain.step(tokens[:, t], bounds[:, t], keep_selection=True)
        b = split.step(tokens[:, t], bounds[:, t], keep_selection=True)
        same = all(torch.equal(pa, sa) and torch.equal(pp, sp_)
                   for (pa, pp), (sa, sp_) in zip(plain.last_selection, split.last_selection))
        agree += int(same)
        if same:
            assert torch.allclose(a[0].float(), b[0].float(), atol=0.25, rtol=0.05), t
    assert agree >= steps - 2          # rounding may flip a rare near-tie
    assert_status_clear()


def test_query_projection_inside_norm_reduce_tracks_separate_launches():
    """The decode step with the next layer's query projection inside norm-reduce (default for
    small batches) against the step with separate tensor-core projections: same selections, logits
    within bf16 noise."""
    from relation_lm.inference.stateful_decode import StatefulDecoder

    model = _small_model(seed=17)
    B, steps = 4, 24
    g = torch.Generator().manual_seed(29)
    tokens = torch.randint(0, 500, (B, steps), generator=g).cuda()
    bounds = torch.randint(0, 16, (B, steps), generator=g).cuda()
    separate = StatefulDecoder(model, B, "cuda", torch.bfloat16, fused_query=False, layer_tail=False)
    fused = StatefulDecoder(model, B, "cuda", torch.bfloat16, layer_tail=False)
    assert fused.fused_query and not separate.fused_query
    agree = 0
    for t in range(steps):
        a = separate.step(tokens[:, t], bounds[:, t], keep_selection=True)
        b = fused.step(tokens[:, t], bounds[:, t], keep_selection=True)
        same = all(torch.equal(pa, sa) and torch.equal(pp, sp_)
                   for (pa, pp), (sa, sp_) in zip(separate.last_selection, fused.last_selection))
        agree += int(same)
        if same:
            assert torch.allclose(a[0].float(), b[0].float(), atol=0.25, rtol=0.05), t
    assert agree >= steps - 2          # rounding may flip a rare near-tie
    assert_status_clear()


@pytest.mark.parametrize("mapped", [True, False])
def test_host_transfer_graph_equals_the_plain_greedy_step(mapped):
    """``capture_host_io`` / ``step_host``: ids from pinned host memory in, chosen tokens in pinned
    host memory out, all inside one graph; same tokens as ``step_greedy`` on device tensors.  Mapped:
    the head kernel writes the choices into the pinned memory itself; otherwise a copy node does."""
    from relation_lm.inference.stateful_decode import StatefulDecoder

    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM

    # d_model 256: the head projection's greedy launch (whose output the mapped form redirects) applies
    model = RoutedRelationLM(RoutedRelationConfig(vocab_size=500, boundary_vocab_size=16, d_model=256, layers=2,
                                                  max_context=96, block_size=8, local_window=16, top_blocks=2), seed=19)
    B, steps = 3, 12
    g = torch.Generator().manual_seed(31)
    tokens = torch.randint(0, 500, (B, steps), generator=g)
    bounds = torch.randint(0, 16, (B, steps), generator=g)
    plain = StatefulDecoder(model, B, "cuda", torch.bfloat16)
    hosted = StatefulDecoder(model, B, "cuda", torch.bfloat16)
    hosted.capture_host_io(mapped=mapped)
    assert hosted.skinny and hosted.host_io_mapped == mapped
    assert int(hosted.position.item()) == 0
    for t in range(steps):
        want = plain.step_greedy(tokens[:, t].cuda(), bounds[:, t].cuda())
        hosted.host_tokens.copy_(tokens[:, t])
        hosted.host_boundaries.copy_(bounds[:, t])
        got = hosted.step_host()
        assert torch.equal(got, want.cpu()), t
    assert int(hosted.position.item()) == steps == int(plain.position.item())
    assert_status_clear()


@pytest.mark.parametrize("name", ["stack_two_layers", "stack_single_layer_d256"])
def test_fp32_decode_reproduces_the_dense_reference_stack(golden, name):
    """The GPU step (fp32) against the reference's dense ``StackedRelationLayers`` outputs stored in
    the golden file: full-history window, no remote blocks — anchors and finite-score partners
    identical at every position and layer, the stack's output within 2e-5."""
    import cases
    from relation_lm.inference.stateful_decode import StatefulDecoder
    from test_oracle_stack import compare_with_dense_reference, stack_model

    entry = golden[name]
    case = entry["case"]
    x = cases.make_inputs(case)
    assert cases.checksum(x) == entry["input_sha256"]
    model = stack_model(case)
    assert cases.checksum(dict(model.state_dict())) == entry["outputs"]["model_sha256"]
    decoder = StatefulDecoder(model, case["batch"], "cuda", torch.float32)
    compare_with_dense_reference(entry, decoder, x["tokens"], x["boundaries"], to_device=lambda v: v.cuda())
    assert_status_clear()


@pytest.mark.parametrize("strict", [False, True])
def test_single_layer_fp32_configuration_matches_cpu_port_at_every_position(strict):
    """The single-layer fp32 configuration as a composed layer: d_model 256, hidden 1024, context
    128, block 16, window 32, 2 remote blocks, K = 8, batch 1 — selections identical and the
    reduced state (the residual stream after the layer, through the final LayerNorm) within 2e-5
    of the CPU port at every position."""
    from oracle.decode_port import OracleDecoder
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM
    from relation_lm.inference.stateful_decode import StatefulDecoder

    cfg = RoutedRelationConfig(vocab_size=300, boundary_vocab_size=16, d_model=256, layers=1, max_context=128,
                               block_size=16, local_window=32, top_blocks=2, strict_valid=strict)
    model = RoutedRelationLM(cfg, seed=1001)
    gpu = StatefulDecoder(model, 1, "cuda", torch.float32)
    cpu = OracleDecoder(model, 1, torch.float32)
    g = torch.Generator().manual_seed(1001)
    tokens = torch.randint(0, 300, (1, 128), generator=g)
    bounds = torch.randint(0, 16, (1, 128), generator=g)
    for t in range(128):
        gpu.step(tokens[:, t].cuda(), bounds[:, t].cuda(), keep_selection=True)
        cpu.step(tokens[:, t], bounds[:, t])
        (ga, gp), (ca, cp) = gpu.last_selection[0], cpu.last_selection[0]
        assert torch.equal(ga.cpu(), ca) and torch.equal(gp.cpu(), cp), t
        assert torch.allclose(gpu.last_final.cpu(), cpu.last_final, atol=2e-5, rtol=1e-5), t
    assert_status_clear()


def test_single_launch_layer_tail_decode_tracks_the_multi_launch_step():
    """The default small-batch step (one cluster launch per layer for the whole relation tail, hidden
    states on chip, second-layer output kept in fp32) against the step built from separate launches
    (relation hidden, library GEMM rounded to 16 bits, norm-reduce): same selections except for rare
    near-ties, logits within 16-bit noise; and the captured graph replays it bit for bit."""
    from relation_lm.inference.stateful_decode import StatefulDecoder

    model = _small_model(seed=23)
    B, steps = 4, 32
    g = torch.Generator().manual_seed(37)
    tokens = torch.randint(0, 500, (B, steps), generator=g).cuda()
    bounds = torch.randint(0, 16, (B, steps), generator=g).cuda()
    separate = StatefulDecoder(model, B, "cuda", torch.bfloat16, layer_tail=False)
    single = StatefulDecoder(model, B, "cuda", torch.bfloat16)
    if not single.layer_tail:
        pytest.skip("thread-block clusters of this size are not available on this device")
    graphed = StatefulDecoder(model, B, "cuda", torch.bfloat16)
    graphed.capture()
    agree = 0
    for t in range(steps):
        a = separate.step(tokens[:, t], bounds[:, t], keep_selection=True)
        b = single.step(tokens[:, t], bounds[:, t], keep_selection=True)
        graphed.static_tokens.copy_(tokens[:, t])
        graphed.static_boundaries.copy_(bounds[:, t])
        graphed.replay()
        assert torch.equal(b[0], graphed.static_token_logits), t
        same = all(torch.equal(pa, sa) and torch.equal(pp, sp_)
                   for (pa, pp), (sa, sp_) in zip(separate.last_selection, single.last_selection))
        agree += int(same)
        if same:
            assert torch.allclose(a[0].float(), b[0].float(), atol=0.25, rtol=0.05), t
    assert agree >= steps - 3
    assert_status_clear()


def test_one_launch_per_layer_equals_select_then_tail_bit_for_bit():
    """The selector run in front of the tail inside the tail's cluster changes no arithmetic: logits
    and selections of every step equal those of the two-launch form."""
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM
    from relation_lm.inference.stateful_decode import StatefulDecoder

    cfg = RoutedRelationConfig()
    model = RoutedRelationLM(cfg, seed=77)
    B, steps = 5, 80
    g = torch.Generator().manual_seed(78)
    tokens = torch.randint(0, cfg.vocab_size, (B, steps), generator=g).cuda()
    bounds = torch.randint(0, cfg.boundary_vocab_size, (B, steps), generator=g).cuda()
    two = StatefulDecoder(model, B, "cuda", torch.bfloat16, whole_layer=False)
    one = StatefulDecoder(model, B, "cuda", torch.bfloat16, whole_layer=True)
    if not one.whole_layer:
        pytest.skip("the one-launch layer is not available for this configuration on this device")
    assert two.layer_tail and not two.whole_layer
    graphed = StatefulDecoder(model, B, "cuda", torch.bfloat16, whole_layer=True)
    graphed.capture()
    for t in range(steps):
        a = two.step(tokens[:, t], bounds[:, t], keep_selection=True)
        b = one.step(tokens[:, t], bounds[:, t], keep_selection=True)
        graphed.static_tokens.copy_(tokens[:, t])
        graphed.static_boundaries.copy_(bounds[:, t])
        graphed.replay()
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), t
        assert torch.equal(b[0], graphed.static_token_logits), t
        for (pa, pp), (sa, sp_) in zip(two.last_selection, one.last_selection):
            assert torch.equal(pa, sa) and torch.equal(pp, sp_), t
    assert_status_clear()


def test_l2_prefetch_branch_changes_no_value():
    """The optional side-stream L2 prefetch at the head of a step (off by default) is invisible in the
    results, eagerly and through a captured graph."""
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM
    from relation_lm.inference.stateful_decode import StatefulDecoder

    cfg = RoutedRelationConfig()
    model = RoutedRelationLM(cfg, seed=91)
    B, steps = 3, 40
    g = torch.Generator().manual_seed(92)
    tokens = torch.randint(0, cfg.vocab_size, (B, steps), generator=g).cuda()
    bounds = torch.randint(0, cfg.boundary_vocab_size, (B, steps), generator=g).cuda()
    plain = StatefulDecoder(model, B, "cuda", torch.bfloat16)
    eager = StatefulDecoder(model, B, "cuda", torch.bfloat16, prefetch=True)
    graphed = StatefulDecoder(model, B, "cuda", torch.bfloat16, prefetch=True)
    assert not plain.prefetch and eager.prefetch
    graphed.capture()
    for t in range(steps):
        a = plain.step(tokens[:, t], bounds[:, t])
        b = eager.step(tokens[:, t], bounds[:, t])
        graphed.static_tokens.copy_(tokens[:, t])
        graphed.static_boundaries.copy_(bounds[:, t])
        graphed.replay()
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), t
        assert torch.equal(a[0], graphed.static_token_logits), t
    assert_status_clear()
