"""GPU parity of the relation-reduce tail vs the CPU oracle and the reference kernels' golden
outputs.  Tolerances: 2e-5 max-abs for fp32 inputs, 1e-2 relative for bf16 inputs."""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

import cases
import oracle
from gpu_util import assert_rel_close, assert_status_clear, position_tensor, to_cuda

pytestmark = pytest.mark.gpu

FP32_ATOL = 2.0e-5


def _names(kind):
    return [n for n, c in cases.all_cases().items() if c["kind"] == kind]


def _close(got, want, low):
    got, want = got.float().cpu(), want.float()
    if low:
        assert_rel_close(got, want, 1e-2)        # 16-bit operands: 1e-2 of the row's largest magnitude
    else:
        assert torch.allclose(got, want, atol=FP32_ATOL, rtol=1e-5), (got - want).abs().max()


@pytest.mark.parametrize("name", _names("reduce"))
def test_hidden_kernels_match_golden_and_oracle(golden, name):
    from relation_lm.kernels.relation_reduce import (factor_relation_first_layer,
                                                     relation_hidden_cache_update,
                                                     relation_hidden_cached)

    entry = golden[name]
    case, ref = entry["case"], entry["outputs"]
    x = cases.make_inputs(case)
    assert cases.checksum(x) == entry["input_sha256"]
    low = case["dtype"] != "fp32"
    factors = factor_relation_first_layer(x["first_weight"], x["first_bias"], case["relation_dim"])
    expanded = F.linear(x["operand_cache"].float(), factors.expanded_weight.float(),
                        factors.expanded_bias.float()).to(x["operand_cache"].dtype)
    xg = to_cuda(x)
    fg = factor_relation_first_layer(xg["first_weight"], xg["first_bias"], case["relation_dim"])
    hidden = relation_hidden_cached(expanded.cuda(), xg["operand_cache"], xg["anchor_index"],
                                    xg["partner_index"], fg.product_weight)
    want, _ = oracle.relation_hidden(expanded, x["operand_cache"], x["anchor_index"],
                                     x["partner_index"], factors.product_weight)
    _close(hidden, want, low)
    _close(hidden, ref["hidden_cached"], low)
    t = case["position"]
    mutable = expanded.clone()
    mutable[:, t].zero_()
    mg = mutable.cuda()
    updated = relation_hidden_cache_update(
        mg, xg["operand_cache"], xg["anchor_index"], xg["partner_index"], fg.anchor_weight,
        fg.partner_weight, fg.product_weight, fg.first_bias, position_tensor(t))
    want_u, want_cache = oracle.relation_hidden(
        mutable, x["operand_cache"], x["anchor_index"], x["partner_index"], factors.product_weight,
        factors.anchor_weight, factors.partner_weight, factors.first_bias, position=t)
    _close(updated, want_u, low)
    _close(updated, ref["hidden_updated"], low)
    _close(mg[:, t], want_cache[:, t], low)
    _close(mg[:, t], ref["expanded_row"], low)
    rest = mg.float().cpu()
    rest[:, t] = 0
    assert torch.equal(rest, mutable.float())          # only the current row is written
    assert_status_clear()


@pytest.mark.parametrize("batch", [1, 8])
@pytest.mark.parametrize("k_out", [5, 8])
def test_reduce_tail_like_the_reference_test(batch, k_out):
    """Context 512, relation_dim 128, hidden 2304, output 576 (the reference's fixture,
    tests/test_relation_reduce_gpu.py:46-160): factorised kernels vs the unfactorised layer."""
    from relation_lm.kernels.relation_reduce import (factor_relation_first_layer,
                                                     relation_hidden_cache_update,
                                                     relation_hidden_cached, relation_norm_reduce)

    g = torch.Generator().manual_seed(20260818 + batch)
    T, R, H, D = 512, 128, 2304, 576
    operand = torch.randn(batch, T, R, generator=g)
    w1, b1 = torch.randn(H, 4 * R, generator=g) * 0.02, torch.randn(H, generator=g) * 0.01
    anchor_index = torch.randint(0, T, (batch,), generator=g, dtype=torch.int32)
    partner_index = torch.randint(0, T, (batch, k_out), generator=g, dtype=torch.int32)
    anchor_index[0] = T - 1
    partner_index[:, 0] = T - 1
    rows = torch.arange(batch)
    a = operand[rows, anchor_index.long()][:, None].expand(-1, k_out, -1)
    p = operand[rows[:, None], partner_index.long()]
    reference_hidden = F.gelu(F.linear(torch.cat((a, p, a * p, a - p), -1).double(), w1.double(), b1.double())).float()
    factors = factor_relation_first_layer(w1.cuda(), b1.cuda(), R)
    expanded = F.linear(operand.cuda(), factors.expanded_weight, factors.expanded_bias)
    hidden = relation_hidden_cached(expanded, operand.cuda(), anchor_index.cuda(),
                                    partner_index.cuda(), factors.product_weight)
    assert torch.allclose(hidden.cpu(), reference_hidden, atol=2e-4, rtol=2e-5)
    mutable = expanded.clone()
    mutable[:, T - 1].zero_()
    updated = relation_hidden_cache_update(
        mutable, operand.cuda(), anchor_index.cuda(), partner_index.cuda(), factors.anchor_weight,
        factors.partner_weight, factors.product_weight, factors.first_bias, position_tensor(T - 1))
    assert torch.allclose(updated.cpu(), reference_hidden, atol=2e-4, rtol=2e-5)
    assert torch.allclose(mutable[:, T - 1], expanded[:, T - 1], atol=2e-4, rtol=2e-5)

    w2, b2 = torch.randn(D, H, generator=g) * 0.02, torch.randn(D, generator=g) * 0.01
    gamma, beta = torch.randn(D, generator=g) * 0.05 + 1.0, torch.randn(D, generator=g) * 0.01
    raw = F.linear(hidden.cpu(), w2, b2)
    scores = torch.randn(batch, k_out, generator=g)
    scores[:, -1] = -torch.inf
    context = relation_norm_reduce(raw.cuda(), scores.cuda(), gamma.cuda(), beta.cuda(),
                                   position_tensor(T - 1), 1e-5)
    want = oracle.relation_norm_reduce(raw, scores, gamma, beta, T - 1, 1e-5)
    assert torch.allclose(context.cpu(), want, atol=FP32_ATOL, rtol=1e-5)
    assert_status_clear()


@pytest.mark.parametrize("name", _names("norm_reduce"))
def test_norm_reduce_matches_golden_and_oracle(golden, name):
    from relation_lm.kernels.relation_reduce import relation_norm_reduce

    entry = golden[name]
    case = entry["case"]
    x = cases.make_inputs(case)
    xg = to_cuda(x)
    for t, ref in entry["outputs"].items():
        got = relation_norm_reduce(xg["raw"], xg["scores"], xg["norm_weight"], xg["norm_bias"],
                                   position_tensor(t), case["eps"])
        want = oracle.relation_norm_reduce(x["raw"], x["scores"], x["norm_weight"], x["norm_bias"],
                                           t, case["eps"])
        assert torch.allclose(got.cpu(), want, atol=FP32_ATOL, rtol=1e-5), (name, t)
        assert torch.allclose(got.cpu(), ref, atol=FP32_ATOL, rtol=1e-5), (name, t)
    assert_status_clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_reduce_tail_low_precision_inputs(dtype):
    """bf16 / fp16 caches and weights at the 512-wide decode shape (hidden 2048), sentinel
    (negative) partner indices included: within 1e-2 relative of the oracle."""
    from relation_lm.kernels.relation_reduce import (factor_relation_first_layer,
                                                     relation_hidden_cached, relation_norm_reduce)

    g = torch.Generator().manual_seed(5150)
    B, T, R, H, D, K = 8, 512, 128, 2048, 512, 8
    operand = torch.randn(B, T, R, generator=g).to(dtype)
    w1, b1 = (torch.randn(H, 4 * R, generator=g) * 0.02).to(dtype), (torch.randn(H, generator=g) * 0.01).to(dtype)
    factors = factor_relation_first_layer(w1, b1, R)
    expanded = F.linear(operand.float(), factors.expanded_weight.float(), factors.expanded_bias.float()).to(dtype)
    anchor_index = torch.randint(0, T, (B,), generator=g, dtype=torch.int32)
    partner_index = torch.randint(0, T, (B, K), generator=g, dtype=torch.int32)
    partner_index[:, -1] = -26          # the empty-slot sentinel must not fault
    hidden = relation_hidden_cached(expanded.cuda(), operand.cuda(), anchor_index.cuda(),
                                    partner_index.cuda(), factors.product_weight.cuda())
    want, _ = oracle.relation_hidden(expanded, operand, anchor_index, partner_index, factors.product_weight)
    assert_rel_close(hidden, want, 1e-2)
    raw = (torch.randn(B, K, D, generator=g)).to(dtype)
    scores = torch.randn(B, K, generator=g)
    scores[:, -1] = -torch.inf
    gamma, beta = torch.ones(D).to(dtype), torch.zeros(D).to(dtype)
    got = relation_norm_reduce(raw.cuda(), scores.cuda(), gamma.cuda(), beta.cuda(), position_tensor(300), 1e-5)
    want = oracle.relation_norm_reduce(raw, scores, gamma, beta, 300, 1e-5)
    assert_rel_close(got, want, 1e-2)
    assert_status_clear()


def test_per_row_forms_match_the_oracle():
    """Prefill forms: rows carry their own sequence index / position (long-context shape:
    block 64 is irrelevant here; d_model 512, hidden 2048, bf16 caches)."""
    from relation_lm.kernels.relation_reduce import (relation_hidden_cached_rows,
                                                     relation_norm_reduce_rows)

    g = torch.Generator().manual_seed(6060)
    B, T, R, H, D, K, N = 3, 256, 128, 2048, 512, 8, 200
    dtype = torch.bfloat16
    operand = torch.randn(B, T, R, generator=g).to(dtype)
    expanded = (torch.randn(B, T, 2 * H, generator=g) * 0.3).to(dtype)
    wm = (torch.randn(H, R, generator=g) * 0.02).to(dtype)
    row_batch = torch.randint(0, B, (N,), generator=g, dtype=torch.int32)
    row_pos = torch.randint(0, T, (N,), generator=g, dtype=torch.int32)
    anchor = (torch.rand(N, generator=g) * (row_pos + 1)).to(torch.int32)
    partner = (torch.rand(N, K, generator=g) * (row_pos[:, None] + 1)).to(torch.int32)
    hidden = relation_hidden_cached_rows(expanded.cuda(), operand.cuda(), anchor.cuda(), partner.cuda(),
                                         wm.cuda(), row_batch.cuda())
    want, _ = oracle.relation_hidden(expanded, operand, anchor, partner, wm, row_batch=row_batch,
                                     row_pos=row_pos)
    assert_rel_close(hidden, want, 1e-2)
    raw = torch.randn(N, K, D, generator=g)
    scores = torch.randn(N, K, generator=g)
    scores[::3, -2:] = -torch.inf
    gamma, beta = torch.rand(D, generator=g) + 0.5, torch.randn(D, generator=g) * 0.1
    ctx = relation_norm_reduce_rows(raw.cuda(), scores.cuda(), gamma.cuda(), beta.cuda(), row_pos.cuda(), 1e-5)
    want_ctx = oracle.relation_norm_reduce(raw, scores, gamma, beta, 0, 1e-5, row_pos=row_pos)
    assert torch.allclose(ctx.cpu(), want_ctx, atol=FP32_ATOL, rtol=1e-5)
    assert_status_clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,K,D", [(8, 8, 512), (5, 5, 768), (40, 8, 1024), (3, 4, 256)])
def test_norm_reduce_residual_with_next_layer_norm(B, K, D, dtype):
    """Residual update and the LayerNorm of the updated rows (the next projection's input) in
    the norm-reduce launch: residual within fp32 tolerance, normalised rows within one 16-bit ulp."""
    from relation_lm.kernels.relation_reduce import relation_norm_reduce_residual_norm

    g = torch.Generator().manual_seed(7700 + B + D)
    raw = torch.randn(B, K, D, generator=g).to(dtype)
    scores = torch.randn(B, K, generator=g)
    scores[::2, -1] = -torch.inf
    gamma, beta = torch.rand(D, generator=g) + 0.5, torch.randn(D, generator=g) * 0.1
    next_w, next_b = torch.rand(D, generator=g) + 0.5, torch.randn(D, generator=g) * 0.1
    hidden = torch.randn(B, D, generator=g) * 2
    mix = torch.tensor(0.37)
    t = 300
    got_hidden = hidden.cuda().clone()
    normalized = torch.empty(B, D, device="cuda", dtype=dtype)
    relation_norm_reduce_residual_norm(raw.cuda(), scores.cuda(), gamma.cuda(), beta.cuda(), position_tensor(t),
                                       1e-5, got_hidden, mix.cuda(), next_w.cuda(), next_b.cuda(), 1e-5,
                                       normalized)
    context = oracle.relation_norm_reduce(raw, scores, gamma, beta, t, 1e-5)
    want_hidden = hidden + mix * context
    assert torch.allclose(got_hidden.cpu(), want_hidden, atol=FP32_ATOL, rtol=1e-5)
    want_norm = F.layer_norm(want_hidden, (D,), next_w, next_b, 1e-5)
    assert_rel_close(normalized, want_norm, 1e-2)
    assert_status_clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,K,D,N", [(8, 8, 512, 256), (1, 8, 512, 256), (5, 5, 768, 192), (3, 4, 1024, 32),
                                     (32, 8, 256, 128)])
def test_norm_reduce_with_the_next_query_projection(B, K, D, N, dtype):
    """Norm-reduce + residual + next LayerNorm + next query projection in one launch (a cluster
    of N / 32 CTAs per row): residual and normalised rows identical to the launch without the
    projection, projected rows equal to the fp32 product of the 16-bit normalised rows."""
    from relation_lm.kernels.relation_reduce import (relation_norm_reduce_residual_norm,
                                                     relation_norm_reduce_residual_norm_project)

    g = torch.Generator().manual_seed(7900 + B + D + N)
    raw = torch.randn(B, K, D, generator=g).to(dtype).cuda()
    scores = torch.randn(B, K, generator=g)
    scores[::2, -1] = -torch.inf
    scores = scores.cuda()
    gamma, beta = (torch.rand(D, generator=g) + 0.5).cuda(), (torch.randn(D, generator=g) * 0.1).cuda()
    next_w, next_b = (torch.rand(D, generator=g) + 0.5).cuda(), (torch.randn(D, generator=g) * 0.1).cuda()
    hidden = (torch.randn(B, D, generator=g) * 2).cuda()
    weight = (torch.randn(N, D, generator=g) * D ** -0.5).to(dtype).cuda()
    mix = torch.tensor(0.37).cuda()
    pos = position_tensor(300)
    plain_hidden, plain_norm = hidden.clone(), torch.empty(B, D, device="cuda", dtype=dtype)
    relation_norm_reduce_residual_norm(raw, scores, gamma, beta, pos, 1e-5, plain_hidden, mix, next_w, next_b,
                                       1e-5, plain_norm)
    got_hidden, got_norm = hidden.clone(), torch.empty(B, D, device="cuda", dtype=dtype)
    projected = torch.full((B, N), float("nan"), device="cuda", dtype=dtype)
    relation_norm_reduce_residual_norm_project(raw, scores, gamma, beta, pos, 1e-5, got_hidden, mix, next_w,
                                               next_b, 1e-5, got_norm, weight, projected)
    assert torch.equal(got_hidden, plain_hidden)
    assert torch.equal(got_norm, plain_norm)
    want = got_norm.double() @ weight.double().T
    assert_rel_close(projected, want.float(), 1e-2)
    assert_status_clear()


@pytest.mark.parametrize("splits", [2, 4])
def test_split_k_second_layer_feeds_norm_reduce(splits):
    """Second relation-MLP layer as a split-K tensor-core GEMM whose fp32 slices (and bias) are
    summed inside norm-reduce: residual and next-layer LayerNorm against the fp32 reference."""
    from relation_lm.kernels.packed_projection import packed_projection_slices
    from relation_lm.kernels.relation_reduce import relation_norm_reduce_residual_norm_slices

    g = torch.Generator().manual_seed(7900 + splits)
    B, K, H, D, t = 8, 8, 2048, 512, 300
    act = torch.randn(B, K, H, generator=g).bfloat16()
    w2 = (torch.randn(D, H, generator=g) * 0.03).bfloat16()
    b2 = torch.randn(D, generator=g) * 0.1
    scores = torch.randn(B, K, generator=g)
    scores[1::3, -2:] = -torch.inf
    gamma, beta = torch.rand(D, generator=g) + 0.5, torch.randn(D, generator=g) * 0.1
    next_w, next_b = torch.rand(D, generator=g) + 0.5, torch.randn(D, generator=g) * 0.1
    hidden = torch.randn(B, D, generator=g)
    mix = torch.tensor(0.61)
    slices = packed_projection_slices(act.cuda().view(B * K, H), w2.cuda(), splits)
    assert slices.shape == (splits, B * K, D) and slices.dtype == torch.float32
    raw = oracle.linear(act.view(B * K, H), w2).view(B, K, D) + b2
    assert torch.allclose(slices.sum(0).cpu().view(B, K, D) + b2, raw, atol=2e-3, rtol=1e-3)
    got_hidden = hidden.cuda().clone()
    normalized = torch.empty(B, D, device="cuda", dtype=torch.bfloat16)
    relation_norm_reduce_residual_norm_slices(slices.view(splits, B, K, D), b2.cuda(), scores.cuda(), gamma.cuda(),
                                              beta.cuda(), position_tensor(t), 1e-5, got_hidden, mix.cuda(),
                                              next_w.cuda(), next_b.cuda(), 1e-5, normalized)
    want_hidden = hidden + mix * oracle.relation_norm_reduce(raw, scores, gamma, beta, t, 1e-5)
    assert torch.allclose(got_hidden.cpu(), want_hidden, atol=2e-3, rtol=1e-3), (got_hidden.cpu() - want_hidden).abs().max()
    want_norm = F.layer_norm(want_hidden, (D,), next_w, next_b, 1e-5)
    assert_rel_close(normalized, want_norm, 1e-2)
    assert_status_clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("N,K,D", [(4096, 8, 512), (2500, 5, 768), (3001, 4, 256), (2048, 8, 1024), (2050, 1, 512)])
def test_many_rows_norm_reduce_matches_the_oracle(N, K, D, dtype):
    """Launches of thousands of rows take the warp-per-row kernel (all of a row's partner rows in flight at
    once, no shared memory): against the oracle on the same 16-bit rows (fp32 tolerance), with empty slots,
    rows without any partner and early positions that limit the active slots; a launch just below the
    threshold (the CTA-per-row kernel) agrees within the same tolerance."""
    from relation_lm.kernels.relation_reduce import relation_norm_reduce_rows

    g = torch.Generator().manual_seed(6500 + N + K + D)
    raw = torch.randn(N, K, D, generator=g).to(dtype)
    scores = torch.randn(N, K, generator=g)
    scores[::3, -1] = -torch.inf
    scores[5::17] = -torch.inf                      # rows without any active partner: context 0
    gamma, beta = torch.rand(D, generator=g) + 0.5, torch.randn(D, generator=g) * 0.1
    row_pos = torch.randint(0, 4096, (N,), generator=g, dtype=torch.int32)
    row_pos[::5] = torch.randint(0, 6, ((N + 4) // 5,), generator=g, dtype=torch.int32)   # k_limit below K
    got = relation_norm_reduce_rows(raw.cuda(), scores.cuda(), gamma.cuda(), beta.cuda(), row_pos.cuda(), 1e-5)
    want = oracle.relation_norm_reduce(raw.float(), scores, gamma, beta, 0, 1e-5, row_pos=row_pos)
    assert torch.allclose(got.cpu(), want, atol=FP32_ATOL, rtol=1e-5)
    assert bool((got[5::17] == 0).all())
    few = relation_norm_reduce_rows(raw[:1000].cuda(), scores[:1000].cuda(), gamma.cuda(), beta.cuda(),
                                    row_pos[:1000].cuda(), 1e-5)
    assert torch.allclose(few, got[:1000], atol=FP32_ATOL, rtol=1e-5)
    assert_status_clear()
