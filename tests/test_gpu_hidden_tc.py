"""GPU parity of the tensor-core form of the relation-hidden kernels (launches with at least
256 (row, partner) pairs and 16-bit caches) against the CPU oracle, through the C ABI.
Tolerance: 1e-2 relative / absolute, the 16-bit bound of the path."""
from __future__ import annotations

import pytest
import torch

import oracle
from gpu_util import assert_rel_close, assert_status_clear, position_tensor

pytestmark = pytest.mark.gpu


def _case(seed, B, T, R, H, K, dtype, t):
    g = torch.Generator().manual_seed(seed)
    operand = torch.randn(B, T, R, generator=g).to(dtype)
    expanded = (torch.randn(B, T, 2 * H, generator=g) * 0.3).to(dtype)
    wm, wa, wp = [(torch.randn(H, R, generator=g) * 0.05).to(dtype) for _ in range(3)]
    bias = (torch.randn(H, generator=g) * 0.1).to(dtype)
    anchor = torch.randint(0, t + 1, (B,), generator=g, dtype=torch.int32)
    partner = torch.randint(0, t + 1, (B, K), generator=g, dtype=torch.int32)
    anchor[::3] = t                      # rows whose anchor is the position being written
    partner[1::4, 0] = t                 # rows with a partner at the position being written
    partner[:, -1] = t - 1000            # empty-slot sentinel (negative): clamped, never faults
    return operand, expanded, wm, wa, wp, bias, anchor, partner


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,K,H,R", [(64, 8, 256, 128), (70, 8, 384, 128), (80, 5, 256, 64),
                                     (100, 4, 128, 128), (32, 16, 256, 128)])
def test_update_form_matches_the_oracle(B, K, H, R, dtype):
    """Hidden rows and the freshly written expanded-cache row, ragged last tiles (rows not a
    multiple of 128 / K, K not a divisor of 128) included."""
    from relation_lm.kernels.relation_reduce import relation_hidden_cache_update

    T, t = 96, 77
    operand, expanded, wm, wa, wp, bias, anchor, partner = _case(9000 + B + K, B, T, R, H, K, dtype, t)
    cache = expanded.cuda().clone()
    got = relation_hidden_cache_update(cache, operand.cuda(), anchor.cuda(), partner.cuda(), wa.cuda(),
                                       wp.cuda(), wm.cuda(), bias.cuda(), position_tensor(t))
    want, want_cache = oracle.relation_hidden(expanded, operand, anchor, partner, wm, wa, wp, bias, position=t)
    assert_rel_close(got, want, 1e-2)
    assert_rel_close(cache, want_cache, 1e-2)
    untouched = torch.ones(T, dtype=torch.bool)
    untouched[t] = False
    assert torch.equal(cache.cpu()[:, untouched], expanded[:, untouched])
    assert_status_clear()


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_cached_form_and_low_precision_output(out_dtype):
    from relation_lm.kernels.relation_reduce import relation_hidden_cache_update_out, relation_hidden_cached

    B, T, R, H, K, t = 48, 64, 128, 512, 8, 40
    dtype = torch.bfloat16
    operand, expanded, wm, wa, wp, bias, anchor, partner = _case(9100, B, T, R, H, K, dtype, t)
    want, _ = oracle.relation_hidden(expanded, operand, anchor, partner, wm)
    if out_dtype == torch.float32:
        got = relation_hidden_cached(expanded.cuda(), operand.cuda(), anchor.cuda(), partner.cuda(), wm.cuda())
    else:
        want, _ = oracle.relation_hidden(expanded, operand, anchor, partner, wm, wa, wp, bias, position=t)
        got = torch.empty(B, K, H, device="cuda", dtype=out_dtype)
        relation_hidden_cache_update_out(got, expanded.cuda().clone(), operand.cuda(), anchor.cuda(),
                                         partner.cuda(), wa.cuda(), wp.cuda(), wm.cuda(), bias.cuda(),
                                         position_tensor(t))
    assert_rel_close(got, want, 1e-2)
    assert_status_clear()


def test_same_results_as_the_small_launch_form():
    """The same rows through the tensor-core form (one launch of 64 sequences) and through the
    CUDA-core form (launches of 8 sequences) agree within the 16-bit bound."""
    from relation_lm.kernels.relation_reduce import relation_hidden_cached_rows

    B, T, R, H, K, t = 64, 64, 128, 256, 8, 63
    dtype = torch.bfloat16
    operand, expanded, wm, _, _, _, anchor, partner = _case(9200, B, T, R, H, K, dtype, t)
    ex, op, wm_d = expanded.cuda(), operand.cuda(), wm.cuda()
    rows = torch.arange(B, dtype=torch.int32)
    big = relation_hidden_cached_rows(ex, op, anchor.cuda(), partner.cuda(), wm_d, rows.cuda())
    parts = [relation_hidden_cached_rows(ex, op, anchor[i:i + 8].cuda(), partner[i:i + 8].cuda(), wm_d,
                                         rows[i:i + 8].cuda()) for i in range(0, B, 8)]
    small = torch.cat(parts)
    assert_rel_close(big, small, 1e-2)
    assert_status_clear()


@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16),
                                             (torch.bfloat16, torch.float16)])
@pytest.mark.parametrize("N,K,H,R", [(6000, 8, 512, 128),      # 375 pair tiles, four hidden tiles
                                     (9001, 5, 256, 64),       # ragged last tile, K that does not divide 128
                                     (20000, 4, 384, 128)])    # three hidden tiles (odd count)
def test_many_rows_form_matches_the_oracle_and_the_per_tile_form(N, K, H, R, dtype, out_dtype):
    """Launches of thousands of rows (a CTA per pair tile walking all hidden tiles through a
    two-stage pipeline) against the oracle on sampled rows, and bit for bit against launches small
    enough to take the one-tile-per-CTA kernel (same contraction, same epilogue arithmetic)."""
    from relation_lm.kernels.relation_reduce import relation_hidden_cached_rows_out

    B, T = 6, 160
    g = torch.Generator().manual_seed(9300 + N + K)
    operand = torch.randn(B, T, R, generator=g).to(dtype)
    expanded = (torch.randn(B, T, 2 * H, generator=g) * 0.3).to(dtype)
    wm = (torch.randn(H, R, generator=g) * 0.05).to(dtype)
    rows = torch.randint(0, B, (N,), generator=g, dtype=torch.int32)
    anchor = torch.randint(0, T, (N,), generator=g, dtype=torch.int32)
    partner = torch.randint(0, T, (N, K), generator=g, dtype=torch.int32)
    partner[::7, -1] = -5                 # empty-slot sentinel: clamped, never faults
    ex, op, wm_d = expanded.cuda(), operand.cuda(), wm.cuda()
    an, pa, rw = anchor.cuda(), partner.cuda(), rows.cuda()
    got = torch.full((N, K, H), float("nan"), device="cuda", dtype=out_dtype)
    relation_hidden_cached_rows_out(got, ex, op, an, pa, wm_d, rw)
    assert bool(torch.isfinite(got.float()).all())
    sample = torch.randperm(N, generator=g)[:300]
    for i in sample.tolist():
        want, _ = oracle.relation_hidden(expanded[rows[i]:rows[i] + 1], operand[rows[i]:rows[i] + 1], anchor[i:i + 1],
                                         partner[i:i + 1].clamp(0, T - 1), wm)
        assert_rel_close(got[i:i + 1], want, 1e-2, f"row {i}")
    step = 2048                            # 128 or fewer pair tiles per launch: the per-tile kernel
    for lo in range(0, N, step):
        part = torch.empty((min(step, N - lo), K, H), device="cuda", dtype=out_dtype)
        relation_hidden_cached_rows_out(part, ex, op, an[lo:lo + step], pa[lo:lo + step], wm_d, rw[lo:lo + step])
        assert torch.equal(part, got[lo:lo + step]), lo
    assert_status_clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("layers,B,H,R", [(3, 8, 256, 128), (2, 70, 384, 64), (1, 1, 128, 128)])
def test_stacked_expanded_cache_append(layers, B, H, R, dtype):
    """All layers' expanded rows of one position in one launch equal the per-layer update of
    the oracle; every other row of the cache stays untouched."""
    from relation_lm.kernels.relation_reduce import expanded_cache_append

    T, t = 40, 23
    g = torch.Generator().manual_seed(9300 + layers + B)
    operand = torch.randn(layers, B, T, R, generator=g).to(dtype)
    expanded = (torch.randn(layers, B, T, 2 * H, generator=g) * 0.3).to(dtype)
    wa, wp = [(torch.randn(layers, H, R, generator=g) * 0.05).to(dtype) for _ in range(2)]
    bias = (torch.randn(layers, H, generator=g) * 0.1).to(dtype)
    cache = expanded.cuda().clone()
    expanded_cache_append(cache, operand.cuda(), wa.cuda(), wp.cuda(), bias.cuda(), position_tensor(t))
    got = cache.cpu()
    anchor = torch.zeros(B, dtype=torch.int32)
    partner = torch.zeros(B, 1, dtype=torch.int32)
    for l in range(layers):
        wm = torch.zeros(H, R).to(dtype)
        _, want = oracle.relation_hidden(expanded[l], operand[l], anchor, partner, wm, wa[l], wp[l], bias[l],
                                         position=t)
        assert_rel_close(got[l], want, 1e-2, f"layer {l}")
    untouched = torch.ones(T, dtype=torch.bool)
    untouched[t] = False
    assert torch.equal(got[:, :, untouched], expanded[:, :, untouched])
    # the same rows with the operands read from packed projection rows (layout of sparse_cache_append)
    from relation_lm.kernels.relation_reduce import expanded_cache_append_packed

    width = 384 + R
    packed = torch.randn(B, layers * width, generator=g).to(dtype)
    for l in range(layers):
        packed[:, l * width + 128:l * width + 128 + R] = operand[l, :, t]
    cache2 = expanded.cuda().clone()
    expanded_cache_append_packed(cache2, packed.cuda(), wa.cuda(), wp.cuda(), bias.cuda(), position_tensor(t))
    assert torch.equal(cache2, cache)
    assert_status_clear()
