"""GPU parity of the selectors: CUDA kernels vs the CPU oracle (bit-exact indices AND scores)
and vs the reference kernels' golden outputs (indices exact, scores within 4e-6)."""
from __future__ import annotations

import pytest
import torch

import cases
import oracle
from gpu_util import (SELECT_KEYS, assert_scores_equal, assert_status_clear, position_tensor, select_args,
                      to_cuda)

pytestmark = pytest.mark.gpu


def _select_cases():
    return [n for n, c in cases.all_cases().items() if c["kind"] == "select"]


def _policy(case):
    return case["local_window"], case["top_blocks"], case["k_out"], case["strict_valid"]


@pytest.mark.parametrize("name", _select_cases())
def test_packed_select_matches_golden_and_oracle(golden, name):
    from relation_lm.kernels.relation_select import relation_select_packed

    entry = golden[name]
    case = entry["case"]
    x = cases.make_inputs(case)
    assert cases.checksum(x) == entry["input_sha256"]
    xg = to_cuda(x)
    for t, ref in entry["outputs"].items():
        a, a_s, p, p_s = relation_select_packed(*select_args(xg), position_tensor(t), *_policy(case))
        oa, oa_s, op, op_s, _ = oracle.relation_select(*select_args(x), t, *_policy(case))
        assert torch.equal(a.cpu(), oa) and torch.equal(p.cpu(), op), (name, t)
        assert_scores_equal(a_s, oa_s)
        assert_scores_equal(p_s, op_s)
        assert torch.equal(a.cpu(), ref["anchor"]) and torch.equal(p.cpu(), ref["partner"]), (name, t)
        finite = torch.isfinite(ref["partner_score"])
        assert torch.allclose(p_s.cpu()[finite], ref["partner_score"][finite], atol=4e-6, rtol=1e-6)
        assert torch.allclose(a_s.cpu(), ref["anchor_score"], atol=4e-6, rtol=1e-6)
    assert_status_clear()


@pytest.mark.parametrize("name", ["select_reftest", "select_c128_strict", "select_top4_k5",
                                  "select_bf16", "select_ties_compat"])
def test_two_operator_path_equals_packed(golden, name):
    """The reference's own GPU test (tests/test_relation_select_gpu.py:33-87): packed == two-op."""
    from relation_lm.kernels.relation_select import relation_select_packed
    from relation_lm.kernels.triton_select import anchor_select, partner_topk

    case = golden[name]["case"]
    xg = to_cuda(cases.make_inputs(case))
    L, top, k, strict = _policy(case)
    batch = torch.arange(case["batch"], device="cuda")
    for t in case["positions"]:
        pos = position_tensor(t)
        anchor, anchor_score = anchor_select(*select_args(xg)[:7], pos, L, top, strict)
        contribution = xg["partner_anchor_cache"][batch, anchor.long()].float()
        base = xg["partner_base"].float()
        partner, partner_score = partner_topk(
            (base[:, :64] + contribution[:, :64]).contiguous(), xg["partner_keys"],
            (base[:, 64:] + contribution[:, 64:]).contiguous(), xg["partner_mean"],
            xg["partner_std"], xg["partner_gamma"], xg["partner_bias"], pos, anchor, L, top, k, strict)
        fused = relation_select_packed(*select_args(xg), pos, L, top, k, strict)
        assert torch.equal(anchor, fused[0]) and torch.equal(partner, fused[2])
        assert torch.equal(anchor_score, fused[1]) and torch.equal(partner_score, fused[3])
    assert_status_clear()


SHAPES = [
    # batch, context, blocks, window, top, k, dtype
    (8, 512, 16, 64, 2, 8, "bf16"),      # ctx-512 decode, block 32
    (8, 512, 64, 16, 2, 8, "fp32"),      # the reference's published policy (block 8, window 16)
    (16, 2048, 32, 128, 2, 8, "bf16"),   # 12-layer decode shape, block 64
    (4, 4096, 64, 128, 4, 8, "bf16"),    # long-context shape, 4 remote blocks
    (4, 2048, 64, 64, 3, 4, "fp16"),     # multi-anchor shape: 3 remote blocks, 4 partners
    (3, 4096, 64, 128, 4, 8, "fp32"),    # largest shared-memory footprint
]


@pytest.mark.parametrize("strict", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_packed_select_matches_oracle_at_baseline_shapes(shape, strict):
    from relation_lm.kernels.relation_select import relation_select_packed

    B, T, NB, L, top, K, dtype = shape
    case = {"kind": "select", "seed": 7000 + T + NB + top, "batch": B, "context": T, "blocks": NB,
            "local_window": L, "top_blocks": top, "k_out": K, "strict_valid": strict, "dtype": dtype}
    x = cases.make_inputs(case)
    xg = to_cuda(x)
    bs = T // NB
    for t in sorted({0, 1, L - 2, L - 1, L, bs - 1, bs, 2 * bs - 1, L + bs, T // 2 + 3, T - 1}):
        a, a_s, p, p_s = relation_select_packed(*select_args(xg), position_tensor(t), L, top, K, strict)
        oa, oa_s, op, op_s, _ = oracle.relation_select(*select_args(x), t, L, top, K, strict)
        assert torch.equal(a.cpu(), oa), (shape, t)
        assert torch.equal(p.cpu(), op), (shape, t)
        assert_scores_equal(a_s, oa_s)
        assert_scores_equal(p_s, op_s)
    assert_status_clear()


@pytest.mark.parametrize("shape", [
    (4, 2048, 32, 128, 2, 8, "bf16"),     # 256 candidates: register tournament of eight per lane, head-per-lane blocks
    (2, 4096, 64, 128, 4, 8, "bf16"),     # 384 candidates: threshold filter, two block scores per lane when picking
    (3, 512, 16, 64, 2, 32, "fp32"),      # 128 candidates, 32 partner slots
    (2, 256, 8, 8, 1, 16, "bf16"),        # more partner slots (16) than some positions have candidates
])
def test_tie_heavy_inputs_keep_the_lowest_position(shape):
    """Quantised inputs (every dot product exact, neighbouring blocks' statistics and every third
    key row duplicated): equal scores everywhere, so block picking, the anchor arg-max and the
    top-K must all break ties the way the oracle does (lowest block, lowest position)."""
    from relation_lm.kernels.relation_select import relation_select_packed

    B, T, NB, L, top, K, dtype = shape
    case = {"kind": "select", "seed": 7300 + T + K, "batch": B, "context": T, "blocks": NB, "local_window": L,
            "top_blocks": top, "k_out": K, "strict_valid": False, "dtype": dtype, "quantize": True}
    x = cases.make_inputs(case)
    xg = to_cuda(x)
    bs = T // NB
    for t in sorted({0, 3, L - 1, L, 2 * bs + 1, T // 2, T - 1}):
        a, a_s, p, p_s = relation_select_packed(*select_args(xg), position_tensor(t), L, top, K, False)
        oa, oa_s, op, op_s, _ = oracle.relation_select(*select_args(x), t, L, top, K, False)
        assert torch.equal(a.cpu(), oa), (shape, t)
        assert torch.equal(p.cpu(), op), (shape, t)
        assert_scores_equal(a_s, oa_s)
        assert_scores_equal(p_s, op_s)
    assert_status_clear()


@pytest.mark.parametrize("strict", [False, True])
def test_rows_form_equals_decode_form_at_every_position(strict):
    """Per-row positions: every t of a context-128 sequence in one launch (fp32, block 16)."""
    from relation_lm.kernels.relation_select import relation_select_packed_rows

    B, T, NB, L, top, K = 2, 128, 8, 32, 2, 8
    case = {"kind": "select", "seed": 7100, "batch": B, "rows": B * T, "context": T, "blocks": NB,
            "local_window": L, "top_blocks": top, "k_out": K, "strict_valid": strict}
    x = cases.make_inputs(case)
    xg = to_cuda(x)
    row_batch = torch.arange(B, dtype=torch.int32).repeat_interleave(T)
    row_pos = torch.arange(T, dtype=torch.int32).repeat(B)
    got = relation_select_packed_rows(*select_args(xg), row_batch.cuda(), row_pos.cuda(), L, top, K, strict)
    want = oracle.relation_select(*select_args(x), 0, L, top, K, strict, row_batch=row_batch, row_pos=row_pos)
    assert torch.equal(got[0].cpu(), want[0]) and torch.equal(got[2].cpu(), want[2])
    assert_scores_equal(got[1], want[1])
    assert_scores_equal(got[3], want[3])
    # size-independent properties: causal, anchor excluded, partners distinct where valid
    anchor, partner, score = got[0].cpu(), got[2].cpu(), got[3].cpu()
    assert torch.all(anchor <= row_pos) and torch.all(anchor >= 0)
    valid = torch.isfinite(score)
    assert torch.all((partner <= row_pos[:, None]) | ~valid)
    assert torch.all((partner != anchor[:, None]) | ~valid)
    assert torch.all(partner[~valid] == (row_pos[:, None].expand_as(partner)[~valid] - L + 1))
    assert torch.all(score[:, :-1] >= score[:, 1:])
    for r in range(0, B * T, 17):
        live = partner[r][valid[r]]
        assert live.unique().numel() == live.numel()
    assert_status_clear()


@pytest.mark.parametrize("dtype", ["bf16", "fp32"])
def test_many_row_launch_equals_short_launches_and_oracle(dtype):
    """A launch of more rows than the SMs hold at once takes the build that stages the partner
    stream in the anchor stream's buffers; it must give what launches of 128 rows (the
    latency-oriented build) give, and what the oracle gives on a sample of the rows."""
    from relation_lm.kernels.relation_select import relation_select_packed_rows

    B, T, NB, L, top, K = 4, 512, 16, 64, 2, 8
    case = {"kind": "select", "seed": 7150, "batch": B, "rows": B * T, "context": T, "blocks": NB,
            "local_window": L, "top_blocks": top, "k_out": K, "strict_valid": False, "dtype": dtype}
    x = cases.make_inputs(case)
    xg = to_cuda(x)
    row_batch = torch.arange(B, dtype=torch.int32).repeat_interleave(T)
    row_pos = torch.arange(T, dtype=torch.int32).repeat(B)
    args = select_args(xg)
    whole = relation_select_packed_rows(*args, row_batch.cuda(), row_pos.cuda(), L, top, K, False)
    rows = B * T
    for r0 in range(0, rows, 128):
        sl = slice(r0, r0 + 128)
        part_args = list(args)
        for i in (0, 2, 7):       # anchor query, anchor router query, partner base: one row per query
            part_args[i] = args[i][sl].contiguous()
        part = relation_select_packed_rows(*part_args, row_batch[sl].cuda(), row_pos[sl].cuda(), L, top, K, False)
        for w, q in zip(whole, part):
            assert torch.equal(w[sl], q), r0
    sample = torch.arange(5, rows, 37)
    cpu_args = list(select_args(x))
    for i in (0, 2, 7):
        cpu_args[i] = cpu_args[i][sample].contiguous()
    want = oracle.relation_select(*cpu_args, 0, L, top, K, False, row_batch=row_batch[sample],
                                  row_pos=row_pos[sample])
    assert torch.equal(whole[0].cpu()[sample], want[0]) and torch.equal(whole[2].cpu()[sample], want[2])
    assert_scores_equal(whole[1][sample.cuda()], want[1])
    assert_scores_equal(whole[3][sample.cuda()], want[3])
    assert_status_clear()


def test_decode_form_of_many_sequences_equals_the_rows_form():
    """600 bf16 sequences in the decode form (one launch: the many-row build of the decode-form
    kernel) against the per-row form of the same queries in launches of 150 rows."""
    from relation_lm.kernels.relation_select import relation_select_packed, relation_select_packed_rows

    B, T, NB, L, top, K, t = 600, 128, 8, 32, 2, 8, 101
    case = {"kind": "select", "seed": 7160, "batch": B, "context": T, "blocks": NB, "local_window": L,
            "top_blocks": top, "k_out": K, "strict_valid": False, "dtype": "bf16"}
    xg = to_cuda(cases.make_inputs(case))
    args = select_args(xg)
    whole = relation_select_packed(*args, position_tensor(t), L, top, K, False)
    for r0 in range(0, B, 150):
        sl = slice(r0, r0 + 150)
        part_args = list(args)
        for i in (0, 2, 7):       # anchor query, anchor router query, partner base: one row per query
            part_args[i] = args[i][sl].contiguous()
        rows = torch.arange(r0, r0 + 150, dtype=torch.int32, device="cuda")
        part = relation_select_packed_rows(*part_args, rows, torch.full_like(rows, t), L, top, K, False)
        for w, q in zip(whole, part):
            assert torch.equal(w[sl], q), r0
    assert_status_clear()


def test_full_window_selection_is_dense_argmax_and_topk():
    """With the window covering the whole history and no remote blocks the routed selection
    must equal dense argmax / top-k of causal scores (the reference's dense models,
    src/relation_lm/models/relation_lm.py:158-167)."""
    from relation_lm.kernels.relation_select import relation_select_packed_rows

    B, T, NB, K = 2, 64, 8, 8
    case = {"kind": "select", "seed": 7200, "batch": B, "rows": B * T, "context": T, "blocks": NB,
            "local_window": T, "top_blocks": 0, "k_out": K, "strict_valid": False}
    x = cases.make_inputs(case)
    xg = to_cuda(x)
    row_batch = torch.arange(B, dtype=torch.int32).repeat_interleave(T)
    row_pos = torch.arange(T, dtype=torch.int32).repeat(B)
    a, _, p, p_s = [v.cpu() for v in relation_select_packed_rows(
        *select_args(xg), row_batch.cuda(), row_pos.cuda(), T, 0, K, False)]
    future = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    aq = x["anchor_query"].view(B, T, 64)
    dense = (torch.einsum("btd,bsd->bts", aq.double(), x["anchor_keys"].double()) * 0.125)
    dense = dense.masked_fill(future[None], -torch.inf)
    assert torch.equal(a.view(B, T).long(), dense.argmax(-1))
    v = x["partner_base"].view(B, T, 128) + x["partner_anchor_cache"][
        torch.arange(B)[:, None], a.view(B, T).long()]
    pd = torch.einsum("btd,bsd->bts", v[..., :64].double(), x["partner_keys"].double()) * 0.125
    pd = pd.masked_fill(future[None], -torch.inf).scatter(2, a.view(B, T, 1).long(), -torch.inf)
    top_scores, top_index = pd.topk(K, dim=-1)
    finite = torch.isfinite(top_scores)
    assert torch.equal(p.view(B, T, K).long()[finite], top_index[finite])
    assert torch.equal(torch.isfinite(p_s.view(B, T, K)), finite)


def test_argument_validation():
    from relation_lm.kernels.relation_select import relation_select_packed

    case = cases.all_cases()["select_top1_k4"]
    xg = to_cuda(cases.make_inputs(case))
    args = select_args(xg)
    pos = position_tensor(5)
    with pytest.raises(ValueError):       # position on the host
        relation_select_packed(*args, torch.tensor(5), 16, 1, 4, False)
    with pytest.raises(ValueError):       # mixed cache dtypes
        bad = list(args)
        bad[1] = bad[1].half()
        relation_select_packed(*bad, pos, 16, 1, 4, False)
    with pytest.raises(ValueError):       # non-contiguous keys
        bad = list(args)
        bad[1] = bad[1].transpose(0, 1).contiguous().transpose(0, 1)
        relation_select_packed(*bad, pos, 16, 1, 4, False)
    with pytest.raises(ValueError):       # working set beyond shared memory
        relation_select_packed(*args, pos, 16, 1000, 4, False)
    # a position outside the cache is reported through the status word, never a fault
    from relation_lm.kernels import _abi
    relation_select_packed(*args, position_tensor(case["context"] + 3), 16, 1, 4, False)
    assert _abi.read_status() == 2
    assert _abi.read_status() == 0


def test_a_bounded_wait_that_expires_reports_timeout_and_leaves_the_context_usable():
    """The expiry path of the kernels' bulk-copy waits, exercised without faulting anything: a
    wait of a few thousand cycles on a barrier nobody completes sets RLM_DEV_TIMEOUT in the
    status word, the kernel returns, and the next launch works."""
    from relation_lm.kernels import _abi

    device = torch.device("cuda", torch.cuda.current_device())
    assert _abi.read_status() == 0
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    _abi.check(_abi.LIB.rlm_selftest_bounded_wait(_abi.ptr(_abi.status_tensor(device)), 4000, _abi.ptr(waited),
                                                  _abi.stream_ptr(device)))
    assert _abi.read_status() == 1                    # RLM_DEV_TIMEOUT, cleared by the read
    assert 4000 < int(waited.item()) < 4_000_000
    with pytest.raises(ValueError):
        _abi.check(_abi.LIB.rlm_selftest_bounded_wait(_abi.ptr(_abi.status_tensor(device)), 1 << 40, None,
                                                      _abi.stream_ptr(device)))
    # the context is intact: an ordinary selection still runs and matches the oracle
    case = cases.all_cases()["select_c512_compat"]
    x = cases.make_inputs(case)
    from relation_lm.kernels.relation_select import relation_select_packed
    got = relation_select_packed(*select_args(to_cuda(x)), position_tensor(300), 64, 2, 8, False)
    want = oracle.relation_select(*select_args(x), 300, 64, 2, 8, False)
    assert torch.equal(got[0].cpu(), want[0]) and torch.equal(got[2].cpu(), want[2])
    assert_status_clear()


@pytest.mark.parametrize("dtype", ["bf16", "fp32"])
@pytest.mark.parametrize("context,blocks,local_window,top_blocks,k_out,strict,query_length", [
    (256, 8, 64, 2, 8, False, 256),       # block 32, window 64
    (256, 8, 64, 2, 8, True, 256),
    (128, 8, 32, 0, 5, False, 128),       # no remote blocks
    (512, 8, 128, 4, 8, False, 500),      # block 64, window 128, 384 candidates; ragged last tile
    (192, 24, 16, 3, 4, True, 70),        # block 8, more than 16 blocks, queries for a prefix only
    (4096, 128, 128, 4, 8, True, 700),    # 128 blocks of statistics: the 16-warp tile does not fit, 8 warps serve
])
def test_whole_sequence_selector_equals_the_per_row_selector(context, blocks, local_window, top_blocks, k_out,
                                                             strict, query_length, dtype):
    """Tiles of consecutive positions (shared staging, a query per warp) against the per-row form: all
    four outputs bit for bit at every position of every sequence, and the oracle on a sample."""
    from relation_lm.kernels.relation_select import relation_select_packed_prefill, relation_select_packed_rows

    B = 3
    if dtype == "fp32" and blocks * 4 * 256 + 2 * (local_window + 32) * 256 > 200 * 1024:
        pytest.skip("fp32 statistics and windows of this shape exceed the shared memory (the per-row kernel serves it)")
    case = {"kind": "select", "seed": 8800 + context + top_blocks, "batch": B, "context": context, "blocks": blocks,
            "rows": B * query_length, "local_window": local_window, "top_blocks": top_blocks, "k_out": k_out,
            "strict_valid": strict, "dtype": dtype, "quantize": dtype == "fp32"}
    x = cases.make_inputs(case)
    xg = to_cuda(x)
    row_batch = torch.arange(B, dtype=torch.int32).repeat_interleave(query_length)
    row_pos = torch.arange(query_length, dtype=torch.int32).repeat(B)
    tiled = relation_select_packed_prefill(*select_args(xg), query_length, local_window, top_blocks, k_out, strict)
    rows = relation_select_packed_rows(*select_args(xg), row_batch.cuda(), row_pos.cuda(), local_window, top_blocks,
                                       k_out, strict)
    for mine, theirs in zip(tiled, rows):
        assert torch.equal(mine.view(torch.int32), theirs.view(torch.int32))
    sample = torch.arange(0, B * query_length, 7)
    want = oracle.relation_select(*[x[k][sample] if x[k].size(0) == B * query_length and k in
                                    ("anchor_query", "anchor_router_query", "partner_base") else x[k]
                                    for k in SELECT_KEYS], 0, local_window, top_blocks, k_out, strict,
                                  row_batch=row_batch[sample], row_pos=row_pos[sample])
    assert torch.equal(tiled[0].cpu()[sample], want[0]) and torch.equal(tiled[2].cpu()[sample], want[2])
    assert_scores_equal(tiled[3][sample.cuda()], want[3])
    assert_status_clear()


@pytest.mark.parametrize("B,T,NB,L,top,K", [
    (8, 512, 16, 64, 2, 8),       # the ctx-512 decode configuration: both key caches resident (128 KB)
    (3, 768, 12, 32, 3, 4),       # block 64; the largest context whose caches still fit
    (2, 256, 16, 128, 4, 8),      # window of half the context
])
def test_decode_form_with_resident_caches_equals_the_rows_form_and_oracle(B, T, NB, L, top, K):
    """bf16 decode launches of at most one row per SM stage the sequence's whole key caches up to the
    position instead of window + picked blocks (no second round of copies): same indices and scores,
    bit for bit, as the per-row form (which stages window and blocks) and as the oracle."""
    from relation_lm.kernels.relation_select import relation_select_packed, relation_select_packed_rows

    case = {"kind": "select", "seed": 7300 + T, "batch": B, "context": T, "blocks": NB, "local_window": L,
            "top_blocks": top, "k_out": K, "strict_valid": True, "dtype": "bf16"}
    x = cases.make_inputs(case)
    xg = to_cuda(x)
    rows = torch.arange(B, dtype=torch.int32).cuda()
    bs = T // NB
    for t in sorted({0, 1, L - 1, L, bs - 1, bs, 2 * bs + 1, T // 2, T - 2, T - 1}):
        got = relation_select_packed(*select_args(xg), position_tensor(t), L, top, K, True)
        ref = relation_select_packed_rows(*select_args(xg), rows, torch.full((B,), t, dtype=torch.int32).cuda(),
                                          L, top, K, True)
        for a, b in zip(got, ref):
            assert torch.equal(a.view(torch.int32) if a.dtype == torch.float32 else a,
                               b.view(torch.int32) if b.dtype == torch.float32 else b), t
        oa, oa_s, op, op_s, _ = oracle.relation_select(*select_args(x), t, L, top, K, True)
        assert torch.equal(got[0].cpu(), oa) and torch.equal(got[2].cpu(), op), t
        assert_scores_equal(got[1], oa_s)
        assert_scores_equal(got[3], op_s)
    assert_status_clear()
