"""The CPU oracle against outputs of the reference project's own kernels.

``tests/golden/reference_kernels.pt`` was produced by running the reference's
Triton kernels through Triton's CPU interpreter (tests/golden/make_golden.py).
Indices must match exactly; scores within the tolerance the reference's own
parity run reports between two implementations of the same math (3.8e-6).
"""
from __future__ import annotations

import pytest
import torch

import cases
import oracle

SCORE_ATOL = 4.0e-6


def _case_names(kind):
    return [n for n, c in cases.all_cases().items() if c["kind"] == kind]


def _inputs(golden, name):
    entry = golden[name]
    x = cases.make_inputs(entry["case"])
    assert cases.checksum(x) == entry["input_sha256"], "seeded inputs drifted from the golden run"
    return entry["case"], x, entry["outputs"]


def _close_scores(a, b, atol=SCORE_ATOL):
    finite = torch.isfinite(b)
    assert torch.equal(torch.isfinite(a), finite)
    assert torch.equal(a[~finite], b[~finite])
    assert torch.allclose(a[finite], b[finite], atol=atol, rtol=1e-6)


@pytest.mark.parametrize("name", _case_names("select"))
def test_select_matches_reference_kernels(golden, name):
    case, x, outputs = _inputs(golden, name)
    args = [x[k] for k in ("anchor_query", "anchor_keys", "anchor_router_query", "anchor_mean",
                           "anchor_std", "anchor_gamma", "anchor_bias", "partner_base",
                           "partner_anchor_cache", "partner_keys", "partner_mean", "partner_std",
                           "partner_gamma", "partner_bias")]
    policy = (case["local_window"], case["top_blocks"], case["k_out"], case["strict_valid"])
    for t, ref in outputs.items():
        a, a_s, p, p_s, _ = oracle.relation_select(*args, t, *policy)
        assert torch.equal(a, ref["anchor"]), (name, t)
        assert torch.equal(p, ref["partner"]), (name, t)
        _close_scores(a_s, ref["anchor_score"])
        _close_scores(p_s, ref["partner_score"])
        # the reference's two-operator path must agree with its packed op, and so must ours
        assert torch.equal(ref["two_anchor"], ref["anchor"])
        assert torch.equal(ref["two_partner"], ref["partner"])
        ta, ta_s = oracle.anchor_select(*args[:7], t, policy[0], policy[1], policy[3])
        assert torch.equal(ta, a) and torch.equal(ta_s, a_s)
        rows = torch.arange(a.numel())
        v = x["partner_base"].float() + x["partner_anchor_cache"].float()[rows, a.long()]
        tp, tp_s = oracle.partner_topk(v[:, :64], x["partner_keys"], v[:, 64:], *args[10:14], t,
                                       a, *policy)
        assert torch.equal(tp, p) and torch.equal(tp_s, p_s)


def test_select_sentinel_slots(golden):
    """Fewer than K candidates: score -inf and index t - L + 1, possibly negative."""
    case, x, outputs = _inputs(golden, "select_c128_compat")
    ref = outputs[0]
    assert torch.all(ref["partner"] == 0 - case["local_window"] + 1)
    assert torch.all(torch.isinf(ref["partner_score"]))
    ref5 = outputs[5]
    assert int(torch.isfinite(ref5["partner_score"]).sum()) == 5


@pytest.mark.parametrize("name", _case_names("router"))
def test_router_update_matches_reference_kernel(golden, name):
    case, x, ref = _inputs(golden, name)
    out, state = oracle.router_cache_update(
        x["anchor_raw"], x["partner_raw"], x["anchor_raw_cache"], x["partner_raw_cache"],
        x["anchor_conv_cache"], x["partner_conv_cache"], x["anchor_mean"], x["anchor_std"],
        x["partner_mean"], x["partner_std"], x["anchor_conv_weight"], x["partner_conv_weight"],
        case["position"], case["block_size"])
    t, blk = case["position"], case["position"] // case["block_size"]
    low = case["dtype"] != "fp32"
    atol = 1.0e-2 if low else 1.0e-6
    assert torch.allclose(out, ref["out"], atol=1.0e-6, rtol=1.0e-6)
    for cache in ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache"):
        assert torch.allclose(state[cache][:, t], ref[cache + "_row"].float(), atol=atol, rtol=1e-6)
        rest = state[cache].clone()
        rest[:, t] = x[cache][:, t].float()
        assert torch.equal(rest, x[cache].float())
    for stat in ("anchor_mean", "anchor_std", "partner_mean", "partner_std"):
        assert torch.allclose(state[stat][:, blk], ref[stat + "_blk"].float(), atol=atol, rtol=1e-6)
        rest = state[stat].clone()
        rest[:, blk] = x[stat][:, blk].float()
        assert torch.equal(rest, x[stat].float())


def test_router_sequence_matches_eager_block_router(golden):
    """T incremental updates == the eager router's conv + block statistics + block scores."""
    case, x, ref = _inputs(golden, "router_sequence")
    B, T, bs = case["batch"], case["context"], case["block_size"]
    nb = T // bs
    st = {n: torch.zeros(B, T, 64) for n in ("anchor_raw_cache", "partner_raw_cache",
                                              "anchor_conv_cache", "partner_conv_cache")}
    st.update({n: torch.zeros(B, nb, 4, 16) for n in ("anchor_mean", "anchor_std",
                                                       "partner_mean", "partner_std")})
    for t in range(T):
        _, st = oracle.router_cache_update(
            x["anchor_raw_seq"][:, t], x["partner_raw_seq"][:, t], st["anchor_raw_cache"],
            st["partner_raw_cache"], st["anchor_conv_cache"], st["partner_conv_cache"],
            st["anchor_mean"], st["anchor_std"], st["partner_mean"], st["partner_std"],
            x["anchor_conv_weight"], x["partner_conv_weight"], t, bs)
        if (t + 1) % bs == 0 or t == T - 1:
            # block scores of the query at t against the stats so far (complete blocks only)
            for b in range(B):
                mine = oracle.block_scores(st["anchor_mean"][b], st["anchor_std"][b],
                                           x["router_query_seq"][b, t], x["gamma"], x["bias"],
                                           t, T, 4, False)
                eager = ref["eager_block_scores"][b, t] + torch.log(torch.tensor(4.0))
                finite = torch.isfinite(eager)
                assert torch.equal(torch.isfinite(mine), finite)
                assert torch.allclose(mine[finite], eager[finite], atol=2e-6, rtol=1e-6)
    for mine, theirs in (("anchor_conv_cache", "anchor_conv_cache"), ("anchor_mean", "anchor_mean"),
                         ("anchor_std", "anchor_std"), ("partner_mean", "partner_mean"),
                         ("partner_std", "partner_std"), ("anchor_conv_cache", "eager_conv"),
                         ("anchor_mean", "eager_mean"), ("anchor_std", "eager_std")):
        assert torch.allclose(st[mine], ref[theirs], atol=1.0e-6, rtol=1.0e-5), (mine, theirs)


@pytest.mark.parametrize("name", _case_names("reduce"))
def test_relation_hidden_matches_reference_kernels(golden, name):
    from relation_lm.kernels.relation_reduce import factor_relation_first_layer

    case, x, ref = _inputs(golden, name)
    factors = factor_relation_first_layer(x["first_weight"], x["first_bias"], case["relation_dim"])
    for field, sha in ref["factor_sha256"].items():
        assert cases.checksum({field: getattr(factors, field)}) == sha, field
    expanded = torch.nn.functional.linear(
        x["operand_cache"].float(), factors.expanded_weight.float(),
        factors.expanded_bias.float()).to(x["operand_cache"].dtype)
    low = case["dtype"] != "fp32"
    atol = 2.0e-2 if low else 2.0e-5
    hidden, _ = oracle.relation_hidden(expanded, x["operand_cache"], x["anchor_index"],
                                       x["partner_index"], factors.product_weight)
    assert torch.allclose(hidden, ref["hidden_cached"], atol=atol, rtol=1e-5)
    t = case["position"]
    mutable = expanded.clone()
    mutable[:, t].zero_()
    updated, cache = oracle.relation_hidden(
        mutable, x["operand_cache"], x["anchor_index"], x["partner_index"],
        factors.product_weight, factors.anchor_weight, factors.partner_weight, factors.first_bias,
        position=t)
    assert torch.allclose(updated, ref["hidden_updated"], atol=atol, rtol=1e-5)
    assert torch.allclose(cache[:, t], ref["expanded_row"].float(), atol=atol, rtol=1e-5)
    rest = cache.clone()
    rest[:, t] = 0
    assert torch.equal(rest, mutable.float())


@pytest.mark.parametrize("name", _case_names("norm_reduce"))
def test_norm_reduce_matches_reference_kernel(golden, name):
    case, x, ref = _inputs(golden, name)
    for t, expected in ref.items():
        got = oracle.relation_norm_reduce(x["raw"], x["scores"], x["norm_weight"],
                                          x["norm_bias"], t, case["eps"])
        assert torch.allclose(got, expected, atol=2.0e-5, rtol=1e-5), (name, t)
    if case.get("all_inactive"):
        assert torch.count_nonzero(ref[511][0]) == 0


@pytest.mark.parametrize("name", _case_names("packed"))
def test_packed_projection_matches_reference(golden, name):
    case, x, ref = _inputs(golden, name)
    packed = torch.cat(x["weights"], dim=0)
    assert cases.checksum({"w": packed}) == ref["packed_weight_sha256"]
    got = oracle.linear(x["memory"], packed).split(ref["split_sizes"], dim=-1)
    for mine, theirs in zip(got, ref["parts"], strict=True):
        assert torch.allclose(mine, theirs, atol=2.0e-5, rtol=2.0e-5)


def test_canonical_exp_log_accuracy():
    """The plain-fp32 exp/log used for block scores stay within a few ulp of libm."""
    lib = oracle.lib()
    xs = torch.linspace(-80.0, 80.0, 4001).tolist() + [0.0, -0.0, 1e-8, -1e-8]
    for v in xs:
        got, want = lib.orc_expf(v), float(torch.tensor(v, dtype=torch.float64).exp())
        assert abs(got - want) <= 4e-7 * want, v
    assert lib.orc_expf(0.0) == 1.0 and lib.orc_expf(-100.0) == 0.0
    ys = torch.logspace(-20, 20, 4001, dtype=torch.float64).tolist() + [1.0, 2.0, 1.5, 1.0000001]
    for v in ys:
        vf = float(torch.tensor(v, dtype=torch.float32))
        got, want = lib.orc_logf(vf), float(torch.tensor(vf, dtype=torch.float64).log())
        assert abs(got - want) <= 4e-7 * max(abs(want), 1e-1), v
    assert lib.orc_logf(1.0) == 0.0


def _multi_anchor_rows(ref):
    B, T, h, _ = ref["anchor_q"].shape
    row_batch = torch.arange(B, dtype=torch.int32).repeat_interleave(T)
    row_pos = torch.arange(T, dtype=torch.int32).repeat(B)
    return B, T, h, row_batch, row_pos


def multi_anchor_dense_check(ref, anchor_rows, partner_rows):
    """Full-window routed selection per slot must reproduce the reference's dense multi-anchor
    block: distinct anchors slot by slot, partners with every active anchor barred."""
    B, T, h, row_batch, row_pos = _multi_anchor_rows(ref)
    N, nb, K = B * T, 3, ref["partner_index"].shape[-1]
    stats = torch.zeros(B, nb, 4, 16)
    gamma, bias, rq = torch.zeros(4), torch.zeros(4, 16), torch.zeros(N, 64)
    active = ref["anchor_active"].reshape(N, h)
    anchors = torch.full((N, h), -1, dtype=torch.int32)
    for s in range(h):
        idx, _ = anchor_rows(ref["anchor_q"][:, :, s].reshape(N, 64).contiguous(),
                             ref["anchor_k"][:, :, s].contiguous(), rq, stats, stats, gamma, bias,
                             row_batch, row_pos, anchors.clone(), T, 0, False)
        idx = torch.where(active[:, s], idx, torch.zeros_like(idx))
        assert torch.equal(idx, ref["anchor_index"].reshape(N, h)[:, s]), s
        anchors[:, s] = torch.where(active[:, s], idx, torch.full_like(idx, -1))
    for s in range(h):
        pidx, pscore = partner_rows(ref["partner_q"][:, :, s].reshape(N, 64).contiguous(),
                                    ref["partner_k"][:, :, s].contiguous(), rq, stats, stats, gamma,
                                    bias, row_batch, row_pos, anchors[:, s].contiguous(), anchors, T, 0, K, False)
        want_active = ref["partner_active"].reshape(N, h, K)[:, s] & active[:, s, None]
        got_active = torch.isfinite(pscore) & active[:, s, None]
        assert torch.equal(got_active, want_active), s
        want = ref["partner_index"].reshape(N, h, K)[:, s]
        assert torch.equal(pidx[want_active], want[want_active]), s


def test_multi_anchor_rules_match_the_dense_reference_block(golden):
    ref = golden["multi_anchor_dense"]["outputs"]

    def anchor_rows(aq, ak, rq, mean, std, gamma, bias, rb, rp, excl, L, top, strict):
        return oracle.anchor_select(aq, ak, rq, mean, std, gamma, bias, 0, L, top, strict,
                                    row_batch=rb, row_pos=rp, exclude_index=excl)

    def partner_rows(pq, pk, rq, mean, std, gamma, bias, rb, rp, anchor, excl, L, top, K, strict):
        return oracle.partner_topk(pq, pk, rq, mean, std, gamma, bias, 0, anchor, L, top, K, strict,
                                   row_batch=rb, row_pos=rp, exclude_index=excl)

    multi_anchor_dense_check(ref, anchor_rows, partner_rows)
