"""The single-launch relation tail of a layer (gather -> product GEMM -> GELU -> second MLP layer ->
norm-reduce -> residual -> next LayerNorm -> next query projection, hidden states on chip) against
the oracle's unfused composition.  16-bit operands with fp32 accumulation: every output within
1e-2 of its row's largest magnitude; two calls in a row give bit-identical results (the
cross-CTA sums have a fixed order)."""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

import oracle
from gpu_util import assert_rel_close, assert_status_clear, position_tensor

pytestmark = pytest.mark.gpu


def _case(B, K, d, R, T, n_query, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    H = 4 * d
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    x = {
        "operand": rn(B, T, R).to(dtype), "expanded": (rn(B, T, 2 * H) * 0.5).to(dtype),
        "wm": (rn(H, R) * 0.08).to(dtype), "w2": (rn(d, H) * 0.03).to(dtype), "b2": (rn(d) * 0.1).to(dtype),
        "anchor": torch.randint(0, T, (B,), generator=g, dtype=torch.int32),
        "partner": torch.randint(0, T, (B, K), generator=g, dtype=torch.int32),
        "scores": rn(B, K), "gamma": torch.rand(d, generator=g) + 0.5, "beta": rn(d) * 0.1,
        "next_w": torch.rand(d, generator=g) + 0.5, "next_b": rn(d) * 0.1,
        "hidden": rn(B, d), "mix": torch.tensor(0.1824),
        "wq": (rn(n_query, d) * 0.05).to(dtype) if n_query else None,
    }
    x["scores"][:, -1] = -torch.inf           # an empty slot, with the selector's (negative) sentinel index
    x["partner"][:, -1] = -7
    if B > 1:
        x["scores"][1] = -torch.inf           # a sequence without any partner: context 0
    return x


def _expected(x, t, dtype):
    clamped = x["partner"].clamp(0, x["operand"].size(1) - 1)
    hid, _ = oracle.relation_hidden(x["expanded"], x["operand"], x["anchor"], clamped, x["wm"])
    raw = oracle.linear(hid.to(dtype), x["w2"]) + x["b2"].float()
    context = oracle.relation_norm_reduce(raw, x["scores"], x["gamma"], x["beta"], t, 1e-5)
    hidden = x["hidden"] + x["mix"] * context
    normalized = F.layer_norm(hidden, (hidden.size(1),), x["next_w"], x["next_b"], 1e-5)
    return hidden, normalized


def _run(x, t, dtype):
    from relation_lm.kernels.relation_reduce import relation_layer_tail

    dev = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in x.items()}
    B, d = x["hidden"].shape
    hidden = dev["hidden"].clone()
    normalized = torch.full((B, d), float("nan"), device="cuda", dtype=dtype)
    query = torch.full((B, x["wq"].size(0)), float("nan"), device="cuda", dtype=dtype) if x["wq"] is not None else None
    relation_layer_tail(dev["expanded"], dev["operand"], dev["anchor"], dev["partner"], dev["scores"], dev["wm"],
                        dev["w2"], dev["b2"], dev["gamma"], dev["beta"], position_tensor(t), 1e-5, hidden,
                        dev["mix"], dev["next_w"], dev["next_b"], 1e-5, normalized, dev["wq"], query)
    return hidden, normalized, query


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,K,d,R,T,n_query,t", [
    (8, 8, 512, 128, 96, 256, 95),        # the ctx-512 decode configuration's layer
    (1, 8, 512, 128, 64, 256, 3),         # one sequence, early position (two active partners)
    (3, 5, 256, 128, 40, 256, 39),        # clusters of 8 CTAs, K that does not divide 64
    (13, 8, 128, 128, 50, 256, 20),       # clusters of 4 CTAs, two clusters, 64 query outputs per CTA
    (4, 8, 128, 64, 30, 0, 10),           # relation width 64
    (16, 4, 512, 128, 64, 0, 63),         # no query projection, 8 sequences per cluster (K 4)
])
def test_layer_tail_matches_unfused_oracle(B, K, d, R, T, n_query, t, dtype):
    from relation_lm.kernels.relation_reduce import relation_layer_tail_supported

    if not relation_layer_tail_supported(B, K, R, 4 * d, d, n_query, dtype):
        pytest.skip("clusters of this size are not available on this device")
    x = _case(B, K, d, R, T, n_query, dtype, 5100 + B + d)
    want_hidden, want_norm = _expected(x, t, dtype)
    hidden, normalized, query = _run(x, t, dtype)
    assert_rel_close(hidden, want_hidden, 1e-2, "residual")
    assert_rel_close(normalized, want_norm, 1e-2, "normalized")
    if n_query:
        assert_rel_close(query, oracle.linear(normalized.cpu(), x["wq"]), 1e-2, "query")
    again = _run(x, t, dtype)
    assert torch.equal(hidden, again[0]) and torch.equal(normalized, again[1])
    if n_query:
        assert torch.equal(query, again[2])
    if B > 1:                               # the sequence without partners keeps its residual row
        assert torch.equal(hidden[1].cpu(), x["hidden"][1])
    assert_status_clear()


def test_layer_tail_rejects_shapes_it_does_not_serve():
    from relation_lm.kernels.relation_reduce import relation_layer_tail_supported

    assert not relation_layer_tail_supported(8, 8, 128, 3072, 768, 256, torch.bfloat16)     # d 768
    assert not relation_layer_tail_supported(8, 8, 128, 2048, 512, 256, torch.float32)
    x = _case(2, 8, 768, 128, 16, 0, torch.bfloat16, 1)
    with pytest.raises(ValueError):
        _run(x, 5, torch.bfloat16)


# ---- the selector in front of the tail, one launch for the layer

def _layer_case(B, K, d, R, T, NB, L, top, n_query, dtype, seed):
    import cases

    name = {torch.bfloat16: "bf16", torch.float16: "fp16"}[dtype]
    sel = cases.make_inputs({"kind": "select", "seed": seed, "batch": B, "context": T, "blocks": NB,
                             "local_window": L, "top_blocks": top, "k_out": K, "strict_valid": True, "dtype": name})
    tail = _case(B, K, d, R, T, n_query, dtype, seed + 1)
    return sel, tail


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,K,d,R,T,NB,L,top,n_query", [
    (8, 8, 512, 128, 512, 16, 64, 2, 256),      # the ctx-512 decode configuration's layer
    (1, 8, 512, 128, 512, 16, 64, 2, 256),
    (5, 8, 256, 128, 256, 8, 32, 2, 256),       # clusters of 8 CTAs
    (3, 4, 128, 64, 128, 8, 16, 1, 0),          # clusters of 4 CTAs, relation width 64
    (32, 4, 128, 64, 128, 8, 16, 1, 64),        # 8 clusters of 4 CTAs, a selecting CTA per sequence
])
def test_whole_layer_equals_select_then_tail(B, K, d, R, T, NB, L, top, n_query, dtype):
    from gpu_util import select_args, to_cuda
    from relation_lm.kernels.relation_layer import relation_layer, relation_layer_supported
    from relation_lm.kernels.relation_reduce import relation_layer_tail
    from relation_lm.kernels.relation_select import relation_select_packed

    sel, x = _layer_case(B, K, d, R, T, NB, L, top, n_query, dtype, 6200 + B + d)
    buckets = sel["anchor_bias"].size(1)
    if not relation_layer_supported(B, K, R, 4 * d, d, n_query, dtype, T, NB, buckets, L, top):
        pytest.skip("the selector does not fit in front of the tail for these sizes on this device")
    sg, dev = to_cuda(sel), to_cuda(x)
    for t in (0, 1, L - 1, T // 2 + 3, T - 1):
        pos = position_tensor(t)
        a, a_s, p, p_s = relation_select_packed(*select_args(sg), pos, L, top, K, True)
        want_hidden = dev["hidden"].clone()
        want_norm = torch.zeros(B, d, device="cuda", dtype=dtype)
        want_query = torch.zeros(B, n_query, device="cuda", dtype=dtype) if n_query else None
        relation_layer_tail(dev["expanded"], dev["operand"], a, p, p_s, dev["wm"], dev["w2"], dev["b2"],
                            dev["gamma"], dev["beta"], pos, 1e-5, want_hidden, dev["mix"], dev["next_w"],
                            dev["next_b"], 1e-5, want_norm, dev["wq"], want_query)
        hidden = dev["hidden"].clone()
        norm = torch.full((B, d), float("nan"), device="cuda", dtype=dtype)
        query = torch.full((B, n_query), float("nan"), device="cuda", dtype=dtype) if n_query else None
        ga, ga_s, gp, gp_s = relation_layer(
            *select_args(sg), pos, L, top, K, True, dev["expanded"], dev["operand"], dev["wm"], dev["w2"],
            dev["b2"], dev["gamma"], dev["beta"], 1e-5, hidden, dev["mix"], dev["next_w"], dev["next_b"], 1e-5,
            norm, dev["wq"], query)
        assert torch.equal(ga, a) and torch.equal(gp, p), t
        assert torch.equal(ga_s.view(torch.int32), a_s.view(torch.int32)), t
        assert torch.equal(gp_s.view(torch.int32), p_s.view(torch.int32)), t
        if B <= 4 * (4 * d // 128):
            assert torch.equal(hidden, want_hidden) and torch.equal(norm, want_norm), t
            if n_query:
                assert torch.equal(query, want_query), t
        else:
            # more sequences than 4 clusters' CTAs: the two forms split the sequences over clusters
            # differently, and the order of a cluster's sums depends on its number of rows
            assert_rel_close(hidden, want_hidden, 1e-2, "residual")
            assert_rel_close(norm, want_norm, 1e-2, "normalized")
            if n_query:
                assert_rel_close(query, want_query, 1e-2, "query")
        # and against the oracle's selection on the same inputs
        oa, _, op, _, _ = oracle.relation_select(*select_args(sel), t, L, top, K, True)
        assert torch.equal(ga.cpu(), oa) and torch.equal(gp.cpu(), op), t
    assert_status_clear()


def test_whole_layer_rejects_a_selector_that_does_not_fit():
    from relation_lm.kernels.relation_layer import relation_layer_supported

    # the tail's tile memory is about 50 KB: 64 blocks of statistics + a 128-row window + 4 blocks of 64 keys need more
    assert not relation_layer_supported(4, 8, 128, 512, 128, 0, torch.bfloat16, 4096, 64, 8, 128, 4)
    assert not relation_layer_supported(4, 8, 128, 3072, 768, 0, torch.bfloat16, 128, 8, 8, 16, 1)   # d 768
