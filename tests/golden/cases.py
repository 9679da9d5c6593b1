"""Seeded input builders shared by the golden-vector generator and the tests.

Every case is a plain dict; ``make_inputs(case)`` rebuilds its tensors on CPU
from ``case['seed']`` with a private ``torch.Generator``.  Distributions follow
the reference's own test fixtures (tests/test_relation_select_gpu.py:14-31,
tests/test_router_cache_update_gpu.py:14-37, tests/test_relation_reduce_gpu.py:46-78
of the reference project).
"""
from __future__ import annotations

import hashlib

import torch

_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    return g


def _quantize(t: torch.Tensor) -> torch.Tensor:
    """Multiples of 1/2 in [-2, 2]: every dot product is exact in any order, ties abound."""
    return (t * 2).round().clamp(-4, 4) / 2


def select_inputs(case) -> dict[str, torch.Tensor]:
    g = _gen(case["seed"])
    B, T, NB = case["batch"], case["context"], case["blocks"]
    n = case.get("rows", B)  # query rows (== batch for the decode form)
    buckets = case.get("buckets", 16)
    dtype = _DTYPES[case.get("dtype", "fp32")]
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    ru = lambda *s: torch.rand(*s, generator=g)  # noqa: E731
    x = {
        "anchor_query": rn(n, 64), "anchor_keys": rn(B, T, 64), "anchor_router_query": rn(n, 64),
        "anchor_mean": rn(B, NB, 4, 16), "anchor_std": ru(B, NB, 4, 16),
        "anchor_gamma": rn(4), "anchor_bias": rn(4, buckets),
        "partner_base": rn(n, 128), "partner_anchor_cache": rn(B, T, 128),
        "partner_keys": rn(B, T, 64), "partner_mean": rn(B, NB, 4, 16),
        "partner_std": ru(B, NB, 4, 16), "partner_gamma": rn(4), "partner_bias": rn(4, buckets),
    }
    if case.get("quantize"):
        for k in x:
            if k.endswith("gamma") or k.endswith("bias"):
                continue
            x[k] = _quantize(x[k])
            if k.endswith("std"):
                x[k] = x[k].abs()
        # duplicate neighbouring blocks' statistics and a few key rows: exact ties
        for k in ("anchor_mean", "anchor_std", "partner_mean", "partner_std"):
            x[k][:, 1::2] = x[k][:, 0::2]
        twins = torch.arange(1, T, 3)
        for k in ("anchor_keys", "partner_keys"):
            x[k][:, twins] = x[k][:, twins - 1]
    big = ("anchor_query", "anchor_keys", "anchor_router_query", "anchor_mean", "anchor_std",
           "partner_base", "partner_anchor_cache", "partner_keys", "partner_mean", "partner_std")
    for k in big:
        x[k] = x[k].to(dtype)
    return x


def router_inputs(case) -> dict[str, torch.Tensor]:
    g = _gen(case["seed"])
    B, T, bs, t = case["batch"], case["context"], case["block_size"], case["position"]
    dtype = _DTYPES[case.get("dtype", "fp32")]
    nb = T // bs
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    packed = rn(B, 512).to(dtype)
    x = {"packed": packed, "anchor_raw": packed[:, 384:448], "partner_raw": packed[:, 448:512]}
    for name in ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache"):
        cache = torch.zeros(B, T, 64)
        cache[:, :t] = rn(B, t, 64)
        if case.get("stale_tail"):
            cache[:, t:] = rn(B, T - t, 64)  # rows not yet written hold old data
        x[name] = cache.to(dtype)
    for name in ("anchor_mean", "anchor_std", "partner_mean", "partner_std"):
        x[name] = rn(B, nb, 4, 16).to(dtype)
    x["anchor_conv_weight"] = rn(64, 3) * 0.1
    x["partner_conv_weight"] = rn(64, 3) * 0.1
    return x


def router_sequence_inputs(case) -> dict[str, torch.Tensor]:
    g = _gen(case["seed"])
    B, T = case["batch"], case["context"]
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    return {"anchor_raw_seq": rn(B, T, 64), "partner_raw_seq": rn(B, T, 64),
            "anchor_conv_weight": rn(64, 3) * 0.1, "partner_conv_weight": rn(64, 3) * 0.1,
            "router_query_seq": rn(B, T, 64), "gamma": rn(4), "bias": rn(4, 16)}


def reduce_inputs(case) -> dict[str, torch.Tensor]:
    g = _gen(case["seed"])
    B, T, R, H, K = case["batch"], case["context"], case["relation_dim"], case["hidden_dim"], case["k_out"]
    dtype = _DTYPES[case.get("dtype", "fp32")]
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    t = case["position"]
    anchor_index = torch.randint(0, T, (B,), generator=g, dtype=torch.int32)
    partner_index = torch.randint(0, T, (B, K), generator=g, dtype=torch.int32)
    anchor_index[0] = t            # the reference fixture plants index == position
    partner_index[:, 0] = t
    return {"operand_cache": rn(B, T, R).to(dtype), "first_weight": (rn(H, 4 * R) * 0.02).to(dtype),
            "first_bias": (rn(H) * 0.01).to(dtype), "anchor_index": anchor_index,
            "partner_index": partner_index}


def norm_reduce_inputs(case) -> dict[str, torch.Tensor]:
    g = _gen(case["seed"])
    B, K, D = case["batch"], case["k_out"], case["dim"]
    dtype = _DTYPES[case.get("dtype", "fp32")]
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    scores = rn(B, K)
    scores[:, -1] = -torch.inf     # as the reference fixture
    if case.get("all_inactive"):
        scores[0] = -torch.inf
    return {"raw": rn(B, K, D).to(dtype), "scores": scores,
            "norm_weight": rn(D) * 0.05 + 1.0, "norm_bias": rn(D) * 0.01}


def packed_inputs(case) -> dict:
    g = _gen(case["seed"])
    d, rows = case["d_model"], case["rows"]
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    widths = (64, 64, 128, 128, 64, 64)
    return {"memory": rn(rows, d), "weights": [rn(w, d) * 0.02 for w in widths]}


def multi_anchor_inputs(case) -> dict[str, torch.Tensor]:
    g = _gen(case["seed"])
    B, T, d = case["batch"], case["context"], case["d_model"]
    return {"hidden": torch.randn(B, T, d, generator=g), "memory": torch.randn(B, T, d, generator=g)}


def stack_inputs(case) -> dict[str, torch.Tensor]:
    """Token and boundary ids of a single-anchor layer stack case.  The model itself is rebuilt
    from ``case['model_seed']`` by ``RoutedRelationLM`` (its state dict is hashed in the golden)."""
    g = _gen(case["seed"])
    B, T = case["batch"], case["context"]
    return {"tokens": torch.randint(0, case["vocab"], (B, T), generator=g),
            "boundaries": torch.randint(0, case["boundary_vocab"], (B, T), generator=g)}


def multi_stack_inputs(case) -> dict[str, torch.Tensor]:
    g = _gen(case["seed"])
    B, T, d = case["batch"], case["context"], case["d_model"]
    return {"hidden": torch.randn(B, T, d, generator=g), "memory": torch.randn(B, T, d, generator=g)}


def multi_stack_config_kwargs(case) -> dict:
    """Keyword arguments of ``MultiAnchorConfig`` for a multi-anchor stack case (full-history
    window, no remote blocks: routed selection equals dense selection)."""
    return dict(d_model=case["d_model"], relation_dim=case["relation_dim"], anchors_per_block=case["anchors"],
                partners_per_anchor=case["partners"], depth=case["depth"], max_context=case["context"],
                block_size=case["block_size"], local_window=case["context"], top_blocks=0)


def stack_config_kwargs(case) -> dict:
    """Keyword arguments of ``RoutedRelationConfig`` for a stack case: the local window covers the
    whole history and no remote block is used, so routed selection equals dense selection."""
    return dict(vocab_size=case["vocab"], boundary_vocab_size=case["boundary_vocab"],
                d_model=case["d_model"], layers=case["layers"], max_context=case["context"],
                block_size=case["block_size"], local_window=case["context"], top_blocks=0,
                k_max=case["k_out"])


_BUILDERS = {"select": select_inputs, "stack": stack_inputs, "multi_stack": multi_stack_inputs, "router": router_inputs,
             "router_sequence": router_sequence_inputs, "reduce": reduce_inputs,
             "norm_reduce": norm_reduce_inputs, "packed": packed_inputs,
             "multi_anchor": multi_anchor_inputs}


def make_inputs(case):
    return _BUILDERS[case["kind"]](case)


def checksum(inputs) -> str:
    h = hashlib.sha256()
    for key in sorted(inputs):
        values = inputs[key]
        for v in (values if isinstance(values, (list, tuple)) else [values]):
            v = v.contiguous().reshape(-1)
            raw = v.view(torch.uint8) if v.dtype != torch.bool else v.to(torch.uint8)
            h.update(key.encode())
            h.update(raw.numpy().tobytes())
    return h.hexdigest()


def all_cases() -> dict[str, dict]:
    c: dict[str, dict] = {}

    def select(name, **kw):
        base = {"kind": "select", "buckets": 16, "k_out": 8, "strict_valid": False, "dtype": "fp32"}
        base.update(kw)
        c[name] = base

    # the reference's own GPU test shape (tests/test_relation_select_gpu.py:14-31)
    select("select_reftest", seed=29, batch=4, context=512, blocks=64, local_window=16,
           top_blocks=2, positions=[511])
    select("select_reftest_strict", seed=30, batch=2, context=512, blocks=64, local_window=16,
           top_blocks=2, positions=[447, 448, 511], strict_valid=True)
    # single layer, context 128, block 16, window 32, 2 remote blocks
    early = [0, 1, 5, 15, 16, 30, 31, 32, 33, 47, 48, 63, 64, 100, 127]
    select("select_c128_compat", seed=1001, batch=1, context=128, blocks=8, local_window=32,
           top_blocks=2, positions=early)
    select("select_c128_strict", seed=1001, batch=1, context=128, blocks=8, local_window=32,
           top_blocks=2, positions=early, strict_valid=True)
    # context 512, block 32, window 64
    mid = [31, 62, 63, 64, 95, 96, 300, 511]
    select("select_c512_compat", seed=1002, batch=2, context=512, blocks=16, local_window=64,
           top_blocks=2, positions=mid)
    select("select_c512_strict", seed=1002, batch=2, context=512, blocks=16, local_window=64,
           top_blocks=2, positions=mid, strict_valid=True)
    select("select_top0", seed=1010, batch=2, context=128, blocks=16, local_window=16,
           top_blocks=0, positions=[0, 7, 40, 127])
    select("select_top1_k4", seed=1011, batch=2, context=128, blocks=16, local_window=16,
           top_blocks=1, k_out=4, positions=[3, 16, 40, 127])
    select("select_top4_k5", seed=1012, batch=2, context=256, blocks=32, local_window=32,
           top_blocks=4, k_out=5, positions=[10, 64, 200, 255])
    select("select_top4_strict", seed=1013, batch=2, context=256, blocks=32, local_window=32,
           top_blocks=4, positions=[10, 40, 64, 255], strict_valid=True)
    select("select_bf16", seed=1014, batch=2, context=256, blocks=16, local_window=32,
           top_blocks=2, positions=[20, 100, 255], dtype="bf16")
    select("select_ties_compat", seed=1015, batch=2, context=128, blocks=16, local_window=16,
           top_blocks=2, positions=[5, 17, 60, 127], quantize=True)
    select("select_ties_strict", seed=1016, batch=2, context=128, blocks=16, local_window=16,
           top_blocks=3, positions=[17, 60, 127], quantize=True, strict_valid=True)
    select("select_buckets8", seed=1017, batch=1, context=512, blocks=64, local_window=16,
           top_blocks=2, positions=[200, 511], buckets=8)

    for i, (batch, pos) in enumerate([(1, 0), (2, 1), (1, 2), (2, 7), (2, 8), (1, 95), (2, 96)]):
        c[f"router_p{pos}_b{batch}"] = {"kind": "router", "seed": 2000 + i, "batch": batch,
                                        "context": 128, "block_size": 8, "position": pos,
                                        "dtype": "fp32"}
    c["router_stale_tail"] = {"kind": "router", "seed": 2010, "batch": 2, "context": 128,
                              "block_size": 16, "position": 37, "stale_tail": True, "dtype": "fp32"}
    c["router_bf16"] = {"kind": "router", "seed": 2011, "batch": 2, "context": 128,
                        "block_size": 32, "position": 70, "dtype": "bf16"}
    c["router_sequence"] = {"kind": "router_sequence", "seed": 2020, "batch": 2, "context": 48,
                            "block_size": 8}

    for i, (batch, k) in enumerate([(1, 8), (3, 5)]):
        c[f"reduce_b{batch}_k{k}"] = {"kind": "reduce", "seed": 3000 + i, "batch": batch,
                                      "context": 64, "relation_dim": 128, "hidden_dim": 256,
                                      "k_out": k, "position": 63 if i == 0 else 20, "dtype": "fp32"}
    c["reduce_bf16"] = {"kind": "reduce", "seed": 3002, "batch": 2, "context": 32,
                        "relation_dim": 128, "hidden_dim": 128, "k_out": 8, "position": 31,
                        "dtype": "bf16"}
    for i, (batch, k, dim) in enumerate([(1, 8, 576), (3, 5, 576), (2, 7, 512), (2, 8, 768)]):
        c[f"norm_reduce_b{batch}_k{k}_d{dim}"] = {
            "kind": "norm_reduce", "seed": 4000 + i, "batch": batch, "k_out": k, "dim": dim,
            "eps": 1.0e-5, "positions": [0, 1, 2, 5, 6, 30, 511], "all_inactive": i == 1}
    c["multi_anchor_dense"] = {"kind": "multi_anchor", "seed": 6000, "batch": 2, "context": 24,
                               "d_model": 48, "anchors": 4, "partners": 4}
    # single-anchor relation layers against the reference's dense RelationBlock / StackedRelationLayers
    c["stack_two_layers"] = {"kind": "stack", "seed": 7000, "model_seed": 7001, "batch": 2, "context": 64,
                             "d_model": 128, "layers": 2, "block_size": 8, "k_out": 8, "vocab": 300,
                             "boundary_vocab": 16}
    # the single-layer fp32 configuration: d_model 256, hidden 1024, context 128, block 16, batch 1
    c["stack_single_layer_d256"] = {"kind": "stack", "seed": 7010, "model_seed": 1001, "batch": 1,
                                    "context": 128, "d_model": 256, "layers": 1, "block_size": 16,
                                    "k_out": 8, "vocab": 300, "boundary_vocab": 16}
    # multi-anchor layers against the reference's dense MultiAnchorRelationBlock / RelationBlockStack
    c["multi_stack_dense"] = {"kind": "multi_stack", "seed": 7100, "model_seed": 7101, "batch": 2, "context": 32,
                              "d_model": 64, "relation_dim": 64, "anchors": 4, "partners": 4, "depth": 2,
                              "block_size": 8}
    c["packed_d576"] = {"kind": "packed", "seed": 5000, "rows": 8, "d_model": 576}
    c["packed_d512"] = {"kind": "packed", "seed": 5001, "rows": 3, "d_model": 512}
    return c
