#!/usr/bin/env python3
"""Generate golden vectors from the reference project's own kernels.

Run where the reference checkout is available::

    python tests/golden/make_golden.py --reference /path/to/relation-lm

The reference's seven Triton kernels are executed UNMODIFIED on CPU tensors
through Triton's interpreter (``TRITON_INTERPRET=1``), and its eager modules
(``DistilledBlockRouter``, ``PackedSparseCacheProjection``,
``factor_relation_first_layer``) are called directly.  Triton 3.6's
interpreter mistypes one scalar-compare result as float and then refuses to
``&`` it with a boolean vector; ``_patch_interpreter`` coerces such operands to
bool inside the *interpreter* (the kernels stay as they are).

Inputs are regenerated from a seed by ``tests/golden/cases.py`` (shared with
the tests); each case stores a SHA-256 of its inputs so RNG drift is detected,
and the reference outputs in full.  Output: ``tests/golden/reference_kernels.pt``.
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases  # noqa: E402


def _patch_interpreter() -> None:
    from triton.runtime import interpreter as ti

    original = ti.InterpreterBuilder.binary_op

    def binary_op(self, lhs, rhs, op):
        if op is np.bitwise_and or op is np.bitwise_or:
            a, b = lhs.data, rhs.data
            if a.dtype != b.dtype and (a.dtype == np.bool_ or b.dtype == np.bool_):
                out = op(a.astype(np.bool_), b.astype(np.bool_))
                return ti.TensorHandle(out, lhs.dtype.scalar if a.dtype == np.bool_ else rhs.dtype.scalar)
        return original(self, lhs, rhs, op)

    ti.InterpreterBuilder.binary_op = binary_op


def _next_pow2(n: int) -> int:
    return 1 << max(0, (int(n) - 1).bit_length())


def run_select(case, x):
    from relation_lm.kernels import relation_select as rs
    from relation_lm.kernels import triton_select as ts

    c = case
    B, T, NB = c["batch"], c["context"], c["blocks"]
    bs = T // NB
    L, TOP, K, strict = c["local_window"], c["top_blocks"], c["k_out"], c["strict_valid"]
    cap = _next_pow2(L + TOP * bs)
    max_top = _next_pow2(max(1, TOP))
    out = {}
    for t in c["positions"]:
        pos = torch.tensor(t, dtype=torch.long)
        oa = torch.empty(B, dtype=torch.int32)
        oas = torch.empty(B)
        op = torch.empty(B, K, dtype=torch.int32)
        ops = torch.empty(B, K)
        rs._relation_select_packed_kernel[(B,)](
            x["anchor_query"], x["anchor_keys"], x["anchor_router_query"], x["anchor_mean"],
            x["anchor_std"], x["anchor_gamma"], x["anchor_bias"], x["partner_base"],
            x["partner_anchor_cache"], x["partner_keys"], x["partner_mean"], x["partner_std"],
            x["partner_gamma"], x["partner_bias"], pos, oa, oas, op, ops,
            MAX_T=T, MAX_NB=NB, EXACT_D=64, HEADS=4, HEAD_D=16, REL_BUCKETS=c["buckets"],
            BLOCK_SIZE=bs, LOCAL=L, TOP_BLOCKS=TOP, MAX_TOP=max_top, CANDIDATE_CAPACITY=cap,
            K_OUT=K, STRICT_VALID=strict, num_warps=1)
        # the two-kernel path of the same reference (triton_select.py)
        ta = torch.empty(B, dtype=torch.int32)
        tas = torch.empty(B)
        ts._anchor_select_kernel[(B,)](
            x["anchor_query"], x["anchor_keys"], x["anchor_router_query"], x["anchor_mean"],
            x["anchor_std"], x["anchor_gamma"], x["anchor_bias"], pos, ta, tas,
            MAX_T=T, MAX_NB=NB, EXACT_D=64, HEADS=4, HEAD_D=16, REL_BUCKETS=c["buckets"],
            BLOCK_SIZE=bs, LOCAL=L, TOP_BLOCKS=TOP, STRICT_VALID=strict, num_warps=1)
        contribution = x["partner_anchor_cache"][torch.arange(B), ta.long()].float()
        base = x["partner_base"].float()
        pq = (base[:, :64] + contribution[:, :64]).contiguous()
        rq = (base[:, 64:] + contribution[:, 64:]).contiguous()
        tp = torch.empty(B, K, dtype=torch.int32)
        tps = torch.empty(B, K)
        ts._partner_topk_kernel[(B,)](
            pq, x["partner_keys"], rq, x["partner_mean"], x["partner_std"], x["partner_gamma"],
            x["partner_bias"], pos, ta, tp, tps,
            MAX_T=T, MAX_NB=NB, EXACT_D=64, HEADS=4, HEAD_D=16, REL_BUCKETS=c["buckets"],
            BLOCK_SIZE=bs, LOCAL=L, TOP_BLOCKS=TOP, MAX_TOP=max_top, CANDIDATE_CAPACITY=cap,
            K_OUT=K, STRICT_VALID=strict, num_warps=1)
        out[t] = {"anchor": oa, "anchor_score": oas, "partner": op, "partner_score": ops,
                  "two_anchor": ta, "two_anchor_score": tas, "two_partner": tp,
                  "two_partner_score": tps}
    return out


def run_router(case, x):
    from relation_lm.kernels import router_cache as rc

    B, T, bs = case["batch"], case["context"], case["block_size"]
    state = {k: v.clone() for k, v in x.items()}
    state["anchor_raw"] = state["packed"][:, 384:448]     # strided views, row stride 512
    state["partner_raw"] = state["packed"][:, 448:512]
    out = torch.empty(B, 2, 64)
    rc._router_cache_update_kernel[(B,)](
        state["anchor_raw"], state["partner_raw"], state["anchor_raw_cache"],
        state["partner_raw_cache"], state["anchor_conv_cache"], state["partner_conv_cache"],
        state["anchor_mean"], state["anchor_std"], state["partner_mean"], state["partner_std"],
        state["anchor_conv_weight"], state["partner_conv_weight"],
        torch.tensor(case["position"], dtype=torch.long), out,
        MAX_T=T, MAX_BLOCKS=T // bs, ROUTER_D=64,
        ANCHOR_RAW_STRIDE=state["anchor_raw"].stride(0),
        PARTNER_RAW_STRIDE=state["partner_raw"].stride(0), BLOCK_SIZE=bs, BLOCK_D=64, num_warps=4)
    blk = case["position"] // bs
    t = case["position"]
    result = {"out": out}
    for name in ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache"):
        result[name + "_row"] = state[name][:, t].clone()
        untouched = state[name].clone()
        untouched[:, t] = x[name][:, t]
        assert torch.equal(untouched, x[name]), "reference touched rows other than `position`"
    for name in ("anchor_mean", "anchor_std", "partner_mean", "partner_std"):
        result[name + "_blk"] = state[name][:, blk].clone()
    return result


def run_router_sequence(case, x):
    """T sequential updates from a zero state, then the eager router's own statistics."""
    from relation_lm.kernels import router_cache as rc
    from relation_lm.routing.block_router import BlockRouterConfig, DistilledBlockRouter

    B, T, bs = case["batch"], case["context"], case["block_size"]
    nb = T // bs
    st = {n: torch.zeros(B, T, 64) for n in ("arc", "prc", "acc", "pcc")}
    stats = {n: torch.zeros(B, nb, 4, 16) for n in ("am", "as", "pm", "ps")}
    out = torch.empty(B, 2, 64)
    for t in range(T):
        rc._router_cache_update_kernel[(B,)](
            x["anchor_raw_seq"][:, t].contiguous(), x["partner_raw_seq"][:, t].contiguous(),
            st["arc"], st["prc"], st["acc"], st["pcc"], stats["am"], stats["as"], stats["pm"],
            stats["ps"], x["anchor_conv_weight"], x["partner_conv_weight"],
            torch.tensor(t, dtype=torch.long), out,
            MAX_T=T, MAX_BLOCKS=nb, ROUTER_D=64, ANCHOR_RAW_STRIDE=64, PARTNER_RAW_STRIDE=64,
            BLOCK_SIZE=bs, BLOCK_D=64, num_warps=4)
    router = DistilledBlockRouter(BlockRouterConfig(d_model=64, block_size=bs))
    with torch.no_grad():
        router.anchor_conv.weight.copy_(x["anchor_conv_weight"][:, None, :])
        conv = router._causal_conv(x["anchor_raw_seq"], router.anchor_conv)
        mean, std, _ = router.block_statistics(conv)
        # eager block scores with identity key/query projections (block_router.py:70-101)
        router.anchor_gamma.copy_(x["gamma"])
        router.anchor_bias.copy_(x["bias"])
        eager_scores = router._scores(x["router_query_seq"], x["anchor_raw_seq"],
                                      router.anchor_conv, router.anchor_gamma, router.anchor_bias)
    return {"anchor_conv_cache": st["acc"], "anchor_mean": stats["am"], "anchor_std": stats["as"],
            "partner_mean": stats["pm"], "partner_std": stats["ps"], "eager_conv": conv,
            "eager_mean": mean, "eager_std": std, "eager_block_scores": eager_scores}


def run_reduce(case, x):
    from relation_lm.kernels import relation_reduce as rr

    B, T, R, H, K = case["batch"], case["context"], case["relation_dim"], case["hidden_dim"], case["k_out"]
    factors = rr.factor_relation_first_layer(x["first_weight"], x["first_bias"], R)
    expanded = torch.nn.functional.linear(
        x["operand_cache"].float(), factors.expanded_weight.float(),
        factors.expanded_bias.float()).to(x["operand_cache"].dtype)
    hidden = torch.empty(B, K, H)
    grid = (B, (H + 63) // 64)
    rr._relation_hidden_cached_kernel[grid](
        expanded, x["operand_cache"], x["anchor_index"], x["partner_index"],
        factors.product_weight, hidden, MAX_T=T, RELATION_D=R, HIDDEN_D=H, K_OUT=K, BLOCK_M=16,
        BLOCK_N=64, num_warps=4)
    t = case["position"]
    mutable = expanded.clone()
    mutable[:, t].zero_()
    updated = torch.empty(B, K, H)
    rr._relation_hidden_cache_update_kernel[grid](
        mutable, x["operand_cache"], x["anchor_index"], x["partner_index"], factors.anchor_weight,
        factors.partner_weight, factors.product_weight, factors.first_bias,
        torch.tensor(t, dtype=torch.long), updated, MAX_T=T, RELATION_D=R, HIDDEN_D=H, K_OUT=K,
        BLOCK_M=16, BLOCK_N=64, num_warps=4)
    # the factor tensors are large; a hash pins them (the split is plain tensor arithmetic)
    factor_sha = {name: cases.checksum({name: getattr(factors, name)})
                  for name in ("anchor_weight", "partner_weight", "product_weight", "first_bias",
                               "expanded_weight", "expanded_bias")}
    return {"factor_sha256": factor_sha, "hidden_cached": hidden, "hidden_updated": updated,
            "expanded_row": mutable[:, t].clone()}


def run_norm_reduce(case, x):
    from relation_lm.kernels import relation_reduce as rr

    B, K, D = case["batch"], case["k_out"], case["dim"]
    out = {}
    for t in case["positions"]:
        ctx = torch.empty(B, D)
        rr._relation_norm_reduce_kernel[(B,)](
            x["raw"], x["scores"], x["norm_weight"], x["norm_bias"],
            torch.tensor(t, dtype=torch.long), ctx, OUTPUT_D=D, K_OUT=K, K_BLOCK=_next_pow2(K),
            BLOCK_D=_next_pow2(D), EPS=case["eps"], num_warps=8)
        out[t] = ctx
    return out


def run_packed(case, x):
    from relation_lm.inference import pack_sparse_cache_projection_weights

    projection = pack_sparse_cache_projection_weights(x["weights"])
    parts = projection.project(x["memory"])
    return {"packed_weight_sha256": cases.checksum({"w": projection.weight}),
            "parts": [p.clone() for p in parts],
            "names": list(projection.names), "split_sizes": list(projection.split_sizes)}


def run_multi_anchor(case, x):
    """The reference's dense multi-anchor block (models/multi_relation_blocks.py): its per-slot
    queries / keys are stored as the selector inputs, its indices as the expected result."""
    from relation_lm.models.multi_relation_blocks import (MultiAnchorRelationBlock,
                                                          MultiRelationBlockConfig)

    torch.manual_seed(case["seed"])
    cfg = MultiRelationBlockConfig(d_model=case["d_model"], gate_dim=64, relation_dim=16,
                                   anchors_per_block=case["anchors"],
                                   partners_per_anchor=case["partners"])
    block = MultiAnchorRelationBlock(cfg).eval()
    B, T, h, g = case["batch"], case["context"], case["anchors"], 64
    hidden, memory = x["hidden"], x["memory"]
    with torch.no_grad():
        _, info = block(hidden, memory)
        normalized = block.input_norm(hidden)
        anchor_q = block.anchor_query(normalized).view(B, T, h, g)
        anchor_k = block.anchor_key(memory).view(B, T, h, g)
        anchor = block._gather(memory, info["anchor_index"]) * info["anchor_active"][..., None]
        partner_input = torch.cat((normalized[:, :, None].expand(-1, -1, h, -1), anchor), dim=-1)
        partner_q = torch.stack([layer(partner_input[:, :, i]) for i, layer in enumerate(block.partner_query)], dim=2)
        partner_k = block.partner_key(memory).view(B, T, h, g)
    return {"anchor_q": anchor_q, "anchor_k": anchor_k, "partner_q": partner_q, "partner_k": partner_k,
            "anchor_index": info["anchor_index"].to(torch.int32), "anchor_active": info["anchor_active"],
            "partner_index": info["partner_index"].to(torch.int32), "partner_active": info["partner_active"]}


def _routed_model_module():
    """This repository's parameter container, loaded by file path: its package shares the name
    ``relation_lm`` with the reference's, so it cannot be imported the ordinary way here."""
    import importlib.util

    name = "b200_routed_model"
    if name in sys.modules:
        return sys.modules[name]
    path = HERE.parents[1] / "relation-lm_b200" / "relation_lm" / "inference" / "routed_model.py"
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def run_stack(case, x):
    """The reference's dense single-anchor layers (models/stacked_relation.py:65-136, 152-182) with
    the weights of this repository's seeded ``RoutedRelationLM``: embeddings as
    models/relation_lm.py:130-131, ``memory = LayerNorm(x)``, ``hidden = x``."""
    from relation_lm.models.stacked_relation import RelationBlockConfig, StackedRelationLayers

    rm = _routed_model_module()
    cfg = rm.RoutedRelationConfig(**cases.stack_config_kwargs(case))
    model = rm.RoutedRelationLM(cfg, seed=case["model_seed"]).eval()
    block_cfg = RelationBlockConfig(d_model=cfg.d_model, gate_dim=cfg.gate_dim, relation_dim=cfg.relation_dim,
                                    hidden_dim=cfg.hidden_dim, k_max=cfg.k_max,
                                    mix_logit_init=cfg.mix_logit_init)
    stack = StackedRelationLayers([block_cfg] * cfg.layers).eval()
    for mine, theirs in zip(model.blocks, stack.blocks):
        theirs.load_state_dict({k: v for k, v in mine.state_dict().items() if not k.startswith("router.")})
    stack.final_norm.load_state_dict(model.final_norm.state_dict())
    T = case["context"]
    with torch.no_grad():
        embedded = (model.token_embedding(x["tokens"]) + model.boundary_embedding(x["boundaries"])) \
            * model.input_scale + model.position_embedding[:T]
        memory = model.memory_norm(embedded)
        output, diagnostics = stack(embedded, memory, return_diagnostics=True)
    layers = [{"anchor_index": d["anchor_index"].to(torch.int32), "partner_index": d["partner_index"].to(torch.int32),
               "partner_scores": d["partner_scores"], "partner_weights": d["partner_weights"],
               "active_partner_mask": d["active_partner_mask"]} for d in diagnostics]
    return {"model_sha256": cases.checksum({k: v for k, v in model.state_dict().items()}),
            "layers": layers, "output": output}


def _multi_anchor_module():
    import importlib.util

    name = "b200_multi_anchor"
    if name in sys.modules:
        return sys.modules[name]
    path = HERE.parents[1] / "relation-lm_b200" / "relation_lm" / "inference" / "multi_anchor.py"
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def run_multi_stack(case, x):
    """The reference's dense ``RelationBlockStack`` (models/multi_relation_blocks.py:190-207) with the
    weights of this repository's seeded ``MultiAnchorRoutedStack`` (same parameter names)."""
    from relation_lm.models.multi_relation_blocks import MultiRelationBlockConfig, RelationBlockStack

    ma = _multi_anchor_module()
    cfg = ma.MultiAnchorConfig(**cases.multi_stack_config_kwargs(case))
    mine = ma.MultiAnchorRoutedStack(cfg, seed=case["model_seed"]).eval()
    ref_cfg = MultiRelationBlockConfig(d_model=cfg.d_model, gate_dim=cfg.gate_dim, relation_dim=cfg.relation_dim,
                                       ff_mult=cfg.ff_mult, anchors_per_block=cfg.anchors_per_block,
                                       partners_per_anchor=cfg.partners_per_anchor)
    theirs = RelationBlockStack(ref_cfg, cfg.depth).eval()
    for a, b in zip(mine.blocks, theirs.blocks):
        b.load_state_dict({k: v for k, v in a.state_dict().items() if not k.startswith("router.")})
    theirs.final_norm.load_state_dict(mine.final_norm.state_dict())
    with torch.no_grad():
        output, diagnostics = theirs(x["hidden"], x["memory"])
    layers = [{"anchor_index": d["anchor_index"].to(torch.int32), "anchor_active": d["anchor_active"],
               "partner_index": d["partner_index"].to(torch.int32), "partner_active": d["partner_active"],
               "partner_weight": d["partner_weight"], "slot_weight": d["slot_weight"],
               "relation_context": d["relation_context"]} for d in diagnostics]
    return {"model_sha256": cases.checksum(dict(mine.state_dict())), "layers": layers, "output": output}


RUNNERS = {"select": run_select, "stack": run_stack, "multi_stack": run_multi_stack, "router": run_router, "router_sequence": run_router_sequence,
           "reduce": run_reduce, "norm_reduce": run_norm_reduce, "packed": run_packed,
           "multi_anchor": run_multi_anchor}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of the reference project")
    parser.add_argument("--out", default=str(HERE / "reference_kernels.pt"))
    parser.add_argument("--only", default=None,
                        help="regenerate only the cases whose name starts with this prefix and keep "
                             "the other entries of the existing file")
    args = parser.parse_args()
    sys.path.insert(0, str(Path(args.reference) / "src"))
    _patch_interpreter()
    golden = torch.load(args.out, weights_only=False) if args.only else {}
    for name, case in cases.all_cases().items():
        if args.only and not name.startswith(args.only):
            continue
        inputs = cases.make_inputs(case)
        golden[name] = {"case": case, "input_sha256": cases.checksum(inputs),
                        "outputs": RUNNERS[case["kind"]](case, inputs)}
        print(name, "ok", flush=True)
    torch.save(golden, args.out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
