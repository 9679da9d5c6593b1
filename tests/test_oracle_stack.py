"""The single-anchor relation layer of the decode path against the reference's own dense modules.

``tests/golden/make_golden.py`` ran the reference's ``StackedRelationLayers`` / ``RelationBlock``
(models/stacked_relation.py:65-136, 152-182 of the reference project: arg-max anchor, anchor
scattered to -inf, ``topk``, ``ceil(log2(t + 2))`` active limit, masked softmax, relation MLP,
``hidden + sigmoid(mix) * context``, final LayerNorm) on whole sequences with the weights of this
repository's seeded ``RoutedRelationLM``.  With a local window that covers the whole history and
no remote blocks, routed selection is dense selection, so the stateful step must reproduce the
dense module position by position: anchor and (finite-score) partner indices exactly, partner
scores to 4e-6, the stack's output to 2e-5.  This file checks the CPU port of the step
(``oracle/decode_port.py``); ``tests/test_gpu_decode.py`` runs the same comparison on the GPU.
"""
from __future__ import annotations

import pytest
import torch

import cases


def stack_model(case):
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM

    return RoutedRelationLM(RoutedRelationConfig(**cases.stack_config_kwargs(case)), seed=case["model_seed"])


def compare_with_dense_reference(entry, decoder, tokens, boundaries, to_device=lambda x: x):
    """Steps ``decoder`` over the sequence and compares every position with the dense reference."""
    ref = entry["outputs"]
    T = entry["case"]["context"]
    for t in range(T):
        decoder.step(to_device(tokens[:, t]), to_device(boundaries[:, t]), **decoder_kwargs(decoder))
        for layer, (anchor, partner) in enumerate(decoder.last_selection):
            want = ref["layers"][layer]
            assert torch.equal(anchor.cpu(), want["anchor_index"][:, t]), (t, layer)
            finite = torch.isfinite(want["partner_scores"][:, t])
            assert torch.equal(partner.cpu()[finite], want["partner_index"][:, t][finite]), (t, layer)
        final = decoder.last_final.float().cpu()
        assert torch.allclose(final, ref["output"][:, t], atol=2e-5, rtol=1e-5), \
            (t, (final - ref["output"][:, t]).abs().max())


def decoder_kwargs(decoder):
    return {"keep_selection": True} if hasattr(decoder, "trace") else {}


@pytest.mark.parametrize("name", ["stack_two_layers", "stack_single_layer_d256"])
def test_cpu_port_of_the_step_reproduces_the_dense_reference_stack(golden, name):
    from oracle.decode_port import OracleDecoder

    entry = golden[name]
    case = entry["case"]
    x = cases.make_inputs(case)
    assert cases.checksum(x) == entry["input_sha256"]
    model = stack_model(case)
    assert cases.checksum(dict(model.state_dict())) == entry["outputs"]["model_sha256"]
    decoder = OracleDecoder(model, case["batch"], torch.float32)
    compare_with_dense_reference(entry, decoder, x["tokens"], x["boundaries"])


def test_reference_partner_weights_follow_the_active_limit(golden):
    """The golden diagnostics themselves: weights are zero beyond ``ceil(log2(t + 2))`` partners and
    on non-finite scores, and sum to one elsewhere (models/stacked_relation.py:99-107)."""
    layer = golden["stack_two_layers"]["outputs"]["layers"][0]
    weights, active = layer["partner_weights"], layer["active_partner_mask"]
    T = weights.shape[1]
    limit = torch.ceil(torch.log2(torch.arange(T).float() + 2.0)).long().clamp(1, weights.shape[2])
    ranks = torch.arange(weights.shape[2])
    assert not active[:, ranks[None, :] >= limit[:, None]].any()
    assert torch.equal(weights == 0, ~active)
    has_partner = active.any(-1)
    assert torch.allclose(weights.sum(-1)[has_partner], torch.ones(int(has_partner.sum())), atol=1e-6)
