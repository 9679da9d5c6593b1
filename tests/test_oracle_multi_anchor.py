"""The routed multi-anchor layer pass against the reference's own dense modules.

``tests/golden/make_golden.py`` ran the reference's ``RelationBlockStack`` of
``MultiAnchorRelationBlock`` layers (models/multi_relation_blocks.py:21-207 of the reference
project) on whole sequences with the weights of this repository's seeded
``MultiAnchorRoutedStack``.  With a window that covers the whole history and no remote blocks the
routed pass is the dense pass: distinct anchors chosen slot after slot, all anchors barred from
every partner set, finite-score partner softmax without an active-K limit, slot mixing
renormalised over the active slots, gated residual, final LayerNorm.  This file checks the CPU
port of the pass (``oracle/multi_anchor_port.py``, fp32): anchor indices and activity exactly,
partner indices wherever the reference marks them active, per-layer relation context and the
stack's output to 2e-5.  ``tests/test_gpu_multi_anchor.py`` compares the GPU pass with the port.
"""
from __future__ import annotations

import torch

import cases


def multi_stack(case):
    from relation_lm.inference.multi_anchor import MultiAnchorConfig, MultiAnchorRoutedStack

    return MultiAnchorRoutedStack(MultiAnchorConfig(**cases.multi_stack_config_kwargs(case)), seed=case["model_seed"])


def test_cpu_port_of_the_multi_anchor_pass_reproduces_the_dense_reference_stack(golden):
    from oracle.multi_anchor_port import OracleMultiAnchor

    entry = golden["multi_stack_dense"]
    case, ref = entry["case"], entry["outputs"]
    x = cases.make_inputs(case)
    assert cases.checksum(x) == entry["input_sha256"]
    stack = multi_stack(case)
    assert cases.checksum(dict(stack.state_dict())) == ref["model_sha256"]
    port = OracleMultiAnchor(stack, torch.float32)
    keep: list = []
    out = port.forward(x["hidden"], x["memory"], keep)
    B, T = case["batch"], case["context"]
    for layer, (mine, theirs) in enumerate(zip(keep, ref["layers"])):
        S = case["anchors"]
        assert torch.equal(mine["anchor_active"].view(B, T, S), theirs["anchor_active"]), layer
        assert torch.equal(mine["anchor"].view(B, T, S), theirs["anchor_index"]), layer
        active = theirs["partner_active"]
        assert torch.equal(torch.isfinite(mine["partner_score"]).view(active.shape), active), layer
        assert torch.equal(mine["partner"].view(active.shape)[active], theirs["partner_index"][active]), layer
        assert torch.allclose(mine["context"].view(B, T, -1), theirs["relation_context"], atol=2e-5, rtol=1e-5), layer
    assert torch.allclose(out, ref["output"], atol=2e-5, rtol=1e-5), (out - ref["output"]).abs().max()
    # the invariants of the reference's own test (tests/test_multi_relation_blocks.py:34-42)
    first = keep[0]
    for row in range(0, B * T, 3):
        chosen = first["anchor"][row][first["anchor_active"][row]]
        assert chosen.unique().numel() == chosen.numel()
        live = torch.isfinite(first["partner_score"][row])
        assert not set(first["partner"][row][live].tolist()) & set(chosen.tolist())
