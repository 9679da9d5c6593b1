"""The operators under ``torch.compile(fullgraph=True, mode="reduce-overhead")``.

Modelled on tests/test_router_cache_update_gpu.py:178-233 of the reference project: a module that
owns the persistent state as buffers and calls the operator; the compiled module (traced through
the operators' fake implementations and replayed as a CUDA graph) must return what the eager
module returns and leave every buffer in the same state.  Results are compared bit for bit —
both run the same kernel.
"""
from __future__ import annotations

import pytest
import torch
from torch import nn

import cases
from gpu_util import SELECT_KEYS, assert_status_clear, position_tensor

pytestmark = pytest.mark.gpu

STATE = ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache",
         "anchor_mean", "anchor_std", "partner_mean", "partner_std")


class RouterUpdateModule(nn.Module):
    def __init__(self, case, block_size) -> None:
        super().__init__()
        for name in STATE + ("anchor_conv_weight", "partner_conv_weight"):
            self.register_buffer(name, case[name].clone())
        self.block_size = int(block_size)

    def forward(self, anchor_raw, partner_raw, position):
        from relation_lm.kernels.router_cache import router_cache_update

        return router_cache_update(anchor_raw, partner_raw, *[getattr(self, n) for n in STATE],
                                   self.anchor_conv_weight, self.partner_conv_weight, position, self.block_size)


def _router_case(batch, t, T=512, bs=8):
    g = torch.Generator().manual_seed(20260824 + batch + t)
    case = {}
    for n in STATE[:4]:
        cache = torch.zeros(batch, T, 64)
        cache[:, :t] = torch.randn(batch, t, 64, generator=g)
        case[n] = cache
    for n in STATE[4:]:
        case[n] = torch.zeros(batch, T // bs, 4, 16)
    case["anchor_conv_weight"] = torch.randn(64, 3, generator=g) * 0.1
    case["partner_conv_weight"] = torch.randn(64, 3, generator=g) * 0.1
    case["packed"] = torch.randn(batch, 512, generator=g)
    return case


@pytest.mark.parametrize("batch", [1, 8])
def test_router_cache_update_fullgraph(batch):
    t, bs = 447, 8
    case = _router_case(batch, t, bs=bs)
    eager = RouterUpdateModule(case, bs).cuda().eval()
    compiled_module = RouterUpdateModule(case, bs).cuda().eval()
    compiled = torch.compile(compiled_module, fullgraph=True, mode="reduce-overhead")
    packed = case["packed"].cuda()
    anchor_raw, partner_raw = packed[:, 384:448], packed[:, 448:512]      # stride-512 views
    position = position_tensor(t)
    want = eager(anchor_raw, partner_raw, position)
    for _ in range(3):            # compile, record the graph, replay it: same position, same result
        torch.compiler.cudagraph_mark_step_begin()
        got = compiled(anchor_raw, partner_raw, position).clone()
    torch.cuda.synchronize()
    assert torch.equal(want, got)
    mine = dict(compiled_module.named_buffers())
    for name, buffer in eager.named_buffers():
        assert torch.equal(buffer, mine[name]), name
    assert_status_clear()


class SelectModule(nn.Module):
    def __init__(self, x, policy) -> None:
        super().__init__()
        for name in SELECT_KEYS:
            if name not in ("anchor_query", "anchor_router_query", "partner_base"):
                self.register_buffer(name, x[name].clone())
        self.policy = policy

    def forward(self, anchor_query, anchor_router_query, partner_base, position):
        from relation_lm.kernels.relation_select import relation_select_packed

        return relation_select_packed(
            anchor_query, self.anchor_keys, anchor_router_query, self.anchor_mean, self.anchor_std,
            self.anchor_gamma, self.anchor_bias, partner_base, self.partner_anchor_cache, self.partner_keys,
            self.partner_mean, self.partner_std, self.partner_gamma, self.partner_bias, position, *self.policy)


@pytest.mark.parametrize("strict", [False, True])
def test_relation_select_packed_fullgraph(strict):
    case = {"kind": "select", "seed": 4242, "batch": 4, "context": 512, "blocks": 16, "local_window": 64,
            "top_blocks": 2, "k_out": 8, "strict_valid": strict, "dtype": "bf16"}
    x = cases.make_inputs(case)
    module = SelectModule(x, (64, 2, 8, strict)).cuda().eval()
    compiled = torch.compile(module, fullgraph=True, mode="reduce-overhead")
    queries = [x[n].cuda() for n in ("anchor_query", "anchor_router_query", "partner_base")]
    position = position_tensor(300)
    want = module(*queries, position)
    for t in (300, 301):          # the position is read on the device: a replay sees the new value
        position.fill_(t)
        want = module(*queries, position)
        torch.compiler.cudagraph_mark_step_begin()
        got = [o.clone() for o in compiled(*queries, position)]
        torch.cuda.synchronize()
        for a, b in zip(want, got):
            assert torch.equal(a, b), t
    assert_status_clear()
