"""The fused relation tail (second MLP layer + norm-reduce + residual) vs the oracle's
unfused composition.  16-bit operands, fp32 accumulation: within 1e-2 of the row's largest magnitude."""
from __future__ import annotations

import pytest
import torch

import oracle
from gpu_util import assert_rel_close, assert_status_clear, position_tensor

pytestmark = pytest.mark.gpu


def _case(batch, k_out, hdim, dim, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    hidden_rel = torch.randn(batch, k_out, hdim, generator=g).to(dtype)
    w2 = (torch.randn(dim, hdim, generator=g) * 0.03).to(dtype)
    b2 = (torch.randn(dim, generator=g) * 0.1).to(dtype)
    scores = torch.randn(batch, k_out, generator=g)
    scores[:, -1] = -torch.inf
    gamma = torch.rand(dim, generator=g) + 0.5
    beta = torch.randn(dim, generator=g) * 0.1
    hidden = torch.randn(batch, dim, generator=g)
    mix = torch.tensor(0.1824)
    return hidden_rel, w2, b2, scores, gamma, beta, hidden, mix


def _expected(case, t):
    hidden_rel, w2, b2, scores, gamma, beta, hidden, mix = case
    raw = oracle.linear(hidden_rel, w2) + b2.float()
    context = oracle.relation_norm_reduce(raw, scores, gamma, beta, t, 1e-5)
    return hidden + mix * context


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("batch,k_out,hdim,dim,t", [(8, 8, 2048, 512, 511), (1, 8, 2048, 512, 3),
                                                    (5, 4, 1024, 256, 40), (16, 8, 3072, 768, 2047),
                                                    (40, 8, 2048, 512, 100), (3, 16, 512, 576, 9)])
def test_relation_tail_matches_unfused_oracle(batch, k_out, hdim, dim, t, dtype):
    from relation_lm.kernels.relation_reduce import relation_tail

    case = _case(batch, k_out, hdim, dim, dtype, batch * 31 + hdim + dim)
    hidden_rel, w2, b2, scores, gamma, beta, hidden, mix = case
    want = _expected(case, t)
    dev = [x.cuda() for x in case]
    for call in range(2):        # the second call finds the scratch as the first one left it
        live = dev[6].clone()
        relation_tail(dev[0], dev[1], dev[2], dev[3], dev[4], dev[5], position_tensor(t), 1e-5, live, dev[7])
        assert_rel_close(live, want, 1e-2, f"call {call}")
    assert_status_clear()


def test_relation_tail_rejects_partner_counts_that_split_a_row_tile():
    from relation_lm.kernels.relation_reduce import relation_tail

    case = [x.cuda() for x in _case(4, 5, 512, 256, torch.bfloat16, 1)]
    with pytest.raises(ValueError):
        relation_tail(case[0], case[1], case[2], case[3], case[4], case[5], position_tensor(9), 1e-5,
                      case[6].clone(), case[7])
