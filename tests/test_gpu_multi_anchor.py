"""Routed multi-anchor selection on the GPU: the exclusion rules against the reference's dense
multi-anchor block (golden fixture), and the routed composition against the same composition
built from the oracle (indices bit-exact)."""
from __future__ import annotations

import pytest
import torch

import oracle
from gpu_util import assert_status_clear
from test_oracle_golden import multi_anchor_dense_check

pytestmark = pytest.mark.gpu


def test_exclusion_rules_match_the_dense_reference_block(golden):
    from relation_lm.kernels.triton_select import anchor_select_rows, partner_topk_rows

    ref = golden["multi_anchor_dense"]["outputs"]

    def anchor_rows(aq, ak, rq, mean, std, gamma, bias, rb, rp, excl, L, top, strict):
        idx, score = anchor_select_rows(aq.cuda(), ak.cuda(), rq.cuda(), mean.cuda(), std.cuda(), gamma.cuda(),
                                        bias.cuda(), rb.cuda(), rp.cuda(), excl.cuda(), L, top, strict)
        return idx.cpu(), score.cpu()

    def partner_rows(pq, pk, rq, mean, std, gamma, bias, rb, rp, anchor, excl, L, top, K, strict):
        idx, score = partner_topk_rows(pq.cuda(), pk.cuda(), rq.cuda(), mean.cuda(), std.cuda(), gamma.cuda(),
                                       bias.cuda(), rb.cuda(), rp.cuda(), anchor.cuda(), excl.cuda(), L, top, K, strict)
        return idx.cpu(), score.cpu()

    multi_anchor_dense_check(ref, anchor_rows, partner_rows)
    assert_status_clear()


@pytest.mark.parametrize("strict", [False, True])
def test_routed_multi_anchor_matches_oracle_composition(strict):
    """Multi-anchor shape scaled down: 4 slots x 4 partners, block 32, window 64, 3 remote
    blocks, bf16 caches; every position of 2 sequences of 256."""
    from relation_lm.kernels.multi_select import relation_select_multi_rows

    S, B, T, NB, L, top, K = 4, 2, 256, 8, 64, 3, 4
    g = torch.Generator().manual_seed(4404)
    N = B * T
    dt = torch.bfloat16
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    x = {"aq": rn(N, S, 64).to(dt), "ak": rn(S, B, T, 64).to(dt), "arq": rn(N, S, 64).to(dt),
         "am": rn(S, B, NB, 4, 16).to(dt), "as": rn(S, B, NB, 4, 16).abs().to(dt),
         "ag": rn(S, 4), "ab": rn(S, 4, 16), "pb": rn(N, S, 128).to(dt),
         "pac": rn(S, B, T, 128).to(dt), "pk": rn(S, B, T, 64).to(dt), "pm": rn(S, B, NB, 4, 16).to(dt),
         "ps": rn(S, B, NB, 4, 16).abs().to(dt), "pg": rn(S, 4), "pbias": rn(S, 4, 16)}
    row_batch = torch.arange(B, dtype=torch.int32).repeat_interleave(T)
    row_pos = torch.arange(T, dtype=torch.int32).repeat(B)
    d = {k: v.cuda() for k, v in x.items()}
    got = relation_select_multi_rows(d["aq"], d["ak"], d["arq"], d["am"], d["as"], d["ag"], d["ab"], d["pb"],
                                     d["pac"], d["pk"], d["pm"], d["ps"], d["pg"], d["pbias"],
                                     row_batch.cuda(), row_pos.cuda(), L, top, K, strict)
    # the same composition from oracle calls
    active = torch.arange(S)[None, :] <= row_pos[:, None]
    taken = torch.full((N, S), -1, dtype=torch.int32)
    anchors = torch.zeros(N, S, dtype=torch.int32)
    for s in range(S):
        idx, score = oracle.anchor_select(x["aq"][:, s], x["ak"][s], x["arq"][:, s], x["am"][s], x["as"][s],
                                          x["ag"][s], x["ab"][s], 0, L, top, strict, row_batch=row_batch,
                                          row_pos=row_pos, exclude_index=taken.clone())
        live = active[:, s] & torch.isfinite(score)
        anchors[:, s] = torch.where(live, idx, torch.zeros_like(idx))
        taken[:, s] = torch.where(live, idx, torch.full_like(idx, -1))
        active[:, s] = live
    assert torch.equal(got[0].cpu(), anchors)
    assert torch.equal(got[2].cpu(), active)
    for s in range(S):
        # the kernel adds the anchor's cached row to the query-side base in fp32, like the packed selector
        v = x["pb"][:, s].float() + x["pac"][s][row_batch.long(), anchors[:, s].long()].float()
        idx, score = oracle.partner_topk(v[:, :64], x["pk"][s], v[:, 64:], x["pm"][s], x["ps"][s], x["pg"][s],
                                         x["pbias"][s], 0, taken[:, s], L, top, K, strict, row_batch=row_batch,
                                         row_pos=row_pos, exclude_index=taken)
        live = active[:, s, None] & torch.isfinite(score)
        assert torch.equal(got[5].cpu()[:, s], live), s
        assert torch.equal(got[3].cpu()[:, s][live], idx[live]), s
        assert torch.equal(got[4].cpu()[:, s][live], score[live]), s
    # invariants of the reference's own multi-anchor test (tests/test_multi_relation_blocks.py:34-42)
    a, act, p, pact = got[0].cpu(), got[2].cpu(), got[3].cpu(), got[5].cpu()
    for r in range(0, N, 7):
        chosen = a[r][act[r]]
        assert chosen.unique().numel() == chosen.numel() and torch.all(chosen <= row_pos[r])
        partners = p[r][pact[r]]
        assert torch.all(partners <= row_pos[r])
        assert not set(partners.tolist()) & set(chosen.tolist())
    assert_status_clear()
