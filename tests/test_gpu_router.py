"""GPU parity of ``router_cache_update``: vs the CPU oracle (bit-exact in fp32), vs the
reference kernel's golden outputs, and vs the eager formulation of the reference's own GPU
test (tests/test_router_cache_update_gpu.py:85-176 of the reference project)."""
from __future__ import annotations

import pytest
import torch

import cases
import oracle
from gpu_util import assert_status_clear, position_tensor, to_cuda

pytestmark = pytest.mark.gpu

STATE = ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache",
         "anchor_mean", "anchor_std", "partner_mean", "partner_std")


def _run(xg, t, block_size):
    from relation_lm.kernels.router_cache import router_cache_update

    return router_cache_update(
        xg["anchor_raw"], xg["partner_raw"], *[xg[n] for n in STATE], xg["anchor_conv_weight"],
        xg["partner_conv_weight"], position_tensor(t), block_size)


def _router_cases():
    return [n for n, c in cases.all_cases().items() if c["kind"] == "router"]


@pytest.mark.parametrize("name", _router_cases())
def test_router_update_matches_golden_and_oracle(golden, name):
    entry = golden[name]
    case = entry["case"]
    x = cases.make_inputs(case)
    assert cases.checksum(x) == entry["input_sha256"]
    xg = to_cuda(x)
    xg["anchor_raw"] = xg["packed"][:, 384:448]      # strided views of the packed projection
    xg["partner_raw"] = xg["packed"][:, 448:512]
    assert xg["anchor_raw"].stride(0) == 512
    t, bs = case["position"], case["block_size"]
    out = _run(xg, t, bs)
    want_out, want = oracle.router_cache_update(
        x["anchor_raw"], x["partner_raw"], *[x[n] for n in STATE], x["anchor_conv_weight"],
        x["partner_conv_weight"], t, bs)
    assert torch.equal(out.cpu(), want_out)
    for n in STATE:
        assert torch.equal(xg[n].float().cpu(), want[n]), n   # every row and block, bit for bit
    ref = entry["outputs"]
    blk = t // bs
    low = case["dtype"] != "fp32"
    atol = 1e-2 if low else 1e-6
    assert torch.allclose(out.cpu(), ref["out"], atol=1e-6, rtol=1e-6)
    for n in STATE[:4]:
        assert torch.allclose(xg[n][:, t].float().cpu(), ref[n + "_row"].float(), atol=atol, rtol=1e-6)
    for n in STATE[4:]:
        assert torch.allclose(xg[n][:, blk].float().cpu(), ref[n + "_blk"].float(), atol=atol, rtol=1e-6)
    assert_status_clear()


@pytest.mark.parametrize("batch", [1, 8])
@pytest.mark.parametrize("position_value", [95, 96, 447, 448])
def test_router_update_state_like_the_reference_test(batch, position_value):
    """Context 512, block 8, eager reference with torch mean/std, atol = rtol = 1e-6."""
    T, bs = 512, 8
    g = torch.Generator().manual_seed(20260824 + batch + position_value)
    packed = torch.randn(batch, 512, generator=g).cuda()
    x = {"anchor_raw": packed[:, 384:448], "partner_raw": packed[:, 448:512]}
    for n in STATE[:4]:
        cache = torch.zeros(batch, T, 64)
        cache[:, :position_value] = torch.randn(batch, position_value, 64, generator=g)
        x[n] = cache.cuda()
    for n in STATE[4:]:
        x[n] = torch.zeros(batch, T // bs, 4, 16, device="cuda")
    x["anchor_conv_weight"] = (torch.randn(64, 3, generator=g) * 0.1).cuda()
    x["partner_conv_weight"] = (torch.randn(64, 3, generator=g) * 0.1).cuda()
    before = {n: x[n].clone() for n in STATE}
    out = _run(x, position_value, bs)
    t, blk = position_value, position_value // bs
    for s, (raw, rc, cc, mean, std, w) in enumerate((
            ("anchor_raw", "anchor_raw_cache", "anchor_conv_cache", "anchor_mean", "anchor_std", "anchor_conv_weight"),
            ("partner_raw", "partner_raw_cache", "partner_conv_cache", "partner_mean", "partner_std", "partner_conv_weight"))):
        conv = x[raw] * x[w][:, 2] + before[rc][:, t - 1] * x[w][:, 1] + before[rc][:, t - 2] * x[w][:, 0]
        assert torch.allclose(out[:, s], conv, atol=1e-6, rtol=1e-6)
        assert torch.equal(x[rc][:, t], x[raw])
        assert torch.allclose(x[cc][:, t], conv, atol=1e-6, rtol=1e-6)
        block = before[cc][:, blk * bs:(blk + 1) * bs].clone()
        block[:, t - blk * bs] = conv
        block = block.reshape(batch, bs, 4, 16)
        assert torch.allclose(x[mean][:, blk], block.mean(1), atol=1e-6, rtol=1e-6)
        assert torch.allclose(x[std][:, blk], block.std(1, unbiased=False), atol=1e-6, rtol=1e-6)
    assert_status_clear()


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_incremental_updates_build_the_full_sequence_statistics(dtype):
    """T updates from a zero state == oracle state after the same updates, and (fp32) the
    eager router's conv + block statistics (src/relation_lm/routing/block_router.py:51-68)."""
    B, T, bs = 3, 96, 32
    td = {"fp32": torch.float32, "bf16": torch.bfloat16}[dtype]
    g = torch.Generator().manual_seed(811)
    raw_a = torch.randn(B, T, 64, generator=g).to(td)
    raw_p = torch.randn(B, T, 64, generator=g).to(td)
    w_a, w_p = torch.randn(64, 3, generator=g) * 0.1, torch.randn(64, 3, generator=g) * 0.1
    host = {n: torch.zeros(B, T, 64, dtype=td) for n in STATE[:4]}
    host.update({n: torch.zeros(B, T // bs, 4, 16, dtype=td) for n in STATE[4:]})
    dev = to_cuda(host)
    dev.update(anchor_conv_weight=w_a.cuda(), partner_conv_weight=w_p.cuda())
    ra, rp = raw_a.cuda(), raw_p.cuda()
    for t in range(T):
        dev["anchor_raw"], dev["partner_raw"] = ra[:, t], rp[:, t]
        _run(dev, t, bs)
        _, new = oracle.router_cache_update(raw_a[:, t], raw_p[:, t], *[host[n] for n in STATE],
                                            w_a, w_p, t, bs)
        host = {n: new[n].to(td) for n in STATE}
    for n in STATE:
        assert torch.equal(dev[n].cpu(), host[n]), n
    if dtype == "fp32":
        conv = torch.nn.functional.conv1d(
            torch.nn.functional.pad(raw_a.transpose(1, 2), (2, 0)), w_a[:, None, :], groups=64).transpose(1, 2)
        grouped = conv.view(B, T // bs, bs, 4, 16)
        assert torch.allclose(dev["anchor_conv_cache"].cpu(), conv, atol=1e-6, rtol=1e-5)
        assert torch.allclose(dev["anchor_mean"].cpu(), grouped.mean(2), atol=1e-6, rtol=1e-5)
        assert torch.allclose(dev["anchor_std"].cpu(), grouped.std(2, unbiased=False), atol=1e-6, rtol=1e-5)
    assert_status_clear()


def test_router_update_validation():
    from relation_lm.kernels import _abi

    case = cases.all_cases()["router_p8_b2"]
    xg = to_cuda(cases.make_inputs(case))
    with pytest.raises(ValueError):
        bad = dict(xg)
        bad["anchor_raw"] = xg["packed"][:, 0:128:2]      # inner stride 2
        _run(bad, 8, 8)
    with pytest.raises(ValueError):
        bad = dict(xg)
        bad["anchor_mean"] = xg["anchor_mean"].half()
        _run(bad, 8, 8)
    _run(xg, 4096, 8)                                      # position outside the cache
    assert _abi.read_status() == 2


@pytest.mark.parametrize("dtype,length", [("fp32", 96), ("fp32", 77), ("bf16", 128), ("bf16", 45)])
def test_prefill_equals_sequential_updates(dtype, length):
    """One prefill launch == `length` oracle updates from a zero state, bit for bit, including a
    trailing partial block; the keys come as strided slices of a packed projection."""
    from relation_lm.kernels.router_cache import router_cache_prefill

    B, T, bs = 2, 128, 32
    td = {"fp32": torch.float32, "bf16": torch.bfloat16}[dtype]
    g = torch.Generator().manual_seed(900 + length)
    packed = torch.randn(B, length, 512, generator=g).to(td)
    w_a, w_p = torch.randn(64, 3, generator=g) * 0.1, torch.randn(64, 3, generator=g) * 0.1
    host = {n: torch.zeros(B, T, 64, dtype=td) for n in STATE[:4]}
    host.update({n: torch.zeros(B, T // bs, 4, 16, dtype=td) for n in STATE[4:]})
    dev = to_cuda(host)
    pg = packed.cuda()
    router_cache_prefill(pg[:, :, 384:448], pg[:, :, 448:512], *[dev[n] for n in STATE], w_a.cuda(), w_p.cuda(), bs)
    for t in range(length):
        _, new = oracle.router_cache_update(packed[:, t, 384:448], packed[:, t, 448:512],
                                            *[host[n] for n in STATE], w_a, w_p, t, bs)
        host = {n: new[n].to(td) for n in STATE}
    for n in STATE:
        assert torch.equal(dev[n].cpu(), host[n]), n


@pytest.mark.parametrize("position", [0, 1, 31, 32, 200])
def test_projection_with_state_append_in_its_epilogue_equals_the_two_launch_form(position):
    """``packed_projection_append`` (projection of one decode position for all layers, token-cache rows
    and router update in the epilogue) against ``skinny_projection`` + ``sparse_cache_append``: the
    packed rows and all twelve state tensors bit for bit, stale rows beyond the position included."""
    from relation_lm.kernels.packed_projection import skinny_projection
    from relation_lm.kernels.router_cache import packed_projection_append, sparse_cache_append

    layers, B, T, bs, R, d = 3, 8, 256, 32, 128, 512
    nb, width = T // bs, 384 + R
    g = torch.Generator().manual_seed(8200 + position)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    x = rn(B, d).bfloat16().cuda()
    weight = (rn(layers * width, d) * 0.05).bfloat16().cuda()
    conv_a, conv_p = (rn(layers, 64, 3) * 0.1).cuda(), (rn(layers, 64, 3) * 0.1).cuda()

    def fresh_state():
        gs = torch.Generator().manual_seed(8300 + position)
        tok = [torch.zeros(layers, B, T, w_, dtype=torch.bfloat16, device="cuda") for w_ in (64, 64, R, 128)]
        router = [torch.randn(layers, B, T, 64, generator=gs).bfloat16().cuda() for _ in range(4)]
        stats = [torch.randn(layers, B, nb, 4, 16, generator=gs).bfloat16().cuda() for _ in range(4)]
        return tok, router, stats

    pos = position_tensor(position)
    tok1, router1, stats1 = fresh_state()
    packed1 = packed_projection_append(x, weight, *tok1, *router1, *stats1, conv_a, conv_p, pos, bs)
    tok2, router2, stats2 = fresh_state()
    packed2 = skinny_projection(x, weight)
    sparse_cache_append(packed2, *tok2, *router2, *stats2, conv_a, conv_p, pos, bs)
    assert torch.equal(packed1, packed2)
    for mine, theirs in zip(tok1 + router1 + stats1, tok2 + router2 + stats2):
        assert torch.equal(mine, theirs)
    assert_status_clear()
