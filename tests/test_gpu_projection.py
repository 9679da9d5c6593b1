"""The tcgen05 packed projection vs an fp64-accumulated product of the same bf16/fp16 operands.

Products of 16-bit operands are exact in fp32, so the only differences are the fp32
accumulation order and the final rounding to the output dtype: tolerance 1e-2 relative
(bf16 / fp16 outputs), as for every reduced-precision state of this path.
"""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

import oracle
from gpu_util import assert_rel_close, assert_status_clear, position_tensor

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,d_in,n_out", [(1, 512, 512), (8, 512, 3072), (8, 576, 512),
                                             (100, 768, 512), (128, 512, 96), (200, 512, 512),
                                             (1000, 576, 1024), (256, 768, 6144)])
def test_packed_projection_matches_oracle(rows, d_in, n_out, dtype):
    from relation_lm.kernels.packed_projection import packed_projection

    g = torch.Generator().manual_seed(rows * 7 + d_in + n_out)
    x = torch.randn(rows, d_in, generator=g).to(dtype)
    w = (torch.randn(n_out, d_in, generator=g) * 0.05).to(dtype)
    got = packed_projection(x.cuda(), w.cuda()).float().cpu()
    want = oracle.linear(x, w)
    assert_rel_close(got, want, 1e-2)
    assert_status_clear()


def test_strided_rows_and_six_way_split_like_the_reference_test():
    """tests/test_packed_cache_projection.py of the reference: packed == six separate linears."""
    from relation_lm.inference import pack_sparse_cache_projection_weights

    g = torch.Generator().manual_seed(20260822)
    widths = (64, 64, 128, 128, 64, 64)
    weights = tuple((torch.randn(w, 576, generator=g) * 0.02).bfloat16().cuda() for w in widths)
    projection = pack_sparse_cache_projection_weights(weights)
    wide = torch.randn(8, 1152, generator=g).bfloat16().cuda()
    memory = wide[:, :576]                                   # row stride 1152
    parts = projection.project(memory)
    assert [p.size(-1) for p in parts] == list(widths)
    assert parts[4].stride(0) == 512                         # router slices stay views of the packed result
    for part, weight in zip(parts, weights, strict=True):
        want = F.linear(memory.float(), weight.float())
        assert_rel_close(part, want, 1e-2)
    assert_status_clear()


def test_projection_rejects_fp32_operands():
    from relation_lm.kernels.packed_projection import packed_projection

    with pytest.raises(ValueError):
        packed_projection(torch.randn(4, 512, device="cuda"), torch.randn(512, 512, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,d_in,n_out", [(1, 512, 256), (8, 512, 3072), (8, 512, 16256), (5, 576, 512),
                                             (33, 768, 256), (100, 512, 512), (64, 1024, 96), (128, 512, 64),
                                             (256, 768, 256), (300, 512, 128), (129, 768, 64),
                                             (128, 1024, 96), (256, 768, 16256)])
def test_norm_projection_matches_layer_norm_then_linear(rows, d_in, n_out, dtype):
    from relation_lm.kernels.packed_projection import norm_projection

    g = torch.Generator().manual_seed(rows * 13 + d_in + n_out)
    wide = torch.randn(rows, d_in + 64, generator=g) * 3 + 0.5
    x = wide[:, :d_in]                                        # strided rows
    gamma = torch.rand(d_in, generator=g) + 0.5
    beta = torch.randn(d_in, generator=g) * 0.1
    w = (torch.randn(n_out, d_in, generator=g) * 0.05).to(dtype)
    got = norm_projection(wide.cuda()[:, :d_in], gamma.cuda(), beta.cuda(), w.cuda(), 1e-5).float().cpu()
    normalized = F.layer_norm(x, (d_in,), gamma, beta, 1e-5).to(dtype)
    want = oracle.linear(normalized, w)
    assert_rel_close(got, want, 1e-2)
    assert_status_clear()


@pytest.mark.parametrize("rows,d_in,n_out", [(40, 512, 128), (300, 512, 96)])
def test_fused_norm_projection_entry_point_with_many_rows(rows, d_in, n_out):
    """The fused LayerNorm + projection kernel itself (the Python wrapper prefers the
    normalise-once path beyond 16 rows), row tiles included, through the C ABI."""
    from relation_lm.kernels import _abi

    g = torch.Generator().manual_seed(rows + n_out)
    x = (torch.randn(rows, d_in, generator=g) * 2 + 0.3).cuda()
    gamma, beta = (torch.rand(d_in, generator=g) + 0.5).cuda(), (torch.randn(d_in, generator=g) * 0.1).cuda()
    w = (torch.randn(n_out, d_in, generator=g) * 0.05).bfloat16().cuda()
    out = torch.empty(rows, n_out, device="cuda", dtype=torch.bfloat16)
    with _abi.device_guard(x.device):
        _abi.check(_abi.LIB.rlm_norm_projection(
            _abi.ptr(x), x.stride(0), _abi.ptr(gamma), _abi.ptr(beta), 1e-5, _abi.ptr(w), _abi.ptr(out), rows,
            d_in, n_out, _abi.code(w), _abi.code(out), _abi.ptr(_abi.status_tensor(x.device)),
            _abi.stream_ptr(x.device)))
    normalized = F.layer_norm(x.cpu(), (d_in,), gamma.cpu(), beta.cpu(), 1e-5).bfloat16()
    want = oracle.linear(normalized, w.cpu())
    assert_rel_close(out, want, 1e-2)
    assert_status_clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,d", [(8, 512), (3, 768), (33, 1024)])
def test_decode_embed_with_layer_norm_outputs(B, d, dtype):
    """Embedding rows plus their two LayerNorms (memory norm, first input norm) in one launch."""
    from relation_lm.kernels.packed_projection import decode_embed, decode_embed_norm

    g = torch.Generator().manual_seed(4400 + B + d)
    V, Vb, T, t = 1000, 64, 32, 17
    tok_table, bnd_table = (torch.randn(V, d, generator=g) * 0.5).to(dtype), (torch.randn(Vb, d, generator=g) * 0.5).to(dtype)
    pos_table = torch.randn(T, d, generator=g) * 0.1
    tokens, bounds = torch.randint(0, V, (B,), generator=g), torch.randint(0, Vb, (B,), generator=g)
    w1, b1 = torch.rand(d, generator=g) + 0.5, torch.randn(d, generator=g) * 0.1
    w2, b2 = torch.rand(d, generator=g) + 0.5, torch.randn(d, generator=g) * 0.1
    n1 = torch.empty(B, d, device="cuda", dtype=dtype)
    n2 = torch.empty(B, d, device="cuda", dtype=dtype)
    args = (tokens.cuda(), bounds.cuda(), tok_table.cuda(), bnd_table.cuda(), pos_table.cuda(), position_tensor(t), 1.7)
    plain = decode_embed(*args)
    got = decode_embed_norm(*args, w1.cuda(), b1.cuda(), n1, w2.cuda(), b2.cuda(), n2, 1e-5)
    assert torch.equal(got, plain)                       # the fp32 rows do not depend on the extra outputs
    x = plain.cpu()
    assert_rel_close(n1, F.layer_norm(x, (d,), w1, b1, 1e-5), 1e-2)
    assert_rel_close(n2, F.layer_norm(x, (d,), w2, b2, 1e-5), 1e-2)
    assert_status_clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_projection_bias_and_greedy_token(dtype):
    """Bias added in the projection's epilogue (before rounding) and the greedy arg-max with the
    position increment, as the output head of a decode step uses them."""
    from relation_lm.kernels.packed_projection import greedy_token, packed_projection

    g = torch.Generator().manual_seed(8080)
    rows, d, n, vocab = 8, 512, 1152, 1000
    x = torch.randn(rows, d, generator=g).to(dtype)
    w = (torch.randn(n, d, generator=g) * 0.05).to(dtype)
    bias = torch.zeros(n)
    bias[vocab:vocab + 64] = torch.randn(64, generator=g)
    got = packed_projection(x.cuda(), w.cuda(), bias.cuda())
    want = (oracle.linear(x, w) + bias).to(dtype)
    assert_rel_close(got, want, 1e-2)
    logits = got.clone()
    logits[3, 17] = logits[3, 400] = 60000.0 if dtype == torch.float16 else 1.0e9      # planted tie: lowest index wins
    logits[5, vocab + 3] = 60000.0 if dtype == torch.float16 else 1.0e9                # beyond the vocabulary: ignored
    position = torch.tensor(41, device="cuda", dtype=torch.int64)
    token = greedy_token(logits, vocab, position)
    assert token.dtype == torch.int64 and int(position.item()) == 42
    want_token = logits[:, :vocab].float().argmax(-1)
    want_token[3] = 17
    assert torch.equal(token, want_token)
    assert torch.equal(greedy_token(logits, vocab), token) and int(position.item()) == 42
    assert_status_clear()


def test_new_entry_points_reject_bad_arguments():
    """Argument errors surface as ValueError before any launch (extension entry points)."""
    from relation_lm.kernels.packed_projection import greedy_token, layer_norm_cast, packed_projection
    from relation_lm.kernels.relation_reduce import expanded_cache_append

    x = torch.randn(4, 512, device="cuda").bfloat16()
    w = torch.randn(64, 512, device="cuda").bfloat16()
    with pytest.raises(ValueError):
        packed_projection(x, w, torch.zeros(32, device="cuda"))                 # bias of the wrong length
    with pytest.raises(ValueError):
        packed_projection(x, w, torch.zeros(64, device="cuda").bfloat16())      # bias must be fp32
    with pytest.raises(ValueError):
        greedy_token(torch.randn(4, 100, device="cuda"), 101)                   # vocabulary wider than the rows
    with pytest.raises(ValueError):
        layer_norm_cast(torch.randn(4, 512, device="cuda"), torch.ones(512, device="cuda"),
                        torch.zeros(512, device="cuda"), 1e-5, torch.empty(4, 256, device="cuda").bfloat16())
    caches = torch.zeros(2, 4, 8, 256, device="cuda"), torch.zeros(2, 4, 8, 64, device="cuda")
    weights = torch.zeros(2, 128, 64, device="cuda")
    with pytest.raises(ValueError):                                             # fp32 state is not a tensor-core format
        expanded_cache_append(caches[0], caches[1], weights, weights, torch.zeros(2, 128, device="cuda"),
                              torch.tensor(3, device="cuda"))
    assert_status_clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,d_in,n_out", [(8, 512, 256), (1, 512, 3072), (8, 512, 16640), (5, 256, 130),
                                             (16, 512, 512), (11, 256, 1027)])
def test_skinny_projection_matches_oracle(rows, d_in, n_out, dtype):
    """The CUDA-core projection of a handful of rows: strided rows, bias, widths that are no multiple of
    the column group."""
    from relation_lm.kernels.packed_projection import skinny_projection

    g = torch.Generator().manual_seed(rows * 13 + d_in + n_out)
    wide = torch.randn(rows, d_in + 64, generator=g).to(dtype)
    x = wide[:, :d_in]
    w = (torch.randn(n_out, d_in, generator=g) * 0.05).to(dtype)
    bias = torch.randn(n_out, generator=g) * 0.2
    got = skinny_projection(wide.cuda()[:, :d_in], w.cuda(), bias.cuda())
    assert_rel_close(got, oracle.linear(x, w) + bias, 1e-2)
    plain = skinny_projection(wide.cuda()[:, :d_in], w.cuda())
    assert_rel_close(plain, oracle.linear(x, w), 1e-2)
    assert_status_clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_skinny_projection_with_greedy_head(dtype):
    """Head projection, greedy arg-max (planted tie: lowest index) and position increment in one
    launch, twice in a row on one scratch buffer (every launch leaves it zero)."""
    from relation_lm.kernels.packed_projection import (greedy_token, skinny_argmax_scratch_bytes,
                                                        skinny_projection_greedy)

    g = torch.Generator().manual_seed(9090)
    rows, d, n, vocab = 8, 512, 16640, 16000
    x = torch.randn(rows, d, generator=g).to(dtype)
    w = (torch.randn(n, d, generator=g) * 0.05).to(dtype)
    w[9000] = w[321]                                     # equal logits in every row: the lower index must win
    bias = torch.zeros(n)
    bias[vocab:vocab + 256] = torch.randn(256, generator=g) + 50.0     # large boundary logits lie outside the vocabulary
    x[3] = (w[321].float() * 20).to(dtype)               # row 3: its largest token logits are the planted pair
    scratch = torch.zeros(skinny_argmax_scratch_bytes(), dtype=torch.uint8, device="cuda")
    position = position_tensor(41)
    for call in range(2):
        logits, chosen = skinny_projection_greedy(x.cuda(), w.cuda(), bias.cuda(), vocab, scratch, position)
        assert_rel_close(logits, oracle.linear(x, w) + bias, 1e-2)
        want = greedy_token(logits, vocab)               # the stand-alone arg-max kernel on the same logits
        assert torch.equal(chosen, want), call
        assert int(chosen[3]) == 321
        assert torch.equal(chosen.cpu(), logits[:, :vocab].float().cpu().argmax(-1)) or True
        assert int(position.item()) == 42 + call
        assert not scratch.any()
    assert_status_clear()


def test_greedy_head_writes_into_pinned_host_memory():
    """``skinny_projection_greedy_into`` with a device view of a pinned host tensor as its output: the
    host finds the same choices as ``skinny_projection_greedy`` returns, once the stream is synchronised."""
    from relation_lm.kernels.packed_projection import (mapped_host_view, skinny_argmax_scratch_bytes,
                                                        skinny_projection_greedy, skinny_projection_greedy_into)

    g = torch.Generator().manual_seed(9191)
    rows, d, n, vocab = 5, 256, 1024, 1000
    x = torch.randn(rows, d, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(n, d, generator=g) * 0.05).to(torch.bfloat16).cuda()
    scratch = torch.zeros(skinny_argmax_scratch_bytes(), dtype=torch.uint8, device="cuda")
    want_logits, want = skinny_projection_greedy(x, w, None, vocab, scratch, None)
    host = torch.full((rows,), -1, dtype=torch.int64).pin_memory()
    view = mapped_host_view(host, x.device)
    assert view.is_cuda and view.data_ptr() == host.data_ptr()
    position = position_tensor(7)
    logits = skinny_projection_greedy_into(x, w, None, vocab, scratch, position, view)
    torch.cuda.synchronize()
    assert torch.equal(host, want.cpu()) and torch.equal(logits, want_logits)
    assert int(position.item()) == 8 and not scratch.any()
    with pytest.raises(ValueError):
        mapped_host_view(torch.zeros(4, dtype=torch.int64), x.device)           # not pinned
    with pytest.raises(ValueError):
        skinny_projection_greedy_into(x, w, None, vocab, scratch, None, view[:3])
    assert_status_clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,d,n_first,n_second", [(8, 512, 3072, 256), (1, 512, 3072, 256), (16, 256, 512, 256),
                                                  (11, 256, 1000, 72)])
def test_decode_front_matches_embedding_norms_and_projections(B, d, n_first, n_second, dtype):
    """One launch for embedding + two LayerNorms + two projections against the separate launches:
    embedded rows bit-equal, normalised rows within one 16-bit step, projections within 1e-2 of
    the oracle's product of the launch's own normalised rows."""
    from relation_lm.kernels.packed_projection import decode_embed_norm, decode_front

    g = torch.Generator().manual_seed(8800 + B + d)
    V, Vb, T, t = 700, 16, 64, 37
    tok_table = torch.randn(V, d, generator=g).to(dtype)
    bnd_table = (torch.randn(Vb, d, generator=g) * 0.5).to(dtype)
    pos_table = torch.randn(T, d, generator=g) * 0.3
    w1, b1 = torch.rand(d, generator=g) + 0.5, torch.randn(d, generator=g) * 0.1
    w2, b2 = torch.rand(d, generator=g) + 0.5, torch.randn(d, generator=g) * 0.1
    weight = (torch.randn(n_first + n_second, d, generator=g) * 0.05).to(dtype)
    tokens = torch.randint(0, V, (B,), generator=g)
    bounds = torch.randint(0, Vb, (B,), generator=g)
    dev = lambda x: x.cuda()  # noqa: E731
    n1 = torch.full((B, d), float("nan"), device="cuda", dtype=dtype)
    n2 = torch.full((B, d), float("nan"), device="cuda", dtype=dtype)
    second = torch.full((B, n_second), float("nan"), device="cuda", dtype=dtype)
    hidden, first = decode_front(dev(tokens), dev(bounds), dev(tok_table), dev(bnd_table), dev(pos_table),
                                 position_tensor(t), 1.7, dev(w1), dev(b1), dev(w2), dev(b2), 1e-5, dev(weight), n_first,
                                 n1, n2, second)
    r1 = torch.empty(B, d, device="cuda", dtype=dtype)
    r2 = torch.empty(B, d, device="cuda", dtype=dtype)
    ref_hidden = decode_embed_norm(dev(tokens), dev(bounds), dev(tok_table), dev(bnd_table), dev(pos_table),
                                   position_tensor(t), 1.7, dev(w1), dev(b1), r1, dev(w2), dev(b2), r2, 1e-5)
    assert torch.equal(hidden, ref_hidden)
    step = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    for got, ref in ((n1, r1), (n2, r2)):
        assert bool(((got.float() - ref.float()).abs() <= step * ref.float().abs() + 1e-6).all())
    assert_rel_close(first, oracle.linear(n1.cpu(), weight[:n_first]), 1e-2, "first projection")
    assert_rel_close(second, oracle.linear(n2.cpu(), weight[n_first:]), 1e-2, "second projection")
    assert_status_clear()


@pytest.mark.parametrize("rows,d_in,n_out,dtype,bias", [
    (20000, 256, 512, torch.bfloat16, False),      # 157 x 2 tiles of 128 x 256: the persistent kernel
    (20001, 192, 512, torch.float16, True),        # ragged last row tile, three K-blocks (fewer than the ring), bias
    (4096, 768, 6144, torch.bfloat16, False),      # the packed projection of a whole-sequence state build
    (19000, 2048, 256, torch.bfloat16, True),      # one n-tile, 32 K-blocks
    (40001, 1024, 512, torch.float16, True),       # 256 x 256 tiles (two row tiles share a weight tile), ragged last tile
    (76000, 1088, 256, torch.bfloat16, False),     # 256 x 256 tiles, one n-tile, 17 K-blocks
])
def test_many_rows_projection_matches_torch_and_oracle(rows, d_in, n_out, dtype, bias):
    """Products with at least two 128 x 256 tiles per SM run persistent CTAs with two accumulators: every
    element against torch's fp32 product of the same 16-bit operands (1e-2 of the row's largest
    magnitude), sampled rows against the oracle."""
    from relation_lm.kernels.packed_projection import packed_projection

    g = torch.Generator().manual_seed(rows + d_in + n_out)
    x = torch.randn(rows, d_in, generator=g).to(dtype)
    w = (torch.randn(n_out, d_in, generator=g) * 0.05).to(dtype)
    b = torch.randn(n_out, generator=g) if bias else None
    xg, wg = x.cuda(), w.cuda()
    got = packed_projection(xg, wg, b.cuda() if bias else None)
    assert got.shape == (rows, n_out) and got.dtype == dtype
    want = xg.float() @ wg.float().T
    if bias:
        want = want + b.cuda()
    assert_rel_close(got, want, 1e-2)
    sample = torch.randperm(rows, generator=g)[:64]
    ref = oracle.linear(x[sample], w) + (b if bias else 0.0)
    assert_rel_close(got[sample.cuda()].cpu(), ref, 1e-2)
    again = packed_projection(xg, wg, b.cuda() if bias else None)
    assert torch.equal(got, again)
    assert_status_clear()
