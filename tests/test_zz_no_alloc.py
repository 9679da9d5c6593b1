"""The relation tail for hosts that must not allocate device memory.

``rlm_relation_tail_static`` keeps its split-K accumulator in a device array built into the
library, for callers such as a serving process whose device memory all belongs to its own
pool, a plug-in inside an engine that owns the allocator, or a latency-critical thread that
cannot afford the device-wide synchronisation of cudaMalloc.  This test drives it through the
C ABI exactly as such a caller would (raw pointers, no allocation between the two calls) and
checks it against the caller-scratch entry point ``rlm_relation_tail`` on the same inputs,
twice in a row: the second call finds the array as the first one left it.

The file name sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2.0e-3, 1.0e-2        # the tolerance of tests/test_gpu_tail.py


def _inputs(batch, k_out, hdim, dim, seed):
    g = torch.Generator().manual_seed(seed)
    dev = "cuda"
    hidden_rel = torch.randn(batch, k_out, hdim, generator=g).bfloat16().to(dev)
    w2 = (torch.randn(dim, hdim, generator=g) * 0.03).bfloat16().to(dev)
    b2 = (torch.randn(dim, generator=g) * 0.1).bfloat16().to(dev)
    scores = torch.randn(batch, k_out, generator=g)
    scores[:, -1] = -torch.inf
    gamma = (torch.rand(dim, generator=g) + 0.5).to(dev)
    beta = (torch.randn(dim, generator=g) * 0.1).to(dev)
    hidden = torch.randn(batch, dim, generator=g).to(dev)
    mix = torch.tensor(0.1824, device=dev)
    position = torch.tensor(300, device=dev, dtype=torch.int64)
    return hidden_rel, w2, b2, scores.to(dev), gamma, beta, hidden, mix, position


def _oracle_expected(x, t):
    import oracle

    hidden_rel, w2, b2, scores, gamma, beta, hidden, mix, _ = [v.cpu() for v in x]
    raw = oracle.linear(hidden_rel, w2) + b2.float()
    context = oracle.relation_norm_reduce(raw, scores, gamma, beta, t, 1e-5)
    return hidden + mix * context


def _call_static(lib, x, residual, status, stream):
    hidden_rel, w2, b2, scores, gamma, beta, _, mix, position = x
    batch, k_out, hdim = hidden_rel.shape
    return lib.rlm_relation_tail_static(
        hidden_rel.data_ptr(), w2.data_ptr(), b2.data_ptr(), scores.data_ptr(), gamma.data_ptr(),
        beta.data_ptr(), position.data_ptr(), 1e-5, residual.data_ptr(), mix.data_ptr(), None,
        batch, k_out, w2.size(0), hdim, 1, status.data_ptr(), stream)


def _call_with_scratch(lib, x, residual, scratch, status, stream):
    hidden_rel, w2, b2, scores, gamma, beta, _, mix, position = x
    batch, k_out, hdim = hidden_rel.shape
    return lib.rlm_relation_tail(
        hidden_rel.data_ptr(), w2.data_ptr(), b2.data_ptr(), scores.data_ptr(), gamma.data_ptr(),
        beta.data_ptr(), position.data_ptr(), 1e-5, residual.data_ptr(), mix.data_ptr(), None,
        scratch.data_ptr(), scratch.numel(), batch, k_out, w2.size(0), hdim, 1, status.data_ptr(), stream)


def test_static_scratch_entry_matches_caller_scratch_entry_twice():
    from relation_lm.kernels import _abi

    lib = _abi.LIB
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    first = _inputs(8, 8, 2048, 512, seed=4101)
    second = _inputs(5, 4, 1024, 768, seed=4102)          # other sizes: reuses the array differently
    scratch = torch.zeros(int(lib.rlm_relation_tail_scratch_bytes(8, 8, 768)), dtype=torch.uint8, device="cuda")
    # every buffer exists before the first call: nothing is allocated between or during the calls
    outs = [(x[6].clone(), x[6].clone()) for x in (first, second)]
    for x, (mine, theirs) in zip((first, second), outs):
        assert _call_static(lib, x, mine, status, stream) == 0, lib.rlm_last_error().decode()
        assert _call_with_scratch(lib, x, theirs, scratch, status, stream) == 0, lib.rlm_last_error().decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for x, (mine, theirs) in zip((first, second), outs):
        assert not torch.equal(mine, x[6])                 # the residual was updated
        assert torch.allclose(mine, theirs, atol=ATOL, rtol=RTOL), (mine - theirs).abs().max()
        # and against the CPU oracle's unfused composition, like tests/test_gpu_tail.py
        want = _oracle_expected(x, 300)
        assert torch.allclose(mine.cpu(), want, atol=ATOL, rtol=RTOL), (mine.cpu() - want).abs().max()
    # after the warm-up calls above, further calls leave the free device memory where it was
    again = [x[6].clone() for x in (first, second)]
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for x, mine in zip((first, second), again):
        assert _call_static(lib, x, mine, status, stream) == 0, lib.rlm_last_error().decode()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    for mine, (earlier, _) in zip(again, outs):
        assert torch.allclose(mine, earlier, atol=ATOL, rtol=RTOL)


def test_static_scratch_entry_rejects_problems_beyond_its_array():
    from relation_lm.kernels import _abi

    lib = _abi.LIB
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    too_many_rows = _inputs(17, 8, 512, 256, seed=4103)    # 136 rows > 128
    rc = _call_static(lib, too_many_rows, too_many_rows[6].clone(), status, stream)
    assert rc == -2 and b"128 rows" in lib.rlm_last_error()
    # a shape the kernel cannot tile is refused before anything reaches the stream
    odd_width = _inputs(4, 8, 512, 96, seed=4104)          # d_model not a multiple of 64
    untouched = odd_width[6].clone()
    assert _call_static(lib, odd_width, untouched, status, stream) == -2
    torch.cuda.synchronize()
    assert torch.equal(untouched, odd_width[6])
