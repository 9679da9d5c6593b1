"""``relation_lm::packed_projection`` — the packed sparse-cache projection on the tensor cores.

``out = x @ weight.T`` for bfloat16 / float16 operands: a hand-written sm_100a kernel
(TMA tile loads, ``tcgen05.mma`` with the accumulator in tensor memory).  It stands where the
reference project calls ``F.linear`` in ``PackedSparseCacheProjection.project``
(src/relation_lm/inference/packed_cache.py:52-57) and also serves the query-side router
projections.
"""
from __future__ import annotations

import torch
from torch import Tensor

from relation_lm.kernels import _abi


@torch.library.custom_op("relation_lm::packed_projection", mutates_args=(), device_types="cuda")
def packed_projection(x: Tensor, weight: Tensor) -> Tensor:
    """``x [rows, d] @ weight [n, d].T`` → ``[rows, n]`` in the operands' dtype (fp32 accumulate)."""
    device = _abi.require_cuda_rows(x=x)
    _abi.require_cuda_contiguous(weight=weight)
    if weight.device != device or weight.dim() != 2 or weight.size(1) != x.size(1):
        raise ValueError("weight must be [n_out, d_in] on the device of x")
    if x.dtype != weight.dtype or x.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("packed_projection takes bfloat16 or float16 operands of one dtype")
    rows, d_in = x.shape
    n_out = weight.size(0)
    out = torch.empty((rows, n_out), device=device, dtype=x.dtype)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_packed_projection(
            _abi.ptr(x), x.stride(0), _abi.ptr(weight), _abi.ptr(out), rows, d_in, n_out,
            _abi.code(x), _abi.code(out), _abi.ptr(_abi.status_tensor(device)),
            _abi.stream_ptr(device)))
    return out


@packed_projection.register_fake
def _(x, weight):
    return x.new_empty((x.size(0), weight.size(0)))
