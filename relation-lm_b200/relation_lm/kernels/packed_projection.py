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

_FUSED_NORM_ROWS = 16    # beyond this many rows normalising once beats normalising in every column tile


@torch.library.custom_op("relation_lm::packed_projection", mutates_args=(), device_types="cuda")
def packed_projection(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    """``x [rows, d] @ weight [n, d].T (+ bias [n])`` → ``[rows, n]`` in the operands' dtype (fp32
    accumulate; the optional fp32 bias is added before the result is rounded)."""
    device = _abi.require_cuda_rows(x=x)
    _abi.require_cuda_contiguous(weight=weight)
    if weight.device != device or weight.dim() != 2 or weight.size(1) != x.size(1):
        raise ValueError("weight must be [n_out, d_in] on the device of x")
    if x.dtype != weight.dtype or x.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("packed_projection takes bfloat16 or float16 operands of one dtype")
    rows, d_in = x.shape
    n_out = weight.size(0)
    if bias is not None:
        _abi.require_cuda_contiguous(bias=bias)
        if bias.dtype != torch.float32 or bias.numel() != n_out or bias.device != device:
            raise ValueError("bias must be float32 [n_out] on the device of x")
    out = torch.empty((rows, n_out), device=device, dtype=x.dtype)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_packed_projection(
            _abi.ptr(x), x.stride(0), _abi.ptr(weight), _abi.ptr(bias), _abi.ptr(out), rows, d_in, n_out,
            _abi.code(x), _abi.code(out), 1, _abi.ptr(_abi.status_tensor(device)),
            _abi.stream_ptr(device)))
    return out


@packed_projection.register_fake
def _(x, weight, bias=None):
    return x.new_empty((x.size(0), weight.size(0)))


@torch.library.custom_op("relation_lm::packed_projection_slices", mutates_args=(), device_types="cuda")
def packed_projection_slices(x: Tensor, weight: Tensor, splits: int) -> Tensor:
    """Split-K form for few rows and a long reduction: ``splits`` CTAs share an output tile and the
    result comes back as fp32 slices ``[splits, rows, n]`` whose sum is ``x @ weight.T`` (the consumer,
    ``relation_norm_reduce_residual_norm_slices``, adds them up).  ``splits`` divides ``d / 64``."""
    device = _abi.require_cuda_rows(x=x)
    _abi.require_cuda_contiguous(weight=weight)
    if weight.device != device or weight.dim() != 2 or weight.size(1) != x.size(1):
        raise ValueError("weight must be [n_out, d_in] on the device of x")
    if x.dtype != weight.dtype or x.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("packed_projection takes bfloat16 or float16 operands of one dtype")
    rows, d_in = x.shape
    n_out = weight.size(0)
    out = torch.empty((int(splits), rows, n_out), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_packed_projection(
            _abi.ptr(x), x.stride(0), _abi.ptr(weight), None, _abi.ptr(out), rows, d_in, n_out,
            _abi.code(x), _abi.code(out), int(splits), _abi.ptr(_abi.status_tensor(device)),
            _abi.stream_ptr(device)))
    return out


@packed_projection_slices.register_fake
def _(x, weight, splits):
    return x.new_empty((splits, x.size(0), weight.size(0)), dtype=torch.float32)


@torch.library.custom_op("relation_lm::layer_norm_cast", mutates_args=("out",), device_types="cuda")
def layer_norm_cast(x: Tensor, norm_weight: Tensor, norm_bias: Tensor, norm_eps: float, out: Tensor) -> None:
    """``out = layer_norm(x)`` for fp32 rows ``[rows, d]`` into a bfloat16 / float16 matrix."""
    device = _abi.require_cuda_rows(x=x)
    _abi.require_cuda_contiguous(norm_weight=norm_weight, norm_bias=norm_bias, out=out)
    if x.dtype != torch.float32 or norm_weight.dtype != torch.float32 or norm_bias.dtype != torch.float32:
        raise ValueError("layer_norm_cast takes fp32 rows and fp32 LayerNorm parameters")
    if out.shape != x.shape or norm_weight.numel() != x.size(1):
        raise ValueError("out must have the shape of x and the norm parameters [d]")
    rows, d_in = x.shape
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_layer_norm_cast(
            _abi.ptr(x), x.stride(0), _abi.ptr(norm_weight), _abi.ptr(norm_bias), float(norm_eps),
            _abi.ptr(out), rows, d_in, _abi.code(out), _abi.stream_ptr(device)))


@layer_norm_cast.register_fake
def _(x, norm_weight, norm_bias, norm_eps, out):
    return None


@torch.library.custom_op("relation_lm::norm_projection", mutates_args=(), device_types="cuda")
def norm_projection(x: Tensor, norm_weight: Tensor, norm_bias: Tensor, weight: Tensor,
                    norm_eps: float) -> Tensor:
    """``layer_norm(x) @ weight.T`` in one launch for fp32 rows: the rows are normalised in
    fp32, rounded to the weight dtype and multiplied on the tensor cores."""
    device = _abi.require_cuda_rows(x=x)
    _abi.require_cuda_contiguous(norm_weight=norm_weight, norm_bias=norm_bias, weight=weight)
    if x.dtype != torch.float32 or norm_weight.dtype != torch.float32 or norm_bias.dtype != torch.float32:
        raise ValueError("norm_projection takes fp32 rows and fp32 LayerNorm parameters")
    if weight.dim() != 2 or weight.size(1) != x.size(1) or norm_weight.numel() != x.size(1):
        raise ValueError("weight must be [n_out, d_in] and the norm parameters [d_in]")
    rows, d_in = x.shape
    if rows > _FUSED_NORM_ROWS:
        # normalise once into a 16-bit matrix, then the TMA-fed GEMM
        normalized = torch.empty((rows, d_in), device=device, dtype=weight.dtype)
        layer_norm_cast(x, norm_weight, norm_bias, norm_eps, normalized)
        return packed_projection(normalized, weight)
    out = torch.empty((rows, weight.size(0)), device=device, dtype=weight.dtype)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_norm_projection(
            _abi.ptr(x), x.stride(0), _abi.ptr(norm_weight), _abi.ptr(norm_bias), float(norm_eps),
            _abi.ptr(weight), _abi.ptr(out), rows, d_in, weight.size(0), _abi.code(weight),
            _abi.code(out), _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out


@norm_projection.register_fake
def _(x, norm_weight, norm_bias, weight, norm_eps):
    return x.new_empty((x.size(0), weight.size(0)), dtype=weight.dtype)


@torch.library.custom_op("relation_lm::decode_embed", mutates_args=(), device_types="cuda")
def decode_embed(tokens: Tensor, boundaries: Tensor, token_table: Tensor, boundary_table: Tensor,
                 position_table: Tensor, position: Tensor, scale: float) -> Tensor:
    """``(token_table[tokens] + boundary_table[boundaries]) * scale + position_table[position]``
    for one decode position, ``[B, d]`` fp32."""
    device = _abi.require_cuda_contiguous(tokens=tokens, boundaries=boundaries,
                                          token_table=token_table, boundary_table=boundary_table,
                                          position_table=position_table)
    _abi.require_position(position, device)
    if tokens.dtype != torch.int64 or boundaries.dtype != torch.int64 or position_table.dtype != torch.float32:
        raise ValueError("ids must be int64 and the position table float32")
    batch, d_model = tokens.numel(), token_table.size(1)
    out = torch.empty((batch, d_model), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_decode_embed(
            _abi.ptr(tokens), _abi.ptr(boundaries), _abi.ptr(token_table), _abi.ptr(boundary_table),
            _abi.ptr(position_table), _abi.ptr(position), float(scale), _abi.ptr(out), batch, d_model,
            token_table.size(0), boundary_table.size(0), position_table.size(0),
            _abi.same_dtype("embedding table", token_table, boundary_table),
            None, None, None, None, None, None, 0.0, 0,
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out


@decode_embed.register_fake
def _(tokens, boundaries, token_table, boundary_table, position_table, position, scale):
    return token_table.new_empty((tokens.numel(), token_table.size(1)), dtype=torch.float32)


@torch.library.custom_op("relation_lm::decode_embed_norm", mutates_args=("normalized1", "normalized2"),
                         device_types="cuda")
def decode_embed_norm(tokens: Tensor, boundaries: Tensor, token_table: Tensor, boundary_table: Tensor,
                      position_table: Tensor, position: Tensor, scale: float, norm1_weight: Tensor,
                      norm1_bias: Tensor, normalized1: Tensor, norm2_weight: Tensor, norm2_bias: Tensor,
                      normalized2: Tensor, norm_eps: float) -> Tensor:
    """``decode_embed`` that also writes two LayerNorms of the embedded rows as 16-bit matrices
    (``normalized1`` with the memory norm for the packed projection, ``normalized2`` with the first
    layer's input norm for its query projection); returns the fp32 rows."""
    device = _abi.require_cuda_contiguous(tokens=tokens, boundaries=boundaries,
                                          token_table=token_table, boundary_table=boundary_table,
                                          position_table=position_table, norm1_weight=norm1_weight,
                                          norm1_bias=norm1_bias, normalized1=normalized1,
                                          norm2_weight=norm2_weight, norm2_bias=norm2_bias,
                                          normalized2=normalized2)
    _abi.require_position(position, device)
    if tokens.dtype != torch.int64 or boundaries.dtype != torch.int64 or position_table.dtype != torch.float32:
        raise ValueError("ids must be int64 and the position table float32")
    batch, d_model = tokens.numel(), token_table.size(1)
    for t in (norm1_weight, norm1_bias, norm2_weight, norm2_bias):
        if t.dtype != torch.float32 or t.numel() != d_model:
            raise ValueError("LayerNorm parameters must be float32 [d_model]")
    if normalized1.shape != (batch, d_model) or normalized2.shape != (batch, d_model) \
            or normalized1.dtype != normalized2.dtype:
        raise ValueError("normalized outputs must be [B, d_model] of one 16-bit dtype")
    out = torch.empty((batch, d_model), device=device, dtype=torch.float32)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_decode_embed(
            _abi.ptr(tokens), _abi.ptr(boundaries), _abi.ptr(token_table), _abi.ptr(boundary_table),
            _abi.ptr(position_table), _abi.ptr(position), float(scale), _abi.ptr(out), batch, d_model,
            token_table.size(0), boundary_table.size(0), position_table.size(0),
            _abi.same_dtype("embedding table", token_table, boundary_table),
            _abi.ptr(norm1_weight), _abi.ptr(norm1_bias), _abi.ptr(normalized1),
            _abi.ptr(norm2_weight), _abi.ptr(norm2_bias), _abi.ptr(normalized2), float(norm_eps),
            _abi.code(normalized1), _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return out


@decode_embed_norm.register_fake
def _(tokens, boundaries, token_table, boundary_table, position_table, position, scale, norm1_weight,
      norm1_bias, normalized1, norm2_weight, norm2_bias, normalized2, norm_eps):
    return token_table.new_empty((tokens.numel(), token_table.size(1)), dtype=torch.float32)


def l2_prefetch(tensors: list[Tensor]) -> None:
    """Issue L2 prefetches for up to 16 CUDA tensors (their storage from the first element to the last), in
    order, on the current stream (extension; see ``rlm_l2_prefetch``).  Not a registered operator: it has no
    outputs and no effect on values."""
    import ctypes

    tensors = [t for t in tensors if t is not None and t.numel() > 0]
    if not tensors:
        return
    if len(tensors) > 16:
        raise ValueError("at most 16 tensors per call")
    device = tensors[0].device
    for t in tensors:
        if not t.is_cuda or t.device != device or not t.is_contiguous():
            raise ValueError("l2_prefetch takes contiguous CUDA tensors of one device")
    ranges = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    sizes = (ctypes.c_int64 * len(tensors))(*[t.numel() * t.element_size() for t in tensors])
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_l2_prefetch(ranges, sizes, len(tensors), _abi.stream_ptr(device)))


def decode_front_supported(batch: int, d_model: int, n_first: int, dtype: torch.dtype) -> bool:
    return batch <= 16 and d_model in (256, 512) and n_first % 8 == 0 and dtype in (torch.bfloat16, torch.float16)


@torch.library.custom_op("relation_lm::decode_front", mutates_args=("norm1_out", "norm2_out", "out_second"),
                         device_types="cuda")
def decode_front(tokens: Tensor, boundaries: Tensor, token_table: Tensor, boundary_table: Tensor,
                 position_table: Tensor, position: Tensor, scale: float, norm1_weight: Tensor, norm1_bias: Tensor,
                 norm2_weight: Tensor, norm2_bias: Tensor, norm_eps: float, weight: Tensor, n_first: int,
                 norm1_out: Tensor, norm2_out: Tensor, out_second: Tensor) -> tuple[Tensor, Tensor]:
    """The front of a decode step in one launch (extension): embedding of one position, two LayerNorms
    of the embedded rows and one projection of each — ``weight[:n_first]`` of the ``norm1`` rows (returned,
    ``[B, n_first]``) and ``weight[n_first:]`` of the ``norm2`` rows (into ``out_second``).  Also returns
    the embedded rows (fp32) and stores the two normalised copies.  At most 16 rows, ``d`` 256 or 512."""
    device = _abi.require_cuda_contiguous(
        tokens=tokens, boundaries=boundaries, token_table=token_table, boundary_table=boundary_table,
        position_table=position_table, norm1_weight=norm1_weight, norm1_bias=norm1_bias, norm2_weight=norm2_weight,
        norm2_bias=norm2_bias, weight=weight, norm1_out=norm1_out, norm2_out=norm2_out, out_second=out_second)
    _abi.require_position(position, device)
    if tokens.dtype != torch.int64 or boundaries.dtype != torch.int64:
        raise ValueError("token and boundary ids must be int64")
    batch, d_model = tokens.numel(), token_table.size(1)
    n_total = weight.size(0)
    n_first = int(n_first)
    if boundaries.numel() != batch or boundary_table.size(1) != d_model or position_table.size(1) != d_model \
            or weight.dim() != 2 or weight.size(1) != d_model or not 0 < n_first < n_total \
            or norm1_out.shape != (batch, d_model) or norm2_out.shape != (batch, d_model) \
            or out_second.shape != (batch, n_total - n_first):
        raise ValueError("decode_front: inconsistent shapes")
    for name, t in (("position_table", position_table), ("norm1_weight", norm1_weight), ("norm1_bias", norm1_bias),
                    ("norm2_weight", norm2_weight), ("norm2_bias", norm2_bias)):
        if t.dtype != torch.float32 or (name != "position_table" and t.numel() != d_model):
            raise ValueError(f"{name} must be float32 of the model width")
    dtype = _abi.same_dtype("16-bit operand", token_table, boundary_table, weight, norm1_out, norm2_out, out_second)
    hidden = torch.empty((batch, d_model), device=device, dtype=torch.float32)
    out_first = torch.empty((batch, n_first), device=device, dtype=weight.dtype)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_decode_front(
            _abi.ptr(tokens), _abi.ptr(boundaries), _abi.ptr(token_table), _abi.ptr(boundary_table),
            _abi.ptr(position_table), _abi.ptr(position), float(scale), _abi.ptr(norm1_weight), _abi.ptr(norm1_bias),
            _abi.ptr(norm2_weight), _abi.ptr(norm2_bias), float(norm_eps), _abi.ptr(weight), _abi.ptr(hidden),
            _abi.ptr(norm1_out), _abi.ptr(norm2_out), _abi.ptr(out_first), _abi.ptr(out_second), batch, d_model,
            n_first, n_total - n_first, token_table.size(0), boundary_table.size(0), position_table.size(0), dtype,
            _abi.ptr(_abi.status_tensor(device)), _abi.stream_ptr(device)))
    return hidden, out_first


@decode_front.register_fake
def _(tokens, boundaries, token_table, boundary_table, position_table, position, scale, norm1_weight, norm1_bias,
      norm2_weight, norm2_bias, norm_eps, weight, n_first, norm1_out, norm2_out, out_second):
    batch = tokens.numel()
    return (token_table.new_empty((batch, token_table.size(1)), dtype=torch.float32),
            weight.new_empty((batch, n_first)))


def greedy_token(logits: Tensor, vocab: int, position: Tensor | None = None) -> Tensor:
    """``logits[:, :vocab].argmax(-1)`` (ties to the lowest index) as int64 ``[rows]``; with
    ``position`` (a 0-d int64 device tensor) the position is advanced by one in the same launch."""
    return _greedy_token(logits, vocab, position)


@torch.library.custom_op("relation_lm::greedy_token", mutates_args=("position",), device_types="cuda")
def _greedy_token(logits: Tensor, vocab: int, position: Tensor | None) -> Tensor:
    device = _abi.require_cuda_rows(logits=logits)
    if logits.dim() != 2 or not 1 <= vocab <= logits.size(1):
        raise ValueError("logits must be [rows, >= vocab]")
    if position is not None:
        _abi.require_position(position, device)
    out = torch.empty((logits.size(0),), device=device, dtype=torch.int64)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_greedy_token(
            _abi.ptr(logits), logits.stride(0), _abi.ptr(out), _abi.ptr(position), logits.size(0),
            int(vocab), _abi.code(logits), _abi.stream_ptr(device)))
    return out


@_greedy_token.register_fake
def _(logits, vocab, position):
    return logits.new_empty((logits.size(0),), dtype=torch.int64)


def skinny_projection_supported(rows: int, d_in: int, dtype: torch.dtype) -> bool:
    """Whether ``skinny_projection`` serves these sizes (a handful of rows, a weight row in registers)."""
    return 1 <= rows <= 16 and d_in in (256, 512) and dtype in (torch.bfloat16, torch.float16)


@torch.library.custom_op("relation_lm::skinny_projection", mutates_args=(), device_types="cuda")
def skinny_projection(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    """``x [rows <= 16, d] @ weight [n, d].T (+ bias)`` on the CUDA cores (extension): for a decode
    batch the product is a stream of the weight matrix, read once by whole warps with no tensor-memory
    or tensor-map set-up.  Same contract as ``packed_projection``; ``d`` must be 256 or 512."""
    device = _abi.require_cuda_rows(x=x)
    _abi.require_cuda_contiguous(weight=weight, bias=bias)
    if weight.dim() != 2 or weight.size(1) != x.size(1) or x.dtype != weight.dtype:
        raise ValueError("weight must be [n_out, d_in] with the dtype of x")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != weight.size(0)):
        raise ValueError("bias must be float32 [n_out]")
    out = torch.empty((x.size(0), weight.size(0)), device=device, dtype=x.dtype)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_skinny_projection(
            _abi.ptr(x), x.stride(0), _abi.ptr(weight), _abi.ptr(bias), _abi.ptr(out), x.size(0), x.size(1),
            weight.size(0), _abi.code(x), 0, None, None, None, _abi.stream_ptr(device)))
    return out


@skinny_projection.register_fake
def _(x, weight, bias=None):
    return x.new_empty((x.size(0), weight.size(0)))


@torch.library.custom_op("relation_lm::skinny_projection_greedy", mutates_args=("scratch", "position"),
                         device_types="cuda")
def skinny_projection_greedy(x: Tensor, weight: Tensor, bias: Tensor | None, vocab: int, scratch: Tensor,
                             position: Tensor | None) -> tuple[Tensor, Tensor]:
    """The output head of a greedy decode step in one launch (extension): ``logits = x @ weight.T + bias``
    and ``next_token = logits[:, :vocab].argmax(-1)`` (lowest index on ties; int64), and with ``position``
    the device position advanced by one.  ``scratch``: a zeroed uint8 tensor of
    ``skinny_argmax_scratch_bytes()`` bytes, allocated once by the caller and left zero by every launch."""
    device = _abi.require_cuda_rows(x=x)
    _abi.require_cuda_contiguous(weight=weight, bias=bias, scratch=scratch)
    if weight.dim() != 2 or weight.size(1) != x.size(1) or x.dtype != weight.dtype:
        raise ValueError("weight must be [n_out, d_in] with the dtype of x")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != weight.size(0)):
        raise ValueError("bias must be float32 [n_out]")
    if scratch.dtype != torch.uint8 or scratch.numel() < skinny_argmax_scratch_bytes():
        raise ValueError("scratch must be a uint8 tensor of skinny_argmax_scratch_bytes() bytes")
    if not 1 <= vocab <= weight.size(0):
        raise ValueError("vocab must lie within the projection's outputs")
    if position is not None:
        _abi.require_position(position, device)
    out = torch.empty((x.size(0), weight.size(0)), device=device, dtype=x.dtype)
    next_token = torch.empty((x.size(0),), device=device, dtype=torch.int64)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_skinny_projection(
            _abi.ptr(x), x.stride(0), _abi.ptr(weight), _abi.ptr(bias), _abi.ptr(out), x.size(0), x.size(1),
            weight.size(0), _abi.code(x), int(vocab), _abi.ptr(scratch), _abi.ptr(next_token), _abi.ptr(position),
            _abi.stream_ptr(device)))
    return out, next_token


@skinny_projection_greedy.register_fake
def _(x, weight, bias, vocab, scratch, position):
    return x.new_empty((x.size(0), weight.size(0))), x.new_empty((x.size(0),), dtype=torch.int64)


@torch.library.custom_op("relation_lm::skinny_projection_greedy_into",
                         mutates_args=("scratch", "position", "next_token"), device_types="cuda")
def skinny_projection_greedy_into(x: Tensor, weight: Tensor, bias: Tensor | None, vocab: int, scratch: Tensor,
                                  position: Tensor | None, next_token: Tensor) -> Tensor:
    """``skinny_projection_greedy`` writing the chosen tokens into the caller's ``next_token`` ``[rows]``
    (int64) — which may be a device view of pinned host memory (``mapped_host_view``): the choice then
    reaches the host without a copy of its own.  Returns the logits."""
    device = _abi.require_cuda_rows(x=x)
    _abi.require_cuda_contiguous(weight=weight, bias=bias, scratch=scratch, next_token=next_token)
    if weight.dim() != 2 or weight.size(1) != x.size(1) or x.dtype != weight.dtype:
        raise ValueError("weight must be [n_out, d_in] with the dtype of x")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != weight.size(0)):
        raise ValueError("bias must be float32 [n_out]")
    if scratch.dtype != torch.uint8 or scratch.numel() < skinny_argmax_scratch_bytes():
        raise ValueError("scratch must be a uint8 tensor of skinny_argmax_scratch_bytes() bytes")
    if not 1 <= vocab <= weight.size(0):
        raise ValueError("vocab must lie within the projection's outputs")
    if next_token.dtype != torch.int64 or next_token.shape != (x.size(0),):
        raise ValueError("next_token must be int64 [rows]")
    if position is not None:
        _abi.require_position(position, device)
    out = torch.empty((x.size(0), weight.size(0)), device=device, dtype=x.dtype)
    with _abi.device_guard(device):
        _abi.check(_abi.LIB.rlm_skinny_projection(
            _abi.ptr(x), x.stride(0), _abi.ptr(weight), _abi.ptr(bias), _abi.ptr(out), x.size(0), x.size(1),
            weight.size(0), _abi.code(x), int(vocab), _abi.ptr(scratch), _abi.ptr(next_token), _abi.ptr(position),
            _abi.stream_ptr(device)))
    return out


@skinny_projection_greedy_into.register_fake
def _(x, weight, bias, vocab, scratch, position, next_token):
    return x.new_empty((x.size(0), weight.size(0)))


class _MappedHost:
    """Pinned host memory presented through ``__cuda_array_interface__`` (with unified addressing the
    device address of pinned memory is its host address)."""

    def __init__(self, host: Tensor) -> None:
        code = {torch.int64: "<i8", torch.int32: "<i4", torch.float32: "<f4", torch.uint8: "|u1"}[host.dtype]
        self.__cuda_array_interface__ = {"shape": tuple(host.shape), "typestr": code,
                                         "data": (host.data_ptr(), False), "version": 2}
        self.host = host


def mapped_host_view(host: Tensor, device: torch.device) -> Tensor:
    """A CUDA tensor over the pinned, contiguous host tensor ``host``: kernels that take it read or write
    the host memory directly (a few bytes of ids in, a few bytes of choices out: cheaper than a copy node
    per transfer in a decode graph).  The host sees a kernel's writes once the stream is synchronised.  The
    view keeps ``host`` alive."""
    if host.is_cuda or not host.is_pinned() or not host.is_contiguous():
        raise ValueError("mapped_host_view takes a pinned, contiguous host tensor")
    holder = _MappedHost(host)
    view = torch.as_tensor(holder, device=device)
    if view.data_ptr() != host.data_ptr() or not view.is_cuda:
        raise RuntimeError("the device view does not alias the host tensor")
    view._mapped_host = holder
    return view


def skinny_argmax_scratch_bytes() -> int:
    return int(_abi.LIB.rlm_skinny_argmax_scratch_bytes())
