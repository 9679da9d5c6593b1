"""CPU oracle for the routed selection-and-reduction path — TEST INFRASTRUCTURE ONLY.

Python binding (ctypes) of ``relation_oracle.c``.  Only the test-suite, the
smoke check and the benchmark's CPU-baseline leg may import this package; the
shipped library never does and has no CPU fallback.

Every function takes CPU torch tensors of any float dtype (bf16/fp16 are
up-cast exactly to fp32, as the GPU kernels do on load) and returns fp32 /
int32 torch tensors.  The algorithms follow the reference kernels cited in
``relation_oracle.c``; the outputs are pinned by ``tests/golden``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np
import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "liboracle.so"
_lib = None

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def build(force: bool = False) -> Path:
    """Compile ``liboracle.so`` with the Makefile beside this file."""
    src = _HERE / "relation_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _lib.orc_expf.restype = ctypes.c_float
        _lib.orc_expf.argtypes = [ctypes.c_float]
        _lib.orc_logf.restype = ctypes.c_float
        _lib.orc_logf.argtypes = [ctypes.c_float]
    return _lib


def _f32(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().to("cpu", torch.float32).contiguous().numpy())


def _i32(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().to("cpu", torch.int32).contiguous().numpy())


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _rows(n_rows: int, position, row_batch, row_pos):
    if row_batch is None:
        row_batch = torch.arange(n_rows, dtype=torch.int32)
        row_pos = torch.full((n_rows,), int(position), dtype=torch.int32)
    return _i32(row_batch), _i32(row_pos)


def _check(rc: int, name: str) -> None:
    if rc != 0:
        raise ValueError(f"oracle {name} rejected its arguments (code {rc})")


def relation_select(aq, ak, arq, amean, astd, agamma, abias, pbase, pac, pk, pmean, pstd,
                    pgamma, pbias, position, local_window, top_blocks, k_out, strict_valid,
                    row_batch=None, row_pos=None):
    """Fused selection; returns (anchor, anchor_score, partner, partner_score, scored).

    ``scored`` = (anchor key rows scored, partner key rows scored) summed over rows.
    With ``row_batch``/``row_pos`` the queries are per-row ``[N, ...]`` against
    caches ``[B, T, ...]``; otherwise row ``i`` is sequence ``i`` at ``position``.
    """
    n = aq.shape[0]
    n_seq, max_t = ak.shape[0], ak.shape[1]
    nb, buckets = amean.shape[1], abias.shape[1]
    rb, rp = _rows(n, position, row_batch, row_pos)
    arrs = [_f32(x) for x in (aq, ak, arq, amean, astd, agamma, abias, pbase, pac, pk, pmean,
                              pstd, pgamma, pbias)]
    oa = np.empty(n, np.int32)
    oas = np.empty(n, np.float32)
    op = np.empty((n, k_out), np.int32)
    ops = np.empty((n, k_out), np.float32)
    scored = np.zeros(2, np.int64)
    rc = lib().orc_relation_select(n, n_seq, max_t, nb, buckets, _p(rb), _p(rp),
                                   *[_p(a) for a in arrs], int(local_window), int(top_blocks),
                                   int(k_out), int(bool(strict_valid)), _p(oa), _p(oas), _p(op),
                                   _p(ops), _p(scored))
    _check(rc, "relation_select")
    return (torch.from_numpy(oa), torch.from_numpy(oas), torch.from_numpy(op),
            torch.from_numpy(ops), (int(scored[0]), int(scored[1])))


def _exclusions(exclude_index):
    if exclude_index is None or exclude_index.shape[1] == 0:
        return None, 0
    arr = _i32(exclude_index)
    return arr, arr.shape[1]


def anchor_select(aq, ak, rq, mean, std, gamma, bias, position, local_window, top_blocks,
                  strict_valid, row_batch=None, row_pos=None, exclude_index=None):
    n = aq.shape[0]
    rb, rp = _rows(n, position, row_batch, row_pos)
    arrs = [_f32(x) for x in (aq, ak, rq, mean, std, gamma, bias)]
    ex, n_ex = _exclusions(exclude_index)
    oi = np.empty(n, np.int32)
    osc = np.empty(n, np.float32)
    rc = lib().orc_anchor_select(n, ak.shape[0], ak.shape[1], mean.shape[1], bias.shape[1],
                                 _p(rb), _p(rp), *[_p(a) for a in arrs], int(local_window),
                                 int(top_blocks), int(bool(strict_valid)), _p(ex), n_ex, _p(oi), _p(osc))
    _check(rc, "anchor_select")
    return torch.from_numpy(oi), torch.from_numpy(osc)


def partner_topk(pq, pk, rq, mean, std, gamma, bias, position, anchor_index, local_window,
                 top_blocks, k_out, strict_valid, row_batch=None, row_pos=None, exclude_index=None):
    n = pq.shape[0]
    rb, rp = _rows(n, position, row_batch, row_pos)
    arrs = [_f32(x) for x in (pq, pk, rq, mean, std, gamma, bias)]
    anchor = _i32(anchor_index)
    ex, n_ex = _exclusions(exclude_index)
    oi = np.empty((n, k_out), np.int32)
    osc = np.empty((n, k_out), np.float32)
    rc = lib().orc_partner_topk(n, pk.shape[0], pk.shape[1], mean.shape[1], bias.shape[1],
                                _p(rb), _p(rp), *[_p(a) for a in arrs], _p(anchor),
                                int(local_window), int(top_blocks), int(k_out),
                                int(bool(strict_valid)), _p(ex), n_ex, _p(oi), _p(osc))
    _check(rc, "partner_topk")
    return torch.from_numpy(oi), torch.from_numpy(osc)


def block_scores(mean, std, rq, gamma, bias, position, max_t, local_window, strict_valid):
    """Block scores of one query against one sequence's stats ``[NB, 4, 16]``."""
    nb = mean.shape[0]
    out = np.empty(nb, np.float32)
    arrs = [_f32(x) for x in (mean, std, rq, gamma, bias)]
    rc = lib().orc_block_scores(int(max_t), nb, bias.shape[1], int(position),
                                *[_p(a) for a in arrs], int(local_window),
                                int(bool(strict_valid)), _p(out))
    _check(rc, "block_scores")
    return torch.from_numpy(out)


def router_cache_update(anchor_raw, partner_raw, anchor_raw_cache, partner_raw_cache,
                        anchor_conv_cache, partner_conv_cache, anchor_mean, anchor_std,
                        partner_mean, partner_std, anchor_conv_weight, partner_conv_weight,
                        position, block_size, inplace=False, cache_dtype=None, stats_dtype=None):
    """Returns (out, new_state dict).

    Stores are rounded to the dtype of the cache / stats tensors passed in (or to
    ``cache_dtype`` / ``stats_dtype`` when given).  With ``inplace=True`` the eight state
    tensors must be fp32 contiguous CPU tensors and are updated where they lie.
    """
    batch, max_t = anchor_raw_cache.shape[0], anchor_raw_cache.shape[1]
    nb = anchor_mean.shape[1]
    names = ("anchor_raw_cache", "partner_raw_cache", "anchor_conv_cache", "partner_conv_cache",
             "anchor_mean", "anchor_std", "partner_mean", "partner_std")
    tensors = (anchor_raw_cache, partner_raw_cache, anchor_conv_cache, partner_conv_cache,
               anchor_mean, anchor_std, partner_mean, partner_std)
    if inplace:
        if any(t.dtype != torch.float32 or not t.is_contiguous() for t in tensors):
            raise ValueError("inplace update needs fp32 contiguous state")
        state = [t.numpy() for t in tensors]
    else:
        state = [_f32(x).copy() for x in tensors]
    araw, praw = _f32(anchor_raw), _f32(partner_raw)
    aw, pw = _f32(anchor_conv_weight), _f32(partner_conv_weight)
    out = np.empty((batch, 2, 64), np.float32)
    rc = lib().orc_router_cache_update(
        batch, max_t, nb, int(block_size), int(position), _p(araw),
        ctypes.c_int64(araw.shape[1]), _p(praw), ctypes.c_int64(praw.shape[1]),
        *[_p(a) for a in state], _p(aw), _p(pw),
        DTYPE_CODE[cache_dtype or anchor_raw_cache.dtype],
        DTYPE_CODE[stats_dtype or anchor_mean.dtype], _p(out))
    _check(rc, "router_cache_update")
    new_state = {n: torch.from_numpy(a).reshape(t.shape) for n, a, t in zip(names, state, tensors)}
    return torch.from_numpy(out), new_state


def relation_hidden(expanded_cache, operand_cache, anchor_index, partner_index, product_weight,
                    anchor_weight=None, partner_weight=None, first_bias=None, position=None,
                    row_batch=None, row_pos=None, inplace=False, cache_dtype=None):
    """``relation_hidden_cached`` (no weights/position) or ``relation_hidden_cache_update``.

    Returns (hidden ``[N, K, H]``, expanded cache after the update).  With ``inplace=True`` the
    expanded cache must be an fp32 contiguous CPU tensor and is updated where it lies.
    """
    update = anchor_weight is not None
    n, k_out = partner_index.shape
    n_seq, max_t, rdim = operand_cache.shape
    hdim = product_weight.shape[0]
    rb, rp = _rows(n, position if position is not None else 0, row_batch, row_pos)
    if inplace:
        if expanded_cache.dtype != torch.float32 or not expanded_cache.is_contiguous():
            raise ValueError("inplace update needs an fp32 contiguous expanded cache")
        ex = expanded_cache.numpy()
    else:
        ex = _f32(expanded_cache).copy()
    op = _f32(operand_cache)
    ai, pi = _i32(anchor_index), _i32(partner_index)
    wm = _f32(product_weight)
    wa = _f32(anchor_weight) if update else None
    wp = _f32(partner_weight) if update else None
    fb = _f32(first_bias) if update else None
    out = np.empty((n, k_out, hdim), np.float32)
    rc = lib().orc_relation_hidden(n, n_seq, max_t, rdim, hdim, k_out, _p(rb), _p(rp), _p(ex),
                                   _p(op), _p(ai), _p(pi), _p(wa), _p(wp), _p(wm), _p(fb),
                                   int(update), DTYPE_CODE[cache_dtype or expanded_cache.dtype],
                                   _p(out))
    _check(rc, "relation_hidden")
    return torch.from_numpy(out), torch.from_numpy(ex).reshape(expanded_cache.shape)


def relation_norm_reduce(raw, partner_scores, norm_weight, norm_bias, position, norm_eps,
                         row_pos=None):
    n, k_out, dim = raw.shape
    if k_out > 64:
        raise ValueError("oracle supports at most 64 partner slots")
    rp = _i32(torch.full((n,), int(position), dtype=torch.int32) if row_pos is None else row_pos)
    arrs = [_f32(x) for x in (raw, partner_scores, norm_weight, norm_bias)]
    out = np.empty((n, dim), np.float32)
    rc = lib().orc_relation_norm_reduce(n, k_out, dim, _p(rp), *[_p(a) for a in arrs],
                                        ctypes.c_float(norm_eps), _p(out))
    _check(rc, "relation_norm_reduce")
    return torch.from_numpy(out)


def linear(x, weight):
    """``x @ weight.T`` accumulated in double."""
    xs = _f32(x).reshape(-1, x.shape[-1])
    w = _f32(weight)
    out = np.empty((xs.shape[0], w.shape[0]), np.float32)
    rc = lib().orc_linear(xs.shape[0], xs.shape[1], w.shape[0], _p(xs), _p(w), _p(out))
    _check(rc, "linear")
    return torch.from_numpy(out).reshape(*x.shape[:-1], w.shape[0])


def set_threads(n: int) -> None:
    """Limit the OpenMP team used by the oracle (0 = all host threads)."""
    os.environ["OMP_NUM_THREADS"] = str(n) if n > 0 else str(os.cpu_count() or 1)
    try:
        gomp = ctypes.CDLL("libgomp.so.1")
        gomp.omp_set_num_threads(int(n) if n > 0 else int(os.cpu_count() or 1))
    except OSError:
        pass
