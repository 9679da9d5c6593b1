"""Helpers for the GPU parity tests: move seeded CPU inputs to the device, call the operators."""
from __future__ import annotations

import torch

SELECT_KEYS = ("anchor_query", "anchor_keys", "anchor_router_query", "anchor_mean", "anchor_std",
               "anchor_gamma", "anchor_bias", "partner_base", "partner_anchor_cache",
               "partner_keys", "partner_mean", "partner_std", "partner_gamma", "partner_bias")


def to_cuda(x: dict) -> dict:
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in x.items()}


def position_tensor(t: int) -> torch.Tensor:
    return torch.tensor(int(t), device="cuda", dtype=torch.long)


def select_args(x: dict) -> list:
    return [x[k] for k in SELECT_KEYS]


def assert_status_clear() -> None:
    from relation_lm.kernels import _abi

    assert _abi.read_status() == 0, "a kernel reported a device-side error"


def assert_scores_equal(got: torch.Tensor, want: torch.Tensor) -> None:
    """Bit-for-bit equality of fp32 scores (infinities included)."""
    assert torch.equal(got.cpu().view(torch.int32), want.view(torch.int32)), \
        (got.cpu() - want).abs().nan_to_num(0).max()


def assert_rel_close(got: torch.Tensor, want: torch.Tensor, rel: float = 1.0e-2, what: str = "") -> None:
    """Relative-to-the-row bound: every element of ``got`` lies within ``rel`` times the largest
    magnitude of its own row of ``want`` (rows = last dimension).  Unlike ``atol + rtol * |x|``
    the bound does not loosen for rows of small values."""
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    scale = want.abs().amax(-1, keepdim=True)
    err = (got - want).abs()
    bound = rel * scale + 1.0e-7
    assert bool((err <= bound).all()), (what, float((err / (scale + 1.0e-30)).max()))
