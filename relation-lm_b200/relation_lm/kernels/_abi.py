"""ctypes binding of ``librelation_lm_b200.so`` (declared in include/relation_lm_b200.h)."""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

ABI_VERSION = 2          # RLM_ABI_VERSION of include/relation_lm_b200.h this binding was written against
_LIB_PATH = Path(__file__).resolve().parents[2] / "lib" / "librelation_lm_b200.so"

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

# name -> argument types, in the order of include/relation_lm_b200.h
PROTOTYPES = {
    "rlm_relation_select_packed": [_P] * 21 + [_L] * 3 + [_I] * 13 + [_P, _P],
    "rlm_anchor_select": [_P] * 11 + [_I] + [_P] * 2 + [_I] * 12 + [_P, _P],
    "rlm_partner_topk": [_P] * 12 + [_I] + [_P] * 2 + [_I] * 13 + [_P, _P],
    "rlm_router_cache_update": [_P, _L, _P, _L] + [_P] * 12 + [_I] * 8 + [_P, _P],
    "rlm_relation_hidden_cached": [_P] * 7 + [_I] * 9 + [_P, _P],
    "rlm_relation_hidden_cache_update": [_P] * 10 + [_I] * 8 + [_P, _P],
    "rlm_relation_norm_reduce": [_P] * 6 + [_F, _P, _P, _P, _P, _P, _F, _P, _I, _I, _L, _P] + [_I] * 5 + [_P, _P],
    "rlm_relation_norm_reduce_project": [_P] * 5 + [_F, _P, _P, _P, _P, _F, _P, _P, _P, _I, _I, _P] + [_I] * 5 + [_P, _P],
    "rlm_router_cache_prefill": [_P, _L, _L, _P, _L, _L] + [_P] * 10 + [_I] * 9 + [_P],
    "rlm_packed_projection": [_P, _L, _P, _P, _P] + [_I] * 6 + [_P, _P],
    "rlm_greedy_token": [_P, _L, _P, _P] + [_I] * 3 + [_P],
    "rlm_norm_projection": [_P, _L, _P, _P, _F, _P, _P] + [_I] * 5 + [_P, _P],
    "rlm_set_programmatic_launch": [_I],
    "rlm_expanded_cache_append": [_P] * 6 + [_I] * 6 + [_P, _P],
    "rlm_expanded_cache_append_packed": [_P, _P, _L, _I, _I] + [_P] * 4 + [_I] * 6 + [_P, _P],
    "rlm_layer_norm_cast": [_P, _L, _P, _P, _F, _P] + [_I] * 3 + [_P],
    "rlm_relation_tail": [_P] * 7 + [_F] + [_P] * 4 + [_L] + [_I] * 5 + [_P, _P],
    "rlm_relation_tail_static": [_P] * 7 + [_F] + [_P] * 3 + [_I] * 5 + [_P, _P],
    "rlm_decode_embed": [_P] * 6 + [_F, _P] + [_I] * 6 + [_P] * 6 + [_F, _I] + [_P, _P],
    "rlm_sparse_cache_append": [_P, _L, _I] + [_P] * 16 + [_I] * 9 + [_P, _P],
    "rlm_selftest_bounded_wait": [_P, _L, _P, _P],
    "rlm_relation_select_packed_prefill": [_P] * 18 + [_L] * 3 + [_I] * 13 + [_P, _P],
    "rlm_relation_select_multi_rows": [_P] * 21 + [_L] * 3 + [_I] * 14 + [_P, _P],
    "rlm_relation_select_multi_prefill": [_P] * 19 + [_L] * 3 + [_I] * 14 + [_P, _P],
    "rlm_slot_mix_residual": [_P] * 5 + [_I] * 3 + [_P],
    "rlm_skinny_projection": [_P, _L, _P, _P, _P] + [_I] * 5 + [_P] * 4,
    "rlm_packed_projection_append": [_P, _L, _P, _P, _I] + [_P] * 15 + [_I] * 7 + [_P, _P],
    "rlm_l2_prefetch": [_P, _P, _I, _P],
    "rlm_state_slide": [_P, _P, _P, _P, _P, _I, _P],
    "rlm_decode_front": [_P] * 6 + [_F] + [_P] * 4 + [_F] + [_P] * 6 + [_I] * 8 + [_P, _P],
    "rlm_relation_layer_tail_supported": [_I] * 7,
    "rlm_relation_layer_tail": [_P] * 11 + [_F, _P, _P, _P, _P, _F, _P, _P, _P] + [_I] * 8 + [_P, _P],
    "rlm_relation_layer_supported": [_I] * 12,
    "rlm_relation_layer": [_P] * 19 + [_L] * 3 + [_I] * 6 + [_P] * 7 + [_F, _P, _P, _P, _P, _F, _P, _P, _P]
                          + [_I] * 8 + [_P, _P],
}


def _load() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `make -C {_LIB_PATH.parents[1] / 'csrc'}` "
            "(nvcc, sm_100a).  relation_lm has no fallback implementation.")
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, argtypes in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int
    lib.rlm_abi_version.restype = ctypes.c_int
    lib.rlm_last_error.restype = ctypes.c_char_p
    lib.rlm_launch_count.restype = ctypes.c_int64
    lib.rlm_skinny_argmax_scratch_bytes.argtypes = []
    lib.rlm_skinny_argmax_scratch_bytes.restype = ctypes.c_int64
    lib.rlm_relation_tail_scratch_bytes.argtypes = [_I, _I, _I]
    lib.rlm_relation_tail_scratch_bytes.restype = ctypes.c_int64
    if lib.rlm_abi_version() != ABI_VERSION:
        raise ImportError("librelation_lm_b200.so has an unexpected ABI version")
    return lib


LIB = _load()

_STATUS: dict[int, torch.Tensor] = {}


def status_tensor(device: torch.device) -> torch.Tensor:
    """Per-device int32 word the kernels OR device-side error bits into."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _STATUS.get(index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
        _STATUS[index] = word
    return word


def read_status(device: torch.device | None = None, clear: bool = True) -> int:
    """Synchronise and return the device-side error bits (0 = none).

    Bit 1: a bounded wait on a bulk copy expired; bit 2: a position or row index
    lay outside the caches.  The affected rows were left unwritten.
    """
    device = device or torch.device("cuda", torch.cuda.current_device())
    word = status_tensor(device)
    value = int(word.item())
    if clear and value:
        word.zero_()
    return value


def launch_count() -> int:
    """Kernels launched by the library in this process."""
    return int(LIB.rlm_launch_count())


def set_programmatic_launch(enabled: bool) -> bool:
    """Switch programmatic dependent launch of the library's kernels on or off; returns the
    previous setting.  While it is on, the caches, block statistics and position given to a
    selector must not be written by the kernel launched just before it on the same stream."""
    return bool(LIB.rlm_set_programmatic_launch(1 if enabled else 0))


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device):
    return torch.cuda.current_stream(device).cuda_stream


def code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}; use float32, bfloat16 or float16") from None


def same_dtype(name: str, *tensors: torch.Tensor) -> int:
    first = tensors[0].dtype
    if any(t.dtype != first for t in tensors):
        raise ValueError(f"{name} tensors must share one dtype, got {[t.dtype for t in tensors]}")
    return code(tensors[0])


def require_cuda_rows(**tensors: torch.Tensor) -> torch.device:
    """2-D CUDA tensors whose rows are dense (unit inner stride); the row stride is free."""
    device = None
    for name, t in tensors.items():
        if not t.is_cuda:
            raise NotImplementedError(
                f"{name} is on {t.device}: relation_lm operators run on CUDA devices only")
        if t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"{name} must be 2-D with unit inner stride")
        if device is not None and t.device != device:
            raise ValueError(f"{name} is on {t.device}, expected {device}")
        device = t.device
    return device


def require_cuda_contiguous(**tensors: torch.Tensor) -> torch.device:
    device = None
    for name, t in tensors.items():
        if t is None:
            continue
        if not t.is_cuda:
            raise NotImplementedError(
                f"{name} is on {t.device}: relation_lm operators run on CUDA devices only")
        if device is None:
            device = t.device
        elif t.device != device:
            raise ValueError(f"{name} is on {t.device}, expected {device}")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    return device


def check(rc: int) -> None:
    if rc == 0:
        return
    message = LIB.rlm_last_error().decode() or f"status {rc}"
    if rc in (-1, -2, -3, -4, -5, -7):
        raise ValueError(message)
    raise RuntimeError(message)


def require_position(position: torch.Tensor, device: torch.device) -> None:
    if position.device != device or position.dtype != torch.int64 or position.numel() != 1:
        raise ValueError("position must be a one-element int64 tensor on the operands' device")


class device_guard:
    """Makes ``device`` current for the launch when it is not already."""

    def __init__(self, device: torch.device):
        self.device = device
        self.previous = None

    def __enter__(self):
        current = torch.cuda.current_device()
        if self.device.index is not None and self.device.index != current:
            self.previous = current
            torch.cuda.set_device(self.device.index)

    def __exit__(self, *exc):
        if self.previous is not None:
            torch.cuda.set_device(self.previous)
