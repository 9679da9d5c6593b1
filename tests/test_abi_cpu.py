"""CPU-side checks of the boundary: the library loads, exports what the header declares,
registers the reference's operator names and schemas, and refuses CPU tensors."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "relation_lm_b200.h"
LIBRARY = ROOT / "relation-lm_b200" / "lib" / "librelation_lm_b200.so"


def _declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(rlm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    assert LIBRARY.exists(), "build the library first: python -c 'import __graft_entry__ as g; g.build()'"
    lib = ctypes.CDLL(str(LIBRARY))
    names = _declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    lib.rlm_abi_version.restype = ctypes.c_int
    from relation_lm.kernels import _abi

    assert lib.rlm_abi_version() == _abi.ABI_VERSION == 2


def test_binding_prototypes_cover_the_header():
    from relation_lm.kernels import _abi

    bound = set(_abi.PROTOTYPES) | {"rlm_abi_version", "rlm_last_error", "rlm_launch_count",
                                    "rlm_relation_tail_scratch_bytes", "rlm_skinny_argmax_scratch_bytes"}
    assert set(_declared_symbols()) <= bound


EXPECTED_SCHEMAS = {
    ("relation_lm", "relation_select_packed"):
        "(Tensor anchor_query, Tensor anchor_keys, Tensor anchor_router_query, Tensor anchor_block_mean, "
        "Tensor anchor_block_std, Tensor anchor_gamma, Tensor anchor_bias, Tensor partner_base, "
        "Tensor partner_anchor_cache, Tensor partner_keys, Tensor partner_block_mean, Tensor partner_block_std, "
        "Tensor partner_gamma, Tensor partner_bias, Tensor position, SymInt local_window, SymInt top_blocks, "
        "SymInt k_out, bool strict_valid) -> (Tensor, Tensor, Tensor, Tensor)",
    ("relation_lm", "relation_hidden_cached"):
        "(Tensor expanded_cache, Tensor operand_cache, Tensor anchor_index, Tensor partner_index, "
        "Tensor product_weight) -> Tensor",
    ("relation_lm", "relation_hidden_cache_update"):
        "(Tensor(a0!) expanded_cache, Tensor operand_cache, Tensor anchor_index, Tensor partner_index, "
        "Tensor anchor_weight, Tensor partner_weight, Tensor product_weight, Tensor first_bias, "
        "Tensor position) -> Tensor",
    ("relation_lm", "relation_norm_reduce"):
        "(Tensor raw, Tensor partner_scores, Tensor norm_weight, Tensor norm_bias, Tensor position, "
        "float norm_eps) -> Tensor",
    ("relation_lm", "router_cache_update"):
        "(Tensor anchor_raw, Tensor partner_raw, Tensor(a2!) anchor_raw_cache, Tensor(a3!) partner_raw_cache, "
        "Tensor(a4!) anchor_conv_cache, Tensor(a5!) partner_conv_cache, Tensor(a6!) anchor_mean, "
        "Tensor(a7!) anchor_std, Tensor(a8!) partner_mean, Tensor(a9!) partner_std, Tensor anchor_conv_weight, "
        "Tensor partner_conv_weight, Tensor position, SymInt block_size) -> Tensor",
    ("relationlex", "anchor_select"):
        "(Tensor anchor_query, Tensor anchor_keys, Tensor router_query, Tensor block_mean, Tensor block_std, "
        "Tensor gamma, Tensor bias, Tensor position, SymInt local_window, SymInt top_blocks, "
        "bool strict_valid) -> (Tensor, Tensor)",
    ("relationlex", "partner_topk"):
        "(Tensor partner_query, Tensor partner_keys, Tensor router_query, Tensor block_mean, Tensor block_std, "
        "Tensor gamma, Tensor bias, Tensor position, Tensor anchor_index, SymInt local_window, "
        "SymInt top_blocks, SymInt k_out, bool strict_valid) -> (Tensor, Tensor)",
}


def test_operator_schemas_match_the_reference():
    """Schemas printed from the reference's registered ops (its kernels/*.py decorators)."""
    import relation_lm.kernels.relation_reduce  # noqa: F401
    import relation_lm.kernels.relation_select  # noqa: F401
    import relation_lm.kernels.router_cache  # noqa: F401
    import relation_lm.kernels.triton_select  # noqa: F401

    for (namespace, name), expected in EXPECTED_SCHEMAS.items():
        schema = str(getattr(getattr(torch.ops, namespace), name).default._schema)
        assert schema == f"{namespace}::{name}{expected}", schema


def test_operators_refuse_cpu_tensors():
    from relation_lm.kernels.relation_reduce import relation_norm_reduce

    with pytest.raises(NotImplementedError):
        relation_norm_reduce(torch.randn(1, 8, 16), torch.randn(1, 8), torch.ones(16),
                             torch.zeros(16), torch.tensor(3), 1e-5)


def test_helper_functions_follow_the_reference():
    from relation_lm.inference import pack_sparse_cache_projection_weights
    from relation_lm.kernels.relation_reduce import (
        factor_relation_first_layer,
        recommended_relation_cache_mode,
    )

    assert recommended_relation_cache_mode(1) == "fused_update"
    assert recommended_relation_cache_mode(8) == "separate_update"
    with pytest.raises(ValueError):
        recommended_relation_cache_mode(0)
    with pytest.raises(ValueError):
        factor_relation_first_layer(torch.randn(8, 30), torch.randn(8), 8)
    with pytest.raises(ValueError):
        pack_sparse_cache_projection_weights((torch.randn(4, 8), torch.randn(4, 9)), names=("a", "b"))
    # exact factorisation identity on CPU tensors
    g = torch.Generator().manual_seed(7)
    w, b = torch.randn(32, 64, generator=g), torch.randn(32, generator=g)
    f = factor_relation_first_layer(w, b, 16)
    a, p = torch.randn(5, 16, generator=g), torch.randn(5, 16, generator=g)
    direct = torch.nn.functional.linear(torch.cat((a, p, a * p, a - p), -1), w, b)
    split = (torch.nn.functional.linear(a, f.anchor_weight, f.first_bias)
             + torch.nn.functional.linear(p, f.partner_weight)
             + torch.nn.functional.linear(a * p, f.product_weight))
    assert torch.allclose(direct, split, atol=1e-5)


def test_programmatic_launch_switch_belongs_to_the_calling_thread():
    """A decode loop that turns programmatic launch on in its own thread must not change how
    another thread's operators are launched, whatever the interleaving."""
    import threading

    from relation_lm.kernels import _abi

    assert _abi.set_programmatic_launch(False) is False
    seen = {}
    a_on, b_done = threading.Event(), threading.Event()

    def decoder_thread():
        seen["a_before"] = _abi.set_programmatic_launch(True)
        a_on.set()
        b_done.wait(10)
        seen["a_restore"] = _abi.set_programmatic_launch(False)     # what this thread had set: True

    def other_thread():
        a_on.wait(10)
        seen["b_sees"] = _abi.set_programmatic_launch(False)        # untouched by the first thread
        b_done.set()

    threads = [threading.Thread(target=decoder_thread), threading.Thread(target=other_thread)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(20)
    assert seen == {"a_before": False, "a_restore": True, "b_sees": False}
    assert _abi.set_programmatic_launch(False) is False              # and the main thread never saw it
