"""CPU-only checks of the C-ABI boundary and of the host-side argument validation (no compute calls)."""

import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            with open(os.path.join(inc, fn)) as f:
                text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
            names |= set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    from nki_library_b200 import _lib
    lib = _lib.load_library()
    declared = _declared_symbols()
    assert len(declared) >= 18
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == declared
    assert lib.b200moe_version() >= 100
    assert lib.b200moe_last_error() is not None


def test_sf_bytes_query():
    from nki_library_b200 import _lib
    lib = _lib.load_library()
    assert lib.b200moe_sf_bytes(128, 128) == 512
    assert lib.b200moe_sf_bytes(129, 4096) == 2 * 32 * 512
    assert lib.b200moe_group_tokens_workspace_bytes(32768, 128) >= 128 * 128 * 4


def test_invalid_arguments_return_status_and_message():
    from nki_library_b200 import _lib
    lib = _lib.load_library()
    rc = lib.b200moe_router_topk(None, 1, None, None, 4, 128, 8, 2, 1, 1, 0, None, 0, None, None, 0, 0, None, 0, None)
    assert rc == -1 and b"must not be null" in lib.b200moe_last_error()
    rc = lib.b200moe_router_topk(1, 1, 1, None, 4, 128, 8, 2, 1, 1, 0, None, 0, None, None, 0, 7, None, 0, None)
    assert rc == -1 and b"path must be 0, 1 or 2" in lib.b200moe_last_error()
    with pytest.raises(AssertionError, match=r"\[INTERNAL_ERROR\] \[NCC_INKI016\] Kernel validation exception"):
        _lib.call("b200moe_combine", None, None, 1, 1, 8, None, None)


def test_python_api_mirrors_reference_names_and_defaults():
    import inspect

    import nki_library_b200 as m
    sig = inspect.signature(m.moe_cte._fn)
    names = list(sig.parameters)
    assert names[:8] == ["hidden_states", "expert_affinities_masked", "gate_up_proj_weight", "down_proj_weight",
                         "token_position_to_id", "block_to_expert", "block_size", "spec"]
    assert sig.parameters["activation_function"].default == m.ActFnType.SiLU
    assert sig.parameters["expert_affinities_scaling_mode"].default == m.ExpertAffinityScaleMode.POST_SCALE
    sig = inspect.signature(m.moe_tkg._fn)
    assert list(sig.parameters)[:6] == ["hidden_input", "expert_gate_up_weights", "expert_down_weights",
                                        "expert_affinities", "expert_index", "is_all_expert"]
    assert sig.parameters["expert_affinities_scaling_mode"].default == m.ExpertAffinityScaleMode.NO_SCALE
    sig = inspect.signature(m.router_topk._fn)
    assert list(sig.parameters)[:10] == ["x", "w", "w_bias", "router_logits", "expert_affinities", "expert_index",
                                         "act_fn", "k", "x_hbm_layout", "x_sb_layout"]
    assert [e.value for e in m.MoECTEImplementation] == list(range(7))
    assert m.get_n_blocks(256, 2, 4, 128, 2) == 8 and m.get_n_blocks(4096, 2, 8, 512) == 23
    assert m.get_n_blocks(8192, 8, 256, 128) == 766 and m.get_n_blocks(32768, 8, 128, 256) == 1151
    assert m.moe_cte[2] is m.moe_cte._fn  # kernel[grid] call form


def test_cpu_tensors_are_rejected_not_silently_computed():
    import nki_library_b200 as m
    with pytest.raises(AssertionError, match="CUDA"):
        m.find_nonzero_indices(torch.zeros(8, 4))
    with pytest.raises(AssertionError, match="CUDA"):
        m.cumsum(torch.zeros(8, 4))
    with pytest.raises(AssertionError, match="CUDA"):
        m.moe_cte(torch.zeros(1), torch.zeros(1), None, None, torch.zeros(1), torch.zeros(1), 128,
                  m.MoECTESpec(m.MoECTEImplementation.shard_on_block))
    with pytest.raises(AssertionError, match="pre-scale"):
        m.moe_tkg(torch.zeros(4, 512), None, None, torch.zeros(4, 8), torch.zeros(4, 2), False,
                  expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.PRE_SCALE)
