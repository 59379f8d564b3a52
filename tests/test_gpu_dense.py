"""The non-MX variants of ``moe_cte`` / ``moe_tkg`` (bf16 and fp8-row weights, PRE_SCALE) on the dense tcgen05
kernels, against outputs of the reference's ``moe_cte_torch_ref`` / ``moe_tkg_torch_ref`` (tests/golden/mx_ref.npz,
parts ``dense_cte`` and ``dense_tkg``).  Tolerance: max|a - ref| / max|ref| <= 2e-2; the GPU rounds the SwiGLU
product to bf16 before the down projection (its operand type) where the CPU reference keeps fp32."""

import os

import numpy as np
import pytest
import torch

import golden_inputs as gi
from moe_testlib import max_rel

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
TOL = 2e-2
_ACTS = {"silu": "SiLU", "swish": "Swish", "gelu": "GELU", "gelu_tanh": "GELU_Tanh_Approx"}


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(GOLD, "mx_ref.npz"))


def _w(a, kind):
    t = torch.from_numpy(a).cuda()
    return t.to(torch.float8_e4m3fn) if kind == "fp8row" else t.to(torch.bfloat16)


@pytest.mark.parametrize("impl", [1, 0])
@pytest.mark.parametrize("name", list(gi.DENSE_CTE_CASES))
def test_dense_moe_cte_matches_reference_torch_ref(name, impl, gold):
    import nki_library_b200 as m
    c = gi.DENSE_CTE_CASES[name]
    d = gi.dense_cte_inputs(name)
    T, E, B = c["T"], c["E"], c["B"]
    fp8 = c["weights"] == "fp8row"
    g_hi, g_lo, u_hi, u_lo = c["clamps"]
    impl_enum = m.MoECTEImplementation.shard_on_i_hybrid if c["hybrid"] else m.MoECTEImplementation.shard_on_block
    mode = {"post": m.ExpertAffinityScaleMode.POST_SCALE, "pre": m.ExpertAffinityScaleMode.PRE_SCALE,
            "none": m.ExpertAffinityScaleMode.NO_SCALE}[c["scaling"]]
    qc = None
    if fp8:
        qc = m.QuantizationConfig(torch.from_numpy(d["gate_up_scale"].reshape(E, 1, -1)).cuda(),
                                  torch.from_numpy(d["down_scale"].reshape(E, 1, -1)).cuda())
    out = m.moe_cte(torch.from_numpy(d["hidden"]).to(torch.bfloat16).cuda(),
                    torch.from_numpy(d["aff"]).to(torch.bfloat16).cuda().reshape(-1, 1), _w(d["gate_up"], c["weights"]),
                    _w(d["down"], c["weights"]), torch.from_numpy(gold[f"dense_cte/{name}/tpi"]).cuda(),
                    torch.from_numpy(gold[f"dense_cte/{name}/block_to_expert"]).cuda(), B, m.MoECTESpec(impl_enum),
                    conditions=torch.from_numpy(gold[f"dense_cte/{name}/conditions"]).cuda() if c["hybrid"] else None,
                    gate_and_up_proj_bias=None if d["bias_gu"] is None else torch.from_numpy(d["bias_gu"]).cuda(),
                    down_proj_bias=None if d["bias_d"] is None else torch.from_numpy(d["bias_d"]).cuda(),
                    quantization_config=qc, activation_function=getattr(m.ActFnType, _ACTS[c["act"]]),
                    skip_dma=m.SkipMode(c["skip_token"], False), expert_affinities_scaling_mode=mode,
                    gate_clamp_upper_limit=g_hi, gate_clamp_lower_limit=g_lo, up_clamp_upper_limit=u_hi,
                    up_clamp_lower_limit=u_lo, _impl=impl, _check_status=True)
    assert out.shape[0] == (T if c["skip_token"] else T + 1) and out.dtype == torch.bfloat16
    assert max_rel(out[:T].float().cpu().numpy(), gold[f"dense_cte/{name}/out"]) <= TOL


@pytest.mark.parametrize("name", list(gi.DENSE_TKG_CASES))
def test_dense_moe_tkg_matches_reference_torch_ref(name, gold):
    import nki_library_b200 as m
    d = gi.dense_tkg_inputs(name)
    fp8 = d["weights"] == "fp8row"
    g_hi, _, u_hi, u_lo = d["clamps"]
    out = m.moe_tkg(torch.from_numpy(d["hidden"]).to(torch.bfloat16).cuda(), _w(d["gate_up"], d["weights"]),
                    _w(d["down"], d["weights"]), torch.from_numpy(d["aff"]).cuda(),
                    torch.from_numpy(d["expert_index"]).cuda(), d["all_expert"],
                    rank_id=torch.zeros((1, 1), dtype=torch.int32, device="cuda"),
                    expert_gate_up_bias=torch.from_numpy(d["bias_gu"]).cuda(),
                    expert_down_bias=torch.from_numpy(d["bias_d"]).cuda(),
                    expert_gate_up_weights_scale=torch.from_numpy(d["gate_up_scale"]).cuda() if fp8 else None,
                    expert_down_weights_scale=torch.from_numpy(d["down_scale"]).cuda() if fp8 else None,
                    expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.POST_SCALE,
                    activation_fn=getattr(m.ActFnType, _ACTS[d["act"]]), gate_clamp_upper_limit=g_hi,
                    up_clamp_upper_limit=u_hi, up_clamp_lower_limit=u_lo, _check_status=True)
    assert max_rel(out.float().cpu().numpy(), gold[f"dense_tkg/{name}/out"]) <= TOL


def test_dense_pre_scale_is_rejected_by_decode_and_mx_prefill():
    """The decode kernels have no pre-scale mode (core/moe/moe_tkg/moe_tkg.py notes); the MX prefill kernels neither."""
    import nki_library_b200 as m
    d = gi.dense_tkg_inputs("sel_t8_bf16_silu")
    with pytest.raises(AssertionError):
        m.moe_tkg(torch.from_numpy(d["hidden"]).to(torch.bfloat16).cuda(), _w(d["gate_up"], "bf16"), _w(d["down"], "bf16"),
                  torch.from_numpy(d["aff"]).cuda(), torch.from_numpy(d["expert_index"]).cuda(), False,
                  expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.PRE_SCALE)
