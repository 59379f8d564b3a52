"""The CUDA path against outputs of the reference's own CPU code (tests/golden/mx_ref.npz).

These fixtures were produced by running the reference's ``quantize_to_mx``,
``generate_blockwise_numpy_golden`` and ``_moe_tkg_mx_ref`` on the seeded inputs of
``tests/golden_inputs.py`` (see tests/golden/make_golden_mx.py); nothing here goes through
the repo's own oracle except the pure layout permutations that build reference-format
tensors.  Every call goes through the drop-in entry points (``moe_cte`` / ``moe_tkg``) with
tensors in the reference's storage.  Output tolerance: max|a - ref| / max|ref| <= 2e-2
(the reference's own bar for these outputs is 5e-2, test_moe_bwmm_mx_cte.py:287-288).
"""

import os

import numpy as np
import pytest
import torch

import golden_inputs as gi
from moe_testlib import max_rel, sf_atoms_to_rows
from oracle import mx

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
TOL = 2e-2


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(GOLD, "mx_ref.npz"))


def _bf16(bits):
    return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).float().numpy()


def _reference_storage(inp, uint_alias=True):
    """Rows-form weights -> the tensors a caller of the reference passes (x4 words as int32 = the uint32 alias
    dtype of test_moe_bwmm_mx_cte.py:118-126, scales uint8, biases in the folded layouts), on the GPU."""
    gw, gs = mx.rows_to_ref_gate_up(inp["w1_codes"], inp["w1_scales"])
    dw, ds = mx.rows_to_ref_down(inp["w2_codes"], inp["w2_scales"])
    t = dict(gate_up=torch.from_numpy(gw.view(np.int32)).cuda(), gate_up_scale=torch.from_numpy(gs).cuda(),
             down=torch.from_numpy(dw.view(np.int32)).cuda(), down_scale=torch.from_numpy(ds).cuda(),
             bias_gu=None, bias_d=None)
    if inp["bias_gu"] is not None:
        E, _, I = inp["bias_gu"].shape
        P = 128 if I > 512 else I // 4
        ref_b = np.ascontiguousarray(inp["bias_gu"].reshape(E, 2, I // (P * 4), P, 4).transpose(0, 3, 1, 2, 4))
        t["bias_gu"] = torch.from_numpy(ref_b).to(torch.bfloat16).cuda()
        t["bias_d"] = torch.from_numpy(inp["bias_d"]).to(torch.bfloat16).cuda()
    return t


def test_quantise_kernel_matches_reference_quantize_to_mx(gold):
    """The MXFP8 activation quantiser, bit for bit, on the reference's own output for data with zero blocks,
    subnormals, rounding ties, clipping maxima and 44 binades of range.  The reference's 8 x 4 blocks of the
    ``[P, F]`` array become rows of 32 contiguous elements: row = column group, K = (row group, row, column)."""
    from nki_library_b200 import _lib
    x = gi.mx_quantize_input()
    P, F = x.shape
    rows = x.reshape(P // 8, 8, F // 4, 4).transpose(2, 0, 1, 3).reshape(F // 4, P * 4)
    h = torch.from_numpy(rows).to(torch.bfloat16)
    assert torch.equal(h.float(), torch.from_numpy(rows)), "the fixture input must be bf16-exact"
    n, K = rows.shape
    lib = _lib.load_library()
    codes = torch.empty((n, K), dtype=torch.uint8, device="cuda")
    sf = torch.zeros(lib.b200moe_sf_bytes(n, K), dtype=torch.uint8, device="cuda")
    _lib.call("b200moe_gather_quantize_mxfp8", _lib.ptr(h.cuda()), n, K, None, n, 0, _lib.ptr(codes), _lib.ptr(sf), None,
              _lib.stream_ptr())
    got_c = codes.cpu().numpy().reshape(F // 4, P // 8, 8, 4).transpose(1, 2, 0, 3).reshape(P, F)
    got_s = sf_atoms_to_rows(sf.cpu().numpy(), n, K).T  # [P/8, F/4]
    assert np.array_equal(got_s, gold["quantize/scales"])
    assert np.array_equal(got_c, gold["quantize/codes"])
    # the token-major twin of the same kernel
    inv = torch.arange(n, dtype=torch.int32, device="cuda").reshape(n, 1)
    codes2 = torch.empty_like(codes)
    sf2 = torch.zeros_like(sf)
    _lib.call("b200moe_scatter_quantize_mxfp8", _lib.ptr(h.cuda()), n, K, _lib.ptr(inv), 1, n, 0, _lib.ptr(codes2),
              _lib.ptr(sf2), None, _lib.stream_ptr())
    assert torch.equal(codes, codes2) and torch.equal(sf, sf2)


_ACTS = {"silu": "SiLU", "swish": "Swish", "gelu": "GELU", "gelu_tanh": "GELU_Tanh_Approx"}


@pytest.mark.parametrize("name", list(gi.MX_LAYER_CASES))
def test_moe_cte_matches_reference_blockwise_golden(name, gold):
    """``moe_cte`` on reference-format tensors against ``generate_blockwise_numpy_golden``: configuration 1 plain
    and in unit-vector style, and two of the reference's own MX vectors (H=3072, I=384, B=256; E=128 top-4 with
    Swish, bias and a one-sided gate clamp; E=2 top-2 with the dynamic block loop and ``n_static_blocks=2``)."""
    import nki_library_b200 as m
    c = gi.MX_LAYER_CASES[name]
    inp = gi.mx_layer_inputs(name)
    st = _reference_storage(inp)
    T, E, B = c["T"], c["E"], c["B"]
    g_hi, g_lo, u_hi, u_lo = c["clamps"]
    spec = m.MoECTESpec(m.MoECTEImplementation.shard_on_block_mx,
                        shard_on_block=m.ShardOnBlockConfig(n_static_blocks=2 if c["dynamic"] else -1))
    out = m.moe_cte(torch.from_numpy(inp["hidden"]).to(torch.bfloat16).cuda(),
                    torch.from_numpy(inp["aff"]).to(torch.bfloat16).cuda().reshape(-1, 1), st["gate_up"], st["down"],
                    torch.from_numpy(gold[f"grouping/{name}/tpi"]).cuda(),
                    torch.from_numpy(gold[f"grouping/{name}/block_to_expert"]).cuda(), B, spec,
                    conditions=torch.from_numpy(gold[f"grouping/{name}/conditions"]).cuda() if c["dynamic"] else None,
                    gate_and_up_proj_bias=st["bias_gu"], down_proj_bias=st["bias_d"],
                    quantization_config=m.QuantizationConfig(st["gate_up_scale"], st["down_scale"]),
                    activation_function=getattr(m.ActFnType, _ACTS[c["act"]]), skip_dma=m.SkipMode(c["skip_token"], False),
                    gate_clamp_upper_limit=g_hi, gate_clamp_lower_limit=g_lo, up_clamp_upper_limit=u_hi,
                    up_clamp_lower_limit=u_lo, _check_status=True)
    assert out.shape[0] == (T if c["skip_token"] else T + 1)
    got = out[:T].float().cpu().numpy()
    if c["sample"] is not None:
        got = got[gi.sample_rows(name, T, c["sample"])]
    assert max_rel(got, _bf16(gold[f"layer/{name}/out_bf16_bits"])) <= TOL


@pytest.mark.parametrize("name", list(gi.MX_DECODE_CASES))
def test_moe_tkg_matches_reference_moe_tkg_mx_ref(name, gold):
    """``moe_tkg`` on reference-format tensors against ``_moe_tkg_mx_ref``: selective and all-expert, bias,
    one-sided gate clamp, SiLU / Swish / GELU / GELU-tanh, and the reference's MXFP8 selective vector shape
    (H=3072, I=1536, top-8)."""
    import nki_library_b200 as m
    d = gi.mx_decode_inputs(name)
    st = _reference_storage(d)
    g_hi, g_lo, u_hi, u_lo = d["clamps"]
    out = m.moe_tkg(torch.from_numpy(d["hidden"]).to(torch.bfloat16).cuda(), st["gate_up"], st["down"],
                    torch.from_numpy(d["aff"]).cuda(), torch.from_numpy(d["expert_index"]).cuda(), d["all_expert"],
                    rank_id=torch.zeros((1, 1), dtype=torch.int32, device="cuda"),
                    expert_gate_up_bias=st["bias_gu"], expert_down_bias=st["bias_d"],
                    expert_gate_up_weights_scale=st["gate_up_scale"], expert_down_weights_scale=st["down_scale"],
                    expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.POST_SCALE,
                    activation_fn=getattr(m.ActFnType, _ACTS[d["act"]]), gate_clamp_upper_limit=g_hi,
                    gate_clamp_lower_limit=g_lo, up_clamp_upper_limit=u_hi, up_clamp_lower_limit=u_lo,
                    _check_status=True)
    assert max_rel(out.float().cpu().numpy(), gold[f"decode/{name}/out"]) <= TOL
