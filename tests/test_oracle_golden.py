"""The CPU oracle against fixtures produced by the reference's own torch references."""

import hashlib
import json
import os

import numpy as np
import pytest
import torch

import golden_inputs as gi
from oracle import moe, mx, routing

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def router_gold():
    return np.load(os.path.join(GOLD, "router_topk_ref.npz"))


@pytest.fixture(scope="module")
def digests():
    with open(os.path.join(GOLD, "grouping_ref_digests.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def small():
    return np.load(os.path.join(GOLD, "grouping_ref_small.npz"))


@pytest.mark.parametrize("name", list(gi.ROUTER_CASES))
def test_router_oracle_matches_reference(name, router_gold):
    T, H, E, k, act, has_bias, pre_norm, l1 = gi.ROUTER_CASES[name]
    x, w, b = gi.router_inputs(T, H, E, has_bias)
    act_id = routing.SOFTMAX if act == "softmax" else routing.SIGMOID
    logits, idx, aff = routing.router_topk(x, w, b, k, act_id, pre_norm, l1)
    # logits: matmul summation order may differ between hosts -> tolerance, not bytes
    np.testing.assert_allclose(logits.numpy(), router_gold[name + "/logits"], rtol=0, atol=2e-5)
    # top-K and affinities are exact functions of the logits: feed the stored ones
    idx2, aff2 = routing.router_from_logits(torch.from_numpy(router_gold[name + "/logits"]), k, act_id, pre_norm, l1)
    assert np.array_equal(idx2.numpy().astype(np.int32), router_gold[name + "/index"])
    np.testing.assert_allclose(aff2.numpy(), router_gold[name + "/aff"], rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("name", list(gi.NONZERO_CASES))
def test_find_nonzero_oracle_matches_reference(name, digests, small):
    T, E, top_k, dtype, cs, nc = gi.NONZERO_CASES[name]
    inp = gi.sparse_input(T, E, top_k, dtype)
    ind, cnt = routing.find_nonzero_indices(inp, 0 if cs is None else cs, nc)
    d = digests["find_nonzero_indices"][name]
    assert _digest(ind) == d["indices"] and _digest(cnt) == d["counts"]
    if name + "/indices" in small:
        assert np.array_equal(ind, small[name + "/indices"])


@pytest.mark.parametrize("name", list(gi.FLATTEN_CASES))
def test_indexed_flatten_oracle_matches_reference(name, digests):
    kw = gi.flatten_inputs(*gi.FLATTEN_CASES[name])
    out = routing.indexed_flatten(kw["input_tensor"], kw["f_len"], kw["output_len"], kw["row_offsets"],
                                  kw["row_offsets_start"] or 0, kw["padding_val"])
    assert _digest(out) == digests["indexed_flatten"][name]


@pytest.mark.parametrize("name", list(gi.CHAIN_CASES))
def test_group_tokens_oracle_matches_reference_chain(name, digests, small):
    T, E, K, B = gi.CHAIN_CASES[name]
    mask = gi.routing_mask(T, E, K)
    N = gi.n_blocks(T, K, E, B)
    assert N == routing.get_n_blocks(T, K, E, B)
    tpi, b2e, cond, counts = routing.group_tokens(mask, B, N)
    assert _digest(tpi) == digests["grouping_chain"][name]
    if name + "/tpi" in small:
        assert np.array_equal(tpi, small[name + "/tpi"])
    # block_to_expert / conditions invariants of the reference generator
    bpe = -(-counts.astype(np.int64) // B)
    n_pad = N - bpe.sum()
    assert np.all(np.diff(b2e) >= 0) and b2e[-1] == E - 1 and len(b2e) == N
    assert cond.shape == (N + 2,) and cond.sum() == N - n_pad and np.all(np.diff(cond) <= 0)


def test_e4m3_codec_against_ml_dtypes():
    ml_dtypes = pytest.importorskip("ml_dtypes")
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(50000).astype(np.float32) * s for s in (1e-4, 1e-2, 1, 40, 300)])
    x = np.clip(x, -448, 448)
    assert np.array_equal(mx.e4m3_encode(x), x.astype(ml_dtypes.float8_e4m3fn).view(np.uint8))
    codes = np.arange(256, dtype=np.uint8)
    vals = mx.e4m3_decode(codes)
    ok = ~np.isnan(vals)
    assert np.array_equal(mx.e4m3_encode(vals[ok]), codes[ok])
    assert np.array_equal(vals[ok], codes[ok].view(ml_dtypes.float8_e4m3fn).astype(np.float32))


def test_element_decoders_match_reference_unpackers():
    """e2m1 / e5m2 / e4m3 decoding against the reference's unpack_float4_x4, unpack_float8_e5m2_x4 and
    unpack_float8_e4m3fn_x4 run over every 16-bit fp4 word and every byte (fixture mx_element_decode_ref.npz)."""
    g = np.load(os.path.join(GOLD, "mx_element_decode_ref.npz"))
    words = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    nib = np.stack([(words >> (4 * j)) & 0xF for j in range(4)], axis=-1).reshape(256, 1024).astype(np.uint8)
    got = mx.e2m1_decode(nib)
    assert np.array_equal(got, g["e2m1_x4"]) and np.array_equal(np.signbit(got), np.signbit(g["e2m1_x4"]))
    # the packed image used on the device is the reference's x4 word
    assert np.array_equal(mx.pack_e2m1(nib).view(np.uint16), words)
    assert np.array_equal(mx.unpack_e2m1(mx.pack_e2m1(nib)), nib)
    every = np.arange(256, dtype=np.uint8)
    assert np.array_equal(mx.e5m2_decode(every), g["e5m2_x4"][0])
    ours = mx.e4m3_decode(every)
    finite = ~np.isnan(ours)
    # 0x7F / 0xFF are NaN in e4m3fn (and on the tensor cores); the reference's unpacker reads them as +-480
    assert list(np.flatnonzero(~finite)) == [0x7F, 0xFF]
    assert np.array_equal(ours[finite], g["e4m3_x4"][0][finite])


@pytest.mark.parametrize("fmt", ["e5m2", "e2m1"])
def test_reference_storage_round_trip_other_formats(fmt):
    """rows -> reference x4 storage -> rows for 8-bit and 4-bit element words."""
    from moe_testlib import make_rows_weights_fmt
    E, H, I = 2, 1024, 512
    c1, s1, c2, s2 = make_rows_weights_fmt(E, H, I, fmt, seed=3)
    gw, gs = mx.rows_to_ref_gate_up(c1, s1, fmt)
    dw, ds = mx.rows_to_ref_down(c2, s2, fmt)
    assert gw.dtype == (np.uint16 if fmt == "e2m1" else np.uint32) and gw.shape == (E, 128, 2, H // 512, I)
    assert dw.shape == (E, 128, 1, H) and gs.shape == (E, 16, 2, H // 512, I)
    if fmt == "e2m1":
        g4 = np.stack([(gw >> (4 * j)) & 0xF for j in range(4)], axis=-1).astype(np.uint8)
        d4 = np.stack([(dw >> (4 * j)) & 0xF for j in range(4)], axis=-1).astype(np.uint8)
    else:
        g4, d4 = gw.view(np.uint8).reshape(*gw.shape, 4), dw.view(np.uint8).reshape(*dw.shape, 4)
    rc1, rs1 = mx.ref_gate_up_to_rows(g4, gs)
    rc2, rs2 = mx.ref_down_to_rows(d4, ds)
    assert np.array_equal(rc1, c1) and np.array_equal(rs1, s1) and np.array_equal(rc2, c2) and np.array_equal(rs2, s2)


def test_quantize_rule_known_answers():
    # largest element 1.0 (biased exponent 127) -> scale byte 119, codes = x * 2^8 clipped to 448
    x = np.zeros((1, 32), dtype=np.float32)
    x[0, :4] = [1.0, -0.5, 1.75, 2.0**-9]
    codes, scales = mx.quantize_mx_rows(x)
    assert scales[0, 0] == 127 - 8
    assert list(mx.e4m3_decode(codes[0, :4])) == [256.0, -128.0, 448.0, 0.5]
    z, zs = mx.quantize_mx_rows(np.zeros((2, 64), dtype=np.float32))
    assert not z.any() and not zs.any()  # all-zero block: scale byte 0 (mx_torch_common.py:213)


def test_contiguous_blocks_equal_reference_blocks():
    """8x4 blocks of the reference's folded view == 32 contiguous elements in packed order."""
    rng = np.random.default_rng(1)
    R, H = 8, 1024
    x = torch.from_numpy(rng.standard_normal((R, H)).astype(np.float32) * 3).bfloat16().float().numpy()
    nt = H // 512
    folded = x.reshape(R, 4, nt, 128).transpose(3, 2, 0, 1).reshape(128, -1)
    rq, rs = mx.quantize_to_mx_ref_blocks(folded)  # [128, nt*R*4], [16, nt*R]
    cq, cs = mx.quantize_mx_rows(x[:, mx.hidden_packed_order(H)])  # [R, H], [R, H/32]
    rq = rq.reshape(128, nt, R, 4).transpose(2, 1, 0, 3).reshape(R, H)
    rs = rs.reshape(16, nt, R).transpose(2, 1, 0).reshape(R, H // 32)
    assert np.array_equal(rq, cq) and np.array_equal(rs, cs)


@pytest.mark.parametrize("I", [256, 1024])
def test_rows_oracle_equals_reference_layout_recipe(I):
    rng = np.random.default_rng(2)
    H, R, E = 1024, 16, 2
    hid = torch.from_numpy(rng.standard_normal((R, H)).astype(np.float32)).bfloat16().float().numpy()
    c1, s1 = mx.quantize_mx_rows((rng.standard_normal((E * 2 * I, H)) * 0.02).astype(np.float32))
    c2, s2 = mx.quantize_mx_rows((rng.standard_normal((E * H, I)) * 0.02).astype(np.float32))
    c1, s1 = c1.reshape(E, 2, I, H), s1.reshape(E, 2, I, H // 32)
    c2, s2 = c2.reshape(E, H, I), s2.reshape(E, H, I // 32)
    gw, gs = mx.rows_to_ref_gate_up(c1, s1)
    dw, ds = mx.rows_to_ref_down(c2, s2)
    a, b = mx.ref_gate_up_to_rows(gw, gs)
    assert np.array_equal(a, c1) and np.array_equal(b, s1)
    a, b = mx.ref_down_to_rows(dw, ds)
    assert np.array_equal(a, c2) and np.array_equal(b, s2)
    pI = 128 if I > 512 else I // 4
    bgu = rng.uniform(-2, 0.5, (E, 2, I)).astype(np.float32)
    bref = bgu.reshape(E, 2, I // (pI * 4), pI, 4).transpose(0, 3, 1, 2, 4)
    assert np.array_equal(mx.ref_gate_up_bias_to_rows(bref), bgu)
    bd = rng.uniform(-1, 1, (E, H)).astype(np.float32)
    for e in range(E):
        y_ref = moe.ref_layout_expert_mlp(hid, gw[e], gs[e], dw[e], ds[e], bref[e], bd[e], act=moe.SWISH,
                                          gate_clamp=(-7, 7), up_clamp=(-7, 7))
        y = moe.expert_mlp_rows(hid[:, mx.hidden_packed_order(H)], moe.ExpertWeights(c1, s1, c2, s2, e), bgu[e], bd[e],
                                act=moe.SWISH, gate_clamp=(-7, 7), up_clamp=(-7, 7), round_inter_bf16=False)
        assert np.abs(y - y_ref).max() <= 1e-5 * np.abs(y_ref).max()


# ---------------------------------------------------------------------------
# MX arithmetic against outputs of the reference's own CPU code
# (tests/golden/mx_ref.npz, written by tests/golden/make_golden_mx.py)
# ---------------------------------------------------------------------------
@pytest.fixture(scope="module")
def mx_gold():
    return np.load(os.path.join(GOLD, "mx_ref.npz"))


def _rel(a, ref):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(ref, np.float64)).max() / max(np.abs(ref).max(), 1e-30))


def test_mx_quantize_matches_reference_quantize_to_mx(mx_gold):
    """Codes and scales of ``quantize_to_mx`` (core/utils/mx_torch_common.py:157-221), bit for bit, on data with
    zero blocks, fp32 subnormals, e4m3 rounding ties, clipping block maxima and 44 binades of dynamic range."""
    x = gi.mx_quantize_input()
    codes, scales = mx.quantize_to_mx_ref_blocks(x)
    assert np.array_equal(scales, mx_gold["quantize/scales"])
    assert np.array_equal(codes, mx_gold["quantize/codes"])
    # the 1 x 32 block form the CUDA kernels use is the same arithmetic on the transposed-and-folded view
    xb = gi.bf16_round(np.random.default_rng(3).standard_normal((64, 256)))
    c2, s2 = mx.quantize_to_mx_ref_blocks(xb)
    assert np.array_equal(c2, mx_gold["quantize/bf16_codes"]) and np.array_equal(s2, mx_gold["quantize/bf16_scales"])


def test_mx_quantize_test_twin_differs_only_on_tiny_blocks(mx_gold):
    """test/utils/mx_utils.py:56-99 is the same rule except that a block whose largest biased exponent is below 8
    (all zeros, fp32 subnormals, magnitudes under 2^-119) gets the wrapped byte ``(e_max - 8) mod 256`` where the
    src/ function clips to 0; the oracle follows src/."""
    codes, scales = mx.quantize_to_mx_ref_blocks(gi.mx_quantize_input())
    twin_s = mx_gold["quantize/test_twin_scales"]
    differs = twin_s != scales
    assert differs.sum() > 0 and np.all(twin_s[differs] >= 248) and np.all(scales[differs] == 0)
    keep = np.repeat(np.repeat(~differs, 8, 0), 4, 1)
    assert np.array_equal(codes[keep], mx_gold["quantize/test_twin_codes"][keep])


def test_mx_matmul_matches_reference(mx_gold):
    sc, mc, ss, ms = gi.mx_matmul_input()
    got = moe._ref_mx_contract(sc, mc, ss, ms)
    assert _rel(got, mx_gold["matmul/mx_matmul"]) <= 1e-6
    assert _rel(got, mx_gold["matmul/nc_matmul_mx_golden"]) <= 1e-6


def _projection_inputs(I):
    """The seeded inputs of ``projection_fixture`` in tests/golden/make_golden_mx.py."""
    import math
    H, R = 512, 16
    rng = np.random.default_rng(100 + I)
    c1, s1 = gi.mx_encode_rows((rng.standard_normal((2 * I, H)) * 0.05).astype(np.float32))
    c2, s2 = gi.mx_encode_rows((rng.standard_normal((H, I)) * 0.05).astype(np.float32))
    gw, gs = mx.rows_to_ref_gate_up(c1.reshape(1, 2, I, H), s1.reshape(1, 2, I, H // 32))
    dw, ds = mx.rows_to_ref_down(c2.reshape(1, H, I), s2.reshape(1, H, I // 32))
    hidden = gi.bf16_round(rng.standard_normal((R, H)))
    P = 128 if I > 512 else I // 4
    nt = math.ceil(I / 512)
    bias_g = gi.bf16_round(rng.uniform(-1, 1, (P, nt, 4)))
    bias_d = gi.bf16_round(rng.uniform(-1, 1, (1, H)))
    inter = (rng.standard_normal((128, nt, R, 4)) * 0.5).astype(np.float32)
    if I < 512:
        inter[I // 4:] = 0
    return dict(H=H, I=I, R=R, gw=mx._as_bytes_x4(gw[0]), gs=gs[0], dw=mx._as_bytes_x4(dw[0]), ds=ds[0],
                hidden=hidden, bias_g=bias_g, bias_d=bias_d, inter=inter, rows=(c1, s1, c2, s2))


@pytest.mark.parametrize("I", [256, 1024])
def test_projection_goldens_match_reference(I, mx_gold):
    """``_gate_up_proj_golden_mx`` / ``_down_proj_golden_mx`` (test_mlp_common.py:550-682) and the src torch
    references ``gate_up_proj_mxfp4_torch_ref`` / ``down_proj_mxfp4_torch_ref`` (mlp_proj_mxfp4_torch.py:52-187)."""
    p = _projection_inputs(I)
    gate = moe.ref_layout_gate_or_up(p["hidden"], p["gw"][:, 0], p["gs"][:, 0], p["bias_g"], p["H"], I)
    assert _rel(gate, mx_gold[f"proj/i{I}/gate_test_golden"]) <= 1e-6
    assert _rel(gate, mx_gold[f"proj/i{I}/gate_src_ref"]) <= 1e-6
    down = moe.ref_layout_down(p["inter"], p["dw"], p["ds"], p["bias_d"], p["H"], I)
    assert _rel(down, mx_gold[f"proj/i{I}/down_test_golden"]) <= 1e-6
    assert _rel(down, mx_gold[f"proj/i{I}/down_src_ref"]) <= 1e-6
    # ... and the plain-rows form the CUDA kernels are compared with gives the same gate values
    c1, s1, c2, s2 = p["rows"]
    H = p["H"]
    ew = moe.ExpertWeights(c1.reshape(1, 2, I, H), s1.reshape(1, 2, I, H // 32), c2.reshape(1, H, I),
                           s2.reshape(1, H, I // 32), 0)
    xq, xs = mx.quantize_mx_rows(p["hidden"][:, mx.hidden_packed_order(H)])
    g_rows = mx.dequantize_mx_rows(xq, xs) @ ew.w1[0].T       # [R, I] in packed I order, no bias
    ref = mx_gold[f"proj/i{I}/gate_test_golden"] - np.pad(p["bias_g"], ((0, 128 - p["bias_g"].shape[0]), (0, 0), (0, 0)))[:, :, None, :]
    nt = ref.shape[1]
    P = 128 if I > 512 else I // 4
    ref_rows = ref[:P].transpose(2, 1, 0, 3).reshape(p["R"], nt * P * 4)  # [R, (tile, p, q)] = packed I order
    assert _rel(g_rows, ref_rows) <= 1e-5


@pytest.mark.parametrize("name", list(gi.MX_LAYER_CASES))
def test_block_assignment_matches_reference_generator(name, mx_gold):
    """``generate_token_position_to_id_and_experts`` (test_moe_cte_common.py:199-264) run on the case's routing:
    token_position_to_id, block_to_expert and the MX ``conditions`` vector, bit for bit."""
    c = gi.MX_LAYER_CASES[name]
    _, mask, _ = gi.mx_layer_routing(name)
    N = routing.get_n_blocks(c["T"], c["K"], c["E"], c["B"])
    tpi, b2e, cond, _ = routing.group_tokens(mask, c["B"], N, skip_token=c["skip_token"], mx_conditions=True)
    assert np.array_equal(tpi, mx_gold[f"grouping/{name}/tpi"])
    assert np.array_equal(b2e, mx_gold[f"grouping/{name}/block_to_expert"])
    assert np.array_equal(cond, mx_gold[f"grouping/{name}/conditions"])


_ACT = {"silu": moe.SILU, "swish": moe.SWISH, "gelu": moe.GELU, "gelu_tanh": moe.GELU_TANH}


def _clamps(c):
    g_hi, g_lo, u_hi, u_lo = c
    return (g_lo, g_hi), (u_lo, u_hi)


@pytest.mark.parametrize("name", list(gi.MX_DECODE_CASES))
def test_decode_oracle_matches_reference_moe_tkg_mx_ref(name, mx_gold):
    """``_moe_tkg_mx_ref`` (core/moe/moe_tkg/moe_tkg_torch.py:299-442): selective and all-expert, bias, Swish,
    one-sided gate clamp.  Same quantised operands; only fp32 summation order differs."""
    d = gi.mx_decode_inputs(name)
    gc, uc = _clamps(d["clamps"])
    out = moe.moe_tkg_rows(d["hidden"], d["aff"], d["expert_index"], d["w1_codes"], d["w1_scales"], d["w2_codes"],
                           d["w2_scales"], d["bias_gu"], d["bias_d"], _ACT[d["act"]], gc, uc,
                           h_order=mx.hidden_packed_order(d["H"]), round_inter_bf16=False,
                           is_all_expert=d["all_expert"])
    assert _rel(out, mx_gold[f"decode/{name}/out"]) <= 1e-5


@pytest.mark.parametrize("name", list(gi.MX_LAYER_CASES))
def test_prefill_oracle_matches_reference_blockwise_golden(name, mx_gold):
    """``generate_blockwise_numpy_golden`` (test/integration/nkilib/core/moe/moe_cte/test_utils.py:474-735) with
    the arguments ``golden_moe_bwmm_mx_cte`` passes.  The reference's own bar for this output is 5e-2 of the
    output range (test_moe_bwmm_mx_cte.py:287-288); the restatement differs only in summation order and in
    summing a token's rows in fp32 before one bf16 rounding (the golden adds bf16 to bf16 block by block)."""
    c = gi.MX_LAYER_CASES[name]
    inp = gi.mx_layer_inputs(name)
    ref = torch.from_numpy(mx_gold[f"layer/{name}/out_bf16_bits"].view(np.int16)).view(torch.bfloat16).float().numpy()
    gc, uc = _clamps(c["clamps"])
    kw = dict(bias_gu=inp["bias_gu"], bias_d=inp["bias_d"], act=_ACT[c["act"]], gate_clamp=gc, up_clamp=uc,
              h_order=mx.hidden_packed_order(c["H"]), round_inter_bf16=False)
    if c["sample"] is None:
        out = moe.moe_cte_rows(inp["hidden"], inp["aff"], inp["w1_codes"], inp["w1_scales"], inp["w2_codes"],
                               inp["w2_scales"], mx_gold[f"grouping/{name}/tpi"],
                               mx_gold[f"grouping/{name}/block_to_expert"], c["B"],
                               mx_gold[f"grouping/{name}/conditions"] if c["dynamic"] else None, **kw)[:c["T"]]
    else:
        rows = gi.sample_rows(name, c["T"], c["sample"])
        out = moe.moe_cte_tokens(rows, inp["hidden"], inp["aff"], inp["w1_codes"], inp["w1_scales"], inp["w2_codes"],
                                 inp["w2_scales"], inp["expert_index"], **kw)
    assert out.shape == ref.shape
    assert _rel(gi.bf16_round(out), ref) <= 8e-3  # two bf16 steps at the largest output


def test_large_operand_dequantise_equals_table_lookup():
    """The torch conversion used for operands of a million elements or more gives the bytes of the lookup table."""
    rng = np.random.default_rng(5)
    codes = rng.integers(0, 256, (2048, 1024), dtype=np.uint8)
    scales = rng.integers(100, 140, (2048, 32), dtype=np.uint8)
    fast = mx.dequantize_mx_rows(codes, scales)
    slow = np.concatenate([mx.dequantize_mx_rows(codes[i:i + 256], scales[i:i + 256]) for i in range(0, 2048, 256)])
    assert np.array_equal(fast, slow, equal_nan=True)


# ---------------------------------------------------------------------------
# Non-MX (bf16 / fp8-row) variants against the reference's torch references
# ---------------------------------------------------------------------------
from oracle import dense  # noqa: E402

_DENSE_ACT = {"silu": dense.SILU, "swish": dense.SWISH, "gelu": dense.GELU, "gelu_tanh": dense.GELU_TANH}
_DENSE_SCALING = {"post": dense.POST_SCALE, "pre": dense.PRE_SCALE, "none": dense.NO_SCALE}


@pytest.mark.parametrize("name", list(gi.DENSE_CTE_CASES))
def test_dense_prefill_oracle_matches_reference_moe_cte_torch_ref(name, mx_gold):
    """``moe_cte_torch_ref`` (core/moe/moe_cte/moe_cte_torch.py:26-242): bf16 and fp8-row weights, POST_SCALE and
    PRE_SCALE, bias, clamps, the hybrid variant's ``conditions``; block assignment from the reference's generator."""
    c = gi.DENSE_CTE_CASES[name]
    d = gi.dense_cte_inputs(name)
    N = routing.get_n_blocks(c["T"], c["K"], c["E"], c["B"])
    tpi, b2e, cond, _ = routing.group_tokens(d["mask"], c["B"], N, skip_token=c["skip_token"], mx_conditions=False)
    assert np.array_equal(tpi, mx_gold[f"dense_cte/{name}/tpi"])
    assert np.array_equal(b2e, mx_gold[f"dense_cte/{name}/block_to_expert"])
    assert np.array_equal(cond, mx_gold[f"dense_cte/{name}/conditions"])
    g_hi, g_lo, u_hi, u_lo = c["clamps"]
    E = c["E"]
    out = dense.moe_cte_dense(
        d["hidden"], d["aff"], d["gate_up"], d["down"], tpi, b2e, c["B"], cond if c["hybrid"] else None, d["bias_gu"],
        d["bias_d"], None if d["gate_up_scale"] is None else d["gate_up_scale"].reshape(E, 1, -1),
        None if d["down_scale"] is None else d["down_scale"].reshape(E, 1, -1), _DENSE_ACT[c["act"]], (g_lo, g_hi),
        (u_lo, u_hi), _DENSE_SCALING[c["scaling"]], c["skip_token"])
    assert _rel(out, mx_gold[f"dense_cte/{name}/out"]) <= 1e-5


@pytest.mark.parametrize("name", list(gi.DENSE_TKG_CASES))
def test_dense_decode_oracle_matches_reference_moe_tkg_torch_ref(name, mx_gold):
    """``moe_tkg_torch_ref`` on non-MX weights (core/moe/moe_tkg/moe_tkg_torch.py:36-297): selective and all-expert,
    bf16 and fp8-row."""
    d = gi.dense_tkg_inputs(name)
    g_hi, _, u_hi, u_lo = d["clamps"]
    out = dense.moe_tkg_dense(d["hidden"], d["aff"], d["expert_index"], d["gate_up"], d["down"], d["bias_gu"],
                              d["bias_d"], _DENSE_ACT[d["act"]], g_hi, (u_lo, u_hi), d["gate_up_scale"], d["down_scale"],
                              True, d["all_expert"])
    assert _rel(out, mx_gold[f"dense_tkg/{name}/out"]) <= 1e-5
