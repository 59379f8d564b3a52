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
