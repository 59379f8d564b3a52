"""Grouped MXFP8 expert contractions, prefill (moe_cte) and decode (moe_tkg), against the CPU oracle.

Output tolerance of this build: max|out - ref| / max|ref| <= 2e-2 on identical
quantised inputs (the reference's own test bar for this path is 5e-2,
test_moe_bwmm_mx_cte.py:287-288).
"""

import numpy as np
import pytest
import torch

from moe_testlib import bf16_values, make_routing, make_rows_weights, max_rel, sf_atoms_to_rows
from oracle import moe, mx, routing

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _prep(m, w_np, bias_gu=None, bias_d=None):
    t = [torch.from_numpy(a).cuda() for a in w_np]
    return m.prepare_from_rows(*t, bias_gu=None if bias_gu is None else torch.from_numpy(bias_gu).cuda(),
                               bias_d=None if bias_d is None else torch.from_numpy(bias_d).cuda())


def _run_gemm1(m, weights, x_np, b2e_np, B, impl, act=0, clamps=(None,) * 4):
    """Quantise rows x_np [n_pos, H] (identity gather) and run the gate/up contraction; returns m codes/scales."""
    from nki_library_b200 import _lib, pipeline
    n_pos, H = x_np.shape
    ws = pipeline.BlockWorkspace(n_pos, H, weights.I, "cuda")
    hidden = torch.from_numpy(x_np).to(torch.bfloat16).cuda()
    b2e = torch.from_numpy(b2e_np.astype(np.int32)).cuda()
    st = _lib.stream_ptr()
    _lib.call("b200moe_gather_quantize_mxfp8", _lib.ptr(hidden), n_pos, H, None, n_pos, 0, _lib.ptr(ws.xq),
              _lib.ptr(ws.x_sf), _lib.ptr(ws.tile_flags), st)
    c = [pipeline._clamp(v) for v in clamps]
    _lib.call("b200moe_grouped_gemm1_swiglu", _lib.ptr(ws.xq), _lib.ptr(ws.x_sf), _lib.ptr(weights.w1),
              _lib.ptr(weights.w1_sf), weights.w_format, _lib.ptr(weights.bias_gu), _lib.ptr(b2e), None, _lib.ptr(ws.tile_flags),
              len(b2e_np), B, weights.E, H, weights.I, act, c[0], c[1], c[2], c[3], _lib.ptr(ws.mq), _lib.ptr(ws.m_sf),
              _lib.ptr(ws.status[1:]), impl, None, st)
    torch.cuda.synchronize()
    assert ws.status.cpu().tolist()[1] == 0, "a device-side wait expired"
    return ws.mq.cpu().numpy(), sf_atoms_to_rows(ws.m_sf.cpu().numpy(), n_pos, weights.I)


@pytest.mark.parametrize("impl,tile_n", [(1, 256), (0, 256), (0, 128)])
def test_gate_up_swiglu_requantise_vs_oracle(impl, tile_n):
    import nki_library_b200 as m
    from nki_library_b200 import _lib
    if tile_n == 128:
        impl |= _lib.GEMM_TILE_N128
    E, H, I, B = 3, 512, 384, 128
    w_np = make_rows_weights(E, H, I, seed=1)
    rng = np.random.default_rng(0)
    bgu = rng.uniform(-1, 0.5, (E, 2, I)).astype(np.float32)
    weights = _prep(m, w_np, bgu)
    b2e = np.array([0, 2, 2, 1])
    x = bf16_values(rng.standard_normal((len(b2e) * B, H)).astype(np.float32))
    mq, ms = _run_gemm1(m, weights, x, b2e, B, impl, act=moe.SWISH, clamps=(-7.0, 7.0, -7.0, 7.0))
    got = mx.dequantize_mx_rows(mq, ms)
    for b, e in enumerate(b2e):
        ew = moe.ExpertWeights(*w_np, e)
        _, parts = moe.expert_mlp_rows(x[b * B:(b + 1) * B], ew, bgu[e], None, act=moe.SWISH,
                                       gate_clamp=(-7, 7), up_clamp=(-7, 7), return_parts=True)
        ref = mx.dequantize_mx_rows(parts["mq"], parts["ms"])
        sl = slice(b * B, (b + 1) * B)
        assert max_rel(got[sl], ref) <= TOL
        # identical quantised inputs and fp32 accumulation: nearly every code and scale is identical
        assert (ms[sl] == parts["ms"]).mean() > 0.99
        assert (mq[sl] == parts["mq"]).mean() > 0.97


def _cte_case(T, H, I, E, K, B, seed, bias, act, clamp, zipf=None):
    hidden, _, _, idx, aff = make_routing(T, H, E, K, seed, zipf)
    w_np = make_rows_weights(E, H, I, seed)
    rng = np.random.default_rng(seed + 7)
    bgu = rng.uniform(-2.0625, 0.52, (E, 2, I)).astype(np.float32) if bias else None
    bd = rng.uniform(-1.632, 1.4375, (E, H)).astype(np.float32) if bias else None
    return hidden, idx, aff, w_np, bgu, bd


def _oracle_cte(hidden, aff, w_np, tpi, b2e, cond, B, bgu, bd, act, clamp, h_order=None):
    g = (-clamp, clamp) if clamp else (None, None)
    out = moe.moe_cte_rows(hidden, aff, *w_np, tpi, b2e, B, cond, bgu, bd, act, g, g, h_order=h_order)
    return bf16_values(out)


@pytest.mark.parametrize("impl", [1, 0])
@pytest.mark.parametrize("variant", ["plain", "bias_clamp_swish"])
def test_moe_cte_c1_rows_weights(impl, variant):
    """Smallest benchmark configuration: T=256, H=512, I=1024, E=4, top-2, B=128."""
    import nki_library_b200 as m
    T, H, I, E, K, B = 256, 512, 1024, 4, 2, 128
    bias = variant != "plain"
    act = moe.SWISH if bias else moe.SILU
    clamp = 7.0 if bias else None
    hidden, idx, aff, w_np, bgu, bd = _cte_case(T, H, I, E, K, B, 11, bias, act, clamp)
    weights = _prep(m, w_np, bgu, bd)
    N = m.get_n_blocks(T, K, E, B, 2)
    g = m.moe_group_tokens(torch.from_numpy(idx).cuda(), E, B, N, check=True)
    out = m.moe_cte(torch.from_numpy(hidden).to(torch.bfloat16).cuda(),
                    torch.from_numpy(aff).to(torch.bfloat16).cuda().reshape(-1, 1), weights, None,
                    g["token_position_to_id"], g["block_to_expert"], B,
                    m.MoECTESpec(m.MoECTEImplementation.shard_on_block_mx), conditions=g["conditions"],
                    activation_function=m.ActFnType(act), skip_dma=m.SkipMode(True, False),
                    gate_clamp_upper_limit=clamp, gate_clamp_lower_limit=None if clamp is None else -clamp,
                    up_clamp_upper_limit=clamp, up_clamp_lower_limit=None if clamp is None else -clamp,
                    _impl=impl, _check_status=True)
    ref = _oracle_cte(hidden, bf16_values(aff), w_np, g["token_position_to_id"].cpu().numpy(),
                      g["block_to_expert"].cpu().numpy(), g["conditions"].cpu().numpy(), B, bgu, bd, act, clamp)
    assert out.shape == (T, H) and out.dtype == torch.bfloat16
    assert max_rel(out.float().cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("B,T,scatter", [(256, 700, False), (512, 1500, False), (128, 700, False), (128, 900, True),
                                         (384, 1100, False), (256, 700, True)])
def test_moe_cte_cta_pair_mode(B, T, scatter):
    """The cta_group::2 kernel (two CTAs share a weight tile) against the oracle and the single-CTA kernel.

    Blocks of 128 or 384 positions make an expert's 128-row tiles pair up across its blocks, with a half-empty
    last pair for an odd count; ``scatter`` shuffles the block order, so experts are no longer contiguous and
    the kernel walks blocks in the given order (tiles of odd-sized blocks then run one per pair)."""
    import nki_library_b200 as m
    from nki_library_b200 import _lib
    H, I, E, K = 512, 512, 4, 2
    hidden, idx, aff, w_np, bgu, bd = _cte_case(T, H, I, E, K, B, 61, True, moe.SILU, None)
    weights = _prep(m, w_np, bgu, bd)
    N = m.get_n_blocks(T, K, E, B)
    g = m.moe_group_tokens(torch.from_numpy(idx).cuda(), E, B, N, check=True)
    tpi, b2e, cond = g["token_position_to_id"], g["block_to_expert"], g["conditions"]
    if scatter:
        n_act = int(cond[:N].sum().item())
        perm = torch.cat([torch.randperm(n_act, generator=torch.Generator().manual_seed(B + T)), torch.arange(n_act, N)])
        tpi = tpi.view(N, B)[perm.cuda()].reshape(-1).contiguous()
        b2e = b2e[perm.cuda()].contiguous()
    args = (torch.from_numpy(hidden).to(torch.bfloat16).cuda(), torch.from_numpy(aff).cuda().reshape(-1, 1), weights,
            None, tpi, b2e, B, m.MoECTESpec(m.MoECTEImplementation.shard_on_block_mx))
    kw = dict(conditions=cond, skip_dma=m.SkipMode(True, False), _check_status=True)
    single = m.moe_cte(*args, _impl=_lib.GEMM_NO_PAIR, **kw)
    paired = m.moe_cte(*args, _impl=_lib.GEMM_FORCE_PAIR, **kw)
    paired2 = m.moe_cte(*args, _impl=_lib.GEMM_FORCE_PAIR, **kw)
    # the same tiles with the left-over launch folded into half-empty pairs, and with it run strictly afterwards
    folded = m.moe_cte(*args, _impl=_lib.GEMM_FORCE_PAIR | _lib.GEMM_NO_SPLIT, **kw)
    serial = m.moe_cte(*args, _impl=_lib.GEMM_FORCE_PAIR | _lib.GEMM_NO_OVERLAP, **kw)
    assert torch.equal(paired, folded) and torch.equal(paired, serial)
    ref = _oracle_cte(hidden, aff, w_np, tpi.cpu().numpy(), b2e.cpu().numpy(), cond.cpu().numpy(), B, bgu, bd,
                      moe.SILU, None)
    assert max_rel(paired.float().cpu().numpy(), ref) <= TOL
    assert torch.equal(paired, paired2)
    assert max_rel(paired.float().cpu().numpy(), single.float().cpu().numpy()) <= 1e-2


@pytest.mark.parametrize("skip_token", [True, False])
def test_moe_cte_reference_storage_layout(skip_token):
    """Weights in the reference's x4-packed storage, hidden in its logical order, pad id -1 or T."""
    import nki_library_b200 as m
    T, H, I, E, K, B = 200, 1024, 512, 4, 2, 128
    hidden, idx, aff, w_np, bgu, bd = _cte_case(T, H, I, E, K, B, 21, True, moe.SILU, None)
    gw, gs = mx.rows_to_ref_gate_up(w_np[0], w_np[1])
    dw, ds = mx.rows_to_ref_down(w_np[2], w_np[3])
    pI = 128 if I > 512 else I // 4
    bref = np.ascontiguousarray(bgu.reshape(E, 2, I // (pI * 4), pI, 4).transpose(0, 3, 1, 2, 4))
    N = m.get_n_blocks(T, K, E, B, 2)
    g = m.moe_group_tokens(torch.from_numpy(idx).cuda(), E, B, N, skip_token=skip_token, check=True)
    hid_t = torch.from_numpy(hidden).to(torch.bfloat16)
    aff_t = torch.from_numpy(aff).to(torch.bfloat16)
    if not skip_token:
        hid_t = torch.cat([hid_t, torch.zeros(1, H, dtype=torch.bfloat16)])
        aff_t = torch.cat([aff_t, torch.zeros(1, E, dtype=torch.bfloat16)])
    out = m.moe_cte(hid_t.cuda(), aff_t.cuda().reshape(-1, 1), torch.from_numpy(gw.view(np.int32)).cuda(),
                    torch.from_numpy(dw.view(np.int32)).cuda(), g["token_position_to_id"], g["block_to_expert"], B,
                    m.MoECTESpec(m.MoECTEImplementation.shard_on_block_mx), conditions=g["conditions"],
                    gate_and_up_proj_bias=torch.from_numpy(bref).cuda(), down_proj_bias=torch.from_numpy(bd).cuda(),
                    quantization_config=m.QuantizationConfig(torch.from_numpy(gs).cuda(), torch.from_numpy(ds).cuda()),
                    skip_dma=m.SkipMode(skip_token, False), compat_lnc_slabs=True, _check_status=True)
    assert out.shape == (2, T + (0 if skip_token else 1), H) and not out[1].any()
    tpi = g["token_position_to_id"].cpu().numpy()
    ref = _oracle_cte(hidden, bf16_values(aff), w_np, tpi, g["block_to_expert"].cpu().numpy(),
                      g["conditions"].cpu().numpy(), B, bgu, bd, moe.SILU, None, h_order=mx.hidden_packed_order(H))
    assert max_rel(out[0, :T].float().cpu().numpy(), ref) <= TOL


def test_moe_cte_conditions_stop_and_skew():
    """Zipf-skewed routing with many partial blocks; blocks past the first zero condition contribute nothing."""
    import nki_library_b200 as m
    T, H, I, E, K, B = 512, 512, 256, 16, 4, 128
    hidden, idx, aff, w_np, _, _ = _cte_case(T, H, I, E, K, B, 31, False, moe.SILU, None, zipf=1.2)
    weights = _prep(m, w_np)
    N = m.get_n_blocks(T, K, E, B)
    g = m.moe_group_tokens(torch.from_numpy(idx).cuda(), E, B, N, check=True)
    cond = g["conditions"].clone()
    n_active = int(cond.sum().item())
    cond[n_active - 2] = 0  # blocks stop at the first zero: the occupied block after it must not run either
    out = m.moe_cte(torch.from_numpy(hidden).to(torch.bfloat16).cuda(), torch.from_numpy(aff).cuda().reshape(-1, 1),
                    weights, None, g["token_position_to_id"], g["block_to_expert"], B,
                    m.MoECTESpec(m.MoECTEImplementation.shard_on_i_mx), conditions=cond,
                    skip_dma=m.SkipMode(True, False), _check_status=True)
    ref = _oracle_cte(hidden, aff, w_np, g["token_position_to_id"].cpu().numpy(), g["block_to_expert"].cpu().numpy(),
                      cond.cpu().numpy(), B, None, None, moe.SILU, None)
    assert max_rel(out.float().cpu().numpy(), ref) <= TOL
    out2 = m.moe_cte(torch.from_numpy(hidden).to(torch.bfloat16).cuda(), torch.from_numpy(aff).cuda().reshape(-1, 1),
                     weights, None, g["token_position_to_id"], g["block_to_expert"], B,
                     m.MoECTESpec(m.MoECTEImplementation.shard_on_i_mx), conditions=cond,
                     skip_dma=m.SkipMode(True, False))
    assert torch.equal(out, out2)  # deterministic: same bytes on a second run


@pytest.mark.parametrize("mode,I", [("selective", 768), ("all_expert", 768), ("selective", 5120)])
def test_moe_tkg_vs_oracle(mode, I):
    """Decode: T=64 tokens, top-2 of 8 experts (the decode configuration with H, I scaled down; I = 5120 gives the
    gate/up contraction more weight tiles than there are SMs, so CTAs walk several tiles each)."""
    import nki_library_b200 as m
    T, H, E, K = 64, 1024, 8, 2
    hidden, idx, aff, w_np, bgu, bd = _cte_case(T, H, I, E, K, 128, 41, True, moe.SILU, None)
    weights = _prep(m, w_np, bgu, bd)
    hid = torch.from_numpy(hidden).to(torch.bfloat16).cuda()
    aff_t = torch.from_numpy(aff).cuda()
    idx_t = torch.from_numpy(idx).cuda()
    if mode == "selective":
        out = m.moe_tkg(hid, weights, None, aff_t, idx_t, False,
                        expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.POST_SCALE, _check_status=True)
        ref = moe.moe_tkg_rows(hidden, aff, idx, *w_np, bias_gu=bgu, bias_d=bd)
    else:
        out = m.moe_tkg(hid, weights, None, aff_t, idx_t, True, rank_id=torch.zeros((1, 1), dtype=torch.int32, device="cuda"),
                        mask_unselected_experts=True,
                        expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.POST_SCALE, _check_status=True)
        ref = moe.moe_tkg_rows(hidden, aff * routing.mask_from_index(idx, E), None, *w_np, bias_gu=bgu, bias_d=bd,
                               is_all_expert=True)
    assert out.shape == (T, H)
    assert max_rel(out.float().cpu().numpy(), bf16_values(ref)) <= TOL
    with pytest.raises(AssertionError):
        m.moe_tkg(hid, weights, None, aff_t, idx_t, False,
                  expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.PRE_SCALE)


def test_moe_cte_properties_at_mixtral_block_shape():
    """Size-independent checks at the Mixtral prefill configuration's block geometry (B=512, H=4096, K=2, E=8; I cut to 2048)."""
    import nki_library_b200 as m
    from nki_library_b200 import _lib, pipeline
    T, H, I, E, K, B = 2048, 4096, 2048, 8, 2, 512
    hidden, idx, aff, _, _, _ = _cte_case(T, 64, 32, E, K, B, 51, False, 0, None)  # routing only
    rng = np.random.default_rng(5)
    hid = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(torch.bfloat16).cuda()
    # weights quantised on the device with the library's own quantiser (N(0, 0.02), feed layout)
    lib = _lib.load_library()
    def qw(rows, K_):
        w = (torch.randn((rows, K_), device="cuda", generator=torch.Generator("cuda").manual_seed(rows)) * 0.02).to(torch.bfloat16)
        codes = torch.empty((rows, K_), dtype=torch.uint8, device="cuda")
        sf = torch.zeros(lib.b200moe_sf_bytes(rows, K_), dtype=torch.uint8, device="cuda")
        _lib.call("b200moe_gather_quantize_mxfp8", _lib.ptr(w), rows, K_, None, rows, 0, _lib.ptr(codes), _lib.ptr(sf), None,
                  _lib.stream_ptr())
        return codes, sf
    w1, w1_sf = qw(E * 2 * I, H)
    w2, w2_sf = qw(E * H, I)
    weights = m.ExpertWeights(E, H, I, w1.view(E, 2 * I, H), w1_sf, w2.view(E, H, I), w2_sf, None, None, False)
    N = m.get_n_blocks(T, K, E, B)
    g = m.moe_group_tokens(torch.from_numpy(idx).cuda(), E, B, N, check=True)
    spec = m.MoECTESpec(m.MoECTEImplementation.shard_on_block_mx)
    run = lambda h, a: m.moe_cte(h, a.reshape(-1, 1), weights, None, g["token_position_to_id"], g["block_to_expert"], B,
                                 spec, conditions=g["conditions"], skip_dma=m.SkipMode(True, False), _check_status=True)
    aff_t = torch.from_numpy(aff).cuda()
    out = run(hid, aff_t)
    assert torch.isfinite(out.float()).all() and out.float().abs().max() > 0
    assert torch.equal(out, run(hid, aff_t))                                   # run-to-run determinism
    assert torch.equal(run(hid, aff_t * 2).float(), out.float() * 2)           # exact linearity in the affinity (x2)
    assert not run(hid, torch.zeros_like(aff_t)).any()                         # zero affinity -> zero output
    # a sample of tokens against the oracle, weights dequantised from the device buffers
    w1_np = w1.view(E, 2 * I, H).cpu().numpy()
    w2_np = w2.view(E, H, I).cpu().numpy()
    s1 = sf_atoms_to_rows(w1_sf.cpu().numpy(), E * 2 * I, H).reshape(E, 2 * I, H // 32)
    s2 = sf_atoms_to_rows(w2_sf.cpu().numpy(), E * H, I).reshape(E, H, I // 32)
    from moe_testlib import gate_up_dev_rows
    rows = gate_up_dev_rows(I)
    c1 = np.stack([w1_np[:, rows[0]], w1_np[:, rows[1]]], axis=1)
    sc1 = np.stack([s1[:, rows[0]], s1[:, rows[1]]], axis=1)
    sample = rng.choice(T, size=24, replace=False)
    hid_np = hid.float().cpu().numpy()
    ref = moe.moe_tkg_rows(hid_np[sample], aff[sample], idx[sample], c1, sc1, w2_np, s2)
    assert max_rel(out[sample].float().cpu().numpy(), bf16_values(ref)) <= TOL


@pytest.mark.parametrize("with_residual", [False, True])
def test_moe_block_tkg_vs_oracle(with_residual):
    """RMSNorm -> router -> decode experts, against the composite of the reference's torch references."""
    import nki_library_b200 as m
    Bt, S, H, I, E, K = 4, 8, 1024, 512, 8, 2
    T = Bt * S
    rng = np.random.default_rng(71)
    inp = bf16_values(rng.standard_normal((Bt, S, H)).astype(np.float32) * 2.0)
    res = bf16_values(rng.standard_normal((Bt, S, H)).astype(np.float32)) if with_residual else None
    gamma = bf16_values(rng.uniform(0.5, 1.5, (1, H)).astype(np.float32))
    rw = bf16_values((rng.standard_normal((H, E)) * 0.05).astype(np.float32))
    w_np = make_rows_weights(E, H, I, 72)
    weights = _prep(m, w_np)
    to = lambda a: None if a is None else torch.from_numpy(a).to(torch.bfloat16).cuda()
    outs = m.moe_block_tkg(to(inp), to(gamma), to(rw), weights, None, top_k=K,
                           router_act_fn=m.RouterActFnType.SOFTMAX, router_pre_norm=True, norm_topk_prob=True,
                           expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.POST_SCALE, residual=to(res))
    assert len(outs) == (3 if with_residual else 2)
    x = inp.reshape(T, H) if res is None else bf16_values(inp.reshape(T, H) + res.reshape(T, H))
    if with_residual:
        assert np.array_equal(outs[2].float().cpu().numpy(), x)
    normed = bf16_values(routing.rms_norm(torch.from_numpy(x), torch.from_numpy(gamma)).numpy())
    logits, idx, aff = routing.router_topk(torch.from_numpy(normed), torch.from_numpy(rw), None, K, routing.SOFTMAX,
                                           True, True)
    np.testing.assert_allclose(outs[1].cpu().numpy(), logits.numpy(), rtol=0, atol=2e-2 * np.abs(logits.numpy()).max())
    ref = moe.moe_tkg_rows(normed, aff.numpy(), idx.numpy(), *w_np)
    assert max_rel(outs[0].float().cpu().numpy(), bf16_values(ref)) <= 3e-2  # bf16 RMSNorm rounding can move a row


# ---- weights in the reference's other MX element types: float8_e5m2_x4 and float4_e2m1fn_x4 (MXFP4) ----------
def _prep_fmt(m, w_np, fmt, bias_gu=None, bias_d=None):
    c1, s1, c2, s2 = w_np
    if fmt == "e2m1":
        c1, c2 = mx.pack_e2m1(c1), mx.pack_e2m1(c2)
    t = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (c1, s1, c2, s2)]
    return m.prepare_from_rows(*t, bias_gu=None if bias_gu is None else torch.from_numpy(bias_gu).cuda(),
                               bias_d=None if bias_d is None else torch.from_numpy(bias_d).cuda(), w_format=fmt)


def _fmt_case(T, H, I, E, K, seed, fmt, bias=True):
    from moe_testlib import make_rows_weights_fmt
    hidden, _, _, idx, aff = make_routing(T, H, E, K, seed)
    w_np = make_rows_weights_fmt(E, H, I, fmt, seed)
    rng = np.random.default_rng(seed + 7)
    bgu = rng.uniform(-1.0, 0.5, (E, 2, I)).astype(np.float32) if bias else None
    bd = rng.uniform(-1.0, 1.0, (E, H)).astype(np.float32) if bias else None
    return hidden, idx, aff, w_np, bgu, bd


@pytest.mark.parametrize("impl", [1, 0])
@pytest.mark.parametrize("fmt,B,T", [("e5m2", 128, 256), ("e2m1", 128, 256), ("e2m1", 256, 700)])
def test_moe_cte_other_weight_formats(impl, fmt, B, T):
    """e4m3 activations against e5m2 / e2m1 weights, single-CTA (B=128) and CTA-pair (B=256) tiles."""
    import nki_library_b200 as m
    H, I, E, K = 512, 1024, 4, 2
    hidden, idx, aff, w_np, bgu, bd = _fmt_case(T, H, I, E, K, 71, fmt)
    weights = _prep_fmt(m, w_np, fmt, bgu, bd)
    assert weights.w1.shape[-1] == (H // 2 if fmt == "e2m1" else H)
    N = m.get_n_blocks(T, K, E, B)
    g = m.moe_group_tokens(torch.from_numpy(idx).cuda(), E, B, N, check=True)
    out = m.moe_cte(torch.from_numpy(hidden).to(torch.bfloat16).cuda(), torch.from_numpy(aff).cuda().reshape(-1, 1),
                    weights, None, g["token_position_to_id"], g["block_to_expert"], B,
                    m.MoECTESpec(m.MoECTEImplementation.shard_on_block_mx), conditions=g["conditions"],
                    skip_dma=m.SkipMode(True, False), _impl=impl, _check_status=True)
    ref = moe.moe_cte_rows(hidden, aff, *w_np, g["token_position_to_id"].cpu().numpy(),
                           g["block_to_expert"].cpu().numpy(), B, g["conditions"].cpu().numpy(), bgu, bd, w_fmt=fmt)
    assert max_rel(out.float().cpu().numpy(), bf16_values(ref)) <= TOL


@pytest.mark.parametrize("fmt", ["e5m2", "e2m1"])
def test_moe_cte_reference_storage_other_formats(fmt):
    """x4 words of the reference storage: 32 bits of e5m2 bytes (typed torch.float8_e5m2) or 16 bits of e2m1 nibbles."""
    import nki_library_b200 as m
    T, H, I, E, K, B = 200, 1024, 512, 4, 2, 128
    hidden, idx, aff, w_np, _, bd = _fmt_case(T, H, I, E, K, 73, fmt)
    gw, gs = mx.rows_to_ref_gate_up(w_np[0], w_np[1], fmt)
    dw, ds = mx.rows_to_ref_down(w_np[2], w_np[3], fmt)
    if fmt == "e2m1":
        gw_t, dw_t = torch.from_numpy(gw.view(np.int16)).cuda(), torch.from_numpy(dw.view(np.int16)).cuda()
    else:
        gw_t = torch.from_numpy(gw.view(np.uint8)).cuda().view(torch.float8_e5m2)
        dw_t = torch.from_numpy(dw.view(np.uint8)).cuda().view(torch.float8_e5m2)
    N = m.get_n_blocks(T, K, E, B, 2)
    g = m.moe_group_tokens(torch.from_numpy(idx).cuda(), E, B, N, check=True)
    out = m.moe_cte(torch.from_numpy(hidden).to(torch.bfloat16).cuda(), torch.from_numpy(aff).cuda().reshape(-1, 1),
                    gw_t, dw_t, g["token_position_to_id"], g["block_to_expert"], B,
                    m.MoECTESpec(m.MoECTEImplementation.shard_on_block_mx), conditions=g["conditions"],
                    down_proj_bias=torch.from_numpy(bd).cuda(),
                    quantization_config=m.QuantizationConfig(torch.from_numpy(gs).cuda(), torch.from_numpy(ds).cuda()),
                    skip_dma=m.SkipMode(True, False), _check_status=True)
    ref = moe.moe_cte_rows(hidden, aff, *w_np, g["token_position_to_id"].cpu().numpy(),
                           g["block_to_expert"].cpu().numpy(), B, g["conditions"].cpu().numpy(), None, bd,
                           h_order=mx.hidden_packed_order(H), w_fmt=fmt)
    assert max_rel(out.float().cpu().numpy(), bf16_values(ref)) <= TOL


@pytest.mark.parametrize("fmt", ["e5m2", "e2m1"])
def test_moe_tkg_other_weight_formats(fmt):
    """Decode with MXFP4 / e5m2 expert weights (the reference's selective-expert MXFP4 path,
    core/moe/moe_tkg/selective_expert_mx_impl.py:51-518, quantises activations to e4m3 all the same)."""
    import nki_library_b200 as m
    T, H, I, E, K = 64, 1024, 768, 8, 2
    hidden, idx, aff, w_np, bgu, bd = _fmt_case(T, H, I, E, K, 75, fmt)
    weights = _prep_fmt(m, w_np, fmt, bgu, bd)
    out = m.moe_tkg(torch.from_numpy(hidden).to(torch.bfloat16).cuda(), weights, None, torch.from_numpy(aff).cuda(),
                    torch.from_numpy(idx).cuda(), False,
                    expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.POST_SCALE, _check_status=True)
    ref = moe.moe_tkg_rows(hidden, aff, idx, *w_np, bias_gu=bgu, bias_d=bd, w_fmt=fmt)
    assert max_rel(out.float().cpu().numpy(), bf16_values(ref)) <= TOL


def test_host_pipeline_matches_direct_forward():
    """Five different host batches through the overlapped host pipeline (graphs working in place on the two
    staging pairs) give the bytes a direct forward pass gives."""
    import nki_library_b200 as m
    from nki_library_b200.layer import HostPipeline, MoELayer, random_expert_weights
    T, H, I, E, K, B = 256, 512, 512, 4, 2, 128
    dev = torch.device("cuda")
    weights = random_expert_weights(E, H, I, dev, seed=3)
    gen = torch.Generator().manual_seed(5)
    router_w = (torch.randn(H, E, generator=gen) * 0.02).to(torch.bfloat16).to(dev)
    layer = MoELayer(router_w, weights, K, B, T)
    pipe = HostPipeline(layer)
    assert pipe.in_place
    ins = [torch.randn(T, H, generator=gen).to(torch.bfloat16).pin_memory() for _ in range(5)]
    outs = [torch.empty(T, H, dtype=torch.bfloat16).pin_memory() for _ in range(5)]
    for a, b in zip(ins, outs):
        pipe.submit(a, b)
    pipe.drain()
    assert not any(layer.device_status())
    for a, b in zip(ins, outs):
        ref = layer.forward(a.to(dev)).clone()
        torch.cuda.synchronize()
        assert torch.equal(b, ref.cpu())


def test_moe_tkg_all_expert_with_128_local_experts():
    """All-expert decode with more local experts than the combine once held per token (64): every one of the
    128 experts contributes to every token (the reference's all-expert mode goes to E = 128, test_moe_tkg.py:292-294)."""
    import nki_library_b200 as m
    T, H, I, E, K = 4, 512, 128, 128, 4
    hidden, idx, aff, w_np, bgu, bd = _cte_case(T, H, I, E, K, 128, 91, True, moe.SILU, None)
    rng = np.random.default_rng(92)
    aff = bf16_values(rng.random((T, E)).astype(np.float32))  # dense: no expert is masked out
    weights = _prep(m, w_np, bgu, bd)
    out = m.moe_tkg(torch.from_numpy(hidden).to(torch.bfloat16).cuda(), weights, None, torch.from_numpy(aff).cuda(),
                    torch.from_numpy(idx).cuda(), True, rank_id=torch.zeros((1, 1), dtype=torch.int32, device="cuda"),
                    expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.POST_SCALE, _check_status=True)
    ref = moe.moe_tkg_rows(hidden, aff, None, *w_np, bias_gu=bgu, bias_d=bd, is_all_expert=True)
    assert max_rel(out.float().cpu().numpy(), bf16_values(ref)) <= TOL
    # experts 64..127 alone must move the result: a combine that dropped them would return this partial sum
    part = moe.moe_tkg_rows(hidden, aff * (np.arange(E) < 64), None, *w_np, bias_gu=bgu, bias_d=bd, is_all_expert=True)
    assert max_rel(bf16_values(part), bf16_values(ref)) > 10 * TOL


@pytest.mark.parametrize("dynamic", [False, True])
@pytest.mark.parametrize("rank", [0, 1])
def test_moe_tkg_all_expert_rank_slice(rank, dynamic):
    """Expert-parallel slice of the all-expert mode: this rank holds experts [rank * E_L, (rank + 1) * E_L) of E,
    affinity columns are sliced by ``rank_id`` and masked by ``expert_index`` (core/moe/moe_tkg/moe_tkg.py:100-101,
    178-198, moe_tkg_affinity_masking.py:31-117); summing the ranks' outputs gives the full layer.  ``dynamic`` runs
    only the tokens routed to each expert (core/moe/moe_tkg/all_expert_mx_impl.py:276-350): same result."""
    import nki_library_b200 as m
    T, H, I, E, K, G = 96, 512, 256, 8, 2, 2
    E_L = E // G
    hidden, idx, aff, w_np, bgu, bd = _cte_case(T, H, I, E, K, 128, 93, True, moe.SILU, None)
    rng = np.random.default_rng(94)
    aff = bf16_values(rng.random((T, E)).astype(np.float32))  # dense affinities: the mask has to come from expert_index
    sl = slice(rank * E_L, (rank + 1) * E_L)
    local = tuple(a[sl] for a in w_np)
    weights = _prep(m, local, bgu[sl], bd[sl])
    out = m.moe_tkg(torch.from_numpy(hidden).to(torch.bfloat16).cuda(), weights, None, torch.from_numpy(aff).cuda(),
                    torch.from_numpy(idx).cuda(), True, rank_id=torch.full((1, 1), rank, dtype=torch.int32, device="cuda"),
                    mask_unselected_experts=True, expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.POST_SCALE,
                    is_all_expert_dynamic=dynamic, block_size=32 if dynamic else None, _check_status=True)
    masked = aff * routing.mask_from_index(idx, E)
    ref = moe.moe_tkg_rows(hidden, masked, None, *local, bias_gu=bgu[sl], bias_d=bd[sl], is_all_expert=True,
                           expert_offset=rank * E_L)
    assert max_rel(out.float().cpu().numpy(), bf16_values(ref)) <= TOL


@pytest.mark.parametrize("layout", ["rows", "reference"])
def test_moe_block_tkg_all_expert_fused_norm_quantise(layout):
    """All-expert decode block: RMSNorm (+ residual) and the MXFP8 quantisation run as one kernel (the reference's
    rmsnorm_mx_quantize_tkg step, core/moe_block/moe_block_tkg.py:199-218).  The quantised rows must equal what the
    stand-alone quantiser makes of the normalised rows, bit for bit, in the plain and in the packed hidden order;
    the block's output is checked against the composite oracle."""
    import nki_library_b200 as m
    from nki_library_b200 import _lib, pipeline
    Bt, S, H, I, E, K = 3, 8, 1024, 512, 4, 2
    T = Bt * S
    rng = np.random.default_rng(81)
    inp = bf16_values(rng.standard_normal((Bt, S, H)).astype(np.float32) * 2.0)
    res = bf16_values(rng.standard_normal((Bt, S, H)).astype(np.float32))
    gamma = bf16_values(rng.uniform(0.5, 1.5, (1, H)).astype(np.float32))
    rw = bf16_values((rng.standard_normal((H, E)) * 0.05).astype(np.float32))
    w_np = make_rows_weights(E, H, I, 82)
    to = lambda a: None if a is None else torch.from_numpy(a).to(torch.bfloat16).cuda()
    if layout == "rows":
        weights, h_order = _prep(m, w_np), None
    else:
        gw, gs = mx.rows_to_ref_gate_up(w_np[0], w_np[1])
        dw, ds = mx.rows_to_ref_down(w_np[2], w_np[3])
        weights = m.prepare_from_nki(torch.from_numpy(gw.view(np.int32)).cuda(), torch.from_numpy(gs).cuda(),
                                     torch.from_numpy(dw.view(np.int32)).cuda(), torch.from_numpy(ds).cuda())
        h_order = mx.hidden_packed_order(H)
    outs = m.moe_block_tkg(to(inp), to(gamma), to(rw), weights, None, top_k=K, router_act_fn=m.RouterActFnType.SOFTMAX,
                           router_pre_norm=True, norm_topk_prob=False, is_all_expert=True,
                           rank_id=torch.zeros((1, 1), dtype=torch.int32, device="cuda"),
                           expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.POST_SCALE, residual=to(res))
    x = bf16_values(inp.reshape(T, H) + res.reshape(T, H))
    assert np.array_equal(outs[2].float().cpu().numpy(), x)
    normed = bf16_values(routing.rms_norm(torch.from_numpy(x), torch.from_numpy(gamma)).numpy())
    # the fused kernel's codes and scales of expert 0's rows == quantising its own normalised output separately
    ws = pipeline.get_workspace(E * 128, H, I, outs[0].device)
    got_codes = ws.xq[:T].cpu().numpy()
    got_scales = sf_atoms_to_rows(ws.x_sf.cpu().numpy(), E * 128, H)[:T]
    normed_gpu = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    _lib.call("b200moe_rmsnorm", _lib.ptr(to(x.reshape(T, H))), None, _lib.ptr(to(gamma.reshape(-1))), _lib.BF16, T, H, 0,
              1e-6, _lib.ptr(normed_gpu), None, _lib.stream_ptr())
    nv = normed_gpu.float().cpu().numpy()
    ref_codes, ref_scales = mx.quantize_mx_rows(nv if h_order is None else nv[:, h_order])
    assert np.array_equal(got_codes, ref_codes) and np.array_equal(got_scales, ref_scales)
    logits, idx, aff = routing.router_topk(torch.from_numpy(normed), torch.from_numpy(rw), None, K, routing.SOFTMAX,
                                           True, False)
    masked = aff.numpy() * routing.mask_from_index(idx.numpy(), E)
    ref = moe.moe_tkg_rows(normed, masked, None, *w_np, is_all_expert=True, h_order=h_order)
    assert max_rel(outs[0].float().cpu().numpy(), bf16_values(ref)) <= 3e-2
