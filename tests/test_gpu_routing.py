"""CUDA router and grouping kernels against the golden fixtures and the CPU oracle (bit-exact integers)."""

import hashlib
import json
import os

import numpy as np
import pytest
import torch

import golden_inputs as gi
from oracle import routing

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def lib():
    import nki_library_b200 as m
    return m


@pytest.fixture(scope="module")
def digests():
    with open(os.path.join(GOLD, "grouping_ref_digests.json")) as f:
        return json.load(f)


@pytest.fixture(params=["split_k", "tcgen05"])
def router_path(request):
    """Runs a router test on the split-K path and with the single-kernel tcgen05 path forced wherever the shape
    is eligible for it (x [T, H], E <= 256, H % 64 == 0; other shapes fall back by themselves)."""
    return request.param


@pytest.mark.parametrize("name", list(gi.ROUTER_CASES))
@pytest.mark.parametrize("x_layout", [1, 0])
def test_router_topk_vs_reference_fixture(lib, name, x_layout, router_path):
    if router_path == "tcgen05" and x_layout == 0:
        pytest.skip("the tcgen05 path takes x as [T, H] only")
    gold = np.load(os.path.join(GOLD, "router_topk_ref.npz"))
    T, H, E, k, act, has_bias, pre_norm, l1 = gi.ROUTER_CASES[name]
    x, w, b = gi.router_inputs(T, H, E, has_bias)
    act_e = lib.RouterActFnType.SOFTMAX if act == "softmax" else lib.RouterActFnType.SIGMOID
    xd = x.cuda() if x_layout == 1 else x.T.contiguous().cuda()
    logits = torch.empty((T, E), dtype=torch.float32, device="cuda")
    aff = torch.empty((T, E), dtype=torch.float32, device="cuda")
    idx = torch.empty((T, k), dtype=torch.int32, device="cuda")
    outs = lib.router_topk(xd, w.cuda(), None if b is None else b.cuda(), logits, aff, idx, act_e, k, x_layout, 0,
                           router_pre_norm=pre_norm, norm_topk_prob=l1, use_indirect_dma_scatter=True,
                           _path=1 if router_path == "split_k" else 2)
    assert outs[0] is logits and outs[1] is idx and outs[2] is aff
    lg = logits.cpu().numpy()
    # bf16 products are exact in fp32; only the summation order (tensor-core tree, split-K) differs
    np.testing.assert_allclose(lg, gold[name + "/logits"], rtol=0, atol=1e-4)
    # top-K and affinities are exact functions of the logits: the oracle on the GPU's own logits must agree bit for bit
    act_id = routing.SOFTMAX if act == "softmax" else routing.SIGMOID
    o_idx, o_aff = routing.router_from_logits(torch.from_numpy(lg), k, act_id, pre_norm, l1)
    assert np.array_equal(idx.cpu().numpy(), o_idx.numpy().astype(np.int32))
    np.testing.assert_allclose(aff.cpu().numpy(), o_aff.numpy(), rtol=2e-6, atol=1e-7)
    # and against the stored reference outputs wherever the reference's own top-K margin exceeds the logit tolerance
    ref_lg = np.sort(gold[name + "/logits"], axis=1)[:, ::-1]
    safe = (ref_lg[:, :k] - ref_lg[:, 1:k + 1]).min(axis=1) > 4e-4 if k < E else np.ones(T, bool)
    assert np.array_equal(idx.cpu().numpy()[safe], gold[name + "/index"][safe])
    np.testing.assert_allclose(aff.cpu().numpy()[safe], gold[name + "/aff"][safe], rtol=0, atol=1e-4)


def test_router_bf16_outputs_and_eager(lib):
    T, H, E, k = 70, 1024, 64, 4
    x, w, b = gi.router_inputs(T, H, E, True)
    logits = torch.empty((T, E), dtype=torch.bfloat16, device="cuda")
    aff = torch.empty((T, E), dtype=torch.bfloat16, device="cuda")
    idx = torch.empty((T, k), dtype=torch.uint32, device="cuda")
    outs = lib.router_topk(x.cuda(), w.cuda(), b.cuda(), logits, aff, idx, lib.RouterActFnType.SOFTMAX, k, 1, 0,
                           router_pre_norm=True, norm_topk_prob=True, return_eager_affi=True)
    _, o_idx, o_aff = routing.router_topk(x, w, b, k, routing.SOFTMAX, True, True)
    assert np.array_equal(idx.cpu().view(torch.int32).numpy(), o_idx.numpy().astype(np.int32))
    # reference tolerance for the router: |a-b| <= 1e-5 + 2e-2 * max|golden|
    assert np.abs(aff.float().cpu().numpy() - o_aff.numpy()).max() <= 1e-5 + 2e-2 * o_aff.abs().max().item()
    assert outs[3].shape == (T, k)


def test_router_rejects_illegal_arguments(lib):
    x, w, _ = gi.router_inputs(4, 256, 16, False)
    mk = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device="cuda")
    with pytest.raises(AssertionError):  # K > 8 (test_router_topk.py boundary value k=9)
        lib.router_topk(x.cuda(), w.cuda(), None, mk(4, 16), mk(4, 16), mk(4, 9, dt=torch.int32),
                        lib.RouterActFnType.SOFTMAX, 9, 1, 0)
    xb, wb, _ = gi.router_inputs(4, 256, 513, False)
    with pytest.raises(AssertionError):  # E = 513
        lib.router_topk(xb.cuda(), wb.cuda(), None, mk(4, 513), mk(4, 513), mk(4, 4, dt=torch.int32),
                        lib.RouterActFnType.SOFTMAX, 4, 1, 0)
    with pytest.raises(AssertionError):  # sigmoid + ACT2 without indirect scatter
        lib.router_topk(x.cuda(), w.cuda(), None, mk(4, 16), mk(4, 16), mk(4, 4, dt=torch.int32),
                        lib.RouterActFnType.SIGMOID, 4, 1, 0, router_pre_norm=False)
    with pytest.raises(AssertionError):  # CPU tensors: no fallback
        lib.router_topk(x, w, None, mk(4, 16), mk(4, 16), mk(4, 4, dt=torch.int32), lib.RouterActFnType.SOFTMAX, 4, 1, 0)


@pytest.mark.parametrize("name", list(gi.NONZERO_CASES))
def test_find_nonzero_indices_vs_reference(lib, name, digests):
    T, E, top_k, dtype, cs, nc = gi.NONZERO_CASES[name]
    inp = gi.sparse_input(T, E, top_k, dtype)
    kw = {}
    if cs is not None:
        kw = dict(col_start_id=torch.tensor([cs], dtype=torch.int32, device="cuda"), n_cols=nc)
    ind, cnt = lib.find_nonzero_indices(torch.from_numpy(inp).cuda(), **kw)
    d = digests["find_nonzero_indices"][name]
    assert _digest(cnt.cpu().numpy()) == d["counts"]
    assert _digest(ind.cpu().numpy()) == d["indices"]


def test_find_nonzero_ragged_and_empty_columns(lib):
    rng = np.random.default_rng(3)
    T, C = 777, 37  # neither a multiple of the chunk nor of the warp size
    m = (rng.random((T, C)) < 0.1).astype(np.float32) * 0.5
    m[:, 5] = 0  # empty column
    m[:, 6] = 1  # full column
    ind, cnt = lib.find_nonzero_indices(torch.from_numpy(m).to(torch.bfloat16).cuda())
    o_ind, o_cnt = routing.find_nonzero_indices(m)
    assert np.array_equal(ind.cpu().numpy(), o_ind) and np.array_equal(cnt.cpu().numpy(), o_cnt)


@pytest.mark.parametrize("name", list(gi.FLATTEN_CASES))
def test_indexed_flatten_vs_reference(lib, name, digests):
    kw = gi.flatten_inputs(*gi.FLATTEN_CASES[name])
    start = kw["row_offsets_start"]
    out = lib.indexed_flatten(torch.from_numpy(kw["input_tensor"]).cuda(), kw["f_len"], kw["output_len"],
                              torch.from_numpy(kw["row_offsets"]).cuda(),
                              None if start is None else torch.tensor([start], dtype=torch.int32, device="cuda"),
                              kw["padding_val"])
    assert _digest(out.cpu().numpy()) == digests["indexed_flatten"][name]


def test_indexed_flatten_overlap_and_out_of_range(lib):
    inp = np.arange(3 * 64, dtype=np.int32).reshape(3, 64)
    offs = np.array([1, 2, 7], dtype=np.int32)  # rows 0/1 overlap; row 2 partly outside
    out = lib.indexed_flatten(torch.from_numpy(inp).cuda(), 16, 9 * 16 + 5, torch.from_numpy(offs).cuda())
    assert np.array_equal(out.cpu().numpy(), routing.indexed_flatten(inp, 16, 9 * 16 + 5, offs))


def test_cumsum(lib):
    rng = np.random.default_rng(0)
    x = rng.integers(0, 50, size=(3, 1000)).astype(np.int32)
    assert np.array_equal(lib.cumsum(torch.from_numpy(x).cuda()).cpu().numpy(), np.cumsum(x, axis=-1))
    f = rng.integers(0, 9, size=(5, 257)).astype(np.float32)
    assert np.array_equal(lib.cumsum(torch.from_numpy(f).cuda()).cpu().numpy(), np.cumsum(f, axis=-1))


GROUP_SHAPES = {
    "c1": (256, 4, 2, 128), "c2": (4096, 8, 2, 512), "c3_decode": (64, 8, 2, 128),
    "c4": (8192, 256, 8, 128), "c5": (32768, 128, 8, 256), "ragged": (1000, 24, 3, 128), "one_token": (1, 8, 2, 128),
}


@pytest.mark.parametrize("name", list(GROUP_SHAPES))
@pytest.mark.parametrize("mode", ["index", "mask"])
@pytest.mark.parametrize("skip_token", [True, False])
def test_group_tokens_bit_exact(lib, name, mode, skip_token):
    T, E, K, B = GROUP_SHAPES[name]
    mask = gi.routing_mask(T, E, K, seed=5)
    N = routing.get_n_blocks(T, K, E, B)
    if mode == "index":
        idx = np.argsort(-mask, axis=1, kind="stable")[:, :K].astype(np.int32)
        idx = idx[:, ::-1].copy()  # order inside a token must not matter
        g = lib.moe_group_tokens(torch.from_numpy(idx).cuda(), E, B, N, skip_token=skip_token, check=True)
    else:
        aff = (mask * 0.25).astype(np.float32)
        g = lib.moe_group_tokens(torch.from_numpy(aff).cuda(), E, B, N, top_k=K, skip_token=skip_token, check=True)
    tpi, b2e, cond, counts = routing.group_tokens(mask, B, N, skip_token=skip_token)
    assert np.array_equal(g["counts"].cpu().numpy(), counts)
    assert np.array_equal(g["block_to_expert"].cpu().numpy(), b2e)
    assert np.array_equal(g["conditions"].cpu().numpy(), cond)
    assert np.array_equal(g["token_position_to_id"].cpu().numpy(), tpi)
    if mode == "index":
        inv = g["inverse_map"].cpu().numpy()
        pos_e = np.repeat(b2e, B)
        assert (inv >= 0).all()
        assert np.array_equal(tpi[inv], np.repeat(np.arange(T)[:, None], K, axis=1))
        assert np.array_equal(pos_e[inv], idx)


@pytest.mark.parametrize("name", list(gi.CHAIN_CASES))
def test_three_step_grouping_chain_vs_reference(lib, name, digests):
    """find_nonzero_indices -> cumsum -> indexed_flatten, the way the reference's caller chains them."""
    T, E, K, B = gi.CHAIN_CASES[name]
    mask = torch.from_numpy(gi.routing_mask(T, E, K)).cuda()
    ind, cnt = lib.find_nonzero_indices(mask)
    bpe = (cnt + B - 1) // B
    offs = (lib.cumsum(bpe) - bpe).to(torch.int32)
    Tpad = -(-T // B) * B
    ind_p = torch.full((E, Tpad), -1, dtype=torch.int32, device="cuda")
    ind_p[:, :T] = ind
    N = gi.n_blocks(T, K, E, B)
    tpi = lib.indexed_flatten(ind_p, B, N * B, offs)
    assert _digest(tpi.cpu().numpy()) == digests["grouping_chain"][name]
    fused = lib.moe_group_tokens(mask, E, B, N, top_k=K)
    assert torch.equal(fused["token_position_to_id"], tpi)


def test_group_tokens_reports_too_few_blocks(lib):
    idx = torch.zeros((300, 1), dtype=torch.int32, device="cuda")  # 300 tokens on expert 0 need 3 blocks
    g = lib.moe_group_tokens(idx, 4, 128, 2)
    assert int(g["status"].item()) != 0
