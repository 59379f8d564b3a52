"""Shape fuzzing of the integer kernels (bit-exact against the oracle) and full-size property checks."""

import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

from oracle import routing

pytestmark = pytest.mark.gpu


@settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck))
@given(T=st.integers(1, 3000), E=st.integers(1, 300), K=st.integers(1, 8), B=st.sampled_from([1, 128, 256, 512]),
       seed=st.integers(0, 1000), skip=st.booleans())
def test_group_tokens_fuzz(T, E, K, B, seed, skip):
    import nki_library_b200 as m
    K = min(K, E)
    rng = np.random.default_rng(seed)
    bias = rng.standard_normal(E) * 2.0  # skewed expert popularity, some experts empty
    idx = np.argsort(-(rng.random((T, E)) + bias), axis=1, kind="stable")[:, :K].astype(np.int32)
    N = routing.get_n_blocks(T, K, E, B)
    g = m.moe_group_tokens(torch.from_numpy(idx).cuda(), E, B, N, top_k=K, skip_token=skip, check=True)
    tpi, b2e, cond, counts = routing.group_tokens(routing.mask_from_index(idx, E), B, N, skip_token=skip)
    assert np.array_equal(g["token_position_to_id"].cpu().numpy(), tpi)
    assert np.array_equal(g["block_to_expert"].cpu().numpy(), b2e)
    assert np.array_equal(g["conditions"].cpu().numpy(), cond)
    assert np.array_equal(g["counts"].cpu().numpy(), counts)
    inv = g["inverse_map"].cpu().numpy()
    assert np.array_equal(tpi[inv], np.repeat(np.arange(T)[:, None], K, axis=1))


@settings(max_examples=25, deadline=None, suppress_health_check=list(HealthCheck))
@given(T=st.integers(1, 2000), C=st.integers(1, 200), density=st.floats(0.0, 1.0), seed=st.integers(0, 1000))
def test_find_nonzero_fuzz(T, C, density, seed):
    import nki_library_b200 as m
    rng = np.random.default_rng(seed)
    x = (rng.random((T, C)) < density).astype(np.int32) * rng.integers(1, 9, (T, C)).astype(np.int32)
    ind, cnt = m.find_nonzero_indices(torch.from_numpy(x).cuda())
    o_ind, o_cnt = routing.find_nonzero_indices(x)
    assert np.array_equal(ind.cpu().numpy(), o_ind) and np.array_equal(cnt.cpu().numpy(), o_cnt)


@pytest.mark.parametrize("T,H,I,E,K,B,zipf", [(8192, 7168, 2048, 256, 8, 128, 1.2), (32768, 4096, 1536, 128, 8, 256, None),
                                              (140000, 256, 4096, 4, 2, 128, None)])
def test_full_size_layer_properties(T, H, I, E, K, B, zipf):
    """The fine-grained and the 32768-token prefill configurations at full size: grouping bit-exact, the layer deterministic and linear in the affinity,
    and a sample of tokens within tolerance of the oracle (weights read back from the device).  The third shape
    (280000 rows, 32 gate/up weight tiles, a two-slab contraction) gives every CTA pair more tiles than its
    prologue table holds (472 > 448), so the last weight tiles of the last expert go through the on-the-spot
    decode."""
    import nki_library_b200 as m
    from moe_testlib import bf16_values, gate_up_dev_rows, max_rel, sf_atoms_to_rows
    from nki_library_b200.layer import MoELayer, random_expert_weights
    from oracle import moe
    g = torch.Generator().manual_seed(5)
    hidden = torch.randn((T, H), generator=g).to(torch.bfloat16)
    rw = (torch.randn((H, E), generator=g) * 0.02).to(torch.bfloat16)
    bias = None
    if zipf:
        bias = (-zipf * torch.log(torch.randperm(E, generator=g).float() + 1)).to(torch.bfloat16)
    weights = random_expert_weights(E, H, I, "cuda", seed=3)
    layer = MoELayer(rw.cuda(), weights, K, B, T, None if bias is None else bias.cuda())
    x = hidden.cuda()
    out = layer.forward(x).clone()
    assert not any(layer.device_status())
    idx = layer.idx.cpu().numpy()
    aff = layer.aff.cpu().numpy()
    tpi, b2e, cond, _ = routing.group_tokens(routing.mask_from_index(idx, E), B, layer.N)
    assert np.array_equal(layer.tpi.cpu().numpy(), tpi) and np.array_equal(layer.b2e.cpu().numpy(), b2e)
    assert np.array_equal(layer.cond.cpu().numpy(), cond)
    assert torch.equal(out, layer.forward(x))
    assert torch.isfinite(out.float()).all()
    # oracle on a few tokens: only their experts' weights are pulled back and dequantised
    rng = np.random.default_rng(0)
    sample = rng.choice(T, size=6, replace=False)
    if E <= 8:   # make sure the last expert (whose last tiles come latest in the walk) is among the sampled ones
        sample[0] = int(np.nonzero((idx == E - 1).any(axis=1))[0][0])
    experts = np.unique(idx[sample])
    remap = {int(e): i for i, e in enumerate(experts)}
    rows = gate_up_dev_rows(I)
    w1 = weights.w1[torch.from_numpy(experts).cuda().long()].cpu().numpy()
    w2 = weights.w2[torch.from_numpy(experts).cuda().long()].cpu().numpy()
    s1_all = weights.w1_sf.view(E, -1)[torch.from_numpy(experts).cuda().long()].cpu().numpy()
    s2_all = weights.w2_sf.view(E, -1)[torch.from_numpy(experts).cuda().long()].cpu().numpy()
    s1 = np.stack([sf_atoms_to_rows(s1_all[i], 2 * I, H) for i in range(len(experts))])
    s2 = np.stack([sf_atoms_to_rows(s2_all[i], H, I) for i in range(len(experts))])
    c1 = np.stack([w1[:, rows[0]], w1[:, rows[1]]], axis=1)
    sc1 = np.stack([s1[:, rows[0]], s1[:, rows[1]]], axis=1)
    idx_l = np.vectorize(remap.get)(idx[sample]).astype(np.int32)
    aff_l = np.zeros((len(sample), len(experts)), dtype=np.float32)
    for r, t in enumerate(sample):
        for k in range(K):
            aff_l[r, idx_l[r, k]] = aff[t, idx[t, k]]
    ref = moe.moe_tkg_rows(hidden[torch.from_numpy(sample)].float().numpy(), aff_l, idx_l, c1, sc1, w2, s2)
    assert max_rel(out[torch.from_numpy(sample).cuda()].float().cpu().numpy(), bf16_values(ref)) <= 2e-2
