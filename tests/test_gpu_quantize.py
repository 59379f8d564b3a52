"""MXFP8 activation quantisation and weight relayout: codes and scales bit-exact against the CPU oracle."""

import numpy as np
import pytest
import torch

from moe_testlib import bf16_values, gate_up_dev_rows, make_rows_weights, sf_atoms_to_rows
from oracle import mx

pytestmark = pytest.mark.gpu


def _gather_quantize(hidden_np, tpi_np, packed):
    from nki_library_b200 import _lib
    lib = _lib.load_library()
    hidden = torch.from_numpy(hidden_np).to(torch.bfloat16).cuda()
    rows, H = hidden.shape
    n_pos = len(tpi_np) if tpi_np is not None else rows
    tpi = None if tpi_np is None else torch.from_numpy(tpi_np.astype(np.int32)).cuda()
    codes = torch.empty((n_pos, H), dtype=torch.uint8, device="cuda")
    sf = torch.full((lib.b200moe_sf_bytes(n_pos, H),), 0xAB, dtype=torch.uint8, device="cuda")
    flags = torch.full(((n_pos + 127) // 128,), 7, dtype=torch.int32, device="cuda")
    _lib.call("b200moe_gather_quantize_mxfp8", _lib.ptr(hidden), rows, H, _lib.ptr(tpi), n_pos, int(packed),
              _lib.ptr(codes), _lib.ptr(sf), _lib.ptr(flags), _lib.stream_ptr())
    torch.cuda.synchronize()
    return codes.cpu().numpy(), sf_atoms_to_rows(sf.cpu().numpy(), n_pos, H), flags.cpu().numpy()


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("H", [512, 4096])
def test_gather_quantize_bit_exact(packed, H):
    rng = np.random.default_rng(0)
    T = 300
    hidden = bf16_values(rng.standard_normal((T, H)).astype(np.float32) * np.exp(rng.uniform(-6, 6, (T, 1))))
    hidden[3] = 0.0                      # all-zero row -> scale byte 0, codes 0
    hidden[4, :32] = 0.0                 # one zero block
    hidden[5, 7] = 3.0e38                # huge element: block mates flush to 0
    hidden[6, :64] = 2.0 ** -130         # bf16 subnormals
    hidden[7, 0:4] = [448.0, -448.0, 1.0, 2.0 ** -9]
    tpi = rng.integers(0, T, size=640).astype(np.int32)
    tpi[10:40] = -1                      # pads
    tpi[500:] = T + 3                    # out-of-range ids are pads too
    tpi[256:384] = -1                    # a whole 128-position tile of pads
    codes, scales, flags = _gather_quantize(hidden, tpi, packed)
    src = np.where(((tpi >= 0) & (tpi < T))[:, None], hidden[np.clip(tpi, 0, T - 1)], 0.0).astype(np.float32)
    if packed:
        src = src[:, mx.hidden_packed_order(H)]
    o_codes, o_scales = mx.quantize_mx_rows(src)
    assert np.array_equal(scales, o_scales)
    assert np.array_equal(codes, o_codes)
    # per 128-position tile: 1 + index of the last row that holds a token (0 = all pads)
    assert list(flags) == [128, 128, 0, 116, 0]


def test_gather_quantize_identity_rows():
    rng = np.random.default_rng(1)
    hidden = bf16_values(rng.standard_normal((130, 1024)).astype(np.float32))
    codes, scales, _ = _gather_quantize(hidden, None, False)
    o_codes, o_scales = mx.quantize_mx_rows(hidden)
    assert np.array_equal(codes, o_codes) and np.array_equal(scales, o_scales)


@pytest.mark.parametrize("I", [256, 1024])
@pytest.mark.parametrize("layout", ["rows", "nki"])
def test_prepare_weights_layouts(layout, I):
    import nki_library_b200 as m
    E, H = 3, 1024
    c1, s1, c2, s2 = make_rows_weights(E, H, I, seed=2)
    rng = np.random.default_rng(4)
    bgu = rng.uniform(-2, 0.5, (E, 2, I)).astype(np.float32)
    bd = rng.uniform(-1, 1, (E, H)).astype(np.float32)
    if layout == "rows":
        w = m.prepare_from_rows(*(torch.from_numpy(a).cuda() for a in (c1, s1, c2, s2)),
                                bias_gu=torch.from_numpy(bgu).cuda(), bias_d=torch.from_numpy(bd).cuda())
        assert not w.h_packed_order
    else:
        gw, gs = mx.rows_to_ref_gate_up(c1, s1)
        dw, ds = mx.rows_to_ref_down(c2, s2)
        pI = 128 if I > 512 else I // 4
        bref = np.ascontiguousarray(bgu.reshape(E, 2, I // (pI * 4), pI, 4).transpose(0, 3, 1, 2, 4))
        w = m.prepare_from_nki(torch.from_numpy(gw.view(np.int32)).cuda(), torch.from_numpy(gs).cuda(),
                               torch.from_numpy(dw.view(np.int32)).cuda(), torch.from_numpy(ds).cuda(),
                               torch.from_numpy(bref).to(torch.bfloat16).cuda(), torch.from_numpy(bd).cuda())
        assert w.h_packed_order
        bgu = bf16_values(bgu)
    rows = gate_up_dev_rows(I)
    w1 = w.w1.cpu().numpy()
    sf1 = w.w1_sf.cpu().numpy().reshape(E, -1)
    for e in range(E):
        for s in (0, 1):
            assert np.array_equal(w1[e, rows[s]], c1[e, s])
            assert np.array_equal(sf_atoms_to_rows(sf1[e], 2 * I, H)[rows[s]], s1[e, s])
            assert np.array_equal(w.bias_gu.cpu().numpy()[e, rows[s]], bgu[e, s])
    assert np.array_equal(w.w2.cpu().numpy(), c2)
    sf2 = w.w2_sf.cpu().numpy().reshape(E, -1)
    for e in range(E):
        assert np.array_equal(sf_atoms_to_rows(sf2[e], H, I), s2[e])
    assert np.array_equal(w.bias_d.cpu().numpy(), bd)


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("H,K", [(512, 2), (4096, 8), (1024, 1), (96, 3)])
def test_scatter_quantize_equals_gather_quantize(packed, H, K):
    """The token-major kernel (driven by the inverse map) writes, at every occupied position, the bytes the
    position-major kernel writes, and the same per-tile row counts; unoccupied positions keep their old bytes."""
    from nki_library_b200 import _lib
    import nki_library_b200 as m
    if packed and H % 512:
        pytest.skip("the packed hidden order needs H % 512 == 0")
    rng = np.random.default_rng(3)
    T, E, B = 333, 8, 128
    hidden = bf16_values(rng.standard_normal((T, H)).astype(np.float32) * np.exp(rng.uniform(-4, 4, (T, 1))))
    idx = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32)
    N = m.get_n_blocks(T, K, E, B)
    g = m.moe_group_tokens(torch.from_numpy(idx).cuda(), E, B, N, top_k=K, check=True)
    tpi, inv = g["token_position_to_id"], g["inverse_map"]
    n_pos = N * B
    hid = torch.from_numpy(hidden).to(torch.bfloat16).cuda()
    lib = _lib.load_library()

    def buffers():
        return (torch.full((n_pos, H), 0xAB, dtype=torch.uint8, device="cuda"),
                torch.full((lib.b200moe_sf_bytes(n_pos, H),), 0xCD, dtype=torch.uint8, device="cuda"),
                torch.full((n_pos // 128,), 7, dtype=torch.int32, device="cuda"))
    c1, s1, f1 = buffers()
    c2, s2, f2 = buffers()
    _lib.call("b200moe_gather_quantize_mxfp8", _lib.ptr(hid), T, H, _lib.ptr(tpi), n_pos, int(packed), _lib.ptr(c1),
              _lib.ptr(s1), _lib.ptr(f1), _lib.stream_ptr())
    _lib.call("b200moe_scatter_quantize_mxfp8", _lib.ptr(hid), T, H, _lib.ptr(inv), K, n_pos, int(packed),
              _lib.ptr(c2), _lib.ptr(s2), _lib.ptr(f2), _lib.stream_ptr())
    torch.cuda.synchronize()
    occ = (tpi >= 0).cpu().numpy()
    assert torch.equal(f1, f2)
    c1, c2 = c1.cpu().numpy(), c2.cpu().numpy()
    assert np.array_equal(c1[occ], c2[occ])
    r1 = sf_atoms_to_rows(s1.cpu().numpy(), n_pos, H if H % 128 == 0 else (H + 127) // 128 * 128)
    r2 = sf_atoms_to_rows(s2.cpu().numpy(), n_pos, H if H % 128 == 0 else (H + 127) // 128 * 128)
    assert np.array_equal(r1[occ][:, : H // 32], r2[occ][:, : H // 32])
    if H % 128 == 0:
        assert (c2[~occ] == 0xAB).all()   # untouched
