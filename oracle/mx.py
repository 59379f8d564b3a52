"""CPU oracle: MXFP8 (E4M3 codes, block-32 UE8M0 scales) arithmetic and layouts.

Test infrastructure only.  Restates, in numpy, the reference's CPU definition
of MX quantisation and of the MX block-scaled matmul:

* block exponent / scale / clip rule ......... core/utils/mx_torch_common.py:157-221
  (``quantize_to_mx``: ``scale = clip(e_max - 8, 0, 255)``, data divided by
  ``2**(e_max - 8 - 127)``, clipped to +-448, then cast to e4m3fn)
* dequantise-and-contract .................... core/utils/mx_torch_common.py:134-154
  (``mx_matmul``)
* e4m3fn byte decoding ....................... core/utils/mx_torch_common.py:107-131
* x4 packing (byte j of a 32-bit word = element j) core/utils/mx_torch_common.py:114-124
* weight / activation "swizzled" layouts ..... test/integration/nkilib/core/mlp/test_mlp_common.py:550-682

Pinned: ``quantize_to_mx_ref_blocks`` reproduces the reference's own
``quantize_to_mx`` bit for bit and the contraction its ``mx_matmul`` to 1e-6 on
the fixtures in tests/golden/mx_ref.npz (tests/test_oracle_golden.py), which
were produced by running the reference's code with two stand-in packages
(tests/golden/standins).  One declared assumption remains: the fp32 -> e4m3
rounding lives in ``neuron_dtypes.static_cast``, a package the reference does
not vendor; the stand-in and this file use IEEE round-to-nearest-even onto the
e4m3fn grid after the +-448 clip (what ``ml_dtypes.float8_e4m3fn`` and the
GPU's ``cvt.rn.satfinite.e4m3x2.f32`` both do).
"""

from __future__ import annotations

import numpy as np

E4M3_MAX = 448.0
E4M3_MAX_EXP = 8  # exponent of the largest e4m3 binade, mx_torch_common.py:196-200
BLOCK = 32


# --------------------------------------------------------------------------
# e4m3fn scalar codec
# --------------------------------------------------------------------------
def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3fn byte, round-to-nearest-even, saturating at +-448.

    Works on exact binary arithmetic only (frexp / rint), so the result does
    not depend on the host's libm.
    """
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.minimum(np.abs(x).astype(np.float64), E4M3_MAX)
    # subnormal grid: multiples of 2^-9 below 2^-6
    sub = a < 2.0**-6
    q_sub = np.rint(a * 2.0**9).astype(np.int32)  # 0..8 (8 == smallest normal)
    m, e = np.frexp(np.where(sub, 1.0, a))  # a = m * 2^e, m in [0.5, 1)
    e = e - 1  # a = (2m) * 2^e, 2m in [1, 2)
    frac = np.rint((2.0 * m - 1.0) * 8.0).astype(np.int32)  # 0..8
    carry = frac == 8
    e = np.where(carry, e + 1, e)
    frac = np.where(carry, 0, frac)
    q_norm = ((e + 7) << 3) | frac
    q = np.where(sub, q_sub, q_norm)
    q = np.minimum(q, 0x7E)  # 0x7F is NaN in e4m3fn
    q = np.where(np.isnan(x), 0x7F, q)
    return (q.astype(np.uint8) | sign).astype(np.uint8)


def _build_decode_lut() -> np.ndarray:
    b = np.arange(256, dtype=np.int32)
    s = (b >> 7) & 1
    e = (b >> 3) & 0xF
    m = b & 0x7
    sub = (m / 8.0) * 2.0**-6
    nor = (1.0 + m / 8.0) * np.power(2.0, e.astype(np.float64) - 7.0)
    v = np.where(e == 0, sub, nor)
    v = np.where(s == 1, -v, v)
    v = np.where((b & 0x7F) == 0x7F, np.nan, v)
    return v.astype(np.float32)


_E4M3_LUT = _build_decode_lut()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    """e4m3fn byte -> float32 (mx_torch_common.py:107-131)."""
    return _E4M3_LUT[np.asarray(codes, dtype=np.uint8)]


def _build_e5m2_lut() -> np.ndarray:
    """float8_e5m2 byte -> float32: S(1) E(5) M(2), bias 15 (mx_torch_common.py:85-105; like the
    reference's unpack, exponent 31 is decoded as an ordinary binade rather than inf/NaN)."""
    b = np.arange(256, dtype=np.int32)
    s = (b >> 7) & 1
    e = (b >> 2) & 0x1F
    m = b & 0x3
    sub = (m / 4.0) * 2.0**-14
    nor = (1.0 + m / 4.0) * np.power(2.0, e.astype(np.float64) - 15.0)
    v = np.where(e == 0, sub, nor)
    return np.where(s == 1, -v, v).astype(np.float32)


_E5M2_LUT = _build_e5m2_lut()
# float4_e2m1fn nibble -> float32: S(1) E(2) M(1), bias 1, finite only (mx_torch_common.py:31-67)
_E2M1_LUT = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
                     dtype=np.float32)

FORMATS = ("e4m3", "e5m2", "e2m1")


def e5m2_decode(codes: np.ndarray) -> np.ndarray:
    return _E5M2_LUT[np.asarray(codes, dtype=np.uint8)]


def e2m1_decode(nibbles: np.ndarray) -> np.ndarray:
    """One 4-bit code per array element (values 0..15) -> float32."""
    return _E2M1_LUT[np.asarray(nibbles, dtype=np.uint8) & 0xF]


def decode_elements(codes: np.ndarray, fmt: str = "e4m3") -> np.ndarray:
    """Element codes (one per array element, whatever the storage width) -> float32."""
    if fmt == "e4m3":
        return e4m3_decode(codes)
    if fmt == "e5m2":
        return e5m2_decode(codes)
    if fmt == "e2m1":
        return e2m1_decode(codes)
    raise ValueError(fmt)


def pack_e2m1(nibbles: np.ndarray) -> np.ndarray:
    """``[..., K]`` nibbles -> ``[..., K/2]`` bytes, element 2j in the low half of byte j.  This is also the
    memory image of the reference's float4_e2m1fn_x4 words (16 bits, element j in bits 4j..4j+3;
    mx_torch_common.py:70-82)."""
    n = np.asarray(nibbles, dtype=np.uint8) & 0xF
    return (n[..., 0::2] | (n[..., 1::2] << 4)).astype(np.uint8)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    b = np.asarray(packed, dtype=np.uint8)
    out = np.empty(b.shape[:-1] + (b.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = b & 0xF
    out[..., 1::2] = b >> 4
    return out


# --------------------------------------------------------------------------
# block quantisation
# --------------------------------------------------------------------------
def _biased_exponent(x_f32: np.ndarray) -> np.ndarray:
    return ((np.ascontiguousarray(x_f32, dtype=np.float32).view(np.uint32) >> 23) & 0xFF).astype(np.int32)


def quantize_mx_rows(x: np.ndarray):
    """Quantise ``x [R, K]`` (K % 32 == 0) with one scale per 32 contiguous K.

    Returns ``(codes uint8 [R, K], scales uint8 [R, K // 32])``.

    Same arithmetic as ``quantize_to_mx`` (mx_torch_common.py:203-221); only
    the shape of a block differs (1 x 32 here, 8 x 4 of a transposed and
    folded view there).  ``ref_hidden_blocks_equal_contiguous`` in the tests
    shows the two views pick identical element sets once K is taken in the
    reference's packed order.
    """
    x = np.asarray(x, dtype=np.float32)
    R, K = x.shape
    assert K % BLOCK == 0
    xb = x.reshape(R, K // BLOCK, BLOCK)
    e_max = _biased_exponent(xb).max(axis=2)  # [R, K/32]
    scales = np.clip(e_max - E4M3_MAX_EXP, 0, 255).astype(np.uint8)
    factor = np.power(2.0, e_max.astype(np.float64) - E4M3_MAX_EXP - 127.0)
    q = np.clip(xb.astype(np.float64) / factor[:, :, None], -E4M3_MAX, E4M3_MAX)
    codes = e4m3_encode(q.astype(np.float32)).reshape(R, K)
    return codes, scales


def quantize_to_mx_ref_blocks(data: np.ndarray):
    """The reference's own block shape: ``data [P, F]``, blocks of 8 rows x 4 cols.

    Restates mx_torch_common.py:157-221 for e4m3.  Returns
    ``(codes uint8 [P, F], scales uint8 [P // 8, F // 4])``; codes are left as
    one byte per element (the reference packs 4 consecutive F elements into a
    32-bit word, byte j = element j, which is the same memory image).
    """
    d = np.asarray(data, dtype=np.float32)
    P, F = d.shape
    assert P % 8 == 0 and F % 4 == 0
    e = _biased_exponent(d).reshape(P // 8, 8, F // 4, 4).max(axis=(1, 3))
    scales = np.clip(e - E4M3_MAX_EXP, 0, 255).astype(np.uint8)
    factor = np.power(2.0, e.astype(np.float64) - E4M3_MAX_EXP - 127.0)
    fe = np.repeat(np.repeat(factor, 8, axis=0), 4, axis=1)
    q = np.clip(d.astype(np.float64) / fe, -E4M3_MAX, E4M3_MAX)
    return e4m3_encode(q.astype(np.float32)), scales


def dequantize_mx_rows(codes: np.ndarray, scales: np.ndarray, fmt: str = "e4m3") -> np.ndarray:
    """``x_hat = decode(code) * 2**(scale - 127)`` per 32-block (mx_torch_common.py:146-152).
    ``codes`` holds one element code per array element (e2m1: unpacked nibbles)."""
    codes = np.asarray(codes, dtype=np.uint8)
    lead = codes.shape[:-1]
    K = codes.shape[-1]
    if fmt == "e4m3" and codes.size >= (1 << 20):
        # large operands (the timed CPU baseline): the same table lookup and power-of-two product, done by
        # torch's multi-threaded e4m3fn -> fp32 conversion (identical values; NaN codes decode to NaN in both)
        import torch
        v = torch.from_numpy(np.ascontiguousarray(codes)).view(torch.float8_e4m3fn).float().view(*lead, K // BLOCK, BLOCK)
        f = torch.exp2(torch.from_numpy(np.ascontiguousarray(scales)).float() - 127.0)
        return (v * f[..., None]).view(*lead, K).numpy()
    v = decode_elements(codes, fmt).reshape(*lead, K // BLOCK, BLOCK)
    f = np.power(2.0, scales.astype(np.float32) - 127.0).astype(np.float32)
    return (v * f[..., None]).reshape(*lead, K)


def mx_matmul_rows(a_codes, a_scales, b_codes, b_scales) -> np.ndarray:
    """``out[m, n] = sum_k A_hat[m, k] * B_hat[n, k]`` in float32 (both K-major)."""
    a = dequantize_mx_rows(a_codes, a_scales)
    b = dequantize_mx_rows(b_codes, b_scales)
    return a @ b.T


# --------------------------------------------------------------------------
# the reference's storage layouts <-> plain K-major arrays
# --------------------------------------------------------------------------
def hidden_packed_order(H: int) -> np.ndarray:
    """Index vector ``h_of[k']`` giving the hidden column stored at packed position k'.

    The reference folds the hidden axis as ``[4 (q), H/512 (t), 128 (p)]``
    (``reshape(T, 4, H/512, 128)``, bwmm_shard_on_block_mx.py:271 and
    test_mlp_common.py:594) and contracts in the order ``(t, p, q)``:
    ``k' = t*512 + p*4 + q`` holds logical column ``h = q*(H/4) + t*128 + p``.
    One scale covers p in [8g, 8g+8) x q in [0, 4), i.e. 32 consecutive k'.
    """
    assert H % 512 == 0
    nt = H // 512
    t, p, q = np.meshgrid(np.arange(nt), np.arange(128), np.arange(4), indexing="ij")
    return (q * (H // 4) + t * 128 + p).reshape(-1).astype(np.int64)


def inter_packed_order(I: int) -> np.ndarray:
    """``i_of[j]``: logical gate/up output column held at packed intermediate position j.

    test_mlp_common.py:607-624: inside each 512-wide tile (or the single
    I-wide tile when I < 512) logical column ``q*(rows/4) + p`` is stored at
    ``p*4 + q``; the down weight's I axis is already in that packed order
    (test_mlp_common.py:654-661).
    """
    out = np.empty(I, dtype=np.int64)
    if I < 512:
        tiles = [(0, I)]
    else:
        assert I % 512 == 0
        tiles = [(s, 512) for s in range(0, I, 512)]
    for start, rows in tiles:
        assert rows % 4 == 0
        p, q = np.meshgrid(np.arange(rows // 4), np.arange(4), indexing="ij")
        out[start + (p * 4 + q).reshape(-1)] = start + (q * (rows // 4) + p).reshape(-1)
    return out


def _as_bytes_x4(w: np.ndarray) -> np.ndarray:
    """View an x4-packed array (uint32 words or a trailing axis of 4 bytes) as [..., 4] uint8."""
    w = np.ascontiguousarray(w)
    if w.dtype == np.uint8:
        assert w.shape[-1] == 4
        return w
    assert w.dtype.itemsize == 4, "x4-packed fp8 weights are 32-bit words"
    return w.view(np.uint8).reshape(*w.shape, 4)


def ref_gate_up_to_rows(w_x4: np.ndarray, scale: np.ndarray):
    """Reference gate/up storage -> K-major rows.

    ``w_x4 [E, 128(p), 2, H/512(t), I]`` (4 packed bytes = q) and
    ``scale [E, 16(g), 2, H/512(t), I]`` (bwmm_shard_on_block_mx.py docstring,
    test_utils.py:376-381) become ``codes [E, 2, I, H]`` with the H axis in
    packed order k' and the I axis in packed order j, plus
    ``scales [E, 2, I, H/32]``.
    """
    b = _as_bytes_x4(w_x4)  # [E, p, 2, t, I, q]
    E, P, two, nt, I, _ = b.shape
    assert P == 128 and two == 2
    codes = b.transpose(0, 2, 4, 3, 1, 5).reshape(E, 2, I, nt * 512)
    sc = np.asarray(scale, dtype=np.uint8).transpose(0, 2, 4, 3, 1).reshape(E, 2, I, nt * 16)
    perm = inter_packed_order(I)
    return np.ascontiguousarray(codes[:, :, perm, :]), np.ascontiguousarray(sc[:, :, perm, :])


def ref_down_to_rows(w_x4: np.ndarray, scale: np.ndarray):
    """Reference down storage ``[E, p_I, ceil(I/512), H]`` x4 -> ``codes [E, H, I]`` (packed I order)."""
    b = _as_bytes_x4(w_x4)  # [E, p, tile, H, q]
    E, P, nt, H, _ = b.shape
    codes = b.transpose(0, 3, 2, 1, 4).reshape(E, H, nt * P * 4)
    sc = np.asarray(scale, dtype=np.uint8).transpose(0, 3, 2, 1).reshape(E, H, -1)
    return np.ascontiguousarray(codes), np.ascontiguousarray(sc)


def ref_gate_up_bias_to_rows(bias: np.ndarray) -> np.ndarray:
    """``[E, p_I, 2, ceil(I/512), 4]`` -> ``[E, 2, I]`` in packed I order (test_mlp_common.py:626-630)."""
    b = np.asarray(bias, dtype=np.float32)
    E, P, two, nt, four = b.shape
    return np.ascontiguousarray(b.transpose(0, 2, 3, 1, 4).reshape(E, 2, nt * P * 4))


def _x4_words(c4: np.ndarray, fmt: str) -> np.ndarray:
    """``[..., 4]`` element codes -> the reference's x4 word per group: 32 bits of four bytes, or for e2m1
    16 bits of four nibbles (element j in bits 4j..4j+3)."""
    c4 = np.ascontiguousarray(c4, dtype=np.uint8)
    if fmt == "e2m1":
        c = c4.astype(np.uint16) & 0xF
        return (c[..., 0] | (c[..., 1] << 4) | (c[..., 2] << 8) | (c[..., 3] << 12)).astype(np.uint16)
    return c4.view(np.uint32).reshape(c4.shape[:-1])


def rows_to_ref_gate_up(codes: np.ndarray, scales: np.ndarray, fmt: str = "e4m3"):
    """Inverse of ``ref_gate_up_to_rows`` (used to fabricate reference-format test inputs)."""
    E, two, I, H = codes.shape
    nt = H // 512
    perm = inter_packed_order(I)
    inv = np.empty_like(perm)
    inv[perm] = np.arange(I)
    c = codes[:, :, inv, :].reshape(E, 2, I, nt, 128, 4).transpose(0, 4, 1, 3, 2, 5)
    s = scales[:, :, inv, :].reshape(E, 2, I, nt, 16).transpose(0, 4, 1, 3, 2)
    w = _x4_words(c, fmt).reshape(E, 128, 2, nt, I)
    return w, np.ascontiguousarray(s)


def rows_to_ref_down(codes: np.ndarray, scales: np.ndarray, fmt: str = "e4m3"):
    """Inverse of ``ref_down_to_rows``."""
    E, H, I = codes.shape
    P = 128 if I > 512 else I // 4
    nt = I // (P * 4)
    c = codes.reshape(E, H, nt, P, 4).transpose(0, 3, 2, 1, 4)
    s = scales.reshape(E, H, nt, P // 8).transpose(0, 3, 2, 1)
    w = _x4_words(c, fmt).reshape(E, P, nt, H)
    return w, np.ascontiguousarray(s)
