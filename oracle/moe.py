"""CPU oracle: blockwise MXFP8 expert MLP for prefill (moe_cte) and decode (moe_tkg).

Test infrastructure only.  Two restatements live here:

1. ``*_rows`` functions work on plain K-major arrays (codes ``[rows, K]`` with one
   scale per 32 contiguous K).  They are what the CUDA kernels are compared with.
2. ``ref_layout_*`` functions follow the reference's numpy goldens step by step
   in the reference's own storage layout (8 x 4 blocks of a folded, transposed
   view): test/integration/nkilib/core/mlp/test_mlp_common.py:550-682.  They
   exist to show that (1) composed with the layout adapters of ``oracle.mx``
   gives the same numbers, so parity with (1) is parity with the reference.

Per-block recipe ........ test/integration/nkilib/core/moe/moe_cte/test_utils.py:528-725
Decode recipe ........... core/moe/moe_tkg/moe_tkg_torch.py:299-442
Activations ............. core/moe/moe_cte/moe_cte_torch_utils.py:23-42 and
                          moe_tkg_torch.py:341-346 (Swish = x * sigmoid(1.702 x))

Known divergence inside the reference: the device kernel rounds act(gate)*up to
bf16 before re-quantising it (bwmm_shard_on_block_mx.py:1270-1278) while the
numpy golden keeps fp32 (test_utils.py:668-687).  ``round_inter_bf16`` selects
either; the CUDA path follows the device kernel (True).
"""

from __future__ import annotations

import math

import numpy as np
import torch

from . import mx

SILU, GELU, GELU_TANH, SWISH = 0, 1, 2, 3


def _act(x: np.ndarray, kind: int) -> np.ndarray:
    x = x.astype(np.float32)
    if kind == SILU:
        return x / (1.0 + np.exp(-x))
    if kind == SWISH:
        return x / (1.0 + np.exp(-1.702 * x))
    if kind == GELU:
        return torch.nn.functional.gelu(torch.from_numpy(x)).numpy()
    if kind == GELU_TANH:
        return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x**3)))
    raise ValueError(kind)


def _bf16_round(x: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def _mm(a: np.ndarray, b_t: np.ndarray) -> np.ndarray:
    """fp32 ``a @ b_t.T`` through torch (multi-threaded)."""
    return (torch.from_numpy(a) @ torch.from_numpy(b_t).T).numpy()


class ExpertWeights:
    """Dequantised fp32 weights of one expert: ``w1 [2, I, H]``, ``w2 [H, I]``.

    ``fmt`` is the element type of the codes ("e4m3", "e5m2" or "e2m1", one code per array element);
    activations are quantised to e4m3 whatever the weights are (moe_tkg_torch.py:364-370)."""

    def __init__(self, w1_codes, w1_scales, w2_codes, w2_scales, e, fmt="e4m3"):
        self.w1 = mx.dequantize_mx_rows(w1_codes[e], w1_scales[e], fmt)
        self.w2 = mx.dequantize_mx_rows(w2_codes[e], w2_scales[e], fmt)


def expert_mlp_rows(x, ew: ExpertWeights, bias_gu=None, bias_d=None, act=SILU,
                    gate_clamp=(None, None), up_clamp=(None, None), round_inter_bf16=True,
                    return_parts=False):
    """One expert on rows ``x [R, H]`` (fp32 values of bf16 inputs).

    quantise(x) -> gate/up contraction (+bias, clamp) -> act(gate)*up -> quantise
    -> down contraction (+bias).  ``gate_clamp``/``up_clamp`` are ``(lower, upper)``.
    """
    xq, xs = mx.quantize_mx_rows(x)
    xh = mx.dequantize_mx_rows(xq, xs)
    g = _mm(xh, ew.w1[0])
    u = _mm(xh, ew.w1[1])
    if bias_gu is not None:
        g = g + bias_gu[0][None, :]
        u = u + bias_gu[1][None, :]
    if gate_clamp[0] is not None or gate_clamp[1] is not None:
        g = np.clip(g, gate_clamp[0], gate_clamp[1])
    if up_clamp[0] is not None or up_clamp[1] is not None:
        u = np.clip(u, up_clamp[0], up_clamp[1])
    m = _act(g, act) * u
    if round_inter_bf16:
        m = _bf16_round(m)
    mq, ms = mx.quantize_mx_rows(m)
    y = _mm(mx.dequantize_mx_rows(mq, ms), ew.w2)
    if bias_d is not None:
        y = y + bias_d[None, :]
    if return_parts:
        return y, dict(xq=xq, xs=xs, g=g, u=u, m=m, mq=mq, ms=ms)
    return y


def moe_cte_rows(hidden, affinities, w1_codes, w1_scales, w2_codes, w2_scales,
                 token_position_to_id, block_to_expert, block_size, conditions=None,
                 bias_gu=None, bias_d=None, act=SILU, gate_clamp=(None, None), up_clamp=(None, None),
                 h_order=None, post_scale=True, round_inter_bf16=True, max_blocks=None, w_fmt="e4m3"):
    """Prefill layer: ``out[T, H]`` fp32 (caller casts to bf16).

    ``hidden [T or T+1, H]`` fp32 values; ``affinities [rows, E]`` fp32 values;
    pad ids (-1 or >= T) contribute nothing.  The block loop stops at the
    first ``conditions[b] == 0`` (test_utils.py:536-538).  Each block adds
    ``bf16(y * affinity)`` to its tokens' rows (test_utils.py:714-725); the
    running sum is kept in fp32 here and rounded once by the caller, which is
    also what the CUDA combine does.
    """
    hidden = np.asarray(hidden, dtype=np.float32)
    aff = np.asarray(affinities, dtype=np.float32)
    tpi = np.asarray(token_position_to_id).reshape(-1, block_size)
    N = tpi.shape[0]
    E = w1_codes.shape[0]
    T = hidden.shape[0] if aff.shape[0] == hidden.shape[0] and (tpi.max() < hidden.shape[0]) else hidden.shape[0]
    H = hidden.shape[1]
    out = np.zeros((hidden.shape[0], H), dtype=np.float32)
    cache_e, ew = -1, None
    nb = N if max_blocks is None else min(N, max_blocks)
    for b in range(nb):
        if conditions is not None and conditions[b] == 0:
            break
        ids = tpi[b]
        valid = (ids >= 0) & (ids < hidden.shape[0])
        if not valid.any():
            continue
        e = int(block_to_expert[b])
        if e != cache_e:
            ew = ExpertWeights(w1_codes, w1_scales, w2_codes, w2_scales, e, w_fmt)
            cache_e = e
        tok = ids[valid]
        x = hidden[tok]
        if h_order is not None:
            x = x[:, h_order]
        y = expert_mlp_rows(x, ew, None if bias_gu is None else bias_gu[e], None if bias_d is None else bias_d[e],
                            act, gate_clamp, up_clamp, round_inter_bf16)
        if post_scale:
            y = y * aff[tok, e][:, None]
        np.add.at(out, tok, _bf16_round(y))
    return out


def moe_tkg_rows(hidden, affinities, expert_index, w1_codes, w1_scales, w2_codes, w2_scales,
                 bias_gu=None, bias_d=None, act=SILU, gate_clamp=(None, None), up_clamp=(None, None),
                 h_order=None, post_scale=True, round_inter_bf16=True, is_all_expert=False,
                 expert_offset=0, w_fmt="e4m3"):
    """Decode layer, fp32 ``[T, H]``: every (token, k) pair runs its expert on that token alone.

    Selective mode follows moe_tkg_torch.py:432-440 (pairs are independent, so
    pairs of one expert are batched here); all-expert mode follows :425-431 for
    the local experts ``[expert_offset, expert_offset + E_local)``.
    """
    hidden = np.asarray(hidden, dtype=np.float32)
    aff = np.asarray(affinities, dtype=np.float32)
    T, H = hidden.shape
    E = w1_codes.shape[0]
    out = np.zeros((T, H), dtype=np.float32)
    x_all = hidden if h_order is None else hidden[:, h_order]
    idx = None if expert_index is None else np.asarray(expert_index).astype(np.int64)
    for e in range(E):
        ge = e + expert_offset
        if is_all_expert:
            tok = np.arange(T)
        else:
            tok = np.flatnonzero((idx == ge).any(axis=1))
        if tok.size == 0:
            continue
        ew = ExpertWeights(w1_codes, w1_scales, w2_codes, w2_scales, e, w_fmt)
        y = expert_mlp_rows(x_all[tok], ew, None if bias_gu is None else bias_gu[e],
                            None if bias_d is None else bias_d[e], act, gate_clamp, up_clamp, round_inter_bf16)
        if post_scale:
            y = y * aff[tok, ge][:, None]
        out[tok] += y
    return out


# --------------------------------------------------------------------------
# Reference-layout restatement (validation of the layout adapters)
# --------------------------------------------------------------------------
def _ref_mx_contract(stat_codes, mov_codes, stat_scale, mov_scale):
    """``out[i, j] = sum_{k,q} S[k, i, q] M[k, j, q]`` with 8-row x 4 block scales (mx_torch_common.py:134-154).

    ``*_codes [P, F*4]`` bytes (F x4-packed words per row), ``*_scale [P/8, F]``.
    """
    def deq(codes, scale):
        P = codes.shape[0]
        v = mx.e4m3_decode(codes).reshape(P, -1, 4)
        f = np.power(2.0, scale.astype(np.float32) - 127.0)
        f = np.repeat(f, 8, axis=0)[:P]
        return v * f[:, :, None]

    s = deq(stat_codes, stat_scale)
    m = deq(mov_codes, mov_scale)
    return np.einsum("kiq,kjq->ij", s, m, optimize=True)


def ref_layout_gate_or_up(hidden_rows, w_x4_bytes, w_scale, bias, H, I):
    """Follows ``_gate_up_proj_golden_mx`` (test_mlp_common.py:550-632) for unquantised hidden.

    ``hidden_rows [R, H]`` fp32; ``w_x4_bytes [128, H/512, I, 4]`` uint8;
    ``w_scale [16, H/512, I]``; ``bias [p, ceil(I/512), 4]`` or None.
    Returns the reference's folded output ``[128, ceil(I/512), R, 4]``.
    """
    R = hidden_rows.shape[0]
    nt = H // 512
    folded = hidden_rows.reshape(R, 4, nt, 128).transpose(3, 2, 0, 1).reshape(128, -1)
    hq, hs = mx.quantize_to_mx_ref_blocks(folded)  # [128, nt*R*4], [16, nt*R]
    hq = hq.reshape(128, nt, R * 4).transpose(1, 0, 2).reshape(nt * 128, R * 4)
    hs = hs.reshape(16, nt, R).transpose(1, 0, 2).reshape(nt * 16, R)
    wq = w_x4_bytes.transpose(1, 0, 2, 3).reshape(nt * 128, I * 4)
    ws = w_scale.transpose(1, 0, 2).reshape(nt * 16, I)
    res = _ref_mx_contract(wq, hq, ws, hs)  # [I, R]
    n_tiles = math.ceil(I / 512)
    out = np.zeros((128, n_tiles, R, 4), dtype=np.float32)
    for t in range(n_tiles):
        rows = 512 if not (t == n_tiles - 1 and I % 512) else I % 512
        cur = res[t * 512: t * 512 + rows]
        rp = math.ceil(rows / 8) * 8
        if rp > rows:
            cur = np.pad(cur, ((0, rp - rows), (0, 0)))
        out[: rp // 4, t] = cur.reshape(4, rp // 4, R).transpose(1, 2, 0)
    if bias is not None:
        b = np.asarray(bias, dtype=np.float32)
        if b.shape[0] < 128:
            b = np.pad(b, ((0, 128 - b.shape[0]), (0, 0), (0, 0)))
        out += b[:, :, None, :]
    return out


def ref_layout_down(inter_folded, w_x4_bytes, w_scale, bias, H, I):
    """Follows ``_down_proj_golden_mx`` (test_mlp_common.py:635-682).

    ``inter_folded [128, ceil(I/512), R, 4]``; ``w_x4_bytes [p_I, ceil(I/512), H, 4]``;
    ``w_scale [p_I/8, ceil(I/512), H]``.  Returns ``[R, H]``.
    """
    R = inter_folded.shape[2]
    wq = w_x4_bytes.transpose(1, 0, 2, 3).reshape(-1, H * 4)
    ws = w_scale.transpose(1, 0, 2).reshape(-1, H)
    x = inter_folded
    if I < 512:
        x = x[: math.ceil(I / 4)]
    x = x.transpose(1, 0, 2, 3).reshape(-1, R * 4)
    P_al = ws.shape[0] * 8
    if x.shape[0] < P_al:
        x = np.pad(x, ((0, P_al - x.shape[0]), (0, 0)))
    wq = wq[:P_al] if wq.shape[0] >= P_al else np.pad(wq, ((0, P_al - wq.shape[0]), (0, 0)))
    xq, xs = mx.quantize_to_mx_ref_blocks(x)
    res = _ref_mx_contract(xq, wq, xs, ws)  # [R, H]
    if bias is not None:
        res = res + np.asarray(bias, dtype=np.float32).reshape(1, H)
    return res


def ref_layout_expert_mlp(hidden_rows, gate_up_w_x4, gate_up_scale, down_w_x4, down_scale,
                          gate_up_bias=None, down_bias=None, act=SILU,
                          gate_clamp=(None, None), up_clamp=(None, None), round_inter_bf16=False):
    """One block through the reference's golden recipe in reference layout (test_utils.py:582-700).

    ``gate_up_w_x4 [128, 2, H/512, I]`` (uint32 or [...,4] uint8), ``gate_up_scale [16, 2, H/512, I]``,
    ``down_w_x4 [p_I, ceil(I/512), H]``, ``down_scale [p_I/8, ceil(I/512), H]``.
    """
    gw = mx._as_bytes_x4(gate_up_w_x4)
    dw = mx._as_bytes_x4(down_w_x4)
    H = gw.shape[2] * 512
    I = gw.shape[3]
    outs = []
    for s in (0, 1):
        b = None if gate_up_bias is None else np.asarray(gate_up_bias)[:, s]
        outs.append(ref_layout_gate_or_up(hidden_rows, gw[:, s], np.asarray(gate_up_scale)[:, s], b, H, I))
    g, u = outs
    if gate_clamp[0] is not None or gate_clamp[1] is not None:
        g = np.clip(g, gate_clamp[0], gate_clamp[1])
    if up_clamp[0] is not None or up_clamp[1] is not None:
        u = np.clip(u, up_clamp[0], up_clamp[1])
    m = _act(g, act) * u
    if round_inter_bf16:
        m = _bf16_round(m)
    return ref_layout_down(m, dw, np.asarray(down_scale), down_bias, H, I)
