"""CPU oracle: the non-MX expert MLP (bf16 or fp8-row weights) for prefill (moe_cte) and decode (moe_tkg).

Test infrastructure only.  Restates, in torch fp32, the reference's CPU definitions:

* prefill block loop ....... core/moe/moe_cte/moe_cte_torch.py:26-242 (``moe_cte_torch_ref``)
* decode expert MLP ........ core/moe/moe_tkg/moe_tkg_torch.py:226-297 (``_compute_expert_mlp``)
* decode loops ............. core/moe/moe_tkg/moe_tkg_torch.py:146-218
* activations .............. core/moe/moe_cte/moe_cte_torch_utils.py:23-42

Pinned: tests/test_oracle_golden.py compares both functions with outputs of those reference functions run on
the seeded inputs of tests/golden_inputs.py (tests/golden/mx_ref.npz, parts ``dense_cte`` / ``dense_tkg``).
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

SILU, GELU, GELU_TANH, SWISH = 0, 1, 2, 3
NO_SCALE, POST_SCALE, PRE_SCALE = 0, 1, 2


def act(x: torch.Tensor, kind: int) -> torch.Tensor:
    if kind == SILU:
        return F.silu(x)
    if kind == GELU:
        return F.gelu(x)
    if kind == GELU_TANH:
        return F.gelu(x, approximate="tanh")
    if kind == SWISH:
        return x * torch.sigmoid(1.702 * x)
    raise ValueError(kind)


def _t(a):
    return None if a is None else torch.as_tensor(np.asarray(a, dtype=np.float32))


def moe_cte_dense(hidden, affinities, gate_up_w, down_w, token_position_to_id, block_to_expert, block_size,
                  conditions=None, bias_gu=None, bias_d=None, gate_up_scale=None, down_scale=None, act_fn=SILU,
                  gate_clamp=(None, None), up_clamp=(None, None), scaling=POST_SCALE, skip_token=True) -> np.ndarray:
    """Prefill layer of the non-MX variants, fp32 ``[T, H]``.

    ``hidden [T or T+1, H]``, ``affinities [rows, E]``, ``gate_up_w [E, H, 2, I]``, ``down_w [E, I, H]`` (values of
    whatever storage type, as fp32), biases ``[E, 2, I]`` / ``[E, H]``, fp8-row factors ``gate_up_scale [E or 1, 1, 2I]``
    and ``down_scale [E or 1, 1, H]``; clamps are ``(lower, upper)``.  Per block: gather rows (pad ids read a zero
    row), optionally multiply by the bf16 affinity (PRE_SCALE), fp32 matmuls, scale, bias, clamp, act(gate) * up,
    down projection, scale, bias, optional affinity (POST_SCALE), round to bf16, accumulate
    (moe_cte_torch.py:125-225).  The loop stops at the first zero ``conditions``.
    """
    hidden = _t(hidden)
    aff = _t(affinities)
    gw, dw = _t(gate_up_w), _t(down_w)
    E, H, _, I = gw.shape
    gw = gw.reshape(E, H, 2 * I)
    B = block_size
    tpi = torch.as_tensor(np.asarray(token_position_to_id)).long().reshape(-1, B)
    N = tpi.shape[0]
    T = hidden.shape[0] if skip_token else hidden.shape[0] - 1
    rows = hidden.shape[0]
    out = torch.zeros((rows + 1, H), dtype=torch.float32)
    hid = torch.cat([hidden, torch.zeros(1, H)])           # index -1 (skip_token pads) reads the zero row
    af = torch.cat([aff.reshape(-1, E), torch.zeros(1, E)])
    gs = None if gate_up_scale is None else _t(gate_up_scale).reshape(-1, 2 * I)
    ds = None if down_scale is None else _t(down_scale).reshape(-1, H)
    bgu, bd = _t(bias_gu), _t(bias_d)
    for b in range(N):
        if conditions is not None and int(conditions[b]) == 0:
            break
        ids = tpi[b]
        e = int(block_to_expert[b])
        if e >= E:
            continue
        x = hid[ids]
        a = af[ids, e].unsqueeze(1).to(torch.bfloat16).float()   # the reference casts it to the hidden dtype
        if scaling == PRE_SCALE:
            x = a * x
        gu = (x @ gw[e]).reshape(B, 2, I)
        g, u = gu[:, 0].clone(), gu[:, 1].clone()
        if gs is not None:
            s = gs[e if gs.shape[0] == E else 0]
            g *= s[:I]
            u *= s[I:]
        if bgu is not None:
            g += bgu[e, 0]
            u += bgu[e, 1]
        if gate_clamp[0] is not None or gate_clamp[1] is not None:
            g = torch.clamp(g, min=gate_clamp[0], max=gate_clamp[1])
        if up_clamp[0] is not None or up_clamp[1] is not None:
            u = torch.clamp(u, min=up_clamp[0], max=up_clamp[1])
        y = (act(g, act_fn) * u) @ dw[e]
        if ds is not None:
            y = y * ds[e if ds.shape[0] == E else 0]
        if bd is not None:
            y = y + bd[e]
        if scaling == POST_SCALE:
            y = y * a
        out[ids] += y.to(torch.bfloat16).float()
    return out[:T].numpy()


def expert_mlp_dense(x, gate_up_w, down_w, bias_gu=None, bias_d=None, act_fn=SILU, gate_clamp_upper=None,
                     up_clamp=(None, None), gate_up_scale=None, down_scale=None) -> torch.Tensor:
    """One expert of the decode reference (moe_tkg_torch.py:226-297): ``gate_up_w [H, 2, I]``, ``down_w [I, H]``,
    fp8-row factors ``gate_up_scale [2, I]`` / ``down_scale [H]`` folded into the weights first; the gate has an
    upper clamp only."""
    gwt, uwt = gate_up_w[:, 0, :], gate_up_w[:, 1, :]
    if gate_up_scale is not None:
        gwt = gwt * gate_up_scale[0:1]
        uwt = uwt * gate_up_scale[1:2]
    g = x @ gwt
    if bias_gu is not None:
        g = g + bias_gu[0]
    if gate_clamp_upper is not None:
        g = torch.clamp(g, max=gate_clamp_upper)
    g = act(g, act_fn)
    u = x @ uwt
    if bias_gu is not None:
        u = u + bias_gu[1]
    if up_clamp[0] is not None or up_clamp[1] is not None:
        u = torch.clamp(u, min=up_clamp[0], max=up_clamp[1])
    dwt = down_w if down_scale is None else down_w * down_scale.unsqueeze(0)
    y = (g * u) @ dwt
    if bias_d is not None:
        y = y + bias_d
    return y


def moe_tkg_dense(hidden, affinities, expert_index, gate_up_w, down_w, bias_gu=None, bias_d=None, act_fn=SILU,
                  gate_clamp_upper=None, up_clamp=(None, None), gate_up_scale=None, down_scale=None, post_scale=True,
                  is_all_expert=False) -> np.ndarray:
    """Decode layer of the non-MX variants, fp32 ``[T, H]`` (moe_tkg_torch.py:146-218): every (token, k) pair runs
    its expert (pairs of one expert are batched here; rows are independent), all-expert mode runs every expert on
    every token and skips experts whose affinity column is all zero."""
    x = _t(hidden)
    aff = _t(affinities)
    gw, dw = _t(gate_up_w), _t(down_w)
    bgu, bd = _t(bias_gu), _t(bias_d)
    gs, ds = _t(gate_up_scale), _t(down_scale)
    T, H = x.shape
    E = gw.shape[0]
    out = torch.zeros((T, H), dtype=torch.float32)
    idx = None if expert_index is None else torch.as_tensor(np.asarray(expert_index)).long()
    for e in range(E):
        if is_all_expert:
            if float(aff[:, e].sum()) == 0.0:
                continue
            tok = torch.arange(T)
        else:
            tok = torch.nonzero((idx == e).any(dim=1)).flatten()
            if tok.numel() == 0:
                continue
        y = expert_mlp_dense(x[tok], gw[e], dw[e], None if bgu is None else bgu[e], None if bd is None else bd[e],
                             act_fn, gate_clamp_upper, up_clamp, None if gs is None else gs[e],
                             None if ds is None else ds[e])
        if post_scale:
            y = y * aff[tok, e].unsqueeze(1)
        out[tok] += y
    return out.numpy()
