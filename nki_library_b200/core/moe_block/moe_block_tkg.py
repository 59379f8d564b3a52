"""``moe_block_tkg``: RMSNorm -> router_topk -> moe_tkg for token generation, with the reference's signature
(core/moe_block/moe_block_tkg.py:39-75)."""

from __future__ import annotations

from typing import Optional

import torch

import math

from ... import _lib, pipeline
from ...weights import ExpertWeights, prepare_from_nki_cached
from ..moe.moe_tkg.moe_tkg import all_expert_layout, moe_tkg
from ..router_topk.router_topk import router_topk
from ..utils.common_types import ActFnType, ExpertAffinityScaleMode, RouterActFnType
from ..utils.kernel_call import kernel_entry


@kernel_entry
def moe_block_tkg(
    inp: torch.Tensor,
    gamma: torch.Tensor,
    router_weights: torch.Tensor,
    expert_gate_up_weights,
    expert_down_weights,
    shared_expert_gate_w=None,
    shared_expert_up_w=None,
    shared_expert_down_w=None,
    expert_gate_up_weights_scale=None,
    expert_down_weights_scale=None,
    router_bias=None,
    expert_gate_up_bias=None,
    expert_down_bias=None,
    shared_expert_gate_bias=None,
    shared_expert_up_bias=None,
    shared_expert_down_bias=None,
    eps: float = 1e-6,
    top_k: int = 1,
    router_act_fn: RouterActFnType = RouterActFnType.SIGMOID,
    router_pre_norm: bool = True,
    norm_topk_prob: bool = False,
    expert_affinities_scaling_mode: ExpertAffinityScaleMode = ExpertAffinityScaleMode.NO_SCALE,
    hidden_act_fn: ActFnType = ActFnType.SiLU,
    hidden_act_scale_factor: Optional[float] = None,
    hidden_act_bias: Optional[float] = None,
    gate_clamp_upper_limit: Optional[float] = None,
    gate_clamp_lower_limit: Optional[float] = None,
    up_clamp_upper_limit: Optional[float] = None,
    up_clamp_lower_limit: Optional[float] = None,
    router_mm_dtype=torch.bfloat16,
    hidden_actual: Optional[int] = None,
    skip_router_logits: bool = False,
    is_all_expert: bool = False,
    rank_id: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
):
    """Decode MoE block on ``inp [B, S, H]`` (or ``[T, H]``) bf16.

    RMSNorm (fp32 statistics, optional fused residual add) -> ``router_topk`` on the normalised rows ->
    ``moe_tkg`` with the MXFP8 expert weights.  Returns ``(out[, router_logits][, residual_out])`` like the
    reference (moe_block_tkg.py:342-349).  As there, ``router_pre_norm`` also selects masking of unselected
    experts in all-expert mode (moe_block_tkg_torch.py:103-112).  Shared experts are dense bf16 MLPs outside
    the MX path and are rejected, as are ``hidden_act_scale_factor`` / ``hidden_act_bias``.
    """
    A = _lib.kernel_assert
    A(shared_expert_gate_w is None and shared_expert_up_w is None and shared_expert_down_w is None,
      "shared experts are not part of the MX expert path and are not supported")
    A(hidden_act_scale_factor is None and hidden_act_bias is None,
      "hidden_act_scale_factor / hidden_act_bias are not supported")
    _lib.require_cuda(inp, gamma, router_weights, router_bias, residual, rank_id)
    A(inp.dtype == torch.bfloat16, "inp must be bfloat16")
    H = inp.shape[-1]
    x = inp.reshape(-1, H).contiguous()
    T = x.shape[0]
    res = None if residual is None else residual.reshape(-1, H).to(torch.bfloat16).contiguous()
    g = None
    if gamma is not None:
        g = gamma.reshape(-1).contiguous()
        if g.dtype not in (torch.float32, torch.bfloat16):
            g = g.float()
        A(g.numel() == H, "gamma must have H elements")
    normed = torch.empty_like(x)
    residual_out = torch.empty_like(x) if res is not None else None
    g_code = _lib.F32 if g is None else _lib.dtype_code(g)
    h_act = 0 if hidden_actual is None else int(hidden_actual)
    # MX weights in all-expert mode: every token's positions are known before the router runs (token t sits at
    # position e * T_pad + t of every local expert), so the normalised rows are quantised by the kernel that
    # produces them -- the reference's rmsnorm_mx_quantize_tkg step (moe_block_tkg.py:199-218)
    prequantized = None
    mx_weights = isinstance(expert_gate_up_weights, ExpertWeights) or (
        isinstance(expert_gate_up_weights, torch.Tensor) and expert_gate_up_weights.dim() == 5)
    if is_all_expert and mx_weights and H % 128 == 0:
        if not isinstance(expert_gate_up_weights, ExpertWeights):
            A(expert_gate_up_weights_scale is not None and expert_down_weights_scale is not None,
              "Scales must be set when using MX weights")
            expert_gate_up_weights = prepare_from_nki_cached(
                expert_gate_up_weights, expert_gate_up_weights_scale, expert_down_weights, expert_down_weights_scale,
                expert_gate_up_bias, expert_down_bias)
        w = expert_gate_up_weights
        _, _, table = all_expert_layout(T, w.E, x.device)
        n_pos = w.E * math.ceil(T / 128) * 128
        prequantized = pipeline.get_workspace(n_pos, H, w.I, x.device)
        _lib.call("b200moe_rmsnorm_quantize_mxfp8", _lib.ptr(x), _lib.ptr(res), _lib.ptr(g), g_code, T, H, h_act,
                  float(eps), _lib.ptr(normed), _lib.ptr(residual_out), _lib.ptr(table), table.shape[1], n_pos,
                  int(w.h_packed_order), _lib.ptr(prequantized.xq), _lib.ptr(prequantized.x_sf),
                  _lib.ptr(prequantized.tile_flags), _lib.stream_ptr())
    else:
        _lib.call("b200moe_rmsnorm", _lib.ptr(x), _lib.ptr(res), _lib.ptr(g), g_code, T, H, h_act, float(eps),
                  _lib.ptr(normed), _lib.ptr(residual_out), _lib.stream_ptr())

    E = router_weights.shape[1]
    logits = torch.empty((T, E), dtype=torch.float32, device=x.device)
    aff = torch.empty((T, E), dtype=torch.float32, device=x.device)
    idx = torch.empty((T, top_k), dtype=torch.int32, device=x.device)
    router_topk(normed, router_weights.to(torch.bfloat16), router_bias, logits, aff, idx, router_act_fn, top_k, 1, 0,
                router_pre_norm=router_pre_norm, norm_topk_prob=norm_topk_prob, use_indirect_dma_scatter=True)
    out = moe_tkg(normed, expert_gate_up_weights, expert_down_weights, aff, idx, is_all_expert, rank_id=rank_id,
                  expert_gate_up_bias=expert_gate_up_bias, expert_down_bias=expert_down_bias,
                  expert_gate_up_weights_scale=expert_gate_up_weights_scale,
                  expert_down_weights_scale=expert_down_weights_scale, mask_unselected_experts=router_pre_norm,
                  expert_affinities_scaling_mode=expert_affinities_scaling_mode, activation_fn=hidden_act_fn,
                  gate_clamp_upper_limit=gate_clamp_upper_limit, gate_clamp_lower_limit=gate_clamp_lower_limit,
                  up_clamp_upper_limit=up_clamp_upper_limit, up_clamp_lower_limit=up_clamp_lower_limit,
                  _prequantized=prequantized)
    outputs = [out]
    if not skip_router_logits:
        outputs.append(logits)
    if residual_out is not None:
        outputs.append(residual_out)
    return tuple(outputs)
