"""``moe_tkg``: MXFP8 expert MLP for token generation, with the reference's signature
(core/moe/moe_tkg/moe_tkg.py:43-70)."""

from __future__ import annotations

import math
from typing import Optional

import torch

from .... import _lib, pipeline
from ....weights import DenseExpertWeights, ExpertWeights, prepare_dense_cached, prepare_from_nki_cached
from ...utils.common_types import ActFnType, ExpertAffinityScaleMode
from ...utils.kernel_call import kernel_entry
from ..moe_cte.group_tokens import moe_group_tokens
from ..moe_cte.moe_cte_utils import get_n_blocks

_PREFIX = "[MoE TKG Kernel]"
_BLOCK = 128


@kernel_entry
def moe_tkg(
    hidden_input: torch.Tensor,
    expert_gate_up_weights,
    expert_down_weights,
    expert_affinities: torch.Tensor,
    expert_index: torch.Tensor,
    is_all_expert: bool,
    rank_id: Optional[torch.Tensor] = None,
    expert_gate_up_bias: Optional[torch.Tensor] = None,
    expert_down_bias: Optional[torch.Tensor] = None,
    expert_gate_up_weights_scale: Optional[torch.Tensor] = None,
    expert_down_weights_scale: Optional[torch.Tensor] = None,
    hidden_input_scale: Optional[torch.Tensor] = None,
    gate_up_input_scale: Optional[torch.Tensor] = None,
    down_input_scale: Optional[torch.Tensor] = None,
    mask_unselected_experts: bool = False,
    expert_affinities_eager: Optional[torch.Tensor] = None,
    expert_affinities_scaling_mode: ExpertAffinityScaleMode = ExpertAffinityScaleMode.NO_SCALE,
    activation_fn: ActFnType = ActFnType.SiLU,
    output_dtype=None,
    gate_clamp_upper_limit: Optional[float] = None,
    gate_clamp_lower_limit: Optional[float] = None,
    up_clamp_upper_limit: Optional[float] = None,
    up_clamp_lower_limit: Optional[float] = None,
    output_in_sbuf: bool = False,
    is_all_expert_dynamic: bool = False,
    block_size: int = None,
    _impl: int = 0,
    _check_status: bool = False,
    _prequantized=None,
) -> torch.Tensor:
    """Decode MoE expert layer, ``[T, H]`` in, ``[T, H]`` out.

    Selective mode (``is_all_expert=False``) runs each token through its
    ``expert_index[t, :]`` experts; every *active* expert's weights are streamed
    from HBM once, however many tokens picked it.  All-expert mode runs every
    token through the local experts ``[E_L * rank_id, E_L * (rank_id + 1))`` with
    the affinity columns sliced (and optionally masked by ``expert_index``) the
    way ``mask_expert_affinities`` does (core/moe/moe_tkg/moe_tkg_affinity_masking.py:31-117).
    ``is_all_expert_dynamic`` computes, per local expert, only the tokens whose masked affinity is non-zero.
    Weights are the reference's x4-packed MXFP8 tensors with their scales, or a
    prepared :class:`~nki_library_b200.weights.ExpertWeights` passed as
    ``expert_gate_up_weights``.  Non-MX weights -- 4-D ``[E_L, H, 2, I]`` bf16, or fp8 with the per-row factors
    ``[E_L, 2, I]`` / ``[E_L, H]`` in the two scale arguments -- run on the dense bf16 kernels.  SBUF-resident
    tensors, pre-quantised hidden states and static (per-tensor input) quantisation are rejected.
    """
    A = _lib.kernel_assert
    A(not output_in_sbuf, f"{_PREFIX} output_in_sbuf has no meaning on a GPU")
    A(hidden_input_scale is None, f"{_PREFIX} pre-quantised hidden_input (hidden_input_scale) is not supported")
    A(gate_up_input_scale is None and down_input_scale is None,
      f"{_PREFIX} Static quantization is not supported in MoE TKG kernel")
    A(expert_affinities_scaling_mode != ExpertAffinityScaleMode.PRE_SCALE_DELAYED,
      f"{_PREFIX} PRE_SCALE_DELAYED option is only applicable in CTE expert_mlp case")
    A(expert_affinities_scaling_mode != ExpertAffinityScaleMode.PRE_SCALE,
      f"{_PREFIX} Kernel does not support pre-scale mode")
    if is_all_expert_dynamic:
        A(is_all_expert, f"{_PREFIX} is_all_expert_dynamic=True requires is_all_expert=True, but got {is_all_expert=}")
        A(block_size is not None,
          f"{_PREFIX} is_all_expert_dynamic=True requires block_size != None, but got {block_size=}")
    if is_all_expert:
        A(expert_affinities_eager is None,
          f"{_PREFIX} expert_affinities eager mode not supported with is_all_expert=True")
    _lib.require_cuda(hidden_input, expert_affinities, expert_index, rank_id)
    A(hidden_input.dim() == 2, f"{_PREFIX} hidden_input must be [T, H]")
    T, H = hidden_input.shape
    A(T <= 128 or is_all_expert,
      f"{_PREFIX} Currently only batch size * seq len <= 128 is supported (except for all-expert mode)")

    dense = isinstance(expert_gate_up_weights, DenseExpertWeights) or (
        isinstance(expert_gate_up_weights, torch.Tensor) and expert_gate_up_weights.dim() == 4)
    if dense:
        # non-MX weights: bf16 [E_L, H, 2, I] / [E_L, I, H], or fp8 with per-row factors [E_L, 2, I] / [E_L, H]
        # (core/moe/moe_tkg/all_expert_impl.py:65, selective_expert_impl.py:45; CPU definition moe_tkg_torch.py:226-290)
        weights = expert_gate_up_weights if isinstance(expert_gate_up_weights, DenseExpertWeights) else \
            prepare_dense_cached(expert_gate_up_weights, expert_down_weights, expert_gate_up_bias, expert_down_bias,
                                 expert_gate_up_weights_scale, expert_down_weights_scale)
    elif isinstance(expert_gate_up_weights, ExpertWeights):
        weights = expert_gate_up_weights
    else:
        A(expert_gate_up_weights_scale is not None and expert_down_weights_scale is not None,
          f"{_PREFIX} Scales must be set when using MX weights")
        weights = prepare_from_nki_cached(expert_gate_up_weights, expert_gate_up_weights_scale, expert_down_weights,
                                          expert_down_weights_scale, expert_gate_up_bias, expert_down_bias)
    A(weights.H == H, f"{_PREFIX} weight hidden size {weights.H} does not match hidden_input ({H})")
    E_L = weights.E
    post_scale = expert_affinities_scaling_mode == ExpertAffinityScaleMode.POST_SCALE
    hidden = hidden_input.to(torch.bfloat16).contiguous()
    dev = hidden.device
    out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    clamps = ((gate_clamp_lower_limit, gate_clamp_upper_limit), (up_clamp_lower_limit, up_clamp_upper_limit))

    if not is_all_expert:
        idx = expert_index.to(torch.int32).contiguous()
        K = idx.shape[1]
        E = expert_affinities.shape[1]
        A(E == E_L, f"{_PREFIX} selective mode needs all {E} experts local, got {E_L}")
        g = moe_group_tokens(idx, E, _BLOCK, get_n_blocks(T, K, E, _BLOCK), skip_token=True)
        aff = None
        if post_scale:
            aff = expert_affinities.contiguous()
            if aff.dtype not in (torch.float32, torch.bfloat16):
                aff = aff.float()
        _run(weights, hidden, T, weights, g["token_position_to_id"], g["block_to_expert"], g["conditions"],
             _BLOCK, aff, g["inverse_map"], out, activation_fn.value, clamps[0], clamps[1], _impl, _check_status)
    else:
        E = expert_affinities.shape[1]
        if post_scale:
            A(rank_id is not None, f"{_PREFIX} rank_id is required for all-expert mode with affinity scaling")
        # local expert columns [E_L * rank_id, E_L * (rank_id + 1)), taken with a device-side index so that the
        # rank tensor never has to travel to the host (moe_tkg_affinity_masking.py:31-117)
        aff = None
        if post_scale or is_all_expert_dynamic:
            cols = torch.arange(E_L, dtype=torch.int64, device=dev)
            if rank_id is not None:
                cols = cols + rank_id.reshape(-1)[:1].to(torch.int64) * E_L
            aff = expert_affinities.float().index_select(1, cols)
            if mask_unselected_experts:
                sel = torch.zeros((T, E), dtype=torch.float32, device=dev)
                sel.scatter_(1, expert_index.to(torch.int64), 1.0)
                aff = aff * sel.index_select(1, cols)
            aff = aff.contiguous()
        if is_all_expert_dynamic:
            # dynamic control flow: per expert only the tokens routed to it (non-zero masked affinity) are
            # gathered into blocks and computed (all_expert_mx_impl.py:276-350); the block bookkeeping is the
            # prefill grouping on the masked affinities, and the blocks of experts nobody chose never run
            A(block_size > 0 and T % block_size == 0, f"{_PREFIX} block_size must evenly divide T")
            n_blocks = E_L * math.ceil(T / _BLOCK)
            g = moe_group_tokens(aff, E_L, _BLOCK, n_blocks, skip_token=True, want_inverse=False)
            tpi, b2e, cond = g["token_position_to_id"], g["block_to_expert"], g["conditions"]
            table = torch.empty((T, E_L), dtype=torch.int32, device=dev)
            _lib.call("b200moe_build_position_table", _lib.ptr(tpi), _lib.ptr(b2e), _lib.ptr(cond), n_blocks, _BLOCK,
                      T, E_L, _lib.ptr(table), _lib.stream_ptr())
        else:
            tpi, b2e, table = all_expert_layout(T, E_L, dev)
            cond = None
        kw = {}
        if _prequantized is not None and not is_all_expert_dynamic and not dense:
            # the caller (moe_block_tkg) has run the fused RMSNorm + quantise kernel into this workspace
            kw = dict(workspace=_prequantized, prequantized=True)
        _run(weights, hidden, T, weights, tpi, b2e, cond, _BLOCK, aff if post_scale else None, table, out,
             activation_fn.value, clamps[0], clamps[1], _impl, _check_status, **kw)
    if output_dtype is not None and output_dtype != torch.bfloat16:
        return out.to(output_dtype)
    return out


def all_expert_layout(T: int, E_L: int, device):
    """Static block layout of the all-expert mode: every local expert owns ceil(T / 128) blocks that hold tokens
    0..T-1 in order.  Returns ``(token_position_to_id, block_to_expert, table [T, E_L])``."""
    n_sub = math.ceil(T / _BLOCK)
    Tpad = n_sub * _BLOCK
    ids = torch.full((Tpad,), -1, dtype=torch.int32, device=device)
    ids[:T] = torch.arange(T, dtype=torch.int32, device=device)
    tpi = ids.repeat(E_L)
    b2e = torch.arange(E_L, dtype=torch.int32, device=device).repeat_interleave(n_sub)
    table = (torch.arange(E_L, dtype=torch.int32, device=device)[None, :] * Tpad +
             torch.arange(T, dtype=torch.int32, device=device)[:, None]).contiguous()
    return tpi, b2e, table


def _run(weights, *args, **kw):
    """MX weights go through the block-scaled kernels, dense weights through the bf16 ones."""
    if isinstance(weights, DenseExpertWeights):
        return pipeline.run_blocks_dense(*args, **kw)
    return pipeline.run_blocks(*args, **kw)
