"""``moe_cte``: blockwise MXFP8 expert MLP for prefill, with the reference's signature
(core/moe/moe_cte/moe_cte.py:252-277) and spec types (:35-249)."""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Any, Optional

import torch

from .... import _lib, pipeline
from ....weights import DenseExpertWeights, ExpertWeights, prepare_dense_cached, prepare_from_nki_cached
from ...utils.common_types import ActFnType, ExpertAffinityScaleMode
from ...utils.kernel_call import kernel_entry
from .moe_cte_utils import BlockShardStrategy, SkipMode


class MoECTEImplementation(Enum):
    shard_on_block = 0
    shard_on_i = 1
    shard_on_i_hybrid = 2
    shard_on_i_dropping = 3
    shard_on_block_mx = 4
    shard_on_i_mx = 5
    shard_on_i_mx_hybrid = 6


_MX_IMPLEMENTATIONS = (MoECTEImplementation.shard_on_block_mx, MoECTEImplementation.shard_on_i_mx,
                       MoECTEImplementation.shard_on_i_mx_hybrid)


@dataclass
class QuantizationConfig:
    gate_up_proj_scale: Optional[Any] = None
    down_proj_scale: Optional[Any] = None


@dataclass
class ShardOnBlockConfig:
    n_block_per_iter: int = 1
    block_sharding_strategy: BlockShardStrategy = BlockShardStrategy.PING_PONG
    n_static_blocks: int = -1
    n_dynamic_blocks: int = 55


@dataclass
class ShardOnIConfig:
    num_static_block: Optional[int] = None
    n_block_per_iter: int = 1
    is_hybrid: bool = False
    checkpoint_activation: bool = False
    expert_affinity_multiply_on_I: bool = False


@dataclass
class MoECTESpec:
    implementation: MoECTEImplementation
    shard_on_block: Optional[ShardOnBlockConfig] = None
    shard_on_I: Optional[ShardOnIConfig] = None

    def __post_init__(self):
        if self.implementation in (MoECTEImplementation.shard_on_block, MoECTEImplementation.shard_on_block_mx):
            if self.shard_on_block is None:
                self.shard_on_block = ShardOnBlockConfig()
        elif self.shard_on_I is None:
            self.shard_on_I = ShardOnIConfig()


@kernel_entry
def moe_cte(
    hidden_states: torch.Tensor,
    expert_affinities_masked: torch.Tensor,
    gate_up_proj_weight,
    down_proj_weight,
    token_position_to_id: torch.Tensor,
    block_to_expert: torch.Tensor,
    block_size: int,
    spec: MoECTESpec,
    conditions: Optional[torch.Tensor] = None,
    gate_and_up_proj_bias: Optional[torch.Tensor] = None,
    down_proj_bias: Optional[torch.Tensor] = None,
    quantization_config: Optional[QuantizationConfig] = None,
    gate_up_activations_T: Optional[torch.Tensor] = None,
    down_activations: Optional[torch.Tensor] = None,
    activation_function: ActFnType = ActFnType.SiLU,
    skip_dma: SkipMode = SkipMode(False, False),
    compute_dtype: Any = torch.bfloat16,
    is_tensor_update_accumulating: bool = True,
    expert_affinities_scaling_mode: ExpertAffinityScaleMode = ExpertAffinityScaleMode.POST_SCALE,
    gate_clamp_upper_limit: Optional[float] = None,
    gate_clamp_lower_limit: Optional[float] = None,
    up_clamp_upper_limit: Optional[float] = None,
    up_clamp_lower_limit: Optional[float] = None,
    compat_lnc_slabs: bool = False,
    _impl: int = 0,
    _check_status: bool = False,
):
    """Prefill MoE expert layer over pre-grouped token blocks.

    Arguments follow the reference.  ``hidden_states`` is bf16 ``[T, H]``
    (``skip_dma.skip_token``) or ``[T + 1, H]`` with a zero row T;
    ``expert_affinities_masked`` is the flat ``[rows * E, 1]`` table;
    ``gate_up_proj_weight`` / ``down_proj_weight`` are the reference's x4-packed
    MXFP8 tensors with their scales in ``quantization_config`` -- or
    ``gate_up_proj_weight`` may be an already prepared
    :class:`~nki_library_b200.weights.ExpertWeights` (then ``down_proj_weight``
    is ignored).  Blocks run while ``conditions[b] != 0``.  Returns bf16
    ``[rows, H]``; with ``compat_lnc_slabs`` the reference's ``[2, rows, H]``
    (slab 1 zero, bwmm_shard_on_block_mx.py:309-313,495-514).

    The MX implementations (``shard_on_block_mx``, ``shard_on_i_mx``, ``shard_on_i_mx_hybrid``) all map to the
    block-scaled kernels.  The non-MX implementations (``shard_on_block``, ``shard_on_i``, ``shard_on_i_hybrid``,
    ``shard_on_i_dropping``: bf16 weights ``[E, H, 2, I]`` / ``[E, I, H]``, or fp8 weights with per-row factors in
    ``quantization_config``) map to the dense bf16 kernels, which also take ``PRE_SCALE`` (hidden rows multiplied
    by the affinity before the first projection; CPU definition core/moe/moe_cte/moe_cte_torch.py:26-242).  The
    sum over a token's blocks is always taken in fp32 and rounded once, whatever
    ``is_tensor_update_accumulating`` says (with it off the reference lets the last block win, which is the same
    thing whenever a token sits in one block only); ``compute_dtype`` other than bf16 is rejected.
    """
    _lib.kernel_assert(isinstance(spec, MoECTESpec), "spec must be a MoECTESpec")
    _lib.kernel_assert(compute_dtype in (torch.bfloat16, None), "compute_dtype must be bfloat16")
    _lib.kernel_assert(gate_up_activations_T is None and down_activations is None,
                       "activation checkpoint outputs (training) are not supported")
    _lib.kernel_assert(block_size % 128 == 0, f"block_size ({block_size}) must be a multiple of 128")
    _lib.require_cuda(hidden_states, expert_affinities_masked, token_position_to_id, block_to_expert, conditions)
    if spec.implementation not in _MX_IMPLEMENTATIONS or isinstance(gate_up_proj_weight, DenseExpertWeights):
        return _moe_cte_dense(hidden_states, expert_affinities_masked, gate_up_proj_weight, down_proj_weight,
                              token_position_to_id, block_to_expert, block_size, spec, conditions,
                              gate_and_up_proj_bias, down_proj_bias, quantization_config, activation_function, skip_dma,
                              expert_affinities_scaling_mode, (gate_clamp_lower_limit, gate_clamp_upper_limit),
                              (up_clamp_lower_limit, up_clamp_upper_limit), compat_lnc_slabs, _impl, _check_status)
    _lib.kernel_assert(expert_affinities_scaling_mode in (ExpertAffinityScaleMode.POST_SCALE,
                                                          ExpertAffinityScaleMode.NO_SCALE),
                       "only POST_SCALE and NO_SCALE affinity scaling are supported by the MX variants")

    if isinstance(gate_up_proj_weight, ExpertWeights):
        weights = gate_up_proj_weight
    else:
        _lib.kernel_assert(quantization_config is not None, "MX weights need quantization_config with both scales")
        weights = prepare_from_nki_cached(gate_up_proj_weight, quantization_config.gate_up_proj_scale, down_proj_weight,
                                          quantization_config.down_proj_scale, gate_and_up_proj_bias, down_proj_bias)
    E, H = weights.E, weights.H
    _lib.kernel_assert(512 <= H <= 8192 and H % 512 == 0 or not weights.h_packed_order,
                       f"H ({H}) must be a multiple of 512 in [512, 8192]")
    rows = hidden_states.shape[0]
    hidden_rows = rows if skip_dma.skip_token else rows - 1
    N = block_to_expert.numel()
    b2e = block_to_expert.reshape(-1).to(torch.int32).contiguous()
    tpi = token_position_to_id.reshape(-1).to(torch.int32).contiguous()
    if conditions is not None:
        conditions = conditions.reshape(-1).to(torch.int32).contiguous()
        _lib.kernel_assert(conditions.numel() >= N, "conditions must cover every block")
    aff = None
    if expert_affinities_scaling_mode == ExpertAffinityScaleMode.POST_SCALE:
        aff = expert_affinities_masked.reshape(-1).contiguous()
        if aff.dtype not in (torch.float32, torch.bfloat16):
            aff = aff.float()
        _lib.kernel_assert(aff.numel() >= hidden_rows * E, "expert_affinities_masked must hold rows * E values")
    hidden = hidden_states.contiguous()
    out = torch.empty((rows, H), dtype=torch.bfloat16, device=hidden.device)
    table = torch.empty((rows, E), dtype=torch.int32, device=hidden.device)
    _lib.call("b200moe_build_position_table", _lib.ptr(tpi), _lib.ptr(b2e), _lib.ptr(conditions), N, block_size,
              hidden_rows, E, _lib.ptr(table), _lib.stream_ptr())
    if rows != hidden_rows:
        table[hidden_rows:].fill_(-1)
    pipeline.run_blocks(hidden, hidden_rows, weights, tpi, b2e, conditions, block_size, aff, table, out,
                        activation_function.value, (gate_clamp_lower_limit, gate_clamp_upper_limit),
                        (up_clamp_lower_limit, up_clamp_upper_limit), _impl, _check_status)
    if compat_lnc_slabs:
        return torch.stack([out, torch.zeros_like(out)])
    return out


def _moe_cte_dense(hidden_states, expert_affinities_masked, gate_up_proj_weight, down_proj_weight, token_position_to_id,
                   block_to_expert, block_size, spec, conditions, gate_and_up_proj_bias, down_proj_bias,
                   quantization_config, activation_function, skip_dma, scaling_mode, gate_clamp, up_clamp,
                   compat_lnc_slabs, impl, check_status):
    """The non-MX implementations: bf16 (or fp8-row) weights through the dense contractions."""
    if isinstance(gate_up_proj_weight, DenseExpertWeights):
        weights = gate_up_proj_weight
    else:
        q = quantization_config or QuantizationConfig()
        weights = prepare_dense_cached(gate_up_proj_weight, down_proj_weight, gate_and_up_proj_bias, down_proj_bias,
                                       q.gate_up_proj_scale, q.down_proj_scale)
    E, H = weights.E, weights.H
    rows = hidden_states.shape[0]
    hidden_rows = rows if skip_dma.skip_token else rows - 1
    N = block_to_expert.numel()
    b2e = block_to_expert.reshape(-1).to(torch.int32).contiguous()
    tpi = token_position_to_id.reshape(-1).to(torch.int32).contiguous()
    # only the hybrid implementation reads ``conditions``; the others run every block
    if spec.implementation == MoECTEImplementation.shard_on_i_hybrid and conditions is not None:
        conditions = conditions.reshape(-1).to(torch.int32).contiguous()
        _lib.kernel_assert(conditions.numel() >= N, "conditions must cover every block")
    else:
        conditions = None
    aff = None
    pre_scale = scaling_mode in (ExpertAffinityScaleMode.PRE_SCALE, ExpertAffinityScaleMode.PRE_SCALE_DELAYED)
    if scaling_mode != ExpertAffinityScaleMode.NO_SCALE:
        aff = expert_affinities_masked.reshape(-1).contiguous()
        if aff.dtype not in (torch.float32, torch.bfloat16):
            aff = aff.float()
        _lib.kernel_assert(aff.numel() >= hidden_rows * E, "expert_affinities_masked must hold rows * E values")
    hidden = hidden_states.to(torch.bfloat16).contiguous()
    out = torch.empty((rows, H), dtype=torch.bfloat16, device=hidden.device)
    table = torch.empty((rows, E), dtype=torch.int32, device=hidden.device)
    _lib.call("b200moe_build_position_table", _lib.ptr(tpi), _lib.ptr(b2e), _lib.ptr(conditions), N, block_size,
              hidden_rows, E, _lib.ptr(table), _lib.stream_ptr())
    if rows != hidden_rows:
        table[hidden_rows:].fill_(-1)
    pipeline.run_blocks_dense(hidden, hidden_rows, weights, tpi, b2e, conditions, block_size, aff, table, out,
                              activation_function.value, gate_clamp, up_clamp, impl, check_status, pre_scale)
    if compat_lnc_slabs:
        return torch.stack([out, torch.zeros_like(out)])
    return out
