"""``router_topk`` with the reference's signature (core/router_topk/router_topk.py:55-75)."""

from __future__ import annotations

import torch

from ... import _lib
from ..utils.common_types import RouterActFnType
from ..utils.kernel_call import kernel_entry


@kernel_entry
def router_topk(
    x: torch.Tensor,
    w: torch.Tensor,
    w_bias,
    router_logits: torch.Tensor,
    expert_affinities: torch.Tensor,
    expert_index: torch.Tensor,
    act_fn: RouterActFnType,
    k: int,
    x_hbm_layout: int,
    x_sb_layout: int,
    router_pre_norm: bool = True,
    norm_topk_prob: bool = False,
    use_column_tiling: bool = False,
    use_indirect_dma_scatter: bool = False,
    return_eager_affi: bool = False,
    use_PE_broadcast_w_bias: bool = False,
    shard_on_tokens: bool = False,
    skip_store_expert_index: bool = False,
    skip_store_router_logits: bool = False,
    _path: int = 0,
):
    """Router logits, top-K expert ids and affinities, written into the caller's tensors.

    ``x`` is bf16 ``[T, H]`` (``x_hbm_layout == 1``) or ``[H, T]`` (0); ``w`` bf16
    ``[H, E]``; ``w_bias`` ``[1, E]``/``[E]`` or None.  The three outputs are
    caller-allocated (``router_logits [T, E]``, ``expert_index [T, k]`` uint32 or
    int32, ``expert_affinities [T, E]``; fp32 or bf16) and returned as
    ``[router_logits, expert_index, expert_affinities]``
    (router_topk.py:1129-1188).  Flags that only steer Trainium engines
    (``x_sb_layout``, ``use_column_tiling``, ``use_indirect_dma_scatter``,
    ``use_PE_broadcast_w_bias``, ``shard_on_tokens``) are accepted and checked
    for the same illegal combinations, then ignored.  ``_path`` (no reference
    counterpart) forces the logits kernel: 0 by shape, 1 split-K, 2 tcgen05.
    """
    _lib.require_cuda(x, w, w_bias, router_logits, expert_affinities, expert_index)
    _lib.kernel_assert(x.dim() == 2 and w.dim() == 2, "x and w must be 2-D")
    x_is_TH = 1 if x_hbm_layout == 1 else 0
    T, H = (x.shape[0], x.shape[1]) if x_is_TH else (x.shape[1], x.shape[0])
    E = w.shape[1]
    _lib.kernel_assert(w.shape[0] == H, f"w rows ({w.shape[0]}) must equal H ({H})")
    _lib.kernel_assert(x.dtype == w.dtype, f"x dtype ({x.dtype}) must match w dtype ({w.dtype})")
    _lib.kernel_assert(x.dtype == torch.bfloat16, "x and w must be bfloat16")
    _lib.kernel_assert(E <= 512, f"E ({E}) must be <= gemm_moving_fmax (512)")
    _lib.kernel_assert(k >= 1, f"K ({k}) must be >= 1")
    _lib.kernel_assert(k <= 8, f"K ({k}) must be <= 8")
    _lib.kernel_assert(H % 128 == 0, f"H ({H}) must be a multiple of pmax (128)")
    _lib.kernel_assert(
        not (act_fn == RouterActFnType.SIGMOID and not use_indirect_dma_scatter and not router_pre_norm),
        "SIGMOID activation with router_pre_norm=False requires use_indirect_dma_scatter=True")
    _lib.kernel_assert(not skip_store_router_logits, "skip_store_router_logits=True is not currently supported")
    _lib.kernel_assert(not (norm_topk_prob and not router_pre_norm), "norm_topk_prob requires router_pre_norm")
    if w_bias is not None:
        w_bias = w_bias.reshape(1, E).to(torch.bfloat16).contiguous()
    x = x.contiguous()
    w = w.contiguous()
    for out, shape in ((router_logits, (T, E)), (expert_affinities, (T, E)), (expert_index, (T, k))):
        _lib.kernel_assert(out is not None and tuple(out.shape) == shape and out.is_contiguous(),
                           f"output tensor must be contiguous with shape {shape}")
    _lib.kernel_assert(expert_index.dtype in (torch.int32, torch.uint32), "expert_index must be a 32-bit integer tensor")
    ws = torch.empty(_lib.load_library().b200moe_router_workspace_bytes(T, H, E), dtype=torch.uint8, device=x.device)
    _lib.call(
        "b200moe_router_topk", _lib.ptr(x), x_is_TH, _lib.ptr(w), _lib.ptr(w_bias), T, H, E, k, act_fn.value,
        int(router_pre_norm), int(norm_topk_prob), _lib.ptr(router_logits), _lib.dtype_code(router_logits),
        None if skip_store_expert_index else _lib.ptr(expert_index), _lib.ptr(expert_affinities),
        _lib.dtype_code(expert_affinities), int(_path), _lib.ptr(ws), ws.numel(), _lib.stream_ptr())
    outs = [router_logits, expert_index, expert_affinities]
    if return_eager_affi:
        idx = expert_index.to(torch.int64)
        outs.append(expert_affinities.gather(1, idx))
    return outs
