"""Fused token-to-block grouping (find_nonzero_indices + cumsum + indexed_flatten in one call)."""

from __future__ import annotations

from typing import Optional

import torch

from .... import _lib
from .moe_cte_utils import get_n_blocks


def moe_group_tokens(routing: torch.Tensor, num_experts: int, block_size: int, n_blocks: Optional[int] = None,
                     top_k: Optional[int] = None, skip_token: bool = True, mx_conditions: bool = True,
                     want_inverse: bool = True, check: bool = False):
    """Block assignment for the blockwise expert kernels.

    ``routing`` is either ``expert_index [T, K]`` (int32/uint32) or a ``[T, E]``
    mask / masked-affinity tensor (fp32, bf16 or int32; non-zero = routed).
    Returns a dict with ``token_position_to_id [N*B]``, ``block_to_expert [N]``,
    ``conditions``, ``counts [E]`` and, for index routing, ``inverse_map [T, K]``
    -- the same arrays the reference builds with find_nonzero_indices, cumsum and
    indexed_flatten (core/subkernels/find_nonzero_indices.py:34,
    core/subkernels/indexed_flatten.py:28) plus the block bookkeeping of
    test/integration/nkilib/core/moe/moe_cte/test_moe_cte_common.py:199-264.
    """
    _lib.require_cuda(routing)
    T = routing.shape[0]
    index_mode = routing.dtype in (torch.int32, torch.uint32, torch.int64) and routing.shape[1] != num_experts
    if routing.dtype == torch.int64:
        routing = routing.to(torch.int32)
    if top_k is not None and routing.shape[1] == top_k and routing.dtype in (torch.int32, torch.uint32):
        index_mode = True
    E, B = num_experts, block_size
    if index_mode:
        K = routing.shape[1]
    else:
        _lib.kernel_assert(routing.shape[1] == E, "mask routing must be [T, E]")
        K = top_k if top_k is not None else 0
        if routing.dtype not in (torch.float32, torch.bfloat16, torch.int32):
            routing = routing.float()
    routing = routing.contiguous()
    if n_blocks is None:
        _lib.kernel_assert(K > 0, "top_k is needed to size the block list for mask routing")
        n_blocks = get_n_blocks(T, K, E, B)
    N = n_blocks
    dev = routing.device
    lib = _lib.load_library()
    tpi = torch.empty(N * B, dtype=torch.int32, device=dev)
    b2e = torch.empty(N, dtype=torch.int32, device=dev)
    cond = torch.empty(N + 2 if mx_conditions else N + 1, dtype=torch.int32, device=dev)
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    inv = torch.empty((T, K), dtype=torch.int32, device=dev) if (index_mode and want_inverse) else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ws = torch.empty(lib.b200moe_group_tokens_workspace_bytes(T, E), dtype=torch.uint8, device=dev)
    _lib.call("b200moe_group_tokens", _lib.ptr(routing), _lib.ROUTING_INDEX if index_mode else _lib.ROUTING_MASK,
              _lib.I32 if index_mode else _lib.dtype_code(routing), T, E, K if index_mode else 0, B, N,
              int(skip_token), int(mx_conditions), _lib.ptr(tpi), _lib.ptr(b2e), _lib.ptr(cond), _lib.ptr(counts),
              _lib.ptr(inv), _lib.ptr(status), _lib.ptr(ws), ws.numel(), _lib.stream_ptr())
    if check:
        _lib.kernel_assert(int(status.item()) == 0, f"n_blocks ({N}) is too small for this routing")
    return {"token_position_to_id": tpi, "block_to_expert": b2e, "conditions": cond, "counts": counts,
            "inverse_map": inv, "status": status, "n_blocks": N}
