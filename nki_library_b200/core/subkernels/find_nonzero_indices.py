"""``find_nonzero_indices`` with the reference's signature (core/subkernels/find_nonzero_indices.py:34-40)."""

from __future__ import annotations

import torch

from ... import _lib
from ..utils.kernel_call import kernel_entry


@kernel_entry
def find_nonzero_indices(input_tensor: torch.Tensor, col_start_id=None, n_cols=None, chunk_size=None,
                         index_dtype=torch.int32):
    """Per column of ``input_tensor [T, C]``: ascending row ids of non-zeros (-1 padded) and their count.

    Returns ``(indices [C_out, T] int32, nonzero_counts [C_out] int32)``.
    ``col_start_id`` (device int32 ``[1]``) with ``n_cols`` selects a column
    window for expert parallelism; ``chunk_size`` is a Trainium tiling hint and
    is ignored.  None of the reference's shape limits (even C, T multiple of
    the chunk) apply.
    """
    _lib.require_cuda(input_tensor, col_start_id)
    _lib.kernel_assert(input_tensor.dim() == 2, "input_tensor must be [T, C]")
    _lib.kernel_assert(index_dtype == torch.int32, "index_dtype must be int32")
    T, C = input_tensor.shape
    if col_start_id is not None:
        _lib.kernel_assert(n_cols is not None, "n_cols is required with col_start_id")
        col_start_id = col_start_id.reshape(-1).to(torch.int32)
        c_out = int(n_cols)
    else:
        c_out = C if n_cols is None else int(n_cols)
    inp = input_tensor.contiguous()
    if inp.dtype not in (torch.float32, torch.bfloat16, torch.int32):
        inp = inp.to(torch.float32)
    dev = inp.device
    indices = torch.empty((c_out, T), dtype=torch.int32, device=dev)
    counts = torch.empty((c_out,), dtype=torch.int32, device=dev)
    lib = _lib.load_library()
    ws = torch.empty(lib.b200moe_find_nonzero_workspace_bytes(T, c_out), dtype=torch.uint8, device=dev)
    _lib.call("b200moe_find_nonzero_indices", _lib.ptr(inp), _lib.dtype_code(inp), T, C, _lib.ptr(col_start_id), c_out,
              _lib.ptr(indices), _lib.ptr(counts), _lib.ptr(ws), ws.numel(), _lib.stream_ptr())
    return indices, counts
