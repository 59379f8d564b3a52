"""``indexed_flatten`` with the reference's signature (core/subkernels/indexed_flatten.py:28-35)."""

from __future__ import annotations

import torch

from ... import _lib
from ..utils.kernel_call import kernel_entry


@kernel_entry
def indexed_flatten(input_tensor: torch.Tensor, f_len: int, output_len: int, row_offsets: torch.Tensor,
                    row_offsets_start=None, padding_val: int = -1):
    """Write row e of ``input_tensor [E, T]`` in chunks of ``f_len`` at block offsets ``row_offsets[start + e] + p``.

    Returns the flat int32 array of ``output_len`` elements, ``padding_val``
    where nothing was written; where rows overlap the highest row wins and
    chunks outside the output are dropped.  ``T`` must be a multiple of
    ``f_len`` (the reference reshapes rows into chunks); its other shape
    limits (``output_len % 128``, ``(T / f_len) % 16``) do not apply.
    """
    _lib.require_cuda(input_tensor, row_offsets, row_offsets_start)
    _lib.kernel_assert(input_tensor.dim() == 2, "input_tensor must be [E, T]")
    E, T = input_tensor.shape
    _lib.kernel_assert(f_len > 0 and T % f_len == 0, f"T ({T}) must be a multiple of f_len ({f_len})")
    inp = input_tensor.to(torch.int32).contiguous()
    offs = row_offsets.reshape(-1).to(torch.int32).contiguous()
    start = None if row_offsets_start is None else row_offsets_start.reshape(-1).to(torch.int32)
    out = torch.empty((output_len,), dtype=torch.int32, device=inp.device)
    _lib.call("b200moe_indexed_flatten", _lib.ptr(inp), E, T, f_len, output_len, _lib.ptr(offs), offs.numel(),
              _lib.ptr(start), int(padding_val), _lib.ptr(out), _lib.stream_ptr())
    return out
