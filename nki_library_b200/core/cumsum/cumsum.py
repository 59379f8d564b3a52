"""``cumsum`` with the reference's signature (core/cumsum/cumsum.py:29-75)."""

from __future__ import annotations

import torch

from ... import _lib
from ..utils.kernel_call import kernel_entry


@kernel_entry
def cumsum(x: torch.Tensor, axis: int = -1):
    """Inclusive cumulative sum along the last axis, accumulated in fp32."""
    _lib.require_cuda(x)
    _lib.kernel_assert(axis in (-1, x.dim() - 1), "cumsum is only implemented along the last axis")
    xin = x.contiguous()
    if xin.dtype not in (torch.float32, torch.bfloat16, torch.int32):
        xin = xin.to(torch.float32)
    cols = xin.shape[-1]
    rows = xin.numel() // cols
    out = torch.empty_like(xin)
    _lib.call("b200moe_cumsum", _lib.ptr(xin), _lib.dtype_code(xin), rows, cols, _lib.ptr(out), _lib.stream_ptr())
    return out if out.dtype == x.dtype else out.to(x.dtype)
