"""Expert weights in the tensor-core feed format, prepared once per model load.

Two sources are accepted:

* the reference's storage (``gate_up_proj_weight [E, 128, 2, H/512, I]`` x4-packed
  fp8 with ``gate_up_proj_scale [E, 16, 2, H/512, I]``, ``down_proj_weight
  [E, p_I, ceil(I/512), H]`` x4 with ``down_proj_scale [E, p_I/8, ceil(I/512), H]``;
  core/moe/moe_cte/bwmm_shard_on_block_mx.py:70-230).  Its hidden and
  intermediate axes are stored in a packed order; the prepared weights keep
  that order and the activation quantiser gathers hidden columns to match.
* plain rows: fp8 codes ``[E, 2, I, H]`` / ``[E, H, I]`` with one UE8M0 scale per
  32 consecutive contraction elements.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib


@dataclass
class ExpertWeights:
    E: int
    H: int
    I: int
    w1: torch.Tensor       # uint8 [E, 2I, H], gate/up rows interleaved per 32
    w1_sf: torch.Tensor    # uint8 scale atoms
    w2: torch.Tensor       # uint8 [E, H, I]
    w2_sf: torch.Tensor
    bias_gu: Optional[torch.Tensor]  # fp32 [E, 2I] in w1 row order
    bias_d: Optional[torch.Tensor]   # fp32 [E, H]
    h_packed_order: bool   # hidden columns must be gathered in the reference's packed order

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w1, self.w1_sf, self.w2, self.w2_sf))


def _as_u8(t: torch.Tensor) -> torch.Tensor:
    t = t.contiguous()
    return t if t.dtype == torch.uint8 else t.view(torch.uint8)


def _prepare(w1, s1, w2, s2, bias_gu, bias_d, layout, E, H, I) -> ExpertWeights:
    _lib.require_cuda(w1, s1, w2, s2, bias_gu, bias_d)
    dev = w1.device
    lib = _lib.load_library()
    st = _lib.stream_ptr()
    w1_dev = torch.empty((E, 2 * I, H), dtype=torch.uint8, device=dev)
    w1_sf = torch.empty(E * lib.b200moe_sf_bytes(2 * I, H), dtype=torch.uint8, device=dev)
    w2_dev = torch.empty((E, H, I), dtype=torch.uint8, device=dev)
    w2_sf = torch.empty(E * lib.b200moe_sf_bytes(H, I), dtype=torch.uint8, device=dev)
    w1u, s1u, w2u, s2u = _as_u8(w1), _as_u8(s1), _as_u8(w2), _as_u8(s2)
    _lib.call("b200moe_prepare_gate_up", _lib.ptr(w1u), _lib.ptr(s1u), layout, E, H, I, _lib.ptr(w1_dev),
              _lib.ptr(w1_sf), st)
    _lib.call("b200moe_prepare_down", _lib.ptr(w2u), _lib.ptr(s2u), layout, E, H, I, _lib.ptr(w2_dev),
              _lib.ptr(w2_sf), st)
    b_gu = None
    if bias_gu is not None:
        src = bias_gu.contiguous()
        if src.dtype not in (torch.float32, torch.bfloat16):
            src = src.float()
        b_gu = torch.empty((E, 2 * I), dtype=torch.float32, device=dev)
        _lib.call("b200moe_prepare_gate_up_bias", _lib.ptr(src), _lib.dtype_code(src), layout, E, I, _lib.ptr(b_gu), st)
    b_d = None if bias_d is None else bias_d.reshape(E, H).float().contiguous()
    return ExpertWeights(E, H, I, w1_dev, w1_sf, w2_dev, w2_sf, b_gu, b_d, layout == _lib.LAYOUT_NKI_X4)


def prepare_from_rows(w1_codes, w1_scales, w2_codes, w2_scales, bias_gu=None, bias_d=None) -> ExpertWeights:
    """``w1_codes [E, 2, I, H]``, ``w1_scales [E, 2, I, H/32]``, ``w2_codes [E, H, I]``, ``w2_scales [E, H, I/32]``."""
    E, two, I, H = w1_codes.shape
    _lib.kernel_assert(two == 2 and tuple(w2_codes.shape) == (E, H, I), "gate_up must be [E,2,I,H] and down [E,H,I]")
    _lib.kernel_assert(tuple(w1_scales.shape) == (E, 2, I, H // 32) and tuple(w2_scales.shape) == (E, H, I // 32),
                       "scales must hold one byte per 32 contraction elements")
    return _prepare(w1_codes, w1_scales, w2_codes, w2_scales, bias_gu, bias_d, _lib.LAYOUT_ROWS, E, H, I)


def prepare_from_nki(gate_up_proj_weight, gate_up_proj_scale, down_proj_weight, down_proj_scale,
                     gate_and_up_proj_bias=None, down_proj_bias=None) -> ExpertWeights:
    """Reference storage -> feed format.  Shapes are taken from the scale tensors."""
    _lib.kernel_assert(gate_up_proj_scale is not None and down_proj_scale is not None,
                       "MX weights need gate_up_proj_scale and down_proj_scale")
    E, sixteen, two, nt, I = gate_up_proj_scale.shape
    _lib.kernel_assert(sixteen == 16 and two == 2, "gate_up_proj_scale must be [E, 16, 2, H/512, I]")
    H = nt * 512
    pI = 128 if I > 512 else I // 4
    n_tiles = I // 512 if I > 512 else 1
    _lib.kernel_assert(tuple(down_proj_scale.shape) == (E, pI // 8, n_tiles, H),
                       f"down_proj_scale must be {(E, pI // 8, n_tiles, H)}, got {tuple(down_proj_scale.shape)}")
    _lib.kernel_assert(gate_up_proj_weight.numel() * gate_up_proj_weight.element_size() == E * 2 * I * H,
                       "gate_up_proj_weight must hold E*2*I*H fp8 bytes (x4-packed)")
    _lib.kernel_assert(down_proj_weight.numel() * down_proj_weight.element_size() == E * I * H,
                       "down_proj_weight must hold E*I*H fp8 bytes (x4-packed)")
    return _prepare(gate_up_proj_weight, gate_up_proj_scale, down_proj_weight, down_proj_scale,
                    gate_and_up_proj_bias, down_proj_bias, _lib.LAYOUT_NKI_X4, E, H, I)


_cache: dict = {}


def prepare_from_nki_cached(gate_up_proj_weight, gate_up_proj_scale, down_proj_weight, down_proj_scale,
                            gate_and_up_proj_bias=None, down_proj_bias=None) -> ExpertWeights:
    """Memoised on the identity and version of the source tensors (weights are static during inference)."""
    srcs = (gate_up_proj_weight, gate_up_proj_scale, down_proj_weight, down_proj_scale, gate_and_up_proj_bias,
            down_proj_bias)
    key = tuple((t.data_ptr(), tuple(t.shape), t._version) if t is not None else None for t in srcs)
    hit = _cache.get(key)
    if hit is None:
        if len(_cache) > 8:
            _cache.clear()
        hit = prepare_from_nki(*srcs)
        _cache[key] = hit
    return hit
