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

Weights may be e4m3 (default), e5m2 or e2m1 (MXFP4: two elements per byte, so
every contraction axis above is half as many bytes); activations are always
quantised to e4m3, as the reference's ``quantize_mx`` does
(core/utils/mx_torch_common.py:31-133 for the three element types).
"""

from __future__ import annotations

import threading
import weakref
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
    w_format: int = 0      # element format of w1 / w2: _lib.W_E4M3, W_E5M2 or W_E2M1 (nibbles)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w1, self.w1_sf, self.w2, self.w2_sf))


def _as_u8(t: torch.Tensor) -> torch.Tensor:
    t = t.contiguous()
    return t if t.dtype == torch.uint8 else t.view(torch.uint8)


def _format_of(w_format, tensor, bytes_8bit) -> int:
    """Resolve a weight format from an explicit name/code, else from the tensor's dtype and size."""
    names = {"e4m3": _lib.W_E4M3, "e5m2": _lib.W_E5M2, "e2m1": _lib.W_E2M1, "mxfp8": _lib.W_E4M3, "mxfp4": _lib.W_E2M1}
    if w_format is not None:
        code = names.get(w_format, w_format) if isinstance(w_format, str) else int(w_format)
        _lib.kernel_assert(code in (_lib.W_E4M3, _lib.W_E5M2, _lib.W_E2M1), f"unknown weight format {w_format!r}")
        return code
    nbytes = tensor.numel() * tensor.element_size()
    if nbytes * 2 == bytes_8bit:
        return _lib.W_E2M1
    return _lib.W_E5M2 if tensor.dtype == torch.float8_e5m2 else _lib.W_E4M3


def _prepare(w1, s1, w2, s2, bias_gu, bias_d, layout, E, H, I, w_format=_lib.W_E4M3) -> ExpertWeights:
    _lib.require_cuda(w1, s1, w2, s2, bias_gu, bias_d)
    dev = w1.device
    lib = _lib.load_library()
    st = _lib.stream_ptr()
    per = 2 if w_format == _lib.W_E2M1 else 1  # elements per byte
    _lib.kernel_assert(per == 1 or (H % 128 == 0 and I % 128 == 0), "e2m1 weights need H and I to be multiples of 128")
    _lib.kernel_assert(w1.numel() * w1.element_size() * per == E * 2 * I * H and
                       w2.numel() * w2.element_size() * per == E * I * H,
                       "weight tensors do not hold E*2*I*H / E*I*H elements of the given format")
    w1_dev = torch.empty((E, 2 * I, H // per), dtype=torch.uint8, device=dev)
    w1_sf = torch.empty(E * lib.b200moe_sf_bytes(2 * I, H), dtype=torch.uint8, device=dev)
    w2_dev = torch.empty((E, H, I // per), dtype=torch.uint8, device=dev)
    w2_sf = torch.empty(E * lib.b200moe_sf_bytes(H, I), dtype=torch.uint8, device=dev)
    w1u, s1u, w2u, s2u = _as_u8(w1), _as_u8(s1), _as_u8(w2), _as_u8(s2)
    _lib.call("b200moe_prepare_gate_up", _lib.ptr(w1u), _lib.ptr(s1u), layout, w_format, E, H, I, _lib.ptr(w1_dev),
              _lib.ptr(w1_sf), st)
    _lib.call("b200moe_prepare_down", _lib.ptr(w2u), _lib.ptr(s2u), layout, w_format, E, H, I, _lib.ptr(w2_dev),
              _lib.ptr(w2_sf), st)
    b_gu = None
    if bias_gu is not None:
        src = bias_gu.contiguous()
        if src.dtype not in (torch.float32, torch.bfloat16):
            src = src.float()
        b_gu = torch.empty((E, 2 * I), dtype=torch.float32, device=dev)
        _lib.call("b200moe_prepare_gate_up_bias", _lib.ptr(src), _lib.dtype_code(src), layout, E, I, _lib.ptr(b_gu), st)
    b_d = None if bias_d is None else bias_d.reshape(E, H).float().contiguous()
    return ExpertWeights(E, H, I, w1_dev, w1_sf, w2_dev, w2_sf, b_gu, b_d, layout == _lib.LAYOUT_NKI_X4, w_format)


def prepare_from_rows(w1_codes, w1_scales, w2_codes, w2_scales, bias_gu=None, bias_d=None,
                      w_format=None) -> ExpertWeights:
    """``w1_codes [E, 2, I, H]``, ``w1_scales [E, 2, I, H/32]``, ``w2_codes [E, H, I]``, ``w2_scales [E, H, I/32]``;
    with ``w_format="e2m1"`` the code tensors are ``[E, 2, I, H/2]`` and ``[E, H, I/2]`` bytes."""
    E, two, I, _ = w1_scales.shape
    H = w2_scales.shape[1]
    fmt = _format_of(w_format, w1_codes, E * 2 * I * H)
    per = 2 if fmt == _lib.W_E2M1 else 1
    _lib.kernel_assert(two == 2 and tuple(w1_codes.shape) == (E, 2, I, H // per) and
                       tuple(w2_codes.shape) == (E, H, I // per), "gate_up must be [E,2,I,H] and down [E,H,I]")
    _lib.kernel_assert(tuple(w1_scales.shape) == (E, 2, I, H // 32) and tuple(w2_scales.shape) == (E, H, I // 32),
                       "scales must hold one byte per 32 contraction elements")
    return _prepare(w1_codes, w1_scales, w2_codes, w2_scales, bias_gu, bias_d, _lib.LAYOUT_ROWS, E, H, I, fmt)


def prepare_from_nki(gate_up_proj_weight, gate_up_proj_scale, down_proj_weight, down_proj_scale,
                     gate_and_up_proj_bias=None, down_proj_bias=None, w_format=None) -> ExpertWeights:
    """Reference storage -> feed format.  Shapes are taken from the scale tensors; the element format from
    ``w_format`` or, when None, from the weight tensor (half the fp8 byte count = e2m1, ``torch.float8_e5m2`` =
    e5m2, anything else e4m3)."""
    _lib.kernel_assert(gate_up_proj_scale is not None and down_proj_scale is not None,
                       "MX weights need gate_up_proj_scale and down_proj_scale")
    E, sixteen, two, nt, I = gate_up_proj_scale.shape
    _lib.kernel_assert(sixteen == 16 and two == 2, "gate_up_proj_scale must be [E, 16, 2, H/512, I]")
    H = nt * 512
    pI = 128 if I > 512 else I // 4
    n_tiles = I // 512 if I > 512 else 1
    _lib.kernel_assert(tuple(down_proj_scale.shape) == (E, pI // 8, n_tiles, H),
                       f"down_proj_scale must be {(E, pI // 8, n_tiles, H)}, got {tuple(down_proj_scale.shape)}")
    fmt = _format_of(w_format, gate_up_proj_weight, E * 2 * I * H)
    per = 2 if fmt == _lib.W_E2M1 else 1
    _lib.kernel_assert(gate_up_proj_weight.numel() * gate_up_proj_weight.element_size() * per == E * 2 * I * H,
                       "gate_up_proj_weight must hold E*2*I*H x4-packed elements")
    _lib.kernel_assert(down_proj_weight.numel() * down_proj_weight.element_size() * per == E * I * H,
                       "down_proj_weight must hold E*I*H x4-packed elements")
    return _prepare(gate_up_proj_weight, gate_up_proj_scale, down_proj_weight, down_proj_scale,
                    gate_and_up_proj_bias, down_proj_bias, _lib.LAYOUT_NKI_X4, E, H, I, fmt)


_cache: dict = {}  # key -> (weak references to the source tensors, prepared weights)
_cache_lock = threading.RLock()  # re-entrant: a weak-reference callback may fire while the lock is held


def _evict(key) -> None:
    with _cache_lock:
        _cache.pop(key, None)


def prepare_from_nki_cached(gate_up_proj_weight, gate_up_proj_scale, down_proj_weight, down_proj_scale,
                            gate_and_up_proj_bias=None, down_proj_bias=None, w_format=None) -> ExpertWeights:
    """Memoised on the identity and version of the source tensors (weights are static during inference).

    An entry lives exactly as long as its source tensors: each is held by a weak reference whose callback drops
    the entry, so a freed allocation that is handed out again can never be mistaken for the old weights, and a
    model with any number of layers keeps one prepared copy per layer (no size limit, no thrashing)."""
    srcs = (gate_up_proj_weight, gate_up_proj_scale, down_proj_weight, down_proj_scale, gate_and_up_proj_bias,
            down_proj_bias)
    key = tuple((id(t), t.data_ptr(), tuple(t.shape), t._version) if t is not None else None for t in srcs) + (w_format,)
    with _cache_lock:
        hit = _cache.get(key)
    if hit is not None and all(r is None or r() is s for r, s in zip(hit[0], srcs)):
        return hit[1]
    prepared = prepare_from_nki(*srcs, w_format=w_format)
    refs = tuple(None if t is None else weakref.ref(t, lambda _r, k=key: _evict(k)) for t in srcs)
    with _cache_lock:
        _cache[key] = (refs, prepared)
    return prepared


# ---------------------------------------------------------------------------------------------------
# Dense (non-MX) expert weights: bf16, or fp8 with one dequantisation factor per output row ("fp8-row").
# ---------------------------------------------------------------------------------------------------
@dataclass
class DenseExpertWeights:
    """bf16 weights in the tensor-core feed layout of the dense contractions."""
    E: int
    H: int
    I: int
    w1: torch.Tensor                  # bf16 [E, 2I, H], gate/up rows interleaved per 32 like the MX layout
    w2: torch.Tensor                  # bf16 [E, H, I]
    scale_gu: Optional[torch.Tensor]  # fp32 [E, 2I] (interleaved order) or None
    scale_d: Optional[torch.Tensor]   # fp32 [E, H] or None
    bias_gu: Optional[torch.Tensor]   # fp32 [E, 2I] (interleaved order)
    bias_d: Optional[torch.Tensor]    # fp32 [E, H]
    h_packed_order: bool = False

    def nbytes(self) -> int:
        return (self.w1.numel() + self.w2.numel()) * 2


def _interleave_gate_up(t: torch.Tensor) -> torch.Tensor:
    """``[E, 2, I, ...]`` -> ``[E, 2I, ...]`` with rows ordered 32 gate, the matching 32 up, 32 gate, ..."""
    E, two, I = t.shape[:3]
    rest = t.shape[3:]
    return t.reshape(E, 2, I // 32, 32, *rest).transpose(1, 2).reshape(E, 2 * I, *rest).contiguous()


def prepare_dense(gate_up_proj_weight, down_proj_weight, gate_and_up_proj_bias=None, down_proj_bias=None,
                  gate_up_proj_scale=None, down_proj_scale=None) -> DenseExpertWeights:
    """Reference storage of the non-MX variants -> feed layout (once per model load).

    ``gate_up_proj_weight [E, H, 2, I]`` and ``down_proj_weight [E, I, H]`` in bf16 / fp16 / fp32 or an fp8 dtype;
    biases ``[E, 2, I]`` / ``[E, H]``; fp8-row factors ``gate_up_proj_scale [E or 1, 1, 2I]`` (or ``[E, 2, I]``, the
    decode kernels' form) and ``down_proj_scale [E or 1, 1, H]`` (or ``[E, H]``)
    (core/moe/moe_cte/moe_cte_torch.py:163-206, core/moe/moe_tkg/moe_tkg_torch.py:226-290)."""
    _lib.require_cuda(gate_up_proj_weight, down_proj_weight, gate_and_up_proj_bias, down_proj_bias, gate_up_proj_scale,
                      down_proj_scale)
    E, H, two, I = gate_up_proj_weight.shape
    _lib.kernel_assert(two == 2 and I % 32 == 0 and H % 32 == 0,
                       "gate_up_proj_weight must be [E, H, 2, I] with H and I multiples of 32")
    _lib.kernel_assert(tuple(down_proj_weight.shape[:1]) == (E,) and down_proj_weight.shape[-1] == H and
                       down_proj_weight.shape[1] >= I, "down_proj_weight must be [E, I, H]")
    w1 = _interleave_gate_up(gate_up_proj_weight.to(torch.bfloat16).permute(0, 2, 3, 1))      # [E, 2, I, H] -> rows
    w2 = down_proj_weight[:, :I, :].to(torch.bfloat16).transpose(1, 2).contiguous()            # [E, H, I]
    scale_gu = scale_d = None
    if gate_up_proj_scale is not None and gate_up_proj_scale.numel() > 0:
        s = gate_up_proj_scale.float().reshape(-1, 2, I)
        scale_gu = _interleave_gate_up(s.expand(E, 2, I))
        scale_d = down_proj_scale.float().reshape(-1, H).expand(E, H).contiguous()
    bias_gu = None if gate_and_up_proj_bias is None else _interleave_gate_up(gate_and_up_proj_bias.float().reshape(E, 2, I))
    bias_d = None if down_proj_bias is None else down_proj_bias.float().reshape(E, H).contiguous()
    return DenseExpertWeights(E, H, I, w1, w2, scale_gu, scale_d, bias_gu, bias_d)


_dense_cache: dict = {}


def prepare_dense_cached(*srcs) -> DenseExpertWeights:
    """``prepare_dense`` memoised on the identity and version of the source tensors (entries die with them)."""
    key = tuple((id(t), t.data_ptr(), tuple(t.shape), t._version) if t is not None else None for t in srcs)
    with _cache_lock:
        hit = _dense_cache.get(key)
    if hit is not None and all(r is None or r() is s for r, s in zip(hit[0], srcs)):
        return hit[1]
    prepared = prepare_dense(*srcs)

    def drop(_r, k=key):
        with _cache_lock:
            _dense_cache.pop(k, None)

    refs = tuple(None if t is None else weakref.ref(t, drop) for t in srcs)
    with _cache_lock:
        _dense_cache[key] = (refs, prepared)
    return prepared
