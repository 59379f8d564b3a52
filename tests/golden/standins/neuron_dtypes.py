"""Stand-in for the ``neuron_dtypes`` package, used only by ``tests/golden/make_golden.py``.

The reference's CPU goldens call ``neuron_dtypes.static_cast`` to pack fp32
values into the x4 MX element types and to unpack them again.  That package is
not vendored by the reference and is not installable offline, so this module
supplies the one function and the three dtype objects the goldens touch:

* the x4 types are numpy structured dtypes with one field (32-bit word for the
  two fp8 types, 16-bit word for fp4) so that ``.view(np.uint32)`` /
  ``.view(np.uint16)``, reshapes, indexing, dict keys and ``==`` behave the way
  the reference code expects of them;
* fp32 -> element conversion is IEEE round-to-nearest-even with saturation to
  the largest finite value, done by ``ml_dtypes`` (``float8_e4m3fn``,
  ``float8_e5m2``, ``float4_e2m1fn``).  This rounding rule is the single
  declared assumption: the reference never states what the real package does.

Byte j (nibble j) of a word holds element j, as the reference's own unpackers
read it (core/utils/mx_torch_common.py:70-131).
"""

import ml_dtypes
import numpy as np

float8_e4m3fn_x4 = np.dtype([("float8_e4m3fn_x4", "<u4")])
float8_e5m2_x4 = np.dtype([("float8_e5m2_x4", "<u4")])
float4_e2m1fn_x4 = np.dtype([("float4_e2m1fn_x4", "<u2")])
bfloat16 = np.dtype(ml_dtypes.bfloat16)
float8_e4m3fn = np.dtype(ml_dtypes.float8_e4m3fn)
float8_e5m2 = np.dtype(ml_dtypes.float8_e5m2)

ROUNDING = "round-to-nearest-even, saturating (ml_dtypes %s)" % ml_dtypes.__version__

_ELEMENT = {
    float8_e4m3fn_x4: (ml_dtypes.float8_e4m3fn, 448.0),
    float8_e5m2_x4: (ml_dtypes.float8_e5m2, 57344.0),
    float4_e2m1fn_x4: (ml_dtypes.float4_e2m1fn, 6.0),
}


def _is_x4(dtype) -> bool:
    try:
        return np.dtype(dtype) in _ELEMENT
    except TypeError:
        return False


def _pack(values: np.ndarray, x4) -> np.ndarray:
    elem, vmax = _ELEMENT[x4]
    v = np.asarray(values, dtype=np.float32)
    assert v.shape[-1] % 4 == 0, "x4 packing needs a last axis that is a multiple of 4"
    codes = np.clip(v, -vmax, vmax).astype(elem).view(np.uint8)
    c = codes.reshape(v.shape[:-1] + (v.shape[-1] // 4, 4))
    if x4 == float4_e2m1fn_x4:
        c = c.astype(np.uint16) & 0xF
        words = (c[..., 0] | (c[..., 1] << 4) | (c[..., 2] << 8) | (c[..., 3] << 12)).astype("<u2")
    else:
        c = c.astype(np.uint32)
        words = (c[..., 0] | (c[..., 1] << 8) | (c[..., 2] << 16) | (c[..., 3] << 24)).astype("<u4")
    return np.ascontiguousarray(words).view(x4)


def _unpack(words: np.ndarray, x4) -> np.ndarray:
    elem, _ = _ELEMENT[x4]
    if x4 == float4_e2m1fn_x4:
        w = np.ascontiguousarray(words).view("<u2").astype(np.uint16)
        c = np.stack([(w >> s) & 0xF for s in (0, 4, 8, 12)], axis=-1).astype(np.uint8)
    else:
        w = np.ascontiguousarray(words).view("<u4").astype(np.uint32)
        c = np.stack([(w >> s) & 0xFF for s in (0, 8, 16, 24)], axis=-1).astype(np.uint8)
    vals = c.view(elem).astype(np.float32)
    return vals.reshape(words.shape[:-1] + (words.shape[-1] * 4,))


def static_cast(array, dtype):
    """Value-preserving cast; to or from an x4 type the last axis shrinks / grows by four."""
    a = np.asarray(array)
    if _is_x4(dtype):
        return _pack(a.astype(np.float32), np.dtype(dtype))
    if a.dtype in _ELEMENT:
        return _unpack(a, a.dtype).astype(dtype)
    return a.astype(dtype)


class _FInfo:
    def __init__(self, dtype):
        self.dtype = np.dtype(dtype)


def finfo(dtype):
    return _FInfo(dtype)
