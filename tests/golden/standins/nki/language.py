"""Stand-in for ``nki.language``: the dtype names the reference's CPU goldens refer to."""

import numpy as np

from neuron_dtypes import (bfloat16, float4_e2m1fn_x4, float8_e4m3fn, float8_e4m3fn_x4, float8_e5m2,  # noqa: F401
                           float8_e5m2_x4)

float32 = np.dtype(np.float32)
float16 = np.dtype(np.float16)
int32 = np.dtype(np.int32)
uint32 = np.dtype(np.uint32)
uint16 = np.dtype(np.uint16)
uint8 = np.dtype(np.uint8)
int8 = np.dtype(np.int8)


class NKIObject:
    """Base class of the reference's small configuration records (no behaviour is needed on the CPU)."""
