"""Enums shared by the MoE hot-path kernels.

Same names and values as the reference's ``core/utils/common_types.py:32-62``
so call sites can switch imports without touching arguments.
"""

from enum import Enum


class ActFnType(Enum):
    SiLU = 0
    GELU = 1
    GELU_Tanh_Approx = 2
    Swish = 3


class RouterActFnType(Enum):
    SIGMOID = 0
    SOFTMAX = 1

    def __str__(self):
        return self.name.lower()


class ExpertAffinityScaleMode(Enum):
    NO_SCALE = 0
    POST_SCALE = 1
    PRE_SCALE = 2
    PRE_SCALE_DELAYED = 3


class QuantizationType(Enum):
    NONE = 0
    STATIC = 1
    ROW = 2
    MX = 3
    STATIC_MX = 4
    ROW_MX = 5
