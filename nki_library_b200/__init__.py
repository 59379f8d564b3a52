"""B200-native MoE expert hot path behind the nki-library kernel signatures.

Public entry points mirror the reference (paths relative to its root):

=====================  ==========================================================
``router_topk``        core/router_topk/router_topk.py:55
``find_nonzero_indices`` core/subkernels/find_nonzero_indices.py:34
``cumsum``             core/cumsum/cumsum.py:29
``indexed_flatten``    core/subkernels/indexed_flatten.py:28
``moe_cte``            core/moe/moe_cte/moe_cte.py:252
``moe_tkg``            core/moe/moe_tkg/moe_tkg.py:43
``moe_block_tkg``      core/moe_block/moe_block_tkg.py:39
=====================  ==========================================================

All of them run hand-written sm_100a CUDA kernels through the C ABI in
``include/b200moe.h``; there is no CPU implementation in this package.
"""

from .core.cumsum import cumsum  # noqa: F401
from .core.moe.moe_cte import (  # noqa: F401
    BlockShardStrategy,
    MoECTEImplementation,
    MoECTESpec,
    QuantizationConfig,
    ShardOnBlockConfig,
    ShardOnIConfig,
    SkipMode,
    get_n_blocks,
    moe_cte,
    moe_group_tokens,
)
from .core.moe.moe_tkg import moe_tkg  # noqa: F401
from .core.moe_block import moe_block_tkg  # noqa: F401
from .core.router_topk import router_topk  # noqa: F401
from .core.subkernels import find_nonzero_indices, indexed_flatten  # noqa: F401
from .core.utils.common_types import (  # noqa: F401
    ActFnType,
    ExpertAffinityScaleMode,
    QuantizationType,
    RouterActFnType,
)
from .weights import ExpertWeights, prepare_from_nki, prepare_from_rows  # noqa: F401
