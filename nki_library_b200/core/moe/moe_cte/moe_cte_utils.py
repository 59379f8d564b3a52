"""Small types of the prefill kernel's interface (core/moe/moe_cte/moe_cte_utils.py:65-95)."""

import math
from enum import Enum


class SkipMode:
    """``skip_token``: pad id is -1 and ``hidden_states`` has T rows; otherwise the pad id
    is T and ``hidden_states`` carries a zero row T.  ``skip_weight`` (reuse of the previous
    block's weights) is a DMA optimisation with no effect on results."""

    def __init__(self, skip_token: bool = False, skip_weight: bool = False):
        self.skip_token = skip_token
        self.skip_weight = skip_weight


class BlockShardStrategy(Enum):
    HI_LO = 0
    PING_PONG = 1


def get_n_blocks(T: int, top_k: int, E: int, B: int, n_block_per_iter: int = 1) -> int:
    """Static number of blocks for T tokens routed to ``top_k`` of E experts in blocks of B
    (test/integration/nkilib/core/moe/moe_cte/test_moe_cte_common.py:95-98)."""
    N = math.ceil((T * top_k - (E - 1)) / B) + E - 1
    return n_block_per_iter * math.ceil(N / n_block_per_iter)
