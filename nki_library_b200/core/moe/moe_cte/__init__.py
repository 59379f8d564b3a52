from .moe_cte import (  # noqa: F401
    MoECTEImplementation,
    MoECTESpec,
    QuantizationConfig,
    ShardOnBlockConfig,
    ShardOnIConfig,
    moe_cte,
)
from .moe_cte_utils import BlockShardStrategy, SkipMode, get_n_blocks  # noqa: F401
from .group_tokens import moe_group_tokens  # noqa: F401
