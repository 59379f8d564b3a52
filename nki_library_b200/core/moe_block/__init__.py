from .moe_block_tkg import moe_block_tkg  # noqa: F401
