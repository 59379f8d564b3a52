from .moe_tkg import moe_tkg  # noqa: F401
