from .router_topk import router_topk  # noqa: F401
