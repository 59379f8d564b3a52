from .cumsum import cumsum  # noqa: F401
