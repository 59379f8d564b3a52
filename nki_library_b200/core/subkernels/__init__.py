from .find_nonzero_indices import find_nonzero_indices  # noqa: F401
from .indexed_flatten import indexed_flatten  # noqa: F401
