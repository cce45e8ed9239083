"""The list of CUDA libraries the engine can ask for: (source name, defines)."""
from .ops import BASE_LIBRARIES, BF16_LIBRARIES


def all_libraries() -> list:
    return [(name, {}) for name in BASE_LIBRARIES + BF16_LIBRARIES]


def libraries_for(dtype: str) -> list:
    """What a model of this activation dtype needs, so that a first call can
    compile it side by side instead of one file after another."""
    names = BASE_LIBRARIES + (BF16_LIBRARIES if dtype == "bfloat16" else [])
    return [(name, {}) for name in names]
