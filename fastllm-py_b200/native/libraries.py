"""The list of CUDA libraries the engine can ask for: (source name, defines)."""
from .ops import BASE_LIBRARIES, BF16_LIBRARIES

DEFAULT_HEAD_DIMS = (128,)


def all_libraries(head_dims=DEFAULT_HEAD_DIMS) -> list:
    from .attention import libraries as attention_libraries

    libs = [(name, {}) for name in BASE_LIBRARIES + BF16_LIBRARIES]
    for d in head_dims:
        libs += attention_libraries(d)
    return libs


def libraries_for(dtype: str, head_dims=()) -> list:
    """What a model of this activation dtype and these head sizes needs, so that
    a first call can compile it side by side instead of one file after another."""
    from .attention import handles, libraries as attention_libraries
    import torch

    libs = [(name, {}) for name in BASE_LIBRARIES]
    if dtype == "bfloat16":
        libs += [(name, {}) for name in BF16_LIBRARIES]
        for d in sorted(set(head_dims)):
            if handles(torch.bfloat16, d):
                libs += attention_libraries(d)
    return libs
