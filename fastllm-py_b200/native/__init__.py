"""The compiled side of the engine: build + ctypes loading + launch wrappers."""
from . import build, ops, scratch  # noqa: F401
from . import gemm_tc  # noqa: F401
