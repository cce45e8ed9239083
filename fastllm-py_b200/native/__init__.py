"""The compiled side of the engine: build + ctypes loading + launch wrappers."""
import os

from . import build, ops  # noqa: F401
from . import gemm_tc  # noqa: F401


def tensor_core_gemm_enabled() -> bool:
    """The tcgen05 kernel serves bfloat16 products unless FASTLLM_B200_GEMM=simt
    asks for the CUDA-core kernel (a debugging aid: it isolates a wrong result)."""
    return os.environ.get("FASTLLM_B200_GEMM", "tcgen05") != "simt"
