"""The compiled side of the engine: build + ctypes loading + launch wrappers."""
import os

from . import build, ops  # noqa: F401


_HAVE_TC = (build.CSRC / "gemm_tcgen05.cu").exists()


def tensor_core_gemm_enabled() -> bool:
    """The tcgen05 kernel serves bfloat16 products unless FASTLLM_B200_GEMM=simt
    asks for the CUDA-core kernel (a debugging aid: it isolates a wrong result)."""
    return _HAVE_TC and os.environ.get("FASTLLM_B200_GEMM", "tcgen05") != "simt"


def __getattr__(name):
    if name == "gemm_tc":
        from . import gemm_tc
        return gemm_tc
    raise AttributeError(name)
