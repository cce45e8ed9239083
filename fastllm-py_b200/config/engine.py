"""EngineConfig: the options of the engine itself, as opposed to the model's.

fastllm-py passes these as keyword arguments (`Model.load(..., dtype=)`,
fastllm_py/model.py:150-153; `BatchedEngine(model, max_batch, max_len)`,
fastllm_py/batched.py:346).  Here they are one typed object.
"""
from __future__ import annotations

from dataclasses import dataclass

_DTYPES = {"float32": "float32", "fp32": "float32", "bfloat16": "bfloat16", "bf16": "bfloat16"}


def canonical_dtype(name: str) -> str:
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {name!r}") from None


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"           # activations, cache and matrix inputs; "float32" = true 32-bit everywhere
    page_size: int = 16               # tokens per cache page
    max_tokens: int | None = None     # cache pool size in tokens (None: sized from free device memory)
    memory_fraction: float = 0.85     # share of free device memory the pool may take when max_tokens is None
    max_requests: int = 64            # live requests (state slots, block-table rows)
    max_batched_tokens: int = 2048    # token budget of one step
    max_model_len: int | None = None  # longest sequence (None: the model's max_position_embeddings)
    cuda_graph: bool = True           # capture decode-only steps
    check_cache: bool = False         # check mode: pages that go back are overwritten with `cache_poison`
    cache_poison: float = 1.0e4       # ... a value that swamps any softmax or output row it gets into
    status_every: int = 1             # the scheduler reads the kernels' error word every this many steps (0: never)
    device: str = "cuda:0"

    def __post_init__(self):
        self.dtype = canonical_dtype(self.dtype)
        if self.page_size < 1:
            raise ValueError("page_size must be >= 1")
        if self.max_requests < 1:
            raise ValueError("max_requests must be >= 1")
        if self.max_batched_tokens < 1:
            raise ValueError("max_batched_tokens must be >= 1")
