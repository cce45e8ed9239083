"""Sources of tensors by name: a folder of safetensors files, or a seeded random generator.

SafetensorsStore follows fastllm_py/weights.py:19-66: the name -> shard index
comes from model.safetensors.index.json's `weight_map` when present, else from
listing the keys of every *.safetensors file; shards are opened lazily.  Unlike
the reference it converts nothing on the way (weights.py:56-59 upcasts bfloat16
to float32 on the CPU): bfloat16 stays bfloat16, 32-bit stays 32-bit, integer
tables become int32, and float16 (which the kernels do not take) is widened to
float32, which is exact.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

_ST_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16,
              "F64": torch.float64, "I64": torch.int64, "I32": torch.int32, "I16": torch.int16,
              "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}


def kept_dtype(stored: torch.dtype) -> torch.dtype:
    """The dtype a tensor has on the device, given how the checkpoint stores it."""
    if stored in (torch.bfloat16, torch.float32):
        return stored
    if stored in (torch.float16, torch.float64):
        return torch.float32
    if stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return torch.int32
    raise TypeError(f"tensors of dtype {stored} are not supported")


class SafetensorsStore:
    def __init__(self, model_path):
        from safetensors import safe_open

        self._open = safe_open
        self.path = Path(model_path)
        self._index: dict = {}
        self._handles: dict = {}
        index_file = self.path / "model.safetensors.index.json"
        if index_file.exists():
            for name, shard in json.loads(index_file.read_text())["weight_map"].items():
                self._index[name] = self.path / shard
        else:
            for shard in sorted(self.path.glob("*.safetensors")):
                with safe_open(str(shard), framework="pt") as f:
                    for name in f.keys():
                        self._index[name] = shard
        if not self._index:
            raise FileNotFoundError(f"no safetensors found in {self.path}")

    def names(self):
        return self._index.keys()

    def _handle(self, shard):
        if shard not in self._handles:
            self._handles[shard] = self._open(str(shard), framework="pt")
        return self._handles[shard]

    def describe(self, name):
        """(shape, stored dtype) without reading the data."""
        sl = self._handle(self._index[name]).get_slice(name)
        return tuple(sl.get_shape()), _ST_DTYPES.get(sl.get_dtype())

    def get(self, name, device):
        t = self._handle(self._index[name]).get_tensor(name)
        return t.to(device=device, dtype=kept_dtype(t.dtype)).contiguous()

    def close(self):
        self._handles.clear()


class RandomStore:
    """Seeded random tensors for a table of (name -> shape).

    Each tensor has a generator of its own, keyed by (seed, name), so a tensor's
    values do not depend on which others exist or in which order they are made.
    Matrices and tables are N(0, std); vectors (norm weights) are 1 + N(0, norm_std).
    Values are drawn in float32 on the CPU and rounded to `dtype`; `on_device`
    draws on the device instead (other values, for models too large to stage)."""

    def __init__(self, shapes: dict, seed: int, std: float = 0.02, norm_std: float = 0.02,
                 dtype: torch.dtype = torch.bfloat16, on_device: bool = False):
        self.shapes = dict(shapes)
        self.seed = seed
        self.std = std
        self.norm_std = norm_std
        self.dtype = dtype
        self.on_device = on_device

    def names(self):
        return self.shapes.keys()

    def describe(self, name):
        return tuple(self.shapes[name]), self.dtype

    def _seed_for(self, name):
        digest = hashlib.sha256(f"{self.seed}:{name}".encode()).digest()
        return int.from_bytes(digest[:8], "little") & ((1 << 62) - 1)

    def get(self, name, device):
        shape = tuple(self.shapes[name])
        gen_device = device if self.on_device else "cpu"
        gen = torch.Generator(device=gen_device)
        gen.manual_seed(self._seed_for(name))
        if len(shape) == 1:
            t = torch.empty(shape, dtype=torch.float32, device=gen_device).normal_(
                0.0, self.norm_std, generator=gen).add_(1.0)
        elif self.on_device:
            # drawn straight in the target dtype, so no float32 copy of a large matrix is made
            t = torch.empty(shape, dtype=self.dtype, device=gen_device).normal_(
                0.0, self.std, generator=gen)
        else:
            t = torch.empty(shape, dtype=torch.float32, device=gen_device).normal_(
                0.0, self.std, generator=gen)
        return t.to(device=device, dtype=self.dtype).contiguous()
