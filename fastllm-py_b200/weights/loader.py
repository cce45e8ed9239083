"""Loading a model's tensors by name, with one error for everything that is wrong.

fastllm-py loads whatever names exist and lets a missing tensor surface later as
a KeyError in the forward pass, never checks a shape, and ties the head silently
when `lm_head.weight` is absent (fastllm_py/model.py:214-231).  Here the parts
say which tensors they expect and in which shape; the store is compared with
that table before anything is read, and every mismatch is listed at once.
"""
from __future__ import annotations

import json
import weakref
from collections.abc import Mapping
from pathlib import Path

import torch

from .store import RandomStore, SafetensorsStore, kept_dtype


class WeightError(ValueError):
    """The checkpoint does not fit the model.  Attributes list what is wrong."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype, where=""):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.wrong_dtype = sorted(wrong_dtype)
        lines = [f"the tensors{' in ' + where if where else ''} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, the model wants {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  unsupported dtype: {name} is stored as {got}")
        super().__init__("\n".join(lines))


def check_store(expected: dict, store, where="", ignorable=()) -> None:
    from fnmatch import fnmatchcase

    names = set(store.names())
    missing = set(expected) - names
    unexpected = {n for n in names - set(expected)
                  if not any(fnmatchcase(n, pat) for pat in ignorable)}
    wrong_shape, wrong_dtype = [], []
    for name in sorted(set(expected) & names):
        shape, dtype = store.describe(name)
        if tuple(shape) != tuple(expected[name]):
            wrong_shape.append((name, tuple(expected[name]), tuple(shape)))
        try:
            if dtype is None:
                raise TypeError
            kept_dtype(dtype)
        except TypeError:
            wrong_dtype.append((name, str(dtype)))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype, where)


class _TensorsOnDemand(Mapping):
    """name -> device tensor, fetched from the store when asked for and held only as long as
    somebody else holds it: a part that stacks its matrices into one frees the originals on the
    spot, so loading never needs much more memory than the model itself (a 135 GB model fits a
    180 GB device), and two parts that ask for one tensor (tied embeddings) get the same one."""

    def __init__(self, names, store, device):
        self._names = list(names)
        self._store = store
        self._device = device
        self._alive = weakref.WeakValueDictionary()

    def __getitem__(self, name):
        if name not in self._names:
            raise KeyError(name)
        t = self._alive.get(name)
        if t is None:
            t = self._store.get(name, self._device)
            self._alive[name] = t
        return t

    def __iter__(self):
        return iter(self._names)

    def __len__(self):
        return len(self._names)


def load_tensors(expected: dict, store, device, where="", ignorable=()) -> Mapping:
    """name -> device tensor for every expected name, after the check; tensors are read when
    they are asked for."""
    check_store(expected, store, where, ignorable)
    return _TensorsOnDemand(expected, store, device)


def write_model_folder(config, folder, seed: int, std: float = 0.02, norm_std: float = 0.02,
                       dtype: str = "bfloat16"):
    """Random-weights mode: write config.json and model.safetensors for a
    configuration (of any registered architecture) and a seed."""
    from safetensors.torch import save_file

    from ..config.engine import canonical_dtype
    from ..config.registry import architecture_of
    from ..parts import BuildContext, Decoder

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    raw = config.to_hf()
    arch = architecture_of(raw)
    plan = arch.make_plan(config, None)
    tdtype = getattr(torch, canonical_dtype(dtype))
    decoder = Decoder(plan, BuildContext(torch.device("cpu"), tdtype, 16, 1))
    shapes = decoder.expected_tensors()
    store = RandomStore(shapes, seed, std, norm_std, tdtype)
    tensors = {name: store.get(name, "cpu") for name in shapes}
    (folder / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    save_file(tensors, str(folder / "model.safetensors"))
    return folder
