"""Model: the Python entry point, in fastllm-py's manner.

    model = Model.load("path/to/model", dtype="bfloat16")
    new_ids = model.generate(prompt_ids, max_new_tokens=32, temperature=0.7, seed=1)

`Model.load` and `Model.generate` keep the names and meanings of
fastllm_py/model.py:150-153 and :500-504 where they apply to one GPU and
unquantised weights: `dtype`, `max_new_tokens`, `temperature`, `use_graph`,
`stop_ids`, `top_p`, `top_k`, `seed`, `min_p`, `repetition_penalty`,
`frequency_penalty`, `presence_penalty`; generate returns only the new ids and
includes the stop id.  Options of the reference that select what this engine
does not have (device maps over several GPUs, INT4/FP8 quantisation, MoE expert
placement) do not exist here.  New: a list of prompts generates as one batch
through the scheduler, and `Model.from_config` makes a model with seeded random
weights.
"""
from __future__ import annotations

import torch

from . import architectures  # noqa: F401  (registers the architectures)
from .config import EngineConfig, canonical_dtype, load_config
from .config.registry import architecture_of
from .engine import Engine, Scheduler
from .parts import BuildContext, Decoder
from .sampling import Sampler, SamplingParams
from .weights import RandomStore, SafetensorsStore, load_tensors


def _require_gpu(device: str) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError(
            "no CUDA device: this engine runs on an NVIDIA B200 (sm_100a) only; there is no CPU path")
    dev = torch.device(device)
    major, minor = torch.cuda.get_device_capability(dev)
    if major != 10:
        raise RuntimeError(f"device {dev} has compute capability {major}.{minor}; the kernels are "
                           f"built for sm_100a only")
    return dev


class Model:
    def __init__(self, config, plan, decoder: Decoder, engine_config: EngineConfig):
        self.cfg = config
        self.plan = plan
        self.decoder = decoder
        self.engine_config = engine_config
        self.engine = None
        self.sampler = None

    # --------------------------------------------------------------- loading
    @classmethod
    def _build(cls, arch, config, store, engine_config: EngineConfig, where: str):
        dev = _require_gpu(engine_config.device)
        torch.cuda.set_device(dev)
        dtype = getattr(torch, engine_config.dtype)
        names = None if isinstance(store, _RandomSpec) else set(store.names())
        plan = arch.make_plan(config, names)
        max_len = engine_config.max_model_len or plan.max_positions
        ctx = BuildContext(dev, dtype, engine_config.page_size, max_len)
        decoder = Decoder(plan, ctx)
        from .native import build as native_build
        from .native.libraries import libraries_for
        head_dims = [p.head_dim for p in decoder.all_parts() if hasattr(p, "head_dim")]
        native_build.compile_many(libraries_for(engine_config.dtype, head_dims))
        expected = decoder.expected_tensors()
        if isinstance(store, _RandomSpec):
            store = RandomStore(expected, store.seed, store.std, store.norm_std,
                                getattr(torch, canonical_dtype(store.dtype)), on_device=store.on_device)
        decoder.load(load_tensors(expected, store, dev, where, plan.ignorable))
        model = cls(config, plan, decoder, engine_config)
        model._make_engine(max_len)
        return model

    @classmethod
    def load(cls, model_path, dtype: str = "bfloat16", **engine_options) -> "Model":
        """Load config.json and the safetensors of a model folder onto the GPU."""
        engine_config = EngineConfig(dtype=dtype, **engine_options)
        arch, config = load_config(model_path)
        store = SafetensorsStore(model_path)
        try:
            return cls._build(arch, config, store, engine_config, str(model_path))
        finally:
            store.close()

    @classmethod
    def from_config(cls, config, seed: int = 0, std: float = 0.02, norm_std: float = 0.02,
                    weight_dtype: str = "bfloat16", dtype: str = "bfloat16", on_device: bool = True,
                    **engine_options) -> "Model":
        """A model of the given typed configuration with seeded random weights
        made on the device (nothing is written to disk)."""
        engine_config = EngineConfig(dtype=dtype, **engine_options)
        arch = architecture_of(config.to_hf())
        spec = _RandomSpec(seed, std, norm_std, weight_dtype, on_device)
        return cls._build(arch, config, spec, engine_config, "random weights")

    def _make_engine(self, max_len: int):
        ec = self.engine_config
        needs = self.decoder.cache_needs()
        from .cache import CacheManager
        itemsize = 2 if ec.dtype == "bfloat16" else 4
        if ec.max_tokens is not None:
            num_pages = max(1, -(-ec.max_tokens // ec.page_size))
        else:
            per_token = CacheManager.bytes_per_token(needs, ec.page_size, itemsize)
            free, _ = torch.cuda.mem_get_info(self.decoder.ctx.device)
            reserve = 2 << 30                                   # activations, logits, graphs
            budget = max(0, int(free * ec.memory_fraction) - reserve)
            num_pages = max(1, budget // max(1, per_token * ec.page_size)) if per_token else 1
            num_pages = min(num_pages, -(-max_len // ec.page_size) * ec.max_requests)
        self.engine = Engine(self.decoder, ec, max_len, num_pages)
        self.sampler = Sampler(self.decoder.ctx.device, ec.max_requests)

    # ------------------------------------------------------------ generation
    def scheduler(self, token_budget: int | None = None, run_ahead: bool = True) -> Scheduler:
        """`run_ahead`: launch a decode step before the host has read the tokens of the one
        before it (they are taken from the sampler's output on the device); same tokens out."""
        return Scheduler(self.engine, self.sampler, token_budget, run_ahead)

    def generate(self, token_ids, max_new_tokens: int = 32, temperature: float = 0.0,
                 use_graph: bool = True, stop_ids=None, top_p: float = 1.0, top_k: int = 0,
                 seed=None, min_p: float = 0.0, repetition_penalty: float = 1.0,
                 frequency_penalty: float = 0.0, presence_penalty: float = 0.0):
        """New token ids for one prompt (a list of ints) or for several (a list of lists).

        With several prompts request i samples with seed + i when a seed is given."""
        many = len(token_ids) > 0 and isinstance(token_ids[0], (list, tuple)) or \
            (hasattr(token_ids, "ndim") and getattr(token_ids, "ndim") == 2)
        prompts = [list(map(int, p)) for p in token_ids] if many else [list(map(int, token_ids))]
        self.engine.use_graph = bool(use_graph) and self.engine_config.cuda_graph
        sched = self.scheduler()
        ids = []
        for i, p in enumerate(prompts):
            params = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p,
                                    repetition_penalty=repetition_penalty,
                                    frequency_penalty=frequency_penalty,
                                    presence_penalty=presence_penalty,
                                    seed=None if seed is None else seed + i)
            ids.append(sched.add_request(p, max_new_tokens, params, stop_ids or ()))
        out = sched.run()
        return [out[i] for i in ids] if many else out[ids[0]]


class _RandomSpec:
    def __init__(self, seed, std, norm_std, dtype, on_device):
        self.seed, self.std, self.norm_std, self.dtype, self.on_device = \
            seed, std, norm_std, dtype, on_device

    def names(self):
        return None
