"""ModelPlan: a model written down as data.

An architecture's `make_plan(config, tensor_names)` returns one of these.  It
names, for every layer, which mixer, feed-forward, norms and position encoding
it has (kind + sizes + constants + the checkpoint names of its tensors), and in
which order the layers run.  The runtime (`parts.decoder.Decoder`) builds the
parts from the registries in `parts.registry` and never looks at the
architecture again.

fastllm-py derives the same information on the fly inside its one forward
function from the config and from which tensor names exist
(fastllm_py/model.py:399-470); a plan is that decision taken once, up front.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class PartSpec:
    """One part: `kind` selects the class, `params` are its sizes and constants
    (a nested PartSpec is allowed, e.g. a mixer's position encoding), `tensors`
    maps the part's own slot names to tensor names in the checkpoint."""
    kind: str
    params: dict = field(default_factory=dict)
    tensors: dict = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A layer = an arrangement (`block`) of a mixer, a feed-forward and norms."""
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: dict            # role in the block -> PartSpec


@dataclass(frozen=True)
class LayerRun:
    """One entry of the running order.

    `layer` indexes ModelPlan.layers; a layer may be named in several runs.
    `cache` names the cache (or state) this run uses: by default a cache of its
    own; the number of an earlier run to read that run's cache instead, in which
    case this run writes nothing to it."""
    layer: int
    cache: int | None = None


@dataclass
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: list
    order: list
    final_norm: PartSpec
    head: PartSpec
    ignorable: tuple = ()      # fnmatch patterns of checkpoint names that may be present and are not used

    def validate(self):
        n = len(self.layers)
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < n:
                raise ValueError(f"order[{i}] names layer {run.layer}, plan has {n} layers")
            if run.cache is not None:
                if not 0 <= run.cache < i:
                    raise ValueError(f"order[{i}] reads the cache of run {run.cache}, "
                                     f"which is not an earlier run")
                if self.order[run.cache].cache is not None:
                    raise ValueError(f"order[{i}] reads the cache of run {run.cache}, "
                                     f"which has no cache of its own")

    def tensor_names(self):
        """Every checkpoint tensor name the plan uses (a shared name once)."""
        names = []
        seen = set()

        def visit(spec):
            for name in spec.tensors.values():
                if name not in seen:
                    seen.add(name)
                    names.append(name)
            for v in spec.params.values():
                if isinstance(v, PartSpec):
                    visit(v)

        visit(self.embedding)
        for layer in self.layers:
            visit(layer.mixer)
            visit(layer.feed_forward)
            for spec in layer.norms.values():
                visit(spec)
        visit(self.final_norm)
        visit(self.head)
        return names
