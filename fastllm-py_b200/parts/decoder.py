"""Decoder: a ModelPlan turned into parts, and the pass of one step through them.

The pass is the order list of the plan: embed the step's tokens into the
residual stream, run each entry's block against its cache, norm the rows whose
logits are wanted and project them to the vocabulary.  It is
fastllm_py/model.py:437-477 with three differences: it runs a flat batch of
tokens from many requests, it reads and writes the cache through the step's
tables, and it computes logits only at the wanted rows.
"""
from __future__ import annotations

import torch

from .base import BuildContext, ResidualStream
from .plan import ModelPlan
from .registry import build_part, part_class


class Decoder:
    def __init__(self, plan: ModelPlan, ctx: BuildContext):
        plan.validate()
        self.plan = plan
        self.ctx = ctx
        self.hidden = plan.hidden_size
        self.vocab = plan.vocab_size
        self.embedding = build_part("embedding", plan.embedding, ctx)
        self.blocks = [part_class("block", layer.block)(layer, ctx) for layer in plan.layers]
        self.final_norm = build_part("norm", plan.final_norm, ctx)
        self.head = build_part("head", plan.head, ctx)
        self.order = list(plan.order)
        for i, run in enumerate(self.order):
            need = self.blocks[run.layer].mixer.cache_need()
            if run.cache is not None and need is not None:
                raise ValueError(f"order[{i}] reads run {run.cache}'s cache but its layer's mixer "
                                 f"wants a cache of its own")
            if run.cache is None and need is None and \
                    getattr(self.blocks[run.layer].mixer, "shares_cache", False):
                raise ValueError(f"order[{i}]: the layer shares a cache but the run names none")

    # ------------------------------------------------------------------ parts
    def all_parts(self):
        """Every part, nested ones included, each once."""
        out, seen = [], set()

        def visit(p):
            if id(p) in seen:
                return
            seen.add(id(p))
            out.append(p)
            for c in p.children():
                visit(c)

        visit(self.embedding)
        for b in self.blocks:
            visit(b)
        visit(self.final_norm)
        visit(self.head)
        return out

    def expected_tensors(self) -> dict:
        """checkpoint name -> shape, over all parts (a name shared by two parts once)."""
        table = {}
        for part in self.all_parts():
            spec = part.spec
            tensors = getattr(spec, "tensors", None)
            if tensors is None:
                continue
            shapes = part.weight_shapes()
            missing = set(shapes) - set(tensors)
            if missing:
                raise ValueError(f"{type(part).__name__}: the plan names no tensor for {sorted(missing)}")
            for slot, shape in shapes.items():
                name = tensors[slot]
                if name in table and tuple(table[name]) != tuple(shape):
                    raise ValueError(f"tensor {name} is wanted as {table[name]} and as {shape}")
                table[name] = tuple(shape)
        return table

    def load(self, tensors_by_name: dict) -> None:
        """Hands every part its tensors.  A part is told beforehand (`shared_slots`) which of its
        slots hold a tensor that another part holds too (a tied embedding table): it must leave
        such a tensor as it is."""
        users: dict = {}
        for part in self.all_parts():
            tensors = getattr(part.spec, "tensors", None)
            if tensors is not None:
                for slot in part.weight_shapes():
                    users[tensors[slot]] = users.get(tensors[slot], 0) + 1
        for part in self.all_parts():
            tensors = getattr(part.spec, "tensors", None)
            if tensors is None:
                continue
            shapes = part.weight_shapes()
            part.shared_slots = frozenset(slot for slot in shapes if users[tensors[slot]] > 1)
            part.load({slot: tensors_by_name[tensors[slot]] for slot in shapes})

    def cache_needs(self) -> dict:
        """run index -> need, for the runs that own a cache or a state."""
        needs = {}
        for i, run in enumerate(self.order):
            if run.cache is None:
                need = self.blocks[run.layer].mixer.cache_need()
                if need is not None:
                    needs[i] = need
        return needs

    @property
    def graph_safe(self) -> bool:
        """False when some part says that its forward decides things on the host from the
        step's host copies (attribute `graph_safe = False`): its steps are never captured."""
        safe = getattr(self, "_graph_safe", None)
        if safe is None:                                    # (the parts are fixed once the decoder is built)
            safe = self._graph_safe = all(getattr(p, "graph_safe", True) for p in self.all_parts())
        return safe

    def _mixers_with(self, hook: str) -> list:
        """The mixers that have `hook`, one per `plan_key` (mixers of equal keys decide alike)."""
        cache = self.__dict__.setdefault("_hooked", {})
        if hook not in cache:
            found, seen = [], set()
            for block in self.blocks:
                mixer = block.mixer
                if not hasattr(mixer, hook):
                    continue
                key = getattr(mixer, "plan_key", None) or id(mixer)
                if key not in seen:
                    seen.add(key)
                    found.append(mixer)
            cache[hook] = found
        return cache[hook]

    def plan_step(self, step) -> None:
        """Before a step is launched: every mixer that decides something on the host for it
        (how to split the keys of a decode kernel, say) does so now and keeps it in `step.plans`."""
        for mixer in self._mixers_with("plan_step"):
            mixer.plan_step(step)

    def graph_key(self, step):
        """What, beside the number of tokens, fixes the launch shapes of a
        decode-only step: each mixer may add its own (a bucket of the longest
        sequence, say).  Steps with equal keys may replay one captured graph."""
        return tuple(mixer.graph_key(step) for mixer in self._mixers_with("graph_key"))

    @property
    def takes_fed_tokens(self) -> bool:
        """True when the embedding part can take a token from the sampler's output on the device."""
        return bool(getattr(self.embedding, "takes_fed_tokens", False))

    def reserve(self, limits, workspace) -> None:
        """Called once when an engine is built: every part sizes its scratch memory, and the
        buffers whose size follows the requests rather than the tokens get their steady size."""
        for part in self.all_parts():
            fn = getattr(part, "reserve", None)
            if fn is not None:
                fn(limits)
        rows = min(limits.max_tokens, limits.max_requests)
        workspace.rows("logits", rows, self.vocab, torch.float32, initial=rows)
        workspace.rows("picked", rows, self.hidden, self.ctx.dtype, initial=rows)

    # ------------------------------------------------------------------- pass
    def forward(self, step) -> torch.Tensor:
        """Logits [wanted rows, vocab] in float32 for the step's tokens."""
        n = step.n_tokens
        ws = step.workspace
        stream = ResidualStream(ws.rows("residual", n, self.hidden, torch.float32),
                                spill=lambda: ws.rows("delta", n, self.hidden, self.ctx.dtype))
        self.embedding.forward(step, stream.x)
        for i, run in enumerate(self.order):
            cache_id = i if run.cache is None else run.cache
            self.blocks[run.layer].forward(stream, step, step.cache_view(cache_id, run.cache is None))
        m = step.n_wanted
        logits = ws.rows("logits", m, self.vocab, torch.float32, initial=64)
        if m > 0:
            picked = ws.rows("picked", m, self.hidden, self.ctx.dtype, initial=64)
            rows = None if step.rows_identity else step.logit_rows
            stream.norm_into(self.final_norm, picked, rows=rows)
            self.head.forward(picked, logits)
        return logits
