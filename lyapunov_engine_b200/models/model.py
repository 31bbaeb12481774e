"""A model built from a description: embedding, the layers in their run order,
final norm, output head; what its cache must hold; and its forward pass over
one step's tokens.

The reference's counterpart is LlamaForCausalLM
(python/lyapunov_engine/models/llama.py:168-225), which is one fixed stack.
"""
from __future__ import annotations

from dataclasses import dataclass

from .. import ops
from ..parts.base import (BLOCKS, EMBEDDINGS, HEADS, NORMS, KVNeed, ModelSpec, ResidualStream, StateNeed,
                          TensorDecl)


@dataclass(frozen=True)
class CacheGroupPlan:
    """Runs whose pages have the same geometry and life share a group: one page
    pool's ids and one block table per request."""
    num_kv_heads: int
    head_dim: int
    window: int | None


@dataclass(frozen=True)
class RunPlan:
    layer: int
    group: int | None        # cache group of its pages (None: the mixer keeps no pages)
    stream: int | None       # which K/V pool pair of the group it uses
    writes: bool             # False when it reads the pages another run writes
    state: int | None        # index of its state buffer (None: no state)


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = EMBEDDINGS.build(spec.embedding)
        self.blocks = [BLOCKS.build(layer.block) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.head = HEADS.build(spec.head)
        self.groups: list[CacheGroupPlan] = []
        self.streams_per_group: list[int] = []
        self.states: list[StateNeed] = []
        self.runs: list[RunPlan] = []
        self._plan_cache()
        # query-tile sizes that the mixers' kernels want listed in every step's integers
        self.tile_sizes: list[int] = sorted({int(t) for b in self.blocks for t in b.mixer.tile_sizes()})
        self._decode_variants: dict[tuple, tuple] = {}

    # ---- what the cache must hold
    def _plan_cache(self) -> None:
        for index, run in enumerate(self.spec.run_order):
            if not 0 <= run.layer < len(self.blocks):
                raise ValueError(f"run order entry {index} names layer {run.layer}; there are {len(self.blocks)}")
            mixer = self.blocks[run.layer].mixer
            need: KVNeed | None = mixer.cache_need()
            state: StateNeed | None = mixer.state_need()
            group = stream = None
            writes = True
            if need is not None:
                if run.reads_cache_of is not None:
                    src = run.reads_cache_of
                    if not 0 <= src < index:
                        raise ValueError(f"run order entry {index} reads the cache of entry {src}, which does not run before it")
                    other = self.runs[src]
                    g = self.groups[other.group] if other.group is not None else None
                    if g is None or (g.num_kv_heads, g.head_dim) != (need.num_kv_heads, need.head_dim):
                        raise ValueError(f"run order entry {index} cannot read the cache of entry {src}: different geometry")
                    group, stream, writes = other.group, other.stream, False
                else:
                    plan = CacheGroupPlan(need.num_kv_heads, need.head_dim, need.window)
                    if plan not in self.groups:
                        self.groups.append(plan)
                        self.streams_per_group.append(0)
                    group = self.groups.index(plan)
                    stream = self.streams_per_group[group]
                    self.streams_per_group[group] += 1
            elif run.reads_cache_of is not None:
                raise ValueError(f"run order entry {index} reads a cache but its mixer keeps no pages")
            state_index = None
            if state is not None:
                state_index = len(self.states)
                self.states.append(state)
            self.runs.append(RunPlan(run.layer, group, stream, writes, state_index))

    # ---- tensors
    def parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def tensors(self) -> list[TensorDecl]:
        seen: dict[str, TensorDecl] = {}
        for part in self.parts():
            for decl in part.tensors():
                if decl.name in seen:
                    if seen[decl.name].shape != decl.shape:
                        raise ValueError(f"tensor {decl.name!r} is declared with shapes {seen[decl.name].shape} and {decl.shape}")
                    continue
                seen[decl.name] = decl
        return list(seen.values())

    def bind(self, get, runtime) -> None:
        self.runtime = runtime
        for part in self.parts():
            part.bind(get, runtime)
        self._decode_variants.clear()

    # ---- one step
    def decode_variant(self, fill: int, num_decode: int, context_bound: int) -> tuple:
        """The mixers' launch choices that depend on how many of a step's
        one-token requests are real (see Mixer.decode_variant)."""
        key = (fill, num_decode, context_bound)
        found = self._decode_variants.get(key)
        if found is None:                      # asked at every step: the mixers answer once per shape
            seen = []
            for b in self.blocks:
                v = b.mixer.decode_variant(fill, num_decode, context_bound)
                if v is not None and v not in seen:
                    seen.append(v)
            found = self._decode_variants[key] = tuple(seen)
        return found

    def forward(self, ctx, cache):
        """Logits [wanted rows, vocab] float32 (None when nothing is wanted).
        ``cache.binding(run_index)`` gives each run its pages and state."""
        for state in cache.states:
            # a request whose first tokens are in this step starts from zero state, whoever held its slot before
            ops.zero_fresh_state(state, ctx.state_slots, ctx.ctx_before, ctx.num_requests)
        resid = self.embedding.forward(ctx)
        stream = ResidualStream(resid)
        for index, run in enumerate(self.runs):
            self.blocks[run.layer].forward(stream, ctx, cache.binding(index))
        if ctx.num_wanted == 0:
            return None
        normed = self.final_norm.apply(stream.resid, stream.pending, rows=ctx.wanted_rows, workspace=ctx.workspace,
                                       key="final_normed")
        return self.head.forward(normed, ctx)
