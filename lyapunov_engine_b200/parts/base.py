"""What a model is made of, and the registries that turn a description into it.

A model is described as data (``ModelSpec``): a list of layers, each naming the
kind and the numbers of its mixer, feed-forward, norms and block arrangement,
and a run order (``RunSpec`` list) that may name a layer twice or let a run
read the cache another run writes.  ``build`` functions look the kinds up in
the registries below; parts get their sizes and constants as arguments and
their tensors by name.  No part knows which model it is in.

Interfaces (all tensors are CUDA tensors; T tokens in the step, H width):

``Norm``
    ``apply(resid, delta=None, rows=None) -> normed``: adds ``delta`` into the
    32-bit residual stream ``resid`` [T, H] when given, returns the normed rows
    in the activations' type.  With ``rows`` it norms those rows only and
    leaves ``resid`` unchanged.
``PositionEncoding``
    ``encode_and_store(qkv, geometry, ctx, kv, write)``: encodes the queries
    (in place) and keys of the fused projection rows and, if ``write``, stores
    keys and values in the paged cache ``kv``.
``Mixer``
    ``cache_need() -> KVNeed | None`` and ``state_need() -> StateNeed | None``
    say what the cache manager must hold for it; ``forward(x, ctx, cache) ->
    y`` mixes the tokens of the step (x, y: [T, H] activations) using
    ``cache.kv`` (pages) and/or ``cache.state`` (one row per state slot).
    State: request b of the step owns row ``ctx.state_slots[b]`` of
    ``cache.state``.  Before the step's first layer the framework zeroes the
    rows of requests whose ``ctx.ctx_before[b]`` is 0 (a new request, or one
    recomputed after pre-emption), so a mixer reads its row unconditionally
    and writes it back.  Rows of a step that stand for no request (padding of a
    fixed-shape batch) carry slot -1: a kernel uses the buffer's last row for
    them, which belongs to nobody, or skips them.  Steps of a model whose
    mixers keep state are never padded with dummy tokens behind a request's
    own.  ``tile_sizes()`` names the query-tile sizes its kernels want listed
    in the step's integers (``ctx.tiles``).
``FeedForward``
    ``forward(x, ctx) -> y``.
``Block``
    ``forward(stream, ctx, cache)``: arranges norms, mixer and feed-forward
    around the residual stream (``stream.resid`` 32-bit plus a ``pending``
    delta not yet added).
Every part also has ``tensors() -> list[TensorDecl]`` (what it reads from the
checkpoint, with shapes, for checking and for random weights) and
``bind(get, runtime)`` (takes its tensors, already on the device).

The reference's modules read a shared config object in their constructors
(python/lyapunov_engine/models/llama.py:35-48,110-117,126-134).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable


# ---------------------------------------------------------------- description
@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: dict = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer and a feed-forward.  All
    sizes, constants and tensor names sit in the parts' params."""
    block: PartSpec


@dataclass(frozen=True)
class RunSpec:
    """One entry of the run order: run ``layer``; ``reads_cache_of`` names an
    earlier entry (by its index in the run order) whose cache this run reads
    instead of writing one of its own."""
    layer: int
    reads_cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    run_order: tuple[RunSpec, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    config_json: dict = field(default_factory=dict, compare=False)


# ---------------------------------------------------------------- tensors
@dataclass(frozen=True)
class TensorDecl:
    """A checkpoint tensor a part reads.  ``role`` decides the type it is kept
    in: "matrix" in the engine's compute type (bfloat16 or float32); "vector"
    (norm weights and the like) always 32-bit, so one stored in 32 bits stays
    exactly so; "int_table" as int32.  ``init`` is how random weights fill it:
    "normal", "ones", "ones_jitter" or "zeros".  ``alias_of`` names the tensor
    that stands in when the checkpoint has none of this name (a tied head)."""
    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    alias_of: str | None = None


@dataclass(frozen=True)
class KVNeed:
    """Keys and values in pages: ``window`` None keeps every key."""
    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one row of ``shape`` per slot."""
    shape: tuple[int, ...]
    dtype: Any = None  # torch dtype; None: float32


class Part:
    def tensors(self) -> list[TensorDecl]:
        return []

    def bind(self, get: Callable[[str], Any], runtime) -> None:
        pass


class Norm(Part):
    def apply(self, resid, delta=None, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    def encode_and_store(self, qkv, geometry, ctx, kv, write: bool) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> KVNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def tile_sizes(self) -> list[int]:
        """Query-tile sizes its kernels want: for each, ``ctx.tiles[size]`` lists
        (request of each tile, first query token of the tile within the
        request, number of tiles, how many of them belong to requests that
        bring several tokens), those of several tokens first."""
        return []

    def decode_variant(self, fill: int, num_decode: int, context_bound: int):
        """What of this mixer's launches depends on how many of a step's
        ``num_decode`` one-token requests are real (``fill``; the others pad
        the step to a fixed shape): any hashable, None if nothing.  Steps of
        fixed shape that are captured once and replayed are kept apart by it;
        ``forward`` finds the same number in ``ctx.decode_fill`` and must make
        the same choice from it."""
        return None

    def forward(self, x, ctx, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, stream, ctx, cache) -> None:
        raise NotImplementedError


class ResidualStream:
    """The 32-bit residual stream of a step and the last sub-layer's output
    that has not been added to it yet (the next norm adds it)."""
    __slots__ = ("resid", "pending")

    def __init__(self, resid, pending=None):
        self.resid = resid
        self.pending = pending


# ---------------------------------------------------------------- registries
class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: dict[str, Callable] = {}

    def register(self, kind: str, factory: Callable | None = None):
        def put(f):
            self._items[kind] = f
            return f
        return put(factory) if factory is not None else put

    def build(self, spec: PartSpec, **extra):
        if spec.kind not in self._items:
            raise KeyError(f"no {self.what} of kind {spec.kind!r} is registered "
                           f"(known: {', '.join(sorted(self._items)) or 'none'})")
        return self._items[spec.kind](**spec.params, **extra)

    def __contains__(self, kind: str) -> bool:
        return kind in self._items

    def kinds(self) -> list[str]:
        return sorted(self._items)


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")

register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register
