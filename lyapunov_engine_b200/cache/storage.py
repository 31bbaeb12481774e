"""The cache on the device and its manager on the host.

For every cache group of the model (layers whose pages have the same geometry
and life: all keys, or a window of them) there is one pool of page ids,
managed by the C++ ``BlockSpaceManager``, and per run of the model that writes
pages a pair of pools K, V of shape [pages + 1, kv_heads, page, head_dim] (the
reference's layout, python/lyapunov_engine/engine/llm_engine.py:143-158).  A
page id means that page in every pool of the group.  The extra last page
belongs to nobody: padding rows of fixed-shape decode batches write there, and
block-table entries that a window has released point there.

Beside the pages, every request holds one state slot; a mixer that declares
per-request state of fixed size gets a buffer [slots + 1, *shape] and finds
its row by the request's slot (the last row again belongs to padding).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import build


@dataclass
class KVStream:
    k: torch.Tensor
    v: torch.Tensor
    page_size: int
    group: int


@dataclass
class CacheBinding:
    """What one run of a layer sees of the cache."""
    kv: KVStream | None
    write: bool
    state: torch.Tensor | None


class DeviceCache:
    def __init__(self, model, runtime, num_blocks: int, block_size: int, max_num_seqs: int):
        host = build.load_host()
        self.model = model
        self.block_size = int(block_size)
        self.num_blocks = int(num_blocks)
        self.max_num_seqs = int(max_num_seqs)
        groups = [host.CacheGroupSpec(block_size=self.block_size, window=int(g.window or 0), num_blocks=self.num_blocks)
                  for g in model.groups]
        self.manager = host.BlockSpaceManager(groups, self.max_num_seqs)
        self.streams: list[list[KVStream]] = []
        for gi, g in enumerate(model.groups):
            pools = []
            for _ in range(model.streams_per_group[gi]):
                shape = (self.num_blocks + 1, g.num_kv_heads, self.block_size, g.head_dim)
                pools.append(KVStream(torch.zeros(shape, dtype=runtime.dtype, device=runtime.device),
                                      torch.zeros(shape, dtype=runtime.dtype, device=runtime.device),
                                      self.block_size, gi))
            self.streams.append(pools)
        self.states = [torch.zeros((self.max_num_seqs + 1, *need.shape), dtype=need.dtype or torch.float32,
                                   device=runtime.device) for need in model.states]
        self._bindings = []
        for run in model.runs:
            kv = self.streams[run.group][run.stream] if run.group is not None else None
            state = self.states[run.state] if run.state is not None else None
            self._bindings.append(CacheBinding(kv, run.writes, state))

    def binding(self, run_index: int) -> CacheBinding:
        return self._bindings[run_index]

    def bytes(self) -> int:
        total = 0
        for pools in self.streams:
            for s in pools:
                total += 2 * s.k.numel() * s.k.element_size()
        for s in self.states:
            total += s.numel() * s.element_size()
        return total

    @staticmethod
    def bytes_per_block(model, dtype: torch.dtype, block_size: int) -> int:
        width = 2 if dtype == torch.bfloat16 else 4
        total = 0
        for gi, g in enumerate(model.groups):
            total += 2 * model.streams_per_group[gi] * g.num_kv_heads * block_size * g.head_dim * width
        return total
