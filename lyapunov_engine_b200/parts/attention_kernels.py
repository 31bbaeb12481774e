"""Chooses the attention kernel for a step.

float32: the FP32-pipe kernel for every shape.  bfloat16: the tensor-core
kernels where they apply (portions of prompts; single decoded tokens split over
the keys), else the same generic kernel.  All of them read keys and values
through the block table and give the same result up to rounding.
"""
from __future__ import annotations

from .. import ops

GENERIC_TILE = 16


def tile_sizes() -> list[int]:
    """Query-tile sizes the kernels want listed in the step's integers."""
    return [GENERIC_TILE]


def prepare(head_dim: int) -> None:
    """Compiles and loads the kernels for this head size (first use only)."""
    ops.attention_lib(head_dim)


def run(out, qkv, ctx, kv, num_heads, num_kv_heads, head_dim, window, scale) -> None:
    tiles = ctx.tiles[GENERIC_TILE]
    ops.attention_generic(out, qkv, qkv.stride(0), kv.k, kv.v, ctx.block_tables[kv.group], ctx.cu_q, ctx.ctx_before,
                          tiles[0], tiles[1], tiles[2], num_heads, num_kv_heads, head_dim, kv.page_size, window,
                          scale, ctx.status)
