"""Chooses the attention kernels for a step.

float32: the FP32-pipe kernel for every shape.  bfloat16 with head sizes up to
128: the tensor-core kernels, one for the requests that bring several tokens
(portions of prompts: the tcgen05 / TMA kernel for head sizes 64 and 128 and
pages of 8..128 keys, else the mma.sync kernel) and a split-key one for the
requests that bring a single decoded token; in a mixed step both run, each on
its own requests.  Other
cases (bfloat16 with larger heads) use the generic kernel.  All of them read
keys and values through the block table and give the same result up to
rounding.
"""
from __future__ import annotations

import os

import torch

from .. import ops

GENERIC_TILE = 16
PREFILL_TILE = 128
DECODE_KEYS_PER_SPLIT = 256     # a split is worth its launch from about four tiles of keys
DECODE_MAX_SPLITS = 64
USE_TC_ATTENTION = os.environ.get("LYAPUNOV_TC_ATTENTION", "1") not in ("0", "")
DECODE_BLOCKS_PER_SM = 2        # blocks of the decode kernel that a multiprocessor holds at once (by their shared memory)


def tile_sizes() -> list[int]:
    """Query-tile sizes the kernels want listed in the step's integers."""
    return [GENERIC_TILE, PREFILL_TILE]


def prepare(head_dim: int) -> None:
    """Compiles and loads the kernels for this head size (first use only)."""
    ops.attention_lib(head_dim)


def decode_splits(num_requests: int, num_heads: int, num_kv_heads: int, context_bound: int) -> int:
    """The fewest splits whose blocks fill the GPU in whole waves (a last wave
    that is mostly empty costs as much as a full one)."""
    group = num_heads // num_kv_heads
    blocks = num_requests * num_kv_heads * ((group + 15) // 16)
    by_keys = max(1, (context_bound + DECODE_KEYS_PER_SPLIT - 1) // DECODE_KEYS_PER_SPLIT)
    limit = max(1, min(by_keys, DECODE_MAX_SPLITS))
    best, best_fill = 1, 0.0
    resident = DECODE_BLOCKS_PER_SM * ops.sm_count()
    for splits in range(1, limit + 1):
        waves = blocks * splits / resident
        fill = waves / -(-waves // 1)        # waves / ceil(waves)
        if fill >= 0.85:
            return splits
        if fill > best_fill + 1e-9:
            best, best_fill = splits, fill
    return best


def run(out, qkv, ctx, kv, num_heads, num_kv_heads, head_dim, window, scale) -> None:
    table = ctx.block_tables[kv.group]
    if out.dtype == torch.bfloat16 and ops.attention_mma_available(head_dim):
        req, q0, n_tiles, n_multi = ctx.tiles[PREFILL_TILE]
        if n_multi:
            prefill = (ops.attention_prefill_tc_bf16 if USE_TC_ATTENTION and ops.attention_tc_available(head_dim, kv.page_size)
                       else ops.attention_prefill_bf16)
            prefill(out, qkv, qkv.stride(0), kv.k, kv.v, table, ctx.cu_q, ctx.ctx_before, req, q0, n_multi, num_heads,
                    num_kv_heads, head_dim, kv.page_size, window, scale, ctx.status)
        if ctx.num_decode:
            splits = decode_splits(ctx.num_decode, num_heads, num_kv_heads, ctx.context_bound)
            floats = ops.attention_decode_scratch_floats(head_dim, ctx.num_decode, num_heads, splits)
            scratch = ctx.workspace.get("attention_scratch", (floats,), torch.float32) if floats else None
            requests = None if ctx.num_decode == ctx.num_requests else ctx.decode_requests
            ops.attention_decode_bf16(out, scratch, qkv, qkv.stride(0), kv.k, kv.v, table, ctx.cu_q, ctx.ctx_before,
                                      requests, ctx.num_decode, num_heads, num_kv_heads, head_dim, kv.page_size,
                                      window, scale, splits, ctx.status)
        return
    req, q0, n_tiles, _ = ctx.tiles[GENERIC_TILE]
    ops.attention_generic(out, qkv, qkv.stride(0), kv.k, kv.v, table, ctx.cu_q, ctx.ctx_before, req, q0, n_tiles,
                          num_heads, num_kv_heads, head_dim, kv.page_size, window, scale, ctx.status)
