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
# 0: a partly filled step of fixed shape cuts the keys as the full step does (one graph per shape)
SPLITS_BY_FILL = os.environ.get("LYAPUNOV_SPLITS_BY_FILL", "1") not in ("0", "")
DECODE_CLUSTER_SPLITS = 8       # up to this many splits merge inside a thread-block cluster; more need a second kernel
DECODE_WAVE_FILL = 0.97         # the part of the resident blocks that a wave can count on inside a step
DECODE_WAVE_US = 5.0            # a wave's fixed time
DECODE_KEY_US = 0.0075          # a block's time per key of head size 64 (keys and values, latency-bound)
DECODE_MERGE_US = 1.5           # the second kernel of splits beyond a cluster
DECODE_BYTES_PER_US = 6.5e6     # what all blocks together read from memory
DECODE_SMALL_FORM_FILL = 0.9       # the part of its resident blocks that a wave of the form with 16-key tiles can count on
DECODE_SMALL_FORM_SHARING = 0.4    # what each block sharing the multiprocessor adds to such a block's time per key
DECODE_SMALL_FORM_CLUSTER_US = 4.0  # what a wave of clusters of such blocks costs more than one of single blocks


def tile_sizes() -> list[int]:
    """Query-tile sizes the kernels want listed in the step's integers."""
    return [GENERIC_TILE, PREFILL_TILE]


def prepare(head_dim: int) -> None:
    """Compiles and loads the kernels for this head size (first use only)."""
    ops.attention_lib(head_dim)


def choose_decode_splits(blocks: int, context_bound: int, head_dim: int, resident, resident_small=None, sms: int = 148) -> int:
    """The number of splits with the least estimated time.

    ``blocks``: thread blocks before splitting; ``resident(splits)``: blocks the
    device holds at once at that split count.  The blocks run in waves; a wave
    takes a fixed time plus the time of a split's keys, so more splits shorten
    the wave until their blocks no longer fit in one, and then a second wave
    costs more than the shorter keys save.  A step's kernels overlap at their
    edges, so the last few places of a wave are not counted on.

    ``resident_small(splits)`` (None: there is no such form): the same of the
    form with 16-key tiles, which the launcher takes where even the unsplit
    blocks of the usual form do not fit at once (``sms``: multiprocessors).
    Its blocks are half as large and twice as many run at once; a block's time
    per key grows with the blocks that share its multiprocessor, and a cluster
    of them costs more to merge.

    The constants are measured on decode steps of the 1B layer sizes at 4,096
    keys: batches 1 to 32 with every split count from 1 to 8, batches 36 to 128
    in both forms with 1 to 4 splits."""
    by_keys = max(1, (context_bound + DECODE_KEYS_PER_SPLIT - 1) // DECODE_KEYS_PER_SPLIT)
    limit = max(1, min(by_keys, DECODE_MAX_SPLITS))
    # however the keys are cut, all of them cross the memory bus once
    floor = blocks * context_bound * 4 * head_dim / DECODE_BYTES_PER_US
    small = resident_small is not None and blocks > resident(1)
    best, best_cost = 1, float("inf")
    for splits in range(1, limit + 1):
        keys = -(-context_bound // splits)
        key_us = DECODE_KEY_US * head_dim / 64
        if small:
            places = max(1, int(DECODE_SMALL_FORM_FILL * resident_small(splits)))
            sharing = min(4.0, min(blocks * splits, places) / sms)
            wave_us = DECODE_WAVE_US + (DECODE_SMALL_FORM_CLUSTER_US if splits > 1 else 0.0) \
                + keys * key_us * (1.0 + DECODE_SMALL_FORM_SHARING * sharing)
        else:
            # (single blocks fill a wave to the last place; clusters do not)
            places = max(1, int((DECODE_WAVE_FILL if splits > 1 else 1.0) * resident(splits)))
            wave_us = DECODE_WAVE_US + keys * key_us
        waves = -(-blocks * splits // places)
        cost = max(floor, waves * wave_us)
        if splits > DECODE_CLUSTER_SPLITS:
            cost += DECODE_MERGE_US
        if cost < best_cost - 1e-9:          # on a tie the fewer splits stay
            best, best_cost = splits, cost
    return best


def decode_blocks(num_requests: int, num_heads: int, num_kv_heads: int) -> int:
    """Thread blocks of the decode kernel before the keys are split."""
    return num_requests * num_kv_heads * ((num_heads // num_kv_heads + 15) // 16)


def decode_small_form(num_requests: int, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whether the kernel's form with 16-key tiles runs: where the head size
    has it and even the unsplit blocks of the real requests are more than the
    device holds of the usual form at once."""
    return head_dim <= 64 and decode_blocks(num_requests, num_heads, num_kv_heads) > ops.attention_decode_resident_blocks(head_dim, 1)


def decode_splits(num_requests: int, num_heads: int, num_kv_heads: int, context_bound: int, head_dim: int) -> int:
    blocks = decode_blocks(num_requests, num_heads, num_kv_heads)
    small = (lambda s: ops.attention_decode_resident_blocks(head_dim, s, small=True)) if head_dim <= 64 else None
    return choose_decode_splits(blocks, context_bound, head_dim, lambda s: ops.attention_decode_resident_blocks(head_dim, s),
                                small, ops.sm_count())


def decode_variant(fill: int, num_heads: int, num_kv_heads: int, head_dim: int, context_bound: int):
    """The split count (and the kernel's form, where it is not the usual one)
    of a step in which ``fill`` of the one-token requests are real: dummy
    requests finish at once, so the real ones alone fill the waves (9 real
    requests in a step of 16 take 3 splits, 16 take 2)."""
    if not SPLITS_BY_FILL or not ops.attention_mma_available(head_dim):
        return None
    fill = max(1, fill)
    splits = decode_splits(fill, num_heads, num_kv_heads, context_bound, head_dim)
    # (the kernel's form follows the real requests too)
    return (splits, "small") if decode_small_form(fill, num_heads, num_kv_heads, head_dim) else splits


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
            real = min(ctx.decode_fill, ctx.num_decode) if SPLITS_BY_FILL else 0     # dummy requests finish at once
            splits = decode_splits(real or ctx.num_decode, num_heads, num_kv_heads, ctx.context_bound, head_dim)
            small = decode_small_form(real or ctx.num_decode, num_heads, num_kv_heads, head_dim)
            floats = ops.attention_decode_scratch_floats(head_dim, ctx.num_decode, num_heads, splits)
            scratch = ctx.workspace.get("attention_scratch", (floats,), torch.float32) if floats else None
            requests = None if ctx.num_decode == ctx.num_requests else ctx.decode_requests
            ops.attention_decode_bf16(out, scratch, qkv, qkv.stride(0), kv.k, kv.v, table, ctx.cu_q, ctx.ctx_before,
                                      requests, ctx.num_decode, num_heads, num_kv_heads, head_dim, kv.page_size,
                                      window, scale, splits, ctx.status, small_form=small)
        return
    req, q0, n_tiles, _ = ctx.tiles[GENERIC_TILE]
    ops.attention_generic(out, qkv, qkv.stride(0), kv.k, kv.v, table, ctx.cu_q, ctx.ctx_before, req, q0, n_tiles,
                          num_heads, num_kv_heads, head_dim, kv.page_size, window, scale, ctx.status)
