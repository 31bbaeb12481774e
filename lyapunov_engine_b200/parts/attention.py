"""Grouped-query attention over the paged cache.

One projection [(nh + 2 nkv) hd, H] = rows q || k || v (the reference keeps
three matrices, python/lyapunov_engine/models/llama.py:45-47), position
encoding of q and k fused with the cache write, attention of every query token
over the keys of its request up to its own position (optionally only the last
``window`` of them), output projection.  Scale 1/sqrt(head_dim)
(csrc/bindings.cpp:131-133).  Head h of the queries uses key/value head
h // (nh / nkv) (csrc/kernels/flash_attn_v2.cu:30-31).

The reference runs attention two ways, FlashAttention on the step's own keys
for a whole prompt and PagedAttention for one decoded token
(llama.py:82-104), and its prompt path never writes the cache.  Here there is
one way: write the step's keys and values to the pages, then attend through the
block table; which kernel does it is chosen by the step's shape and the type.
"""
from __future__ import annotations

import torch

from .. import ops
from . import attention_kernels
from .base import KVNeed, Mixer, POSITION_ENCODINGS, PartSpec, TensorDecl, register_mixer


@register_mixer("attention")
class AttentionMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position: PartSpec,
                 q_name: str, k_name: str, v_name: str, o_name: str, window: int | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} groups")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"attention takes head sizes 16..256 in steps of 16, got {head_dim}")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.window = int(window) if window else None
        self.scale = 1.0 / (head_dim ** 0.5)
        self.names = (q_name, k_name, v_name, o_name)
        self.position = POSITION_ENCODINGS.build(position)
        self.w_qkv = self.w_o = None
        self.runtime = None

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    def tile_sizes(self):
        return attention_kernels.tile_sizes()

    def decode_variant(self, fill, num_decode, context_bound):
        if self.runtime is None or self.runtime.dtype != torch.bfloat16:
            return None                       # the float32 kernel takes every shape the same way
        return attention_kernels.decode_variant(fill, self.num_heads, self.num_kv_heads, self.head_dim, context_bound)

    def tensors(self):
        q, k, v, o = self.names
        H, nh, nkv, hd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim
        return [TensorDecl(q, (nh * hd, H)), TensorDecl(k, (nkv * hd, H)), TensorDecl(v, (nkv * hd, H)),
                TensorDecl(o, (H, nh * hd))] + self.position.tensors()

    def bind(self, get, runtime):
        q, k, v, o = self.names
        self.w_qkv = torch.cat([get(q), get(k), get(v)], dim=0).contiguous()
        self.w_o = get(o)
        self.runtime = runtime
        self.position.bind(get, runtime)
        attention_kernels.prepare(self.head_dim)

    def forward(self, x, ctx, cache):
        rt = self.runtime
        nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        T = x.shape[0]
        ws = ctx.workspace
        qkv = ws.get("qkv", (T, (nh + 2 * nkv) * hd), rt.dtype)
        # a position encoding may know how to run the product itself, with its own work in the epilogue
        fused = getattr(self.position, "product_encode_store", None)
        if fused is None or not fused(qkv, x, self.w_qkv, (nh, nkv, hd), ctx, cache.kv, cache.write):
            ops.linear(qkv, x, self.w_qkv, ctx.status)
            self.position.encode_and_store(qkv, (nh, nkv, hd), ctx, cache.kv, cache.write)
        attn = ws.get("attn", (T, nh * hd), rt.dtype)
        attention_kernels.run(attn, qkv, ctx, cache.kv, nh, nkv, hd, self.window, self.scale)
        return ops.linear_for_residual(attn, self.w_o, ws, "mixer_out", ctx.status)
