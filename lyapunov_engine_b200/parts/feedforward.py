"""Gated feed-forward (SwiGLU): down(silu(gate(x)) * up(x)).

Gate and up are one projection [2 I, H], gate rows first, as the reference
fuses them at load (python/lyapunov_engine/models/weight_loader.py:155-163;
python/lyapunov_engine/models/llama.py:109-122).  The activation is computed in
32 bits and rounded once (csrc/kernels/fused_rmsnorm_swiglu.cu:170-176).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorDecl, register_feed_forward


@register_feed_forward("gated_silu")
class GatedFeedForward(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, gate_name: str, up_name: str, down_name: str):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.names = (gate_name, up_name, down_name)
        self.w_gate_up = self.w_down = None
        self.runtime = None

    def tensors(self):
        g, u, d = self.names
        H, I = self.hidden_size, self.intermediate_size
        return [TensorDecl(g, (I, H)), TensorDecl(u, (I, H)), TensorDecl(d, (H, I))]

    def bind(self, get, runtime):
        g, u, d = self.names
        self.w_gate_up = torch.cat([get(g), get(u)], dim=0).contiguous()
        self.w_down = get(d)
        self.runtime = runtime

    def forward(self, x, ctx):
        rt = self.runtime
        T = x.shape[0]
        ws = ctx.workspace
        act = ws.get("ffn_act", (T, self.intermediate_size), rt.dtype)
        ops.gated_linear(act, x, self.w_gate_up, ws, ctx.status)
        return ops.linear_for_residual(act, self.w_down, ws, "ffn_out", ctx.status)
