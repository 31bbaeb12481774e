"""RMSNorm over the 32-bit residual stream (with the residual addition fused).

Reference: rmsnorm (python/lyapunov_engine/ops.py:12-51) and rmsnorm_kernel
(csrc/kernels/fused_rmsnorm_swiglu.cu:15-113); the layer's norm weights there
are bare parameters of the decoder layer (python/lyapunov_engine/models/llama.py:130-134).
"""
from __future__ import annotations

from .. import ops
from .base import Norm, TensorDecl, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, hidden_size: int, eps: float, weight_name: str):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight = None
        self.runtime = None

    def tensors(self):
        return [TensorDecl(self.weight_name, (self.hidden_size,), role="vector", init="ones_jitter")]

    def bind(self, get, runtime):
        self.weight = get(self.weight_name)
        self.runtime = runtime

    def apply(self, resid, delta=None, rows=None, workspace=None, key="normed"):
        n = resid.shape[0] if rows is None else rows.shape[0]
        ws = workspace or self.runtime.workspace
        out = ws.get(key, (n, self.hidden_size), self.runtime.dtype)
        ops.rmsnorm(out, resid, delta, self.weight, self.eps, rows)
        return out
