"""Rotary position encoding: the frequency table and its use on queries and
keys, fused with the cache write.

Frequencies f_j = theta^(-2j/rot) in float32 as the reference builds them
(python/lyapunov_engine/models/llama.py:180-184); angles p * f_j, their cosines
and sines in float32 (llama.py:186-194); rotate-half pairing (llama.py:23-31).
The reference then casts cos/sin to the activations' type and rotates in it;
here the table stays 32-bit and so does the rotation, as in the reference's own
fused kernel (csrc/kernels/fused_rope_paged.cu:26-46).

"llama3" scaling is not in the reference.  By the meaning of its config.json
keys: a frequency whose wavelength 2*pi/f is shorter than original_max /
high_freq_factor is kept; one longer than original_max / low_freq_factor is
divided by ``factor``; in between the two are blended linearly in
original_max / wavelength.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import PositionEncoding, register_position_encoding


def inverse_frequencies(rot: int, theta: float, scaling: dict | None) -> torch.Tensor:
    exponents = torch.arange(0, rot, 2, dtype=torch.float32) / rot
    inv_freq = 1.0 / (theta ** exponents)
    if not scaling:
        return inv_freq
    if scaling.get("rope_type") != "llama3":
        raise ValueError(f"rotary scaling {scaling.get('rope_type')!r} is not supported")
    factor, low, high = float(scaling["factor"]), float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    scaled = []
    for f in inv_freq.tolist():
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            scaled.append(f)
        elif wavelength > original / low:
            scaled.append(f / factor)
        else:
            blend = (original / wavelength - low) / (high - low)
            scaled.append((1.0 - blend) * f / factor + blend * f)
    return torch.tensor(scaled, dtype=torch.float32)


@register_position_encoding("rotary")
class RotaryEncoding(PositionEncoding):
    """``rot`` leading dimensions of each head are rotated (rot = head_dim for
    Llama); the table covers positions 0 .. max_positions - 1."""

    def __init__(self, head_dim: int, theta: float, max_positions: int, scaling: dict | None = None,
                 rot: int | None = None):
        self.head_dim = int(head_dim)
        self.rot = int(rot if rot is not None else head_dim)
        if self.rot % 2 or not 0 < self.rot <= self.head_dim:
            raise ValueError(f"rotary width {self.rot} must be even and at most head_dim {self.head_dim}")
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        self.max_positions = int(max_positions)
        self.table = None

    def build_table(self, max_positions: int | None = None) -> torch.Tensor:
        """[positions, rot] float32 on the CPU: cos(rot/2) || sin(rot/2)."""
        n = int(max_positions or self.max_positions)
        inv_freq = inverse_frequencies(self.rot, self.theta, self.scaling)
        angles = torch.outer(torch.arange(n, dtype=torch.float32), inv_freq)
        return torch.cat((angles.cos(), angles.sin()), dim=-1).contiguous()

    def bind(self, get, runtime):
        n = min(self.max_positions, runtime.max_model_len) if runtime.max_model_len else self.max_positions
        key = ("rotary", self.rot, self.theta, repr(self.scaling), n)
        table = runtime.shared.get(key)
        if table is None:
            table = self.build_table(n).to(runtime.device)
            runtime.shared[key] = table
        self.table = table

    def product_encode_store(self, qkv, x, w_qkv, geometry, ctx, kv, write: bool) -> bool:
        """qkv = x @ w_qkv^T, rotated and stored, as one kernel where that exists
        (few rows, bfloat16, the whole head rotates).  False: nothing was done,
        the caller runs the product and encode_and_store."""
        nh, nkv, hd = geometry
        if not ops.FUSE_ROTARY or x.dtype != torch.bfloat16 or not ops.rotary_product_applies(x, w_qkv, hd, self.table.shape[1]):
            return False
        ops.gemm_skinny_rotary(qkv, x, w_qkv, kv.k if kv is not None else None, kv.v if kv is not None else None, self.table,
                               ctx.positions, ctx.request_of_token,
                               ctx.block_tables[kv.group] if kv is not None else ctx.block_tables[0], nh, nkv, hd,
                               kv.page_size if kv is not None else 1, write and kv is not None, ctx.status)
        return True

    def encode_and_store(self, qkv, geometry, ctx, kv, write: bool) -> None:
        nh, nkv, hd = geometry
        ops.rope_kv_write(qkv, kv.k if kv is not None else None, kv.v if kv is not None else None, self.table,
                          ctx.positions, ctx.request_of_token, ctx.block_tables[kv.group] if kv is not None else ctx.block_tables[0],
                          nh, nkv, hd, kv.page_size if kv is not None else 1, write and kv is not None, ctx.status)
