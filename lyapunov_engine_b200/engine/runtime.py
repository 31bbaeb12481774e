"""What every part of a running model shares: the device, the activations'
type, scratch memory and the device status word."""
from __future__ import annotations

import torch

from .. import ops


class Workspace:
    """Named scratch buffers that are reused step after step and layer after
    layer (layers run one after the other, so one buffer per name is enough).
    A buffer only ever grows; its earlier storage is kept alive when
    ``pin_old`` is set, because a captured CUDA graph may still point into it."""

    def __init__(self, device, pin_old: bool = False):
        self.device = device
        self.pin_old = pin_old
        self._buffers: dict[tuple, torch.Tensor] = {}
        self._views: dict[tuple, torch.Tensor] = {}
        self._old: list[torch.Tensor] = []

    def get(self, name: str, shape, dtype) -> torch.Tensor:
        # the same name, shape and type as before (every layer of a step, every step of a decode): the same view
        view = self._views.get((name, shape, dtype)) if type(shape) is tuple else None
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            if buf is not None and self.pin_old:
                self._old.append(buf)
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self._views = {k: v for k, v in self._views.items() if (k[0], k[2]) != key}   # they point into the old storage
        view = buf[:n].view(*shape)
        if type(shape) is tuple and len(self._views) < 4096:
            self._views[(name, shape, dtype)] = view
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class Runtime:
    def __init__(self, device, dtype: torch.dtype, max_model_len: int | None = None):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ops.KernelError(f"lyapunov_engine_b200 runs on a CUDA device, not on {self.device} "
                                  f"(there is no CPU path)")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be torch.bfloat16 or torch.float32, got {dtype}")
        self.dtype = dtype
        # Library products (bfloat16 with many rows) must add up in 32 bits whatever algorithm the library picks;
        # its default lets split-K partial sums pass through bfloat16.
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self.max_model_len = max_model_len
        self.shared: dict = {}
        self.workspace = Workspace(self.device)
        self.status = ops.new_status(self.device)


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
             "f32": torch.float32}
    if name not in table:
        raise ValueError(f"dtype must be one of {sorted(table)}, got {name!r}")
    return table[name]
