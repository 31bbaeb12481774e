"""Chooses the next token of every sampled request on the device, in one
launch for the whole batch.

Greedy rows and temperature rows go through the same kernel; a step whose rows
are all greedy uses the argmax kernel.  The per-row options travel as small
tensors; nothing comes back to the host but the chosen ids.  The reference
loops over rows in Python with a device-to-host transfer per row
(python/lyapunov_engine/engine/sampling.py:30-70).
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops


class Sampler:
    def __init__(self, device, max_rows: int):
        self.device = device
        self.max_rows = max_rows
        # A ring of pinned buffers: the copy to the device runs when the device gets to it, which may be after
        # the next call has been made (the engine launches steps ahead of reading their results).
        self._hosts = [(torch.empty((max_rows, 6), dtype=torch.int32, pin_memory=True), torch.cuda.Event()) for _ in range(4)]
        self._host_at = 0
        self._dev = torch.empty((max_rows, 6), dtype=torch.int32, device=device)
        self._out = torch.empty(max_rows, dtype=torch.int32, device=device)
        self._scratch = None

    def sample(self, logits: torch.Tensor, params: list, token_indices: list[int]) -> torch.Tensor:
        """``logits`` [n, V] float32; ``params[i]`` the SamplingParams of row i;
        ``token_indices[i]`` the index in its sequence of the token being
        chosen (the generator's counter).  Returns int32 ids [n] on the device."""
        n = logits.shape[0]
        out = self._out[:n]
        if all(p.temperature < 1e-4 for p in params):
            need = ops.argmax_scratch_floats(self.max_rows, logits.shape[1])
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(need, dtype=torch.float32, device=self.device)
            ops.argmax(out, logits, self._scratch)
            return out
        pinned, event = self._hosts[self._host_at]
        self._host_at = (self._host_at + 1) % len(self._hosts)
        event.synchronize()
        host = pinned.numpy()
        f = host.view(np.float32)
        for i, p in enumerate(params):
            f[i, 0] = p.temperature
            f[i, 1] = p.top_p
            host[i, 2] = p.top_k
            seed = int(p.seed) & 0xFFFFFFFFFFFFFFFF
            host[i, 3:5] = np.array([seed & 0xFFFFFFFF, seed >> 32], dtype=np.uint32).view(np.int32)
            host[i, 5] = token_indices[i]
        self._dev[:n].copy_(pinned[:n], non_blocking=True)
        event.record()
        d = self._dev[:n]
        cols = d.t().contiguous()  # [6, n]: each option contiguous
        temperature = cols[0].view(torch.float32)
        top_p = cols[1].view(torch.float32)
        top_k = cols[2]
        seeds = d[:, 3:6].contiguous()
        ops.sample(out, logits, temperature, top_p, top_k, seeds)
        return out
