"""Weights by tensor name, from a model folder or from a seed.

Every part of a model declares the checkpoint tensors it reads
(``TensorDecl``).  ``FolderWeights`` checks all of them against the folder's
safetensors files before anything is copied and raises ONE error that lists
what is missing, what is unexpected and what has the wrong shape.  Types on
the device: "matrix" tensors in the engine's compute type (bfloat16 or
float32), "vector" tensors (norm weights) in float32, so that one stored in 32
bits stays exactly so, "int_table" tensors in int32.

The reference treats every tensor as optional and skips silently what is
missing (python/lyapunov_engine/models/weight_loader.py:91-169).

``RandomWeights`` fills the same declarations from a seed: matrices N(0, std),
norm weights 1 (+ N(0, norm_jitter)); ``write_random_model`` writes such a
model as a folder (config.json, model.safetensors).
"""
from __future__ import annotations

import json
import os

import torch

from ..config.base import read_config_json
from ..parts.base import TensorDecl
from . import safetensors_io

# Buffers some exporters store although they are computed, not learned.
IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


class WeightsError(ValueError):
    pass


def _kept_dtype(decl: TensorDecl, compute_dtype: torch.dtype) -> torch.dtype:
    if decl.role == "matrix":
        return compute_dtype
    if decl.role == "vector":
        return torch.float32
    if decl.role == "int_table":
        return torch.int32
    raise ValueError(f"tensor {decl.name!r}: unknown role {decl.role!r}")


class FolderWeights:
    def __init__(self, folder: str, decls: list[TensorDecl], compute_dtype: torch.dtype, device):
        self.folder = folder
        self.device = device
        self.compute_dtype = compute_dtype
        try:
            self.table = safetensors_io.open_folder(folder)
        except safetensors_io.SafetensorsError as e:
            raise WeightsError(str(e)) from e
        self.decls = {d.name: d for d in decls}
        self._resolved: dict[str, str] = {}
        self._cache: dict[str, torch.Tensor] = {}
        self._check()

    def _check(self) -> None:
        missing, wrong, wrong_type = [], [], []
        used = set()
        for d in self.decls.values():
            source = d.name
            if source not in self.table:
                if d.alias_of is not None and d.alias_of in self.table:
                    source = d.alias_of
                else:
                    missing.append(f"{d.name} {list(d.shape)}" + (f" (or {d.alias_of})" if d.alias_of else ""))
                    continue
            entry = self.table[source]
            used.add(source)
            self._resolved[d.name] = source
            if tuple(entry.shape) != tuple(d.shape):
                wrong.append(f"{source}: the file has {list(entry.shape)}, the model needs {list(d.shape)}")
            floating = entry.dtype in (torch.float32, torch.float16, torch.bfloat16, torch.float64)
            if (d.role == "int_table") == floating:
                wrong_type.append(f"{source}: stored as {entry.dtype}, read as {d.role}")
        unexpected = sorted(n for n in self.table if n not in used and not n.endswith(IGNORED_SUFFIXES))
        if missing or wrong or wrong_type or unexpected:
            lines = [f"{self.folder}: the tensors in the folder do not fit the model"]
            if missing:
                lines.append(f"  missing ({len(missing)}): " + "; ".join(missing))
            if unexpected:
                lines.append(f"  unexpected ({len(unexpected)}): " + "; ".join(unexpected))
            if wrong:
                lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(wrong))
            if wrong_type:
                lines.append(f"  wrong type ({len(wrong_type)}): " + "; ".join(wrong_type))
            raise WeightsError("\n".join(lines))

    def get(self, name: str) -> torch.Tensor:
        decl = self.decls[name]
        source = self._resolved[name]
        key = source
        if key not in self._cache:
            entry = self.table[source]
            host = entry.file.tensor(source)
            self._cache[key] = host.to(device=self.device, dtype=_kept_dtype(decl, self.compute_dtype)).contiguous()
        return self._cache[key]

    def release(self) -> None:
        self._cache.clear()


class RandomWeights:
    """Seeded tensors for the same declarations, made on ``device`` (one
    generator, declarations in order, so a seed gives one model)."""

    def __init__(self, decls: list[TensorDecl], compute_dtype: torch.dtype, device, seed: int, std: float = 0.02,
                 norm_jitter: float = 0.0, tied: bool = True):
        self.decls = {d.name: d for d in decls}
        self.compute_dtype, self.device = compute_dtype, device
        self.std, self.norm_jitter, self.tied = std, norm_jitter, tied
        self.generator = torch.Generator(device=device).manual_seed(int(seed))
        self._cache: dict[str, torch.Tensor] = {}
        for d in decls:  # fixed order of generation
            if d.alias_of is not None and tied:
                continue
            self._cache[d.name] = self._make(d)

    def _make(self, d: TensorDecl) -> torch.Tensor:
        if d.role == "int_table":
            return torch.zeros(d.shape, dtype=torch.int32, device=self.device)
        if d.init == "normal":
            t = torch.randn(d.shape, generator=self.generator, device=self.device, dtype=torch.float32) * self.std
        elif d.init in ("ones", "ones_jitter"):
            t = torch.ones(d.shape, device=self.device, dtype=torch.float32)
            if d.init == "ones_jitter" and self.norm_jitter:
                t += torch.randn(d.shape, generator=self.generator, device=self.device, dtype=torch.float32) * self.norm_jitter
        elif d.init == "zeros":
            t = torch.zeros(d.shape, device=self.device, dtype=torch.float32)
        else:
            raise ValueError(f"tensor {d.name!r}: unknown init {d.init!r}")
        return t.to(_kept_dtype(d, self.compute_dtype))

    def get(self, name: str) -> torch.Tensor:
        d = self.decls[name]
        if name not in self._cache and d.alias_of is not None:
            return self._cache[d.alias_of]
        return self._cache[name]

    def release(self) -> None:
        self._cache.clear()


def write_random_model(folder: str, config: dict, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                       norm_jitter: float = 0.0) -> str:
    """Writes ``folder``/config.json and ``folder``/model.safetensors for the
    architecture that ``config`` (the content of a config.json) names: matrices
    N(0, std), norm weights 1 + N(0, norm_jitter), stored as ``dtype`` (vectors
    as float32).  A tied head is not stored."""
    from ..models.model import Model
    from ..registry import spec_for

    spec = spec_for(config)
    model = Model(spec)
    decls = model.tensors()
    source = RandomWeights(decls, dtype, "cpu", seed, std, norm_jitter, tied=True)
    os.makedirs(folder, exist_ok=True)
    tensors = {d.name: source.get(d.name).contiguous() for d in decls if d.name in source._cache}
    safetensors_io.save_file(tensors, os.path.join(folder, "model.safetensors"), {"format": "pt"})
    out = dict(spec.config_json) if spec.config_json else dict(config)
    out["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[dtype]
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out, f, indent=1)
    return folder


def read_folder_config(folder: str) -> dict:
    return read_config_json(folder)
