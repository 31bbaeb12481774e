"""LlamaConfig: the keys of a Llama checkpoint's config.json, typed.

The reference's ``LlamaConfig`` holds ten fields
(python/lyapunov_engine/models/llama.py:9-20) and its reader neither knows
``rope_scaling`` nor ``tie_word_embeddings`` nor ``eos_token_id``
(python/lyapunov_engine/models/weight_loader.py:23-38; the end-of-sequence id
128001 is fixed in csrc/include/engine/scheduler.hpp:16).  All of them are read
here, and options the engine cannot honour are refused rather than ignored.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json.  ``rope_type`` "default" is no scaling;
    "llama3" rescales each frequency by its wavelength relative to
    ``original_max_position_embeddings``."""

    rope_type: str
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    original_max_position_embeddings: int = 0

    @staticmethod
    def from_dict(raw: dict | None, source: str) -> "RopeScaling | None":
        if raw is None:
            return None
        r = KeyReader(raw, source + ": rope_scaling")
        kind = raw.get("rope_type", raw.get("type"))
        if kind is None:
            raise ConfigError(f"{source}: rope_scaling needs 'rope_type'")
        if kind == "default":
            return None
        if kind != "llama3":
            raise ConfigError(
                f"{source}: rope_scaling.rope_type {kind!r} is not supported "
                f"(supported: 'default', 'llama3')")
        scaling = RopeScaling(
            rope_type="llama3",
            factor=r.number("factor"),
            low_freq_factor=r.number("low_freq_factor"),
            high_freq_factor=r.number("high_freq_factor"),
            original_max_position_embeddings=r.integer("original_max_position_embeddings"),
        )
        if not scaling.high_freq_factor > scaling.low_freq_factor:
            raise ConfigError(f"{source}: rope_scaling.high_freq_factor must exceed low_freq_factor")
        return scaling


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling | None
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...]
    bos_token_id: int | None
    torch_dtype: str | None
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    @staticmethod
    def from_dict(raw: dict, source: str = "config.json") -> "LlamaConfig":
        r = KeyReader(raw, source)
        archs = raw.get("architectures") or []
        architecture = archs[0] if archs else r.string("model_type")
        hidden = r.integer("hidden_size")
        heads = r.integer("num_attention_heads")
        kv_heads = r.integer("num_key_value_heads", default=heads)
        head_dim = r.integer("head_dim", default=None)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"{source}: 'head_dim' is absent and hidden_size {hidden} is not a "
                    f"multiple of num_attention_heads {heads}")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(
                f"{source}: num_attention_heads {heads} is not a multiple of "
                f"num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"{source}: head_dim {head_dim} must be even for rotary encoding")
        act = r.string("hidden_act", default="silu")
        if act != "silu":
            raise ConfigError(f"{source}: hidden_act {act!r} is not supported (the gated "
                              f"feed-forward of this architecture uses 'silu')")
        for key in ("attention_bias", "mlp_bias"):
            if r.boolean(key, default=False):
                raise ConfigError(f"{source}: {key} = true is not supported (projections have no bias)")
        bos = r.integer("bos_token_id", default=None, minimum=0)
        return LlamaConfig(
            architecture=architecture,
            vocab_size=r.integer("vocab_size"),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size"),
            num_hidden_layers=r.integer("num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=r.integer("max_position_embeddings"),
            rms_norm_eps=r.number("rms_norm_eps"),
            rope_theta=r.number("rope_theta"),
            rope_scaling=RopeScaling.from_dict(r.mapping("rope_scaling", default=None), source),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=False),
            eos_token_ids=r.id_list("eos_token_id", default=None),
            bos_token_id=bos,
            torch_dtype=r.string("torch_dtype", default=None),
            raw=dict(raw),
        )

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        out = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            out["rope_scaling"] = {
                "rope_type": s.rope_type, "factor": s.factor,
                "low_freq_factor": s.low_freq_factor, "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": s.original_max_position_embeddings,
            }
        if self.eos_token_ids:
            out["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                   else list(self.eos_token_ids))
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.torch_dtype:
            out["torch_dtype"] = self.torch_dtype
        return out
