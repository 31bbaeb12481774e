"""Tiny configurations, seeded weights and model folders for the tests.

The two tiny configurations differ in every size and option of the
architecture: layer count, width, heads and groups (GQA against MQA), head
size, feed-forward width, vocabulary (none a power of two in tiny-B), the
norms' eps, rope_theta, plain against llama3-scaled RoPE, tied against untied
output head and the cache's page size.  Folders are written with the
``safetensors`` library (the product has its own writer), always into a
temporary directory.
"""
from __future__ import annotations

import json
import os

import torch

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 256,
    "hidden_size": 64,
    "intermediate_size": 192,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "max_position_embeddings": 128,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "rope_scaling": None,
    "tie_word_embeddings": True,
    "hidden_act": "silu",
    "attention_bias": False,
    "mlp_bias": False,
    "bos_token_id": 1,
    "eos_token_id": 2,
    "torch_dtype": "float32",
}
TINY_A_PAGE = 4

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 515,
    "hidden_size": 96,
    "intermediate_size": 328,
    "num_hidden_layers": 3,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "head_dim": 32,
    "max_position_embeddings": 256,
    "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 4.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 32,
    },
    "tie_word_embeddings": False,
    "hidden_act": "silu",
    "attention_bias": False,
    "mlp_bias": False,
    "bos_token_id": 0,
    "eos_token_id": [3, 4],
    "torch_dtype": "float32",
}
TINY_B_PAGE = 8

# tiny-B with every number as the baseline's configuration list states it (vocabulary 512, feed-forward 320;
# weights N(0, 0.02), see the replay tests).  TINY_B above departs from it on purpose: a vocabulary and a
# feed-forward width that are no multiples of 8 or 16, and larger weights with peaked attention, which make a wrong
# key, position or page show.
TINY_B_STATED = dict(TINY_B, vocab_size=512, intermediate_size=320)

# A third shape for long contexts: head size 64 as in the 1B model, more
# groups, a width that is a multiple of 8 only.
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 1000,
    "hidden_size": 136,
    "intermediate_size": 264,
    "num_hidden_layers": 2,
    "num_attention_heads": 6,
    "num_key_value_heads": 3,
    "head_dim": 64,
    "max_position_embeddings": 2048,
    "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 256,
    },
    "tie_word_embeddings": True,
    "hidden_act": "silu",
    "attention_bias": False,
    "mlp_bias": False,
    "bos_token_id": 0,
    "eos_token_id": 1,
    "torch_dtype": "float32",
}
TINY_C_PAGE = 16


# A fourth shape: a head size that is no power of two (48), six heads in three groups, a width and a feed-forward
# that are multiples of 8 only, an odd vocabulary.
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 777,
    "hidden_size": 200,
    "intermediate_size": 296,
    "num_hidden_layers": 2,
    "num_attention_heads": 6,
    "num_key_value_heads": 3,
    "head_dim": 48,
    "max_position_embeddings": 512,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "rope_scaling": None,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
    "attention_bias": False,
    "mlp_bias": False,
    "bos_token_id": 0,
    "eos_token_id": 1,
    "torch_dtype": "float32",
}
TINY_D_PAGE = 8


def head_dim(cfg):
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


def make_weights(cfg: dict, seed: int, std: float = 0.02, norm_std: float = 0.0,
                 qk_gain: float = 1.0) -> dict:
    """Seeded float32 tensors under the checkpoint's tensor names: matrices
    N(0, std), norm weights 1 + N(0, norm_std).  ``qk_gain`` multiplies the
    query and key projections so that attention is peaked and a wrong key, a
    wrong position or a stale page changes the logits visibly."""
    g = torch.Generator().manual_seed(seed)
    H = cfg["hidden_size"]
    I = cfg["intermediate_size"]
    V = cfg["vocab_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = head_dim(cfg)

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (std * gain)

    def norm():
        return 1.0 + torch.randn(H, generator=g) * norm_std if norm_std else torch.ones(H)

    w = {"model.embed_tokens.weight": mat(V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = norm()
        w[p + "self_attn.q_proj.weight"] = mat(nh * hd, H, qk_gain)
        w[p + "self_attn.k_proj.weight"] = mat(nkv * hd, H, qk_gain)
        w[p + "self_attn.v_proj.weight"] = mat(nkv * hd, H)
        w[p + "self_attn.o_proj.weight"] = mat(H, nh * hd)
        w[p + "post_attention_layernorm.weight"] = norm()
        w[p + "mlp.gate_proj.weight"] = mat(I, H)
        w[p + "mlp.up_proj.weight"] = mat(I, H)
        w[p + "mlp.down_proj.weight"] = mat(H, I)
    w["model.norm.weight"] = norm()
    if not cfg.get("tie_word_embeddings", False):
        w["lm_head.weight"] = mat(V, H)
    return w


def write_model_folder(folder: str, cfg: dict, weights: dict, dtype=torch.float32) -> str:
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    cfg = dict(cfg)
    cfg["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()},
              os.path.join(folder, "model.safetensors"))
    return folder


def random_ids(cfg: dict, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
