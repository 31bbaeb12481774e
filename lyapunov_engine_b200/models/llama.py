"""The dense Llama decoder as a description: which parts, with which numbers
and tensor names, in which order.

Layers (python/lyapunov_engine/models/llama.py:125-178): token embedding; per
layer a pre-norm block of grouped-query attention with rotary encoding and a
SiLU-gated feed-forward, RMSNorm before each; final RMSNorm; linear head, tied
to the embedding when config.json says so.  Tensor names are the checkpoint's
own (python/lyapunov_engine/models/weight_loader.py:91-169).
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec


def llama_spec(raw_config: dict) -> ModelSpec:
    c = LlamaConfig.from_dict(raw_config)
    scaling = None
    if c.rope_scaling is not None:
        s = c.rope_scaling
        scaling = {"rope_type": s.rope_type, "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                   "high_freq_factor": s.high_freq_factor,
                   "original_max_position_embeddings": s.original_max_position_embeddings}
    position = PartSpec("rotary", {"head_dim": c.head_dim, "theta": c.rope_theta,
                                   "max_positions": c.max_position_embeddings, "scaling": scaling})
    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec("attention", {
            "hidden_size": c.hidden_size, "num_heads": c.num_attention_heads,
            "num_kv_heads": c.num_key_value_heads, "head_dim": c.head_dim, "position": position,
            "q_name": p + "self_attn.q_proj.weight", "k_name": p + "self_attn.k_proj.weight",
            "v_name": p + "self_attn.v_proj.weight", "o_name": p + "self_attn.o_proj.weight"})
        feed_forward = PartSpec("gated_silu", {
            "hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size,
            "gate_name": p + "mlp.gate_proj.weight", "up_name": p + "mlp.up_proj.weight",
            "down_name": p + "mlp.down_proj.weight"})
        norm1 = PartSpec("rmsnorm", {"hidden_size": c.hidden_size, "eps": c.rms_norm_eps,
                                     "weight_name": p + "input_layernorm.weight"})
        norm2 = PartSpec("rmsnorm", {"hidden_size": c.hidden_size, "eps": c.rms_norm_eps,
                                     "weight_name": p + "post_attention_layernorm.weight"})
        layers.append(LayerSpec(PartSpec("prenorm", {"mixer": mixer, "feed_forward": feed_forward,
                                                     "mixer_norm": norm1, "feed_forward_norm": norm2})))
    return ModelSpec(
        architecture=c.architecture,
        hidden_size=c.hidden_size,
        vocab_size=c.vocab_size,
        max_positions=c.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
                                               "weight_name": "model.embed_tokens.weight"}),
        layers=tuple(layers),
        run_order=tuple(RunSpec(i) for i in range(c.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"hidden_size": c.hidden_size, "eps": c.rms_norm_eps,
                                        "weight_name": "model.norm.weight"}),
        head=PartSpec("linear_head", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
                                      "weight_name": "lm_head.weight",
                                      "tied_to": "model.embed_tokens.weight" if c.tie_word_embeddings else None}),
        eos_token_ids=c.eos_token_ids,
        bos_token_id=c.bos_token_id,
        config_json=c.to_dict(),
    )
