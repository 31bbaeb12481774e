"""Makes tests/golden/*.npz: logits of IanConery/lyapunov-engine's own model
code (python/lyapunov_engine/models/llama.py, eager CPU fallbacks of
python/lyapunov_engine/ops.py) on the tiny random models of tests/fixtures.py.

    python tests/golden/make_golden.py /path/to/lyapunov-engine

Only whole-sequence forwards from position 0 are taken: the reference's decode
branch neither writes the cache nor rotates by the token's position, so it
anchors nothing.  The reference has no llama3 frequency scaling; for the scaled
configuration the scaled ``inv_freq`` of the plain implementation is written
into the reference model's buffer, so that golden anchors everything but that
formula.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import fixtures  # noqa: E402
import plain_llama  # noqa: E402


def reference_logits(ref_root, cfg, weights, ids):
    sys.path.insert(0, os.path.join(ref_root, "python"))
    sys.dont_write_bytecode = True
    from lyapunov_engine.models.llama import LlamaConfig, LlamaForCausalLM
    from lyapunov_engine.models.weight_loader import load_hf_weights_into_model

    rc = LlamaConfig(
        vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"],
        intermediate_size=cfg["intermediate_size"],
        num_hidden_layers=cfg["num_hidden_layers"],
        num_attention_heads=cfg["num_attention_heads"],
        num_key_value_heads=cfg["num_key_value_heads"],
        head_dim=fixtures.head_dim(cfg),
        max_position_embeddings=cfg["max_position_embeddings"],
        rms_norm_eps=cfg["rms_norm_eps"], rope_theta=cfg["rope_theta"])
    model = LlamaForCausalLM(rc)
    load_hf_weights_into_model(model, dict(weights), dtype=torch.float32, device="cpu")
    model.eval()
    if cfg.get("rope_scaling"):
        model.inv_freq.copy_(plain_llama.plain_inv_freq(
            fixtures.head_dim(cfg), cfg["rope_theta"], cfg["rope_scaling"]))
    with torch.no_grad():
        return model(torch.tensor([ids], dtype=torch.long))[0]


CASES = {
    # name: (config, weight seed, std, norm_std, qk_gain, ids seed, length)
    "tiny_a": (fixtures.TINY_A, 0, 0.02, 0.0, 1.0, 100, 49),
    "tiny_b": (fixtures.TINY_B, 1, 0.02, 0.1, 1.0, 101, 64),
    "tiny_b_sharp": (fixtures.TINY_B, 2, 0.08, 0.1, 6.0, 102, 48),
}


def main():
    ref_root = sys.argv[1]
    for name, (cfg, seed, std, norm_std, gain, ids_seed, n) in CASES.items():
        w = fixtures.make_weights(cfg, seed, std, norm_std, gain)
        ids = fixtures.random_ids(cfg, n, ids_seed)
        ref = reference_logits(ref_root, cfg, w, ids)
        mine = plain_llama.plain_forward(cfg, w, ids)
        err = (ref - mine).abs().max().item()
        print(f"{name}: logits {tuple(ref.shape)} max|ref| {ref.abs().max():.4f} "
              f"max|ref - plain| {err:.3e}")
        np.savez_compressed(os.path.join(HERE, name + ".npz"),
                            ids=np.asarray(ids, dtype=np.int32),
                            logits=ref.numpy().astype(np.float32))


if __name__ == "__main__":
    main()
