"""The engine at the layer sizes of the real models (Llama-3.2-1B: width 2048,
32 heads in 8 groups, head 64, feed-forward 8192; Llama-3.2-3B: width 3072, 24
heads in 8 groups, head 128), with few layers and a smaller vocabulary so that
the plain implementation can follow on the CPU.  Replay in every cut, bfloat16
and float32, against the plain implementation."""
import pytest
import torch

import fixtures
import plain_llama
import replay_util as ru

pytestmark = pytest.mark.gpu

SCALING = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
           "original_max_position_embeddings": 8192}


def config(hidden, heads, kv_heads, head_dim, inter, vocab, layers, tied):
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": vocab, "hidden_size": hidden,
            "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": heads,
            "num_key_value_heads": kv_heads, "head_dim": head_dim, "max_position_embeddings": 131072,
            "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": SCALING, "tie_word_embeddings": tied,
            "hidden_act": "silu", "attention_bias": False, "mlp_bias": False, "eos_token_id": 1}


CONFIGS = {
    "1b_layers": (config(2048, 32, 8, 64, 8192, 32064, 2, True), (700, 333, 130, 64)),
    "3b_layers": (config(3072, 24, 8, 128, 8192, 16032, 1, True), (520, 200, 77)),
}


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    cfg, lengths = CONFIGS[request.param]
    w = fixtures.make_weights(cfg, seed=11, std=0.02, norm_std=0.05, qk_gain=2.0)
    folders = {}
    for dtype in (torch.bfloat16, torch.float32):
        d = str(tmp_path_factory.mktemp(request.param + ("16" if dtype == torch.bfloat16 else "32")))
        fixtures.write_model_folder(d, cfg, w, dtype)
        folders[dtype] = d
    requests = {f"r{i}": fixtures.random_ids(cfg, n, 900 + i) for i, n in enumerate(lengths)}
    rounded = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    ref32 = {r: plain_llama.plain_forward(cfg, w, ids) for r, ids in requests.items()}
    ref16 = {r: plain_llama.plain_forward(cfg, rounded, ids, act_dtype=torch.bfloat16, prob_dtype=torch.bfloat16)
             for r, ids in requests.items()}
    short = min(requests, key=lambda r: len(requests[r]))
    r64 = {k: v.double() for k, v in rounded.items()}
    floor = float((plain_llama.plain_forward(cfg, r64, requests[short], act_dtype=torch.bfloat16).float() - ref16[short]).abs().max())
    return dict(cfg=cfg, folders=folders, requests=requests, ref={"float32": ref32, "bfloat16": ref16}, floor=floor,
                prompt_lens={r: max(1, len(ids) - 40) for r, ids in requests.items()})


def check(m, trace, dtype, tmp_path, live, what):
    folder = m["folders"][torch.float32 if dtype == "float32" else torch.bfloat16]
    lens = sorted((len(v) for v in m["requests"].values()), reverse=True)[:live]
    pool = sum((n + 63) // 64 * 64 for n in lens)
    got = ru.run_trace(trace, folder, dtype, str(tmp_path), pool, 16)
    assert len(got) == sum(len(w) for w in trace.wanted)
    if dtype == "float32":
        return ru.compare(got, m["ref"][dtype], atol=2e-4, rtol=2e-4, what=what)
    return ru.compare(got, m["ref"][dtype], atol=3.0 * m["floor"] + 2e-3, rtol=0.0, what=what)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_whole_then_tail(model, dtype, tmp_path):
    check(model, ru.tail_trace(model["requests"], 32), dtype, tmp_path, 1, f"scale {dtype} tail")


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_portions_and_mixed(model, dtype, tmp_path):
    check(model, ru.portions_trace(model["requests"], sizes=(130, 2, 257, 64, 3, 129, 17)), dtype, tmp_path / "p", 1,
          f"scale {dtype} portions")
    trace = ru.mixed_trace(model["requests"], model["prompt_lens"], chunk=200, max_live=4, seed=1)
    check(model, trace, dtype, tmp_path / "m", 4, f"scale {dtype} mixed")
