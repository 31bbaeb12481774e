"""Configuration, registry, safetensors reading/writing and the loader's one
error that lists everything wrong (no GPU needed)."""
import json
import os

import pytest
import torch

import fixtures
from lyapunov_engine_b200 import known_architectures, register_architecture, write_random_model
from lyapunov_engine_b200.config import ConfigError, LlamaConfig
from lyapunov_engine_b200.models.model import Model
from lyapunov_engine_b200.registry import spec_for
from lyapunov_engine_b200.weights import FolderWeights, RandomWeights, WeightsError, safetensors_io


def test_reads_every_key_of_both_tiny_configs():
    a = LlamaConfig.from_dict(fixtures.TINY_A)
    b = LlamaConfig.from_dict(fixtures.TINY_B)
    assert (a.vocab_size, a.hidden_size, a.intermediate_size, a.num_hidden_layers) == (256, 64, 192, 2)
    assert (a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (4, 2, 16)
    assert a.rope_scaling is None and a.tie_word_embeddings and a.eos_token_ids == (2,) and a.rms_norm_eps == 1e-5
    assert b.rope_scaling.factor == 4.0 and b.rope_scaling.original_max_position_embeddings == 32
    assert b.eos_token_ids == (3, 4) and not b.tie_word_embeddings and b.rope_theta == 500000.0
    assert LlamaConfig.from_dict(a.to_dict()) == a and LlamaConfig.from_dict(b.to_dict()) == b


def test_head_dim_and_kv_heads_are_derived_when_absent():
    raw = dict(fixtures.TINY_A)
    del raw["head_dim"], raw["num_key_value_heads"]
    c = LlamaConfig.from_dict(raw)
    assert c.head_dim == 16 and c.num_key_value_heads == 4


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "max_position_embeddings", "rms_norm_eps", "rope_theta"])
def test_a_missing_size_is_an_error_that_names_the_key(key):
    raw = dict(fixtures.TINY_B)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(raw)


@pytest.mark.parametrize("change,match", [
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"), ({"num_key_value_heads": 3}, "multiple"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"vocab_size": "many"}, "vocab_size"), ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
])
def test_options_the_engine_cannot_honour_are_refused(change, match):
    raw = dict(fixtures.TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict(raw)


def test_registry_builds_the_model_by_name_and_rejects_unknown_names():
    assert "LlamaForCausalLM" in known_architectures()
    spec = spec_for(fixtures.TINY_B)
    assert len(spec.layers) == 3 and len(spec.run_order) == 3
    model = Model(spec)
    assert len(model.groups) == 1 and model.streams_per_group == [3]
    assert model.groups[0].num_kv_heads == 1 and model.groups[0].head_dim == 32
    with pytest.raises(ConfigError, match="NoSuchModel.*LlamaForCausalLM"):
        spec_for({"architectures": ["NoSuchModel"]})
    register_architecture("AliasForTest", lambda raw: spec_for(dict(raw, architectures=["LlamaForCausalLM"])))
    assert spec_for(dict(fixtures.TINY_A, architectures=["AliasForTest"])).vocab_size == 256


def test_safetensors_round_trip_against_the_library(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "empty": torch.zeros(0, 4)}
    safetensors_io.save_file(t, str(tmp_path / "mine.safetensors"))
    theirs = load_file(str(tmp_path / "mine.safetensors"))
    assert all(torch.equal(theirs[k], t[k]) for k in t)
    save_file(t, str(tmp_path / "theirs.safetensors"))
    f = safetensors_io.SafetensorsFile(str(tmp_path / "theirs.safetensors"))
    assert all(torch.equal(f.tensor(k), t[k]) for k in t)


def test_truncated_and_duplicate_files_are_errors(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    safetensors_io.save_file({"x": torch.ones(4, 4)}, str(d / "a.safetensors"))
    raw = (d / "a.safetensors").read_bytes()
    (d / "b.safetensors").write_bytes(raw)
    with pytest.raises(safetensors_io.SafetensorsError, match="both"):
        safetensors_io.open_folder(str(d))
    (d / "b.safetensors").write_bytes(raw[:-8])
    with pytest.raises(safetensors_io.SafetensorsError, match="truncated"):
        safetensors_io.open_folder(str(d))
    with pytest.raises(safetensors_io.SafetensorsError, match="no .safetensors"):
        safetensors_io.open_folder(str(tmp_path))


def _decls(cfg):
    return Model(spec_for(cfg)).tensors()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = fixtures.TINY_B
    w = fixtures.make_weights(cfg, 0)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["lm_head.weight"]                                  # untied: nothing stands in for it
    w["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(5, 5)
    w["model.layers.2.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)   # harmless, ignored
    w["model.layers.9.mlp.down_proj.weight"] = torch.zeros(2, 2)
    fixtures.write_model_folder(str(tmp_path), cfg, w)
    with pytest.raises(WeightsError) as e:
        FolderWeights(str(tmp_path), _decls(cfg), torch.float32, "cpu")
    text = str(e.value)
    assert "missing (2)" in text and "model.layers.1.mlp.up_proj.weight [328, 96]" in text and "lm_head.weight" in text
    assert "unexpected (1)" in text and "model.layers.9.mlp.down_proj.weight" in text
    assert "wrong shape (1)" in text and "the file has [5, 5], the model needs [96, 96]" in text
    assert "inv_freq" not in text


def test_kept_types_and_tied_head(tmp_path):
    cfg = fixtures.TINY_A
    w = fixtures.make_weights(cfg, 0, norm_std=0.1)
    fixtures.write_model_folder(str(tmp_path), cfg, w, torch.float32)
    src = FolderWeights(str(tmp_path), _decls(cfg), torch.bfloat16, "cpu")
    assert src.get("model.layers.0.mlp.down_proj.weight").dtype == torch.bfloat16
    norm = src.get("model.norm.weight")
    assert norm.dtype == torch.float32 and torch.equal(norm, w["model.norm.weight"])   # stored in 32 bits, stays so
    assert src.get("lm_head.weight") is src.get("model.embed_tokens.weight")           # an alias, not a copy
    src32 = FolderWeights(str(tmp_path), _decls(cfg), torch.float32, "cpu")
    assert torch.equal(src32.get("model.layers.1.self_attn.k_proj.weight"), w["model.layers.1.self_attn.k_proj.weight"])


def test_random_weights_mode_writes_a_folder_that_loads(tmp_path):
    for cfg in (fixtures.TINY_A, fixtures.TINY_B):
        d = str(tmp_path / str(cfg["hidden_size"]))
        write_random_model(d, cfg, seed=7, dtype=torch.bfloat16, norm_jitter=0.05)
        assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
        raw = json.load(open(os.path.join(d, "config.json")))
        assert LlamaConfig.from_dict(raw) == LlamaConfig.from_dict(dict(cfg, torch_dtype="bfloat16"))
        src = FolderWeights(d, _decls(raw), torch.bfloat16, "cpu")
        e = src.get("model.embed_tokens.weight")
        assert e.dtype == torch.bfloat16 and abs(float(e.float().std()) - 0.02) < 0.002
        assert ("lm_head.weight" in src.table) == (not cfg["tie_word_embeddings"])
        again = str(tmp_path / "again")
        write_random_model(again, cfg, seed=7, dtype=torch.bfloat16, norm_jitter=0.05)
        assert open(os.path.join(d, "model.safetensors"), "rb").read() == open(os.path.join(again, "model.safetensors"), "rb").read()
        # the plain implementation reads the same folder with the library's reader
        import plain_llama
        pcfg, pw = plain_llama.read_model_folder(d)
        assert plain_llama.plain_forward(pcfg, pw, [1, 2, 3]).shape == (3, cfg["vocab_size"])


def test_random_source_is_seeded():
    decls = _decls(fixtures.TINY_A)
    a = RandomWeights(decls, torch.float32, "cpu", 3)
    b = RandomWeights(decls, torch.float32, "cpu", 3)
    c = RandomWeights(decls, torch.float32, "cpu", 4)
    n = "model.layers.1.mlp.gate_proj.weight"
    assert torch.equal(a.get(n), b.get(n)) and not torch.equal(a.get(n), c.get(n))
