"""Generation through the Python entry point and the command line, against the
plain implementation; the scheduler's pre-emption with a real model; each part
of a layer alone."""
import os
import subprocess
import sys

import pytest
import torch

import fixtures
import plain_llama
from lyapunov_engine_b200 import EngineConfig, LLMEngine, SamplingParams, load_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg, seed in (("a", fixtures.TINY_A, 0), ("b", fixtures.TINY_B, 1)):
        w = fixtures.make_weights(cfg, seed, 0.05, 0.1, 4.0)
        d32 = fixtures.write_model_folder(str(tmp_path_factory.mktemp(name + "32")), cfg, w, torch.float32)
        d16 = fixtures.write_model_folder(str(tmp_path_factory.mktemp(name + "16")), cfg, w, torch.bfloat16)
        out[name] = (cfg, w, d32, d16)
    return out


@pytest.mark.parametrize("name,page", [("a", fixtures.TINY_A_PAGE), ("b", fixtures.TINY_B_PAGE)])
def test_greedy_generation_equals_the_plain_implementation(folders, name, page):
    cfg, w, d32, _ = folders[name]
    lens = (5, 17, 33) if name == "a" else (1, 8, 40, 97)
    steps = 16 if name == "a" else 24
    prompts = [fixtures.random_ids(cfg, n, 30 + n) for n in lens]
    # prompts are cut into portions of at most 16 tokens and run beside decoded tokens
    engine = LLMEngine.from_pretrained(d32, dtype="float32", num_blocks=64, block_size=page, max_num_seqs=4,
                                       max_num_batched_tokens=20, max_prefill_chunk=16)
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=steps, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.output_tokens == plain_llama.plain_greedy_generate(cfg, w, p, steps)
        assert o.finished and o.finish_reason == "length" and o.prompt_tokens == p
    st = engine.stats()
    assert st["graph_steps"] > 0 and st["free_blocks"] == 64 and engine.block_manager.audit() == ""


def test_generation_survives_preemption(folders):
    """So few pages that requests are pre-empted and recomputed: the tokens are
    the same as without pressure."""
    cfg, w, d32, _ = folders["a"]
    prompts = [fixtures.random_ids(cfg, n, 70 + n) for n in (9, 14, 11, 6)]
    engine = LLMEngine.from_pretrained(d32, dtype="float32", num_blocks=14, block_size=4, max_num_seqs=4,
                                       max_num_batched_tokens=32)
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.output_tokens == plain_llama.plain_greedy_generate(cfg, w, p, 20), o
    assert engine.stats()["preemptions"] > 0 and engine.block_manager.audit() == ""
    assert engine.block_manager.get_num_free_blocks() == 14


def test_end_of_sequence_stops_and_too_long_fails(folders):
    cfg, w, d32, _ = folders["b"]
    prompt = fixtures.random_ids(cfg, 12, 5)
    free_run = plain_llama.plain_greedy_generate(cfg, w, prompt, 12)
    raw = dict(cfg, eos_token_id=[free_run[4], 9999 % cfg["vocab_size"]])
    import json
    import shutil
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        shutil.copy(os.path.join(d32, "model.safetensors"), d)
        json.dump(raw, open(os.path.join(d, "config.json"), "w"))
        engine = LLMEngine.from_pretrained(d, dtype="float32", num_blocks=32, block_size=8, max_num_seqs=2,
                                           max_num_batched_tokens=64, max_model_len=40)
        o1, o2, o3 = engine.generate([prompt, prompt, fixtures.random_ids(cfg, 40, 6)],
                                     [SamplingParams(temperature=0.0, max_tokens=12),
                                      SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True),
                                      SamplingParams(temperature=0.0, max_tokens=4)])
    first_stop = free_run.index(free_run[4])
    assert o1.output_tokens == free_run[:first_stop + 1] and o1.finish_reason == "stop"
    assert o2.output_tokens == free_run and o2.finish_reason == "length"
    assert o3.finish_reason == "error" and "max_model_len" in o3.error


def test_temperature_sampling_is_seeded_and_batch_independent(folders):
    # float32: its logits are bit-for-bit independent of the batch, so the same
    # uniform number must pick the same token alone and among others
    cfg, w, d32, _ = folders["b"]
    prompts = [fixtures.random_ids(cfg, n, 90 + n) for n in (7, 23, 4)]
    sp = [SamplingParams(temperature=0.9, top_k=40, top_p=0.95, max_tokens=10, ignore_eos=True, seed=100 + i) for i in range(3)]
    engine = LLMEngine.from_pretrained(d32, dtype="float32", num_blocks=64, block_size=8, max_num_seqs=4,
                                       max_num_batched_tokens=64)
    together = [o.output_tokens for o in engine.generate(prompts, sp)]
    alone = [engine.generate([p], [s])[0].output_tokens for p, s in zip(prompts, sp)]
    assert together == alone
    other = engine.generate([prompts[0]], [SamplingParams(temperature=0.9, max_tokens=10, ignore_eos=True, seed=7)])
    assert other[0].output_tokens != together[0] and all(0 <= t < cfg["vocab_size"] for t in other[0].output_tokens)


@pytest.mark.parametrize("count", [3, 9, 11, 21])
def test_decode_graphs_of_partly_filled_buckets(folders, count):
    """Decode steps run as captured graphs of the next power-of-two batch; the
    rows between the live requests and the bucket are dummies.  With 9 to 12
    (or 17 to 28) live requests the list of wanted rows is longer than the
    live requests' own, and must not reach into the block tables behind it:
    every request's tokens equal the plain implementation's."""
    cfg, w, d32, _ = folders["a"]
    engine = LLMEngine.from_pretrained(d32, dtype="float32", num_blocks=count * 20, block_size=fixtures.TINY_A_PAGE,
                                       max_num_seqs=32, max_num_batched_tokens=256)
    prompts = [fixtures.random_ids(cfg, 21 + 2 * i, 700 + i) for i in range(count)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    assert engine.stats()["graph_steps"] >= 5
    for i in (0, 1, count - 1):
        assert outs[i].output_tokens == plain_llama.plain_greedy_generate(cfg, w, prompts[i], 10), i
    assert engine.block_manager.audit() == ""


def test_prompt_portions_as_graphs_of_fixed_shape(folders):
    """A step with one prompt portion (alone or beside decoded tokens) runs as a
    captured graph: the portion padded with dummy tokens to a multiple of 64,
    the decoded tokens with dummy requests.  The dummies write behind the
    request's own tokens and into the page nobody owns; every request's
    tokens equal the plain implementation's, with pages used again."""
    cfg, w, d32, _ = folders["b"]
    engine = LLMEngine.from_pretrained(d32, dtype="float32", num_blocks=48, block_size=fixtures.TINY_B_PAGE,
                                       max_num_seqs=4, max_num_batched_tokens=128, max_prefill_chunk=48)
    lens = (40, 97, 8, 61, 33, 70, 52, 19)
    prompts = [fixtures.random_ids(cfg, n, 900 + n) for n in lens]
    # a request arrives when the one before has had its whole prompt run, so a step holds one portion at most
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    done, nxt, calls = {}, 0, 0
    while nxt < len(prompts) or engine.has_unfinished_requests():
        waiting_for_prompt = any(seq.get_output_len() == 0 for seq, _, _ in engine.active_sequences.values())
        if nxt < len(prompts) and not waiting_for_prompt and len(engine.active_sequences) < 4:
            engine.add_request(str(nxt), prompts[nxt], sp)
            nxt += 1
        for o in engine.step():
            if o.finished:
                done[int(o.request_id)] = o
        calls += 1
        assert calls < 500
    outs = [done[i] for i in range(len(prompts))]
    graphs = engine.runner._prompt_graphs
    assert any(g.graph is not None for g in graphs.values()), "no prompt step was captured"
    assert any(key[1] > 0 for key in graphs), "no mixed step went through a graph"
    for p, o in zip(prompts, outs):
        assert o.output_tokens == plain_llama.plain_greedy_generate(cfg, w, p, 12)
    assert engine.block_manager.audit() == "" and engine.stats()["free_blocks"] == 48


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_give_the_same_tokens(folders, dtype):
    """The engine launches a decode step before it has read the tokens of the
    step before (they pass on the device).  Same tokens, finish reasons and
    number of step() calls as without; a request that stops at an
    end-of-sequence token, one that arrives while others decode, one that is
    aborted, greedy and seeded sampling."""
    cfg, w, d32, d16 = folders["b"]
    folder = d32 if dtype == "float32" else d16
    prompts = [fixtures.random_ids(cfg, n, 300 + n) for n in (9, 17, 5, 12)]
    free_run = plain_llama.plain_greedy_generate(cfg, w, prompts[0], 14)
    raw = dict(cfg, eos_token_id=[free_run[6]])
    import json
    import shutil
    import tempfile
    runs = []
    with tempfile.TemporaryDirectory() as d:
        shutil.copy(os.path.join(folder, "model.safetensors"), d)
        json.dump(raw, open(os.path.join(d, "config.json"), "w"))
        for ahead in (False, True):
            engine = LLMEngine.from_pretrained(d, dtype=dtype, num_blocks=64, block_size=8, max_num_seqs=4,
                                               max_num_batched_tokens=32, lookahead=ahead)
            engine.add_request("stops", prompts[0], SamplingParams(temperature=0.0, max_tokens=14))
            engine.add_request("sampled", prompts[1], SamplingParams(temperature=0.8, top_p=0.9, max_tokens=20, ignore_eos=True, seed=5))
            engine.add_request("aborted", prompts[2], SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True))
            done, calls = {}, 0
            while engine.has_unfinished_requests():
                calls += 1
                if calls == 6:
                    engine.add_request("late", prompts[3], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
                if calls == 9:
                    engine.abort_request("aborted")
                for o in engine.step():
                    if o.finished:
                        done[o.request_id] = (o.output_tokens, o.finish_reason)
                assert calls < 200
            assert engine.block_manager.audit() == "" and engine.block_manager.get_num_free_blocks() == 64
            runs.append((done, calls, engine.stats()["steps_ahead"]))
    assert runs[0][0] == runs[1][0] and runs[0][1] == runs[1][1]
    assert runs[0][2] == 0 and runs[1][2] >= 10
    done = runs[1][0]
    if dtype == "float32":
        assert done["stops"] == (free_run[:free_run.index(free_run[6]) + 1], "stop")
    assert len(done["sampled"][0]) == 20 and len(done["late"][0]) == 8 and done["late"][1] == "length"


@pytest.mark.parametrize("seed", [0, 2, 3, 8])
def test_random_traffic_with_and_without_steps_ahead(folders, seed):
    """Random arrivals, lengths, sampling options, end-of-sequence tokens,
    aborts and page pools small enough to pre-empt: the same tokens and finish
    reasons with every step launched kernel by kernel and read before the next
    is scheduled, and with steps captured as graphs of padded shape and
    launched ahead.  float32, whose logits do not depend on what else is in a
    batch, so every token must agree."""
    import json
    import random
    import shutil
    import tempfile
    cfg, w, d32, _ = folders["b"]
    results = []
    with tempfile.TemporaryDirectory() as d:
        shutil.copy(os.path.join(d32, "model.safetensors"), d)
        json.dump(dict(cfg, eos_token_id=[3, 4, 77, 120, 301]), open(os.path.join(d, "config.json"), "w"))
        for ahead in (False, True):
            rng = random.Random(seed)
            engine = LLMEngine.from_pretrained(d, dtype="float32", num_blocks=rng.choice([12, 20, 48]), block_size=8, max_num_seqs=4,
                                               max_num_batched_tokens=rng.choice([16, 48]), lookahead=ahead, max_model_len=160,
                                               use_cuda_graphs=ahead)
            plan = [(rng.randint(0, 60), f"r{i}", fixtures.random_ids(cfg, rng.randint(1, 40), seed * 100 + i),
                     SamplingParams(temperature=rng.choice([0.0, 0.0, 0.7]), top_p=rng.choice([1.0, 0.9]), top_k=rng.choice([-1, 20]),
                                    max_tokens=rng.randint(1, 30), ignore_eos=rng.random() < 0.3, seed=i)) for i in range(14)]
            aborts = {rng.randint(5, 70): f"r{rng.randint(0, 13)}" for _ in range(3)}
            done, call = {}, 0
            while call < 2000 and (call <= 70 or engine.has_unfinished_requests()):
                call += 1
                for when, rid, prompt, sp in plan:
                    if when == call:
                        engine.add_request(rid, prompt, sp)
                if call in aborts:
                    engine.abort_request(aborts[call])
                for o in engine.step():
                    if o.finished:
                        done[o.request_id] = (tuple(o.output_tokens), o.finish_reason)
            assert engine.block_manager.audit() == "" and not engine.has_unfinished_requests()
            results.append((done, engine.stats()))
    assert results[0][0] == results[1][0] and len(results[0][0]) >= 11
    assert results[0][1]["steps_ahead"] == 0 and results[1][1]["steps_ahead"] > 0
    assert results[0][1]["graph_steps"] == 0 and results[1][1]["graph_steps"] > 0
    assert results[0][1]["preemptions"] == results[1][1]["preemptions"]


def test_command_line(folders):
    cfg, w, d32, _ = folders["a"]
    prompt = fixtures.random_ids(cfg, 9, 3)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "lyapunov"), "generate", "--model", d32, "--prompt-ids",
           ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0", "--dtype", "float32",
           "--block-size", "4", "--num-blocks", "32", "--max-num-seqs", "2", "--max-batched-tokens", "64", "--ignore-eos"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    last = out.stdout.strip().split("\n")[-1]
    assert [int(t) for t in last.split()] == plain_llama.plain_greedy_generate(cfg, w, prompt, 6)


def test_text_prompts_through_the_folders_tokenizer(folders, tmp_path):
    """generate() with strings: encoded by the tokenizer found in the model's
    folder (a word-level one, made here), outputs decoded into ``text``; the
    command line's --prompt goes the same way."""
    import json
    import shutil
    tokenizers = pytest.importorskip("tokenizers")
    pytest.importorskip("transformers")
    cfg, w, d32, _ = folders["a"]
    folder = str(tmp_path / "with_tokenizer")
    shutil.copytree(d32, folder)
    vocab = {f"w{i}": i for i in range(cfg["vocab_size"] - 1)}
    vocab["[UNK]"] = cfg["vocab_size"] - 1
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    tok.save(os.path.join(folder, "tokenizer.json"))
    with open(os.path.join(folder, "tokenizer_config.json"), "w", encoding="utf-8") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "[UNK]"}, f)
    ids = fixtures.random_ids(cfg, 11, 8)
    text = " ".join(f"w{i}" for i in ids)
    engine = LLMEngine.from_pretrained(folder, dtype="float32", num_blocks=32, block_size=4, max_num_seqs=2,
                                       max_num_batched_tokens=64)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    by_text = engine.generate([text], sp)[0]
    want = plain_llama.plain_greedy_generate(cfg, w, ids, 6)
    assert by_text.prompt_tokens == ids and by_text.output_tokens == want
    # (the unknown-word token is a special token, which decoding leaves out)
    assert by_text.text == " ".join(f"w{i}" for i in want if i < cfg["vocab_size"] - 1)
    assert engine.generate([ids], sp)[0].text is None
    cmd = [sys.executable, os.path.join(ROOT, "bin", "lyapunov"), "generate", "--model", folder, "--prompt", text,
           "--max-tokens", "6", "--temperature", "0", "--dtype", "float32", "--block-size", "4", "--num-blocks", "32",
           "--max-num-seqs", "2", "--max-batched-tokens", "64", "--ignore-eos"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip().split("\n")[-1] == by_text.text
    # a model without a folder has no tokenizer to offer
    loaded = load_model(config=cfg, random_seed=1, dtype="float32", device="cuda:0")
    bare = LLMEngine(loaded, EngineConfig(num_blocks=16, block_size=4, max_num_seqs=2, max_num_batched_tokens=32,
                                          dtype="float32", device="cuda:0"))
    with pytest.raises(ValueError, match="tokenizer"):
        bare.generate(["w1 w2"], sp)


def test_command_line_with_random_weights(folders, tmp_path):
    """generate --random-weights: --model names a config.json (or a folder that
    holds one); the weights are those that load_model draws from the seed."""
    import json
    cfg, _, _, _ = folders["b"]
    path = str(tmp_path / "config.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    prompt = fixtures.random_ids(cfg, 7, 5)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "lyapunov"), "generate", "--model", path, "--random-weights", "--seed", "3",
           "--prompt-ids", " ".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0", "--dtype", "float32",
           "--block-size", "8", "--num-blocks", "16", "--max-num-seqs", "2", "--max-batched-tokens", "64", "--ignore-eos"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    got = [int(t) for t in out.stdout.strip().split("\n")[-1].split()]
    loaded = load_model(config=cfg, random_seed=3, dtype="float32", device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(num_blocks=16, block_size=8, max_num_seqs=2, max_num_batched_tokens=64,
                                            dtype="float32", device="cuda:0"))
    want = engine.generate([prompt], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))[0].output_tokens
    assert got == want and len(got) == 5


def test_step_timers(folders):
    """With step timers on, every step's device time is recorded by kind."""
    cfg, _, d32, _ = folders["a"]
    engine = LLMEngine.from_pretrained(d32, dtype="float32", num_blocks=64, block_size=4, max_num_seqs=4,
                                       max_num_batched_tokens=20)
    engine.runner.enable_step_timers()
    engine.generate([fixtures.random_ids(cfg, n, n) for n in (30, 7)], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    timings = engine.runner.step_timings()
    assert len(timings) == engine.runner.num_steps and all(t["ms"] > 0 for t in timings)
    assert {t["kind"] for t in timings} >= {"decode", "prompt"} and sum(t["tokens"] for t in timings) >= 37 + 2 * 5
    summary = engine.stats()["step_ms"]
    assert summary["decode"]["steps"] > 0 and summary["decode"]["mean"] <= summary["decode"]["max"]


def test_warm_up_captures_the_decode_graphs_ahead(folders):
    """After warm_up() a decode step of any batch and context it covered replays
    a captured graph at its first use."""
    cfg, w, d32, _ = folders["a"]
    engine = LLMEngine.from_pretrained(d32, dtype="float32", num_blocks=64, block_size=4, max_num_seqs=4,
                                       max_num_batched_tokens=32, max_model_len=128)
    captured = engine.warm_up()
    runner = engine.runner
    assert captured == len(runner._graphs) > 0 and all(g.graph is not None for g in runner._graphs.values())
    assert engine.block_manager.audit() == "" and engine.block_manager.get_num_free_blocks() == 64
    before = runner.num_captures
    prompts = [fixtures.random_ids(cfg, n, 50 + n) for n in (5, 17, 33)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.output_tokens == plain_llama.plain_greedy_generate(cfg, w, p, 10)
    decode_captures = sum(g.graph is not None for g in runner._graphs.values())
    assert decode_captures == captured, "a decode step needed a graph that warm_up had not captured"
    assert runner.num_captures - before == sum(g.graph is not None for g in runner._prompt_graphs.values())


def test_no_cpu_path():
    from lyapunov_engine_b200 import ops
    with pytest.raises(ops.KernelError, match="CUDA"):
        ops.swiglu(torch.zeros(2, 4), torch.zeros(2, 8))
    with pytest.raises(ops.KernelError, match="CPU"):
        load_model(config=fixtures.TINY_A, random_seed=0, dtype="float32", device="cpu")


# ---- each part of a layer alone, against its plain function
class _Ctx:
    pass


def _runtime(dtype):
    from lyapunov_engine_b200.engine.runtime import Runtime
    return Runtime("cuda:0", dtype, max_model_len=64)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parts_alone(dtype):
    from lyapunov_engine_b200.parts import FEED_FORWARDS, NORMS, POSITION_ENCODINGS, PartSpec
    rt = _runtime(dtype)
    g = torch.Generator().manual_seed(0)
    Hh, Ii, T = 72, 200, 11
    tensors = {"n": 1 + 0.1 * torch.randn(Hh, generator=g), "g": torch.randn(Ii, Hh, generator=g) * 0.1,
               "u": torch.randn(Ii, Hh, generator=g) * 0.1, "d": torch.randn(Hh, Ii, generator=g) * 0.1}

    def get(name):
        t = tensors[name]
        return t.to("cuda:0", torch.float32 if name == "n" else dtype)
    ctx = _Ctx()
    ctx.workspace = rt.workspace
    ctx.status = rt.status
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    rounded = {k: (v if k == "n" else v.to(dtype).float()) for k, v in tensors.items()}

    norm = NORMS.build(PartSpec("rmsnorm", {"hidden_size": Hh, "eps": 1e-6, "weight_name": "n"}))
    assert [d.name for d in norm.tensors()] == ["n"] and norm.tensors()[0].role == "vector"
    norm.bind(get, rt)
    resid = torch.randn(T, Hh, generator=g)
    delta = torch.randn(T, Hh, generator=g).to(dtype)
    r = resid.to("cuda:0")
    out = norm.apply(r, delta.to("cuda:0"))
    torch.testing.assert_close(out.float().cpu(), plain_llama.plain_rmsnorm(resid + delta.float(), tensors["n"], 1e-6), **tol)

    ff = FEED_FORWARDS.build(PartSpec("gated_silu", {"hidden_size": Hh, "intermediate_size": Ii, "gate_name": "g",
                                                     "up_name": "u", "down_name": "d"}))
    assert [d.shape for d in ff.tensors()] == [(Ii, Hh), (Ii, Hh), (Hh, Ii)]
    ff.bind(get, rt)
    x = torch.randn(T, Hh, generator=g).to(dtype)
    y = ff.forward(x.to("cuda:0"), ctx)
    if y.dim() == 3:          # float32 partial sums of a split-K product, for the next norm to add up
        assert y.dtype == torch.float32
        y = y.sum(0)
    want = plain_llama.plain_mlp(x.float(), rounded["g"], rounded["u"], rounded["d"], act_dtype=None if dtype == torch.float32 else dtype)
    torch.testing.assert_close(y.float().cpu(), want, **tol)

    scaling = dict(fixtures.TINY_B["rope_scaling"])
    rope = POSITION_ENCODINGS.build(PartSpec("rotary", {"head_dim": 32, "theta": 500000.0, "max_positions": 64, "scaling": scaling}))
    table = rope.build_table(64)
    inv = plain_llama.plain_inv_freq(32, 500000.0, scaling)
    cos, sin = plain_llama.plain_cos_sin(torch.arange(64), inv)
    assert torch.equal(table[:, :16], cos[:, :16]) and torch.equal(table[:, 16:], sin[:, :16])
