"""The engine at the layer sizes of the real models (Llama-3.2-1B: width 2048,
32 heads in 8 groups, head 64, feed-forward 8192; Llama-3.2-3B: width 3072, 24
heads in 8 groups, head 128), with few layers and a smaller vocabulary so that
the plain implementation can follow on the CPU.  Replay in every cut, bfloat16
and float32, against the plain implementation; and the schedules that only
these sizes reach: prompt portions run as padded graphs of fixed shape on the
tcgen05 kernels (alone and beside decoded tokens), decode batches of 24 and 64
rows on the library's and the tcgen05 products, and greedy generation through
the entry point in bfloat16."""
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
# for the schedules below: the same layers under a small vocabulary (no power of two), since the plain
# implementation computes every place's logits
SMALL_VOCAB = {"1b_layers": config(2048, 32, 8, 64, 8192, 4040, 2, True),
               "3b_layers": config(3072, 24, 8, 128, 8192, 3032, 1, False)}


def make(cfg, tmp_path_factory, name, dtypes=(torch.bfloat16, torch.float32)):
    w = fixtures.make_weights(cfg, seed=11, std=0.02, norm_std=0.05, qk_gain=2.0)
    folders = {}
    for dtype in dtypes:
        d = str(tmp_path_factory.mktemp(name + ("16" if dtype == torch.bfloat16 else "32")))
        fixtures.write_model_folder(d, cfg, w, dtype)
        folders[dtype] = d
    return w, folders


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    cfg, lengths = CONFIGS[request.param]
    w, folders = make(cfg, tmp_path_factory, request.param)
    requests = {f"r{i}": fixtures.random_ids(cfg, n, 900 + i) for i, n in enumerate(lengths)}
    ref32 = {r: plain_llama.plain_forward(cfg, w, ids) for r, ids in requests.items()}
    # the noise is measured on the shorter requests (64-bit sums over the longest take the CPU too long)
    short = dict(sorted(requests.items(), key=lambda kv: len(kv[1]))[:2])
    ref16, noise = ru.bf16_references(cfg, w, short, plain_llama.plain_forward)
    rounded = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    for r, ids in requests.items():
        if r not in ref16:
            ref16[r] = plain_llama.plain_forward(cfg, rounded, ids, act_dtype=torch.bfloat16, prob_dtype=torch.bfloat16)
    return dict(cfg=cfg, folders=folders, requests=requests, ref={"float32": ref32, "bfloat16": ref16}, noise=noise,
                prompt_lens={r: max(1, len(ids) - 40) for r, ids in requests.items()})


def check(m, trace, dtype, tmp_path, live, what, extra=(), pool=None):
    folder = m["folders"][torch.float32 if dtype == "float32" else torch.bfloat16]
    if pool is None:
        lens = sorted((len(v) for v in m["requests"].values()), reverse=True)[:live]
        pool = sum((n + 63) // 64 * 64 for n in lens)
    got = ru.run_trace(trace, folder, dtype, str(tmp_path), pool, 16, extra=extra)
    assert len(got) == sum(len(w) for w in trace.wanted)
    if dtype == "float32":
        return ru.compare(got, m["ref"][dtype], atol=2e-4, rtol=2e-4, what=what)
    return ru.compare_bf16(got, m["ref"][dtype], m["noise"], what)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_whole_then_tail(model, dtype, tmp_path):
    check(model, ru.tail_trace(model["requests"], 32), dtype, tmp_path, 1, f"scale {dtype} tail")


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_portions_and_mixed(model, dtype, tmp_path):
    check(model, ru.portions_trace(model["requests"], sizes=(130, 2, 257, 64, 3, 129, 17)), dtype, tmp_path / "p", 1,
          f"scale {dtype} portions")
    trace = ru.mixed_trace(model["requests"], model["prompt_lens"], chunk=200, max_live=4, seed=1)
    check(model, trace, dtype, tmp_path / "m", 4, f"scale {dtype} mixed")


# ---------------------------------------------------------------- schedules of the real sizes
@pytest.fixture(scope="module", params=sorted(SMALL_VOCAB))
def small(request, tmp_path_factory):
    cfg = SMALL_VOCAB[request.param]
    w, folders = make(cfg, tmp_path_factory, request.param + "s", dtypes=(torch.bfloat16,))
    return dict(name=request.param, cfg=cfg, w=w, folders=folders)


def with_references(small, requests, noise_from):
    ref, noise = ru.bf16_references(small["cfg"], small["w"], {r: requests[r] for r in noise_from}, plain_llama.plain_forward)
    rounded = {k: v.to(torch.bfloat16).float() for k, v in small["w"].items()}
    for r, ids in requests.items():
        if r not in ref:
            ref[r] = plain_llama.plain_forward(small["cfg"], rounded, ids, act_dtype=torch.bfloat16, prob_dtype=torch.bfloat16)
    return dict(small, requests=requests, ref={"bfloat16": ref}, noise=noise)


PORTIONS = (130, 65, 257, 1000)          # none a multiple of 64: padded to 192, 128, 320 and 1024 rows


def test_prompt_portions_as_padded_graphs(small, tmp_path):
    """Prompt portions that ask for one row each run as captured graphs of fixed
    shape: dummy tokens behind the portion, dummy requests beside the decoded
    tokens, on the tcgen05 attention and products.  Every shape occurs twice
    (two prompts cut alike), so its second use is the captured graph; alone,
    beside 3 and beside 20 decoded tokens."""
    cfg = small["cfg"]
    total = sum(PORTIONS)
    decoders = {f"d{i}": fixtures.random_ids(cfg, 24 + 16, 300 + i) for i in range(20)}
    prompts = {f"p{k}{j}": fixtures.random_ids(cfg, total, 400 + 2 * k + j) for k in range(3) for j in range(2)}
    m = with_references(small, {**decoders, **prompts}, noise_from=("d0", "d1", "d2", "d3"))
    t = ru.Trace()
    for rid, ids in decoders.items():                      # their prompts, whole
        t.step([(rid, ids[:24], [23])])
    done = {rid: 24 for rid in decoders}
    for k, beside in enumerate((0, 3, 20)):
        for j in range(2):
            rid, pos = f"p{k}{j}", 0
            for n in PORTIONS:
                entries = [(rid, prompts[rid][pos:pos + n], [n - 1])]
                for d in list(decoders)[:beside]:
                    if done[d] < len(decoders[d]):
                        entries.append((d, decoders[d][done[d]:done[d] + 1], [0]))
                        done[d] += 1
                pos += n
                t.step(entries, end=[rid] if pos == total else [])
    t.step([], end=list(decoders))
    pool = 20 * 64 + 2 * ((total + 63) // 64 * 64)
    check(m, t, "bfloat16", tmp_path, 0, f"{small['name']} padded prompt graphs", extra=("--max-num-seqs", "32"), pool=pool)
    pages = ru.read_pages(str(tmp_path))
    # 3 x 4 shapes, each captured at its second use and replayed for it
    assert pages["prompt_graphs_captured"] >= 12 and pages["graph_steps"] >= 24, pages


@pytest.mark.parametrize("batch", [24, 64])
def test_decode_batches_beyond_the_weight_streaming_kernels(small, batch, tmp_path):
    """Decode steps of 24 and 64 rows: more rows than the weight-streaming
    products take, so the library's products and the tcgen05 gated product run
    them, as graphs of 32 and 64 rows."""
    cfg = small["cfg"]
    lengths = [9 + (7 * i) % 41 for i in range(batch)]
    steps = 5
    requests = {f"q{i}": fixtures.random_ids(cfg, n + steps, 700 + i) for i, n in enumerate(lengths)}
    m = with_references(small, requests, noise_from=("q0", "q1", "q2", "q3", "q4", "q5"))
    t = ru.Trace()
    names = list(requests)
    for at in range(0, batch, 8):                           # prompts, eight to a step
        t.step([(r, requests[r][:lengths[names.index(r)]], [lengths[names.index(r)] - 1]) for r in names[at:at + 8]])
    for s in range(steps):
        t.step([(r, requests[r][n + s:n + s + 1], [0]) for r, n in zip(names, lengths)],
               end=names if s == steps - 1 else [])
    check(m, t, "bfloat16", tmp_path, 0, f"{small['name']} decode batch {batch}", extra=("--max-num-seqs", "64"),
          pool=batch * 64)
    pages = ru.read_pages(str(tmp_path))
    assert pages["graph_steps"] >= steps, pages


def test_partly_filled_decode_steps_have_graphs_of_their_own(small, tmp_path):
    """Five and then three requests decode in steps captured for eight and for
    four rows, at contexts beyond 1,024 keys: the attention kernel cuts the keys
    of five real requests into more splits than those of eight (the dummy
    requests that pad the step finish at once), so these steps get a graph of
    their own beside the full step's, and their logits are the plain
    implementation's all the same."""
    cfg = small["cfg"]
    lengths = [1030 + 9 * i for i in range(5)]
    steps = 6
    requests = {f"f{i}": fixtures.random_ids(cfg, n + steps, 760 + i) for i, n in enumerate(lengths)}
    m = with_references(small, requests, noise_from=("f0", "f1"))
    t = ru.Trace()
    names = list(requests)
    for r, n in zip(names, lengths):
        t.step([(r, requests[r][:n], [n - 1])])
    for s in range(steps):
        live = names if s < 3 else names[:3]                 # two requests end half-way
        t.step([(r, requests[r][n + s:n + s + 1], [0]) for r, n in zip(names, lengths) if r in live],
               end=names[3:] if s == 2 else (names[:3] if s == steps - 1 else []))
    pool = sum((n + steps + 63) // 64 * 64 for n in lengths)
    check(m, t, "bfloat16", tmp_path, 0, f"{small['name']} partly filled decode steps", extra=("--max-num-seqs", "8"), pool=pool)
    pages = ru.read_pages(str(tmp_path))
    shapes = pages["decode_graph_shapes"]
    assert {rows for rows, _, _ in shapes} == {4, 8}, shapes
    from lyapunov_engine_b200.parts.attention_kernels import decode_splits
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    apart = 0
    for rows, fill in ((8, 5), (4, 3)):
        width = next(w for r, w, _ in shapes if r == rows)
        want = decode_splits(fill, nh, nkv, width * 16, hd)
        apart += want != decode_splits(rows, nh, nkv, width * 16, hd)
        assert [rows, width, [want]] in shapes, shapes
    assert apart, "the test's sizes no longer tell a partly filled step from a full one"


def test_greedy_generation_in_bfloat16(small, tmp_path):
    """Through LLMEngine.generate: every token the engine chose must be a
    maximum of the plain implementation's logits at its place, given the same
    tokens before it, up to the rounding noise of bfloat16 (a logit tolerance,
    not a vote over tokens)."""
    from lyapunov_engine_b200 import EngineConfig, LLMEngine, SamplingParams, load_model

    cfg = small["cfg"]
    prompts = [fixtures.random_ids(cfg, n, 800 + n) for n in (3, 40, 150, 21, 260)]
    steps = 24
    loaded = load_model(small["folders"][torch.bfloat16], "bfloat16", "cuda:0", max_model_len=512)
    engine = LLMEngine(loaded, EngineConfig(num_blocks=96, block_size=16, max_num_seqs=4, max_num_batched_tokens=128,
                                            dtype="bfloat16", device="cuda:0", max_model_len=512))
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=steps, ignore_eos=True))
    assert engine.block_manager.audit() == ""
    stats = engine.stats()
    assert stats["graph_steps"] > 0 and stats["steps_ahead"] > 0, stats
    sequences = {f"g{i}": p + o.output_tokens for i, (p, o) in enumerate(zip(prompts, outs))}
    m = with_references(small, sequences, noise_from=("g0", "g3"))
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o.output_tokens) == steps
        logits = m["ref"]["bfloat16"][f"g{i}"]
        for s, tok in enumerate(o.output_tokens):
            row = logits[len(p) + s - 1]
            lead = float(row.max() - row[tok])
            assert lead <= 2 * ru.BF16_MAX_ABS * m["noise"]["max"], \
                (f"prompt {i}, token {s}: the engine chose {tok}, whose plain logit lies {lead:.4f} under the maximum "
                 f"({int(row.argmax())}); rounding explains {2 * ru.BF16_MAX_ABS * m['noise']['max']:.4f}")
