"""Replay through bin/trace_run's program against the plain implementation:
each request whole; the last 32 tokens one by one; portions of changing size;
mixed batches with so few pages that they are used again.  In float32 and in
bfloat16, on tiny configurations that differ in every size and option."""
import os

import pytest
import torch

import fixtures
import plain_llama
import replay_util as ru

pytestmark = pytest.mark.gpu

# name: (config, page, weight seed, std, norm_std, qk_gain)
MODELS = {
    "tiny_a": (fixtures.TINY_A, fixtures.TINY_A_PAGE, 0, 0.05, 0.0, 4.0),
    "tiny_b": (fixtures.TINY_B, fixtures.TINY_B_PAGE, 1, 0.05, 0.1, 3.0),
    "tiny_c": (fixtures.TINY_C, fixtures.TINY_C_PAGE, 2, 0.04, 0.1, 3.0),
    # the stated tiny-B: N(0, 0.02) matrices, norm weights 1 + N(0, 0.1), seed 1, prompts of 1/8/40/97 tokens and
    # 24 decoded tokens each, portions of at most 16 beside decoded tokens, pages of 8
    "tiny_b_stated": (fixtures.TINY_B_STATED, fixtures.TINY_B_PAGE, 1, 0.02, 0.1, 1.0),
    "tiny_d": (fixtures.TINY_D, fixtures.TINY_D_PAGE, 4, 0.04, 0.1, 3.0),
}
LENGTHS = {"tiny_a": (21, 33, 49, 70), "tiny_b": (25, 32, 64, 121), "tiny_c": (40, 65, 130, 300),
           "tiny_b_stated": (25, 32, 64, 121), "tiny_d": (19, 50, 97, 180)}
PROMPTS = {"tiny_a": (5, 17, 33, 38), "tiny_b": (1, 8, 40, 97), "tiny_c": (8, 33, 98, 268),
           "tiny_b_stated": (1, 8, 40, 97), "tiny_d": (3, 18, 65, 148)}

# float32: different summation orders of the same 32-bit arithmetic.
F32_TOL = dict(atol=1e-4, rtol=1e-4)
# bfloat16: the plain implementation rounds its activations to bfloat16 where the
# pipeline stores them (plain_llama.rounded), the softmax numerators included
# (the tensor cores take them as bfloat16).  What is left is which way
# roundings fall: the order of accumulation inside the products, and which
# maximum the numerators were scaled by when they were rounded.  That noise is
# measured, not guessed (replay_util.bf16_references), and the engine's
# distance from the plain implementation is bounded in units of it
# (replay_util.compare_bf16).


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, page, seed, std, norm_std, gain) in MODELS.items():
        w = fixtures.make_weights(cfg, seed, std, norm_std, gain)
        folders = {}
        for dtype in (torch.float32, torch.bfloat16):
            d = str(tmp_path_factory.mktemp(f"{name}_{'f32' if dtype == torch.float32 else 'bf16'}"))
            fixtures.write_model_folder(d, cfg, w, dtype)
            folders[dtype] = d
        requests = {f"r{i}": fixtures.random_ids(cfg, n, 100 + i) for i, n in enumerate(LENGTHS[name])}
        prompt_lens = {f"r{i}": n for i, n in enumerate(PROMPTS[name])}
        ref32 = {r: plain_llama.plain_forward(cfg, w, ids) for r, ids in requests.items()}
        ref16, noise = ru.bf16_references(cfg, w, requests, plain_llama.plain_forward)
        out[name] = dict(cfg=cfg, page=page, folders=folders, requests=requests, prompt_lens=prompt_lens,
                         ref={"float32": ref32, "bfloat16": ref16}, noise=noise)
    return out


def pool_tokens(m, live):
    """Room for the `live` longest requests at once, each rounded up to 64."""
    lens = sorted((len(v) for v in m["requests"].values()), reverse=True)[:live]
    return sum((n + 63) // 64 * 64 for n in lens)


def check(m, trace, dtype, tmp_path, live, what, child=False, pool=None):
    folder = m["folders"][torch.float32 if dtype == "float32" else torch.bfloat16]
    got = ru.run_trace(trace, folder, dtype, str(tmp_path), pool or pool_tokens(m, live), m["page"], child=child)
    ref = m["ref"][dtype]
    expected = sum(len(w) for w in trace.wanted)
    assert len(got) == expected
    if dtype == "float32":
        return ru.compare(got, ref, what=what, **F32_TOL)
    return ru.compare_bf16(got, ref, m["noise"], what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MODELS))
def test_whole(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.whole_trace(m["requests"]), dtype, tmp_path, 1, f"{name} {dtype} whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MODELS))
def test_last_32_one_by_one(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.tail_trace(m["requests"], 32), dtype, tmp_path, 1, f"{name} {dtype} tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MODELS))
def test_portions(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.portions_trace(m["requests"]), dtype, tmp_path, 1, f"{name} {dtype} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MODELS))
def test_mixed_with_page_reuse(models, name, dtype, tmp_path):
    m = models[name]
    # twice the requests, so that those that start late get pages others gave back
    cfg = m["cfg"]
    requests = dict(m["requests"])
    prompt_lens = dict(m["prompt_lens"])
    ref = dict(m["ref"][dtype])
    weights = None
    for i, (rid, ids) in enumerate(list(m["requests"].items())):
        more = fixtures.random_ids(cfg, len(ids), 500 + i)
        requests[rid + "x"] = more
        prompt_lens[rid + "x"] = m["prompt_lens"][rid]
    if weights is None:
        _, _, seed, std, norm_std, gain = MODELS[name]
        weights = fixtures.make_weights(cfg, seed, std, norm_std, gain)
        if dtype == "bfloat16":
            weights = {k: v.to(torch.bfloat16).float() for k, v in weights.items()}
    for rid, ids in requests.items():
        if rid not in ref:
            low = torch.bfloat16 if dtype == "bfloat16" else None
            ref[rid] = plain_llama.plain_forward(cfg, weights, ids, act_dtype=low, prob_dtype=low)
    m2 = dict(m, requests=requests, prompt_lens=prompt_lens, ref={dtype: ref})
    trace = ru.mixed_trace(requests, prompt_lens, chunk=16, max_live=4, seed=3)
    assert any(len(s["entries"]) >= 3 for s in trace.steps)
    assert any(len(e["tokens"]) == 1 for s in trace.steps for e in s["entries"]) and \
        any(len(e["tokens"]) > 1 for s in trace.steps for e in s["entries"])
    # a pool that just holds the trace's peak, so that requests that start late get pages that others gave back
    check(m2, trace, dtype, tmp_path, 4, f"{name} {dtype} mixed", pool=ru.peak_pool_tokens(trace, m["page"]))
    pages = ru.read_pages(str(tmp_path))
    assert pages["allocations"] > pages["pool_pages"] and pages["reuses"] > 0, pages
    assert pages["pool_pages"] - 64 // m["page"] < pages["peak_used_pages"] <= pages["pool_pages"], pages


def test_child_process_as_a_user_runs_it(models, tmp_path):
    m = models["tiny_b"]
    check(m, ru.portions_trace(m["requests"]), "float32", tmp_path, 1, "tiny_b child", child=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(models, dtype, tmp_path):
    """Every token one by one from the very first (a sequence's first tokens,
    then long decoding across many pages)."""
    m = models["tiny_c"]
    ids = m["requests"]["r3"]
    t = ru.Trace()
    for i, tok in enumerate(ids):
        t.step([("r3", [tok], [0])], end=["r3"] if i == len(ids) - 1 else [])
    m1 = dict(m, requests={"r3": ids})
    check(m1, t, dtype, tmp_path, 1, f"tiny_c {dtype} one by one")
