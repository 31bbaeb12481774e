"""Benchmark: decode tokens a second of the engine on Llama-3.2-1B shapes
(random weights, synthetic tokens), one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A step is one decode step of a batch of 8 requests at context 4096.  `value`
times K steps on the device (CUDA events) through the step function and the
sampler; `e2e` times the same through the Python entry point
(LLMEngine.step(): host tokens in, host tokens out).  The line also carries a
2,048-token prefill, decode at batch 1 and 64, and the decode step's HBM
roofline.  Every step reads all weights (2.5 GB) and the live cache, far more
than the 126 MB L2, so nothing is served from cache between timed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048,
    "intermediate_size": 8192, "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
    "bos_token_id": 128000, "eos_token_id": 128001, "torch_dtype": "bfloat16",
}
# The same architecture at the sizes of Llama-3.2-3B and Llama-3.1-8B, for --only runs at further sizes.
LLAMA_3B = dict(LLAMA_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, head_dim=128)
LLAMA_8B = dict(LLAMA_1B, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, head_dim=128,
                tie_word_embeddings=False,
                rope_scaling=dict(LLAMA_1B["rope_scaling"], factor=8.0))
SHAPES = {"1b": LLAMA_1B, "3b": LLAMA_3B, "8b": LLAMA_8B}
CONTEXT = 4096
PREFILL_TOKENS = 2048
BLOCK_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(path) as f:
            raw = json.load(f)
        for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if key in raw and isinstance(raw[key], (int, float)):
                out[key] = float(raw[key])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def mark(self):
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, begin=0, end=None):
        rows = [r for r in self.rows[begin:end] if len(r) >= 7]
        if not rows:
            rows = [r for r in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(int(float(r[0])) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(float(rows[0][1])), "reasons": reasons,
                "samples": len(rows), "power_w": max(float(r[2]) for r in rows)}


def decode_bytes(cfg, batch, context):
    """Bytes one decode step must read: every weight it uses once, and the
    keys and values of the live requests (bfloat16)."""
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I
    weights = 2 * (L * per_layer + V * H) + 4 * (2 * L + 1) * H   # the head's table; the embedding reads `batch` rows
    kv = 2 * batch * context * 2 * nkv * hd * L
    return weights + kv


def prefill_flops(cfg, tokens):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I
    linear = 2 * tokens * L * per_layer + 2 * V * H
    attention = 4 * nh * hd * tokens * (tokens + 1) // 2 * L
    return linear + attention


def make_rig(cfg, context, max_batch, page):
    """A model of the given shapes with random weights, an engine around it with
    room for `max_batch` requests of `context` tokens, and the three timed
    loops (decode steps, prompts, decode steps beside a prompt portion)."""
    import gc
    import types

    import torch

    from lyapunov_engine_b200 import EngineConfig, LLMEngine, SamplingParams, build, load_model, ops

    host = build.load_host()
    num_blocks = (max_batch * (context + 64) + 2 * PREFILL_TOKENS + context) // page
    loaded = load_model(config=cfg, random_seed=0, dtype="bfloat16", device="cuda:0", max_model_len=context + 64)
    engine = LLMEngine(loaded, EngineConfig(num_blocks=num_blocks, block_size=page, max_num_seqs=max_batch,
                                            max_num_batched_tokens=8192, dtype="bfloat16", device="cuda:0",
                                            max_model_len=context + 64))
    runner, manager, sampler = engine.runner, engine.block_manager, engine.sampler
    gen = torch.Generator().manual_seed(0)
    vocab = cfg["vocab_size"]
    # Synthetic cache content: timing does not depend on what the pages hold,
    # but a softmax over zeros would be a degenerate case.
    for pools in engine.cache.streams:
        for s in pools:
            s.k.normal_(0, 1)
            s.v.normal_(0, 1)
    greedy = SamplingParams(temperature=0.0, max_tokens=1 << 30, ignore_eos=True)
    def timed_decode(batch, steps, warmup, context_end):
        """K decode steps of `batch` requests whose last step runs at
        `context_end` tokens: step function + sampler, timed on the device."""
        start_len = context_end - (steps + warmup)
        seqs = []
        for i in range(batch):
            ids = torch.randint(0, vocab, (start_len + 1,), generator=gen).tolist()
            s = host.Sequence(10_000 + i, ids, host.SamplingParams())
            assert manager.grow(s, start_len)
            s.set_num_computed_tokens(start_len)
            seqs.append(s)
        params = [greedy] * batch
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def one_step():
            entries = []
            for s in seqs:
                n = s.get_num_computed_tokens()
                assert manager.grow(s, n + 1)
                entries.append(host.StepEntry(s, n, 1, [0]))
            logits = runner.step(entries)
            ids = sampler.sample(logits, params, [0] * batch)
            for s in seqs:
                s.set_num_computed_tokens(s.get_num_computed_tokens() + 1)
                s.extend_prompt([1])
            return ids

        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        before = dict(ops.counters)
        graph_before = runner.num_graph_steps
        begin.record()
        for _ in range(steps):
            one_step()
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        for s in seqs:
            manager.free(s)
        return ms, runner.num_graph_steps - graph_before, before

    def timed_prefill(tokens, repeats, warmup):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = []
        for r in range(warmup + repeats):
            ids = torch.randint(0, vocab, (tokens,), generator=gen).tolist()
            s = host.Sequence(20_000 + r, ids, host.SamplingParams())
            assert manager.grow(s, tokens)
            torch.cuda.synchronize()
            begin.record()
            logits = runner.step([host.StepEntry(s, 0, tokens, [tokens - 1])])
            sampler.sample(logits, [greedy], [0])
            end.record()
            torch.cuda.synchronize()
            if r >= warmup:
                best.append(begin.elapsed_time(end))
            manager.free(s)
        best.sort()
        return best[len(best) // 2]

    def timed_mixed(batch, steps, warmup, context_end, chunk):
        """K steps of `batch` decoding requests beside one `chunk`-token
        portion of a prompt (a new prompt starts when one is through)."""
        start_len = context_end - (steps + warmup)
        seqs = []
        for i in range(batch):
            ids = torch.randint(0, vocab, (start_len + 1,), generator=gen).tolist()
            s = host.Sequence(30_000 + i, ids, host.SamplingParams())
            assert manager.grow(s, start_len)
            s.set_num_computed_tokens(start_len)
            seqs.append(s)
        prompt_len = context_end // chunk * chunk
        state = {"prompt": None, "made": 0, "keys": 0}
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def one_step(count):
            if state["prompt"] is None:
                ids = torch.randint(0, vocab, (prompt_len,), generator=gen).tolist()
                state["prompt"] = host.Sequence(40_000 + state["made"], ids, host.SamplingParams())
                state["made"] += 1
            pr = state["prompt"]
            done = pr.get_num_computed_tokens()
            assert manager.grow(pr, done + chunk)
            entries = [host.StepEntry(pr, done, chunk, [chunk - 1])]
            for s in seqs:
                n = s.get_num_computed_tokens()
                assert manager.grow(s, n + 1)
                entries.append(host.StepEntry(s, n, 1, [0]))
            logits = runner.step(entries)
            sampler.sample(logits, [greedy] * (batch + 1), [0] * (batch + 1))
            if count:   # keys that the step's queries read: the portion's causal triangle and every decode context
                state["keys"] += chunk * done + chunk * (chunk + 1) // 2 + sum(s.get_num_computed_tokens() + 1 for s in seqs)
            for s in seqs:
                s.set_num_computed_tokens(s.get_num_computed_tokens() + 1)
                s.extend_prompt([1])
            pr.set_num_computed_tokens(done + chunk)
            if done + chunk >= prompt_len:
                manager.free(pr)
                state["prompt"] = None

        for _ in range(warmup):
            one_step(False)
        torch.cuda.synchronize()
        begin.record()
        for _ in range(steps):
            one_step(True)
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        for s in seqs:
            manager.free(s)
        if state["prompt"] is not None:
            manager.free(state["prompt"])
        return ms, state["keys"] / steps

    def close():
        """Gives the device memory back (the next rig may need all of it)."""
        nonlocal engine, loaded, runner, manager, sampler
        engine = loaded = runner = manager = sampler = None
        rig.engine = rig.runner = rig.manager = rig.sampler = None
        gc.collect()
        torch.cuda.empty_cache()

    rig = types.SimpleNamespace(engine=engine, runner=runner, manager=manager, sampler=sampler, host=host, gen=gen, vocab=vocab,
                                timed_decode=timed_decode, timed_prefill=timed_prefill, timed_mixed=timed_mixed, close=close)
    return rig


def leave_out(what, cfg):
    """Replaces one kind of kernel of a decode step by nothing, so that the step
    can be timed without it: the difference to the whole step is what the
    kernel costs inside the chain (the rest computes on stale buffers, which
    changes no launch and no byte moved)."""
    from lyapunov_engine_b200 import ops

    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    product = ops.gemm_skinny

    def products_but(skip):
        def run(out, a, w, splits=1, gated=False):
            if not skip(w, gated):
                product(out, a, w, splits=splits, gated=gated)
        return run
    if what == "norms":
        ops.rmsnorm = lambda *a, **k: None
    elif what == "qkv":
        ops.gemm_skinny_rotary = lambda *a, **k: None
    elif what == "attention":
        ops.attention_decode_bf16 = lambda *a, **k: None
    elif what == "o":
        ops.gemm_skinny = products_but(lambda w, gated: not gated and tuple(w.shape) == (H, cfg["num_attention_heads"] * cfg["head_dim"]) and w.shape[0] < V)
    elif what == "gate_up":
        ops.gemm_skinny = products_but(lambda w, gated: gated)
    elif what == "down":
        ops.gemm_skinny = products_but(lambda w, gated: not gated and tuple(w.shape) == (H, I))
    elif what == "head":
        ops.gemm_skinny = products_but(lambda w, gated: w.shape[0] == V)


def further_points(pk, page, context=8192, steps=24, warmup=6):
    """Decode at batch 1, 8 and 64 and prefill of 2,048 and 8,192 tokens at the
    3B and 8B shapes (context 8192), and the 8B mixed step (64 decoding requests
    beside a 2,048-token portion): tokens a second, with the fraction of the
    HBM or bfloat16 peak each reaches."""
    import torch

    out = {}
    for name in ("3b", "8b"):
        cfg = dict(SHAPES[name])
        # weights, the cache of 65 requests of `context` tokens, activations: leave the size out if it does not fit
        H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
        nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        weights = 2 * (L * ((nh + 2 * nkv) * hd * H + H * nh * hd + 3 * I * H) + (1 if cfg["tie_word_embeddings"] else 2) * cfg["vocab_size"] * H)
        cache = 2 * 2 * nkv * hd * L * (65 * (context + 64) + 2 * PREFILL_TOKENS + context)
        free, _ = torch.cuda.mem_get_info()
        if weights + cache + (6 << 30) > free:
            out[f"{name}_skipped"] = f"needs {(weights + cache) >> 30} GiB of device memory, {free >> 30} GiB are free"
            continue
        rig = make_rig(cfg, context, 65, page)
        for b in (1, 8, 64):
            rig.timed_decode(b, 3, 2, context - 200)          # (captures the graph)
            ms, _, _ = rig.timed_decode(b, steps, warmup, context)
            out[f"{name}_decode_b{b}"] = round(b * 1000.0 / ms, 1)
            out[f"{name}_decode_b{b}_hbm_frac"] = round(decode_bytes(cfg, b, context - (steps - 1) // 2) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        for tokens in (2048, 8192):
            ms = rig.timed_prefill(tokens, 3, 2)
            out[f"{name}_prefill_{tokens}"] = round(tokens * 1000.0 / ms, 1)
            out[f"{name}_prefill_{tokens}_frac"] = round(prefill_flops(cfg, tokens) / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
        if name == "8b":
            ms, _ = rig.timed_mixed(64, 8, 3, context, 2048)
            out["8b_mixed_64_2048"] = round((64 + 2048) * 1000.0 / ms, 1)
            out["8b_mixed_64_2048_ms"] = round(ms, 3)
        rig.close()
        del rig
    return out


def run_ours(args):
    global BLOCK_SIZE, CONTEXT
    import torch
    BLOCK_SIZE = args.page
    if args.only and args.context:
        CONTEXT = args.context

    from lyapunov_engine_b200 import SamplingParams, ops

    cfg = dict(SHAPES[args.shapes if args.only else "1b"])
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    torch.cuda.set_device(0)
    # room for the batches the run times (the prompt beside the decoding requests of a mixed step holds a slot too)
    max_batch = (max(args.batch, args.max_num_seqs, 1) + (args.only == "mixed")) if args.only else 64
    rig = make_rig(cfg, CONTEXT, max_batch, BLOCK_SIZE)
    engine, runner, manager, sampler, host, gen, vocab = rig.engine, rig.runner, rig.manager, rig.sampler, rig.host, rig.gen, rig.vocab
    timed_decode, timed_prefill, timed_mixed = rig.timed_decode, rig.timed_prefill, rig.timed_mixed

    if args.only and args.without:
        leave_out(args.without, cfg)
    if args.only:
        # A short run of one kind of step, for profilers: no CUDA graph, so
        # that every kernel shows as its own launch.
        runner.use_cuda_graphs = not args.no_cuda_graphs
        if args.only == "decode":
            ms, _, _ = timed_decode(args.batch, args.steps, args.warmup, args.context or CONTEXT)
            nbytes = decode_bytes(cfg, args.batch, (args.context or CONTEXT) - (args.steps - 1) // 2)
            print(json.dumps({"only": "decode", "shapes": args.shapes, "batch": args.batch, "context": args.context or CONTEXT,
                              "ms_per_step": round(ms, 4), "tokens_per_s": round(args.batch * 1000.0 / ms, 1),
                              "hbm_frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
                              "layers": cfg["num_hidden_layers"], "cuda_graph": runner.use_cuda_graphs}))
        elif args.only == "mixed":
            chunk = args.tokens or PREFILL_TOKENS
            ms, keys = timed_mixed(args.batch, args.steps, args.warmup, CONTEXT, chunk)
            H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
            nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
            per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * I * H
            flops = 2 * (chunk + args.batch) * L * per_layer + 2 * (args.batch + 1) * cfg["vocab_size"] * H + 4 * nh * hd * keys * L
            nbytes = decode_bytes(cfg, args.batch, CONTEXT - (args.steps - 1) // 2)
            print(json.dumps({"only": "mixed", "shapes": args.shapes, "decoding": args.batch, "portion": chunk, "context": CONTEXT,
                              "ms_per_step": round(ms, 4), "tokens_per_s": round((args.batch + chunk) * 1000.0 / ms, 1),
                              "layers": cfg["num_hidden_layers"],
                              "tflops": round(flops / (ms * 1e-3) / 1e12, 1),
                              "flops_frac": round(flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4),
                              "hbm_frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}))
        else:
            tokens = args.tokens or PREFILL_TOKENS
            ms = timed_prefill(tokens, args.steps, args.warmup)
            print(json.dumps({"only": "prefill", "shapes": args.shapes, "tokens": tokens, "ms": round(ms, 4),
                              "layers": cfg["num_hidden_layers"],
                              "tflops": round(prefill_flops(cfg, tokens) / (ms * 1e-3) / 1e12, 1),
                              "flops_frac": round(prefill_flops(cfg, tokens) / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.3)

    # ---- headline: batch 8 at context 4096
    batch = 8
    kernels_per_step = None
    # captures the graph for this batch outside the timed call, and runs long enough (some 60 ms) for the clocks
    # to come up from idle: the sampler's start above left the GPU waiting, and a short timed run (20 steps are
    # 16 ms) would otherwise sit on the ramp
    timed_decode(batch, 64, 8, CONTEXT - 200)
    ops.counters["own_kernels"] = ops.counters["library_products"] = 0
    m0 = clocks.mark()
    ms8, graph_steps, _ = timed_decode(batch, args.steps, args.warmup, CONTEXT)
    m1 = clocks.mark()
    value = batch * 1000.0 / ms8

    # kernels per decode step: count launches of one eager step of the same shape
    runner.use_cuda_graphs = False
    ops.counters["own_kernels"] = ops.counters["library_products"] = 0
    timed_decode(batch, 1, 0, CONTEXT - 300)
    kernels_per_step = dict(ops.counters)
    runner.use_cuda_graphs = True

    points = {}
    for b in (1, 64):
        timed_decode(b, 4, 2, CONTEXT - 200)
        ms, _, _ = timed_decode(b, args.steps, args.warmup, CONTEXT)
        points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)
        points[f"decode_b{b}_ms"] = round(ms, 4)
        points[f"decode_b{b}_hbm_frac"] = round(decode_bytes(cfg, b, CONTEXT - (args.steps - 1) // 2) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    # ---- prefill of 2,048 tokens
    pre_ms = timed_prefill(PREFILL_TOKENS, 5, 3)
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)}

    # ---- end to end through the entry point: host tokens in, host tokens out
    # The requests live past the timed window (it holds K steps of all `batch` requests and nothing else); they
    # end afterwards four steps apart, and that drain (8 requests down to none, smaller batch buckets) is timed
    # by itself.
    e2e_steps, e2e_warm = args.steps, args.warmup
    ahead_of_window = 8                      # steps in which requests get their first tokens one after the other
    # The prefill of 8 x 4,000 tokens draws the full 1 kW; for some 0.1 s afterwards the power cap holds the SM
    # clock down (1,725 of 1,965 MHz sampled), which a decode step, bound by latencies, feels.  The window
    # measures steady decoding, so untimed decode steps run first until that has passed.
    settle = 200
    prompt_len = CONTEXT - (e2e_steps + e2e_warm + settle) - ahead_of_window - 1   # the window ends at CONTEXT at the latest
    for i in range(batch):
        sp = SamplingParams(temperature=0.0, max_tokens=e2e_steps + e2e_warm + settle + ahead_of_window + 4 * (i + 1),
                            ignore_eos=True)
        engine.add_request(f"bench-{i}", torch.randint(0, vocab, (prompt_len,), generator=gen).tolist(), sp)
    engine.warm_up(contexts=[CONTEXT, CONTEXT + 64], batches=[1, 2, 4, batch])   # as a server does before its first request
    while any(seq.get_output_len() == 0 for seq, _, _ in engine.active_sequences.values()):
        engine.step()                               # prefill (portions under the token budget)
    for _ in range(settle + e2e_warm):
        engine.step()
    torch.cuda.synchronize()
    m2 = clocks.mark()
    d2h0 = engine.d2h_bytes
    t0 = time.perf_counter()
    produced = 0
    slowest = 0.0
    for _ in range(e2e_steps):
        t1 = time.perf_counter()
        produced += len(engine.step())
        slowest = max(slowest, time.perf_counter() - t1)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    m3 = clocks.mark()
    assert produced == batch * e2e_steps, (produced, batch, e2e_steps)
    d2h = (engine.d2h_bytes - d2h0) / e2e_steps
    live = [host.StepEntry(seq, seq.get_num_computed_tokens(), 1, [0]) for seq, _, _ in engine.active_sequences.values()]
    width = runner._table_width(max(e.start for e in live) + 1)    # as the runner packs a captured decode step
    layout = host.pack_step(live, manager, runner.tile_sizes, batch, [min(width, w) for w in runner.fixed_max_blocks], 0, 0)
    h2d = 4 * layout.total
    t0 = time.perf_counter()
    drain_steps = drain_tokens = 0
    while engine.has_unfinished_requests():
        drain_tokens += len(engine.step())
        drain_steps += 1
    torch.cuda.synchronize()
    drain_s = time.perf_counter() - t0
    e2e = {"value": round(produced / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_s * 1000 / e2e_steps, 4),
           "slowest_step_ms": round(slowest * 1000, 3), "settle_steps": settle,
           "sm_mhz": clocks.summary(m2, max(m3, m2 + 1)).get("sm_mhz"),
           "drain": {"steps": drain_steps, "tokens": drain_tokens, "ms_per_step": round(drain_s * 1000 / max(drain_steps, 1), 4)}}
    clocks.stop()

    # ---- further sizes: the same steps at the layer sizes of Llama-3.2-3B and Llama-3.1-8B, context 8192
    if args.points == "all":
        rig.close()
        del rig, engine, runner, manager, sampler
        try:
            points.update(further_points(pk, BLOCK_SIZE))
        except Exception as e:       # the headline does not depend on the further sizes (they need 90 GB of device memory)
            points["further_sizes_failed"] = f"{type(e).__name__}: {str(e)[:160]}"

    # the timed steps run at contexts CONTEXT - steps + 1 .. CONTEXT: count the bytes of their mean
    mean_context = CONTEXT - (args.steps - 1) // 2
    nbytes = decode_bytes(cfg, batch, mean_context)
    achieved = nbytes / (ms8 * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s, Llama-3.2-1B shapes, batch 8, context 4096",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), token ids uniform over the vocabulary",
        "config": {"model": "Llama-3.2-1B shapes", "layers": cfg["num_hidden_layers"], "layers_of_model": layers_full,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": batch,
                   "seq_len": CONTEXT, "page": BLOCK_SIZE, "parallelism": "single GPU",
                   "timing": "CUDA events; working set per step > L2", "cuda_graph": graph_steps > 0,
                   "peaks": pk["source"]},
        "clocks": clocks.summary(m0, m1),
        "e2e": e2e,
        "gpu_launches": kernels_per_step["own_kernels"] * args.steps,
        "library_products": kernels_per_step["library_products"] * args.steps,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": nbytes, "mean_context": mean_context},
        "points": points,
    }
    print(json.dumps(line))
    return 0


def run_reference(args):
    """The unmodified reference (installed under baseline/_ref with its own
    setup.py, CUDA extension built for sm_100 through its TORCH_CUDA_ARCH_LIST
    switch) through its own public API: LlamaForCausalLM with random weights,
    LLMEngine.add_request / step.  Same shapes, batch, context and greedy
    sampling as the other arm; float16, the only type its kernels take."""
    why = reference_unavailable()
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    try:
        line = _reference_line(args)
    except Exception as e:  # the reference's own failure is a result, not a crash of the benchmark
        line = {"impl": "reference", "unavailable": f"the reference failed while running: {type(e).__name__}: {str(e)[:200]}"}
    print(json.dumps(line))
    return 0


def reference_unavailable() -> str:
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "lyapunov_engine")):
        return "IanConery/lyapunov-engine is not installed under baseline/_ref (pip install --no-index --target baseline/_ref of the reference)"
    if not any(f.startswith("_C") and f.endswith(".so") for f in os.listdir(os.path.join(ref, "lyapunov_engine"))):
        return "the reference was installed without its CUDA extension; its engine then returns nothing from step()"
    return ""


def _reference_line(args):
    import torch

    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    from lyapunov_engine.engine.llm_engine import EngineConfig, LLMEngine
    from lyapunov_engine.engine.sampling import SamplingParams
    from lyapunov_engine.models.llama import LlamaConfig, LlamaForCausalLM

    c = LLAMA_1B
    torch.manual_seed(0)
    torch.cuda.set_device(0)
    config = LlamaConfig(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], intermediate_size=c["intermediate_size"],
                         num_hidden_layers=c["num_hidden_layers"], num_attention_heads=c["num_attention_heads"],
                         num_key_value_heads=c["num_key_value_heads"], head_dim=c["head_dim"],
                         max_position_embeddings=c["max_position_embeddings"], rms_norm_eps=c["rms_norm_eps"],
                         rope_theta=c["rope_theta"])
    model = LlamaForCausalLM(config)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 2:
                p.normal_(0.0, 0.02)
    model = model.to(dtype=torch.float16, device="cuda:0").eval()
    batch = 8
    steps, warmup = args.steps, max(args.warmup, 3)
    prompt_len = CONTEXT - (steps + warmup) - 1
    engine = LLMEngine(model, EngineConfig(model_config=config, num_blocks=batch * (CONTEXT // BLOCK_SIZE + 2),
                                           block_size=BLOCK_SIZE, max_num_seqs=64,
                                           max_num_batched_tokens=batch * CONTEXT + 64, dtype=torch.float16,
                                           device="cuda:0"))
    gen = torch.Generator().manual_seed(0)
    sp = SamplingParams(temperature=0.0, max_tokens=steps + warmup + 1, ignore_eos=True)
    for i in range(batch):
        engine.add_request(f"bench-{i}", torch.randint(0, c["vocab_size"], (prompt_len,), generator=gen).tolist(), sp)
    clocks = ClockSampler()
    clocks.start()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.step()                                   # the reference runs every waiting prompt whole in one step
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    m0 = clocks.mark()
    t0 = time.perf_counter()
    begin.record()
    produced = 0
    for _ in range(steps):
        produced += len(engine.step())
    end.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    m1 = clocks.mark()
    clocks.stop()
    ms = begin.elapsed_time(end) / steps
    nbytes = decode_bytes(c, batch, CONTEXT)
    pk = peaks()
    return {
        "impl": "reference",
        "metric": "decode tokens/s, Llama-3.2-1B shapes, batch 8, context 4096",
        "value": round(batch * 1000.0 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic: random weights N(0,0.02), token ids uniform over the vocabulary",
        "config": {"model": "Llama-3.2-1B shapes", "layers": c["num_hidden_layers"], "layers_of_model": c["num_hidden_layers"],
                   "global_batch": batch, "seq_len": CONTEXT, "page": BLOCK_SIZE, "parallelism": "single GPU",
                   "timing": "CUDA events around LLMEngine.step(); working set per step > L2",
                   "note": "the reference's model never writes its KV cache, so its decode reads pages it never filled"},
        "clocks": clocks.summary(m0, m1),
        "e2e": {"value": round(produced / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                "ms_per_step": round(wall * 1000 / steps, 4)},
        "gpu_launches": None,
        "prefill": {"value": round(batch * prompt_len / prefill_s, 1), "tokens": batch * prompt_len, "ms": round(prefill_s * 1000, 2)},
        "roofline": {"bound": "hbm", "achieved": round(nbytes / (ms * 1e-3) / 1e9, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)},
    }


# The reference's serving benchmark (benchmarks/bench_serving.py:10-43: the model; 46-77: what is timed): a small
# Llama with random weights, every request a prompt of 128 tokens (ids 100, 101, ...), 32 tokens generated
# greedily, batches of 1, 4, 8, 16.  TTFT is the first step (all prompts in it), ITL the mean of the steps after
# it, each with a device synchronisation on both sides; tok/s counts prompt and generated tokens over the sum of
# those times.  Here in bfloat16, and each batch runs twice untimed first (kernels compiled, step graphs captured).
SERVING_MODEL = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 32000, "hidden_size": 1024,
    "intermediate_size": 4096, "num_hidden_layers": 8, "num_attention_heads": 16, "num_key_value_heads": 4,
    "head_dim": 64, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "rope_scaling": None, "tie_word_embeddings": False, "hidden_act": "silu", "attention_bias": False,
    "mlp_bias": False, "bos_token_id": 1, "eos_token_id": 2, "torch_dtype": "bfloat16",
}


def run_serving(args):
    import torch

    from lyapunov_engine_b200 import EngineConfig, LLMEngine, SamplingParams, load_model

    prompt_len, generated = 128, 32
    loaded = load_model(config=dict(SERVING_MODEL), random_seed=0, dtype="bfloat16", device="cuda:0", max_model_len=1024)
    rows = []
    for batch in args.batch_sizes:
        engine = LLMEngine(loaded, EngineConfig(num_blocks=2048, block_size=BLOCK_SIZE, max_num_seqs=batch,
                                                max_num_batched_tokens=4096, dtype="bfloat16", device="cuda:0",
                                                max_model_len=1024))
        for run in range(3):        # two untimed runs (a prompt step is captured as a graph at its second use), one timed
            for _ in range(batch):
                engine.add_request([100 + i for i in range(prompt_len)],
                                   SamplingParams(temperature=0.0, max_tokens=generated, ignore_eos=True))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            engine.step()
            torch.cuda.synchronize()
            ttft = (time.perf_counter() - t0) * 1e3
            steps = []
            while engine.has_unfinished_requests():
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                engine.step()
                torch.cuda.synchronize()
                steps.append((time.perf_counter() - t0) * 1e3)
        total_s = (ttft + sum(steps)) / 1e3
        rows.append({"batch": batch, "ttft_ms": round(ttft, 3), "itl_ms": round(sum(steps) / max(len(steps), 1), 4),
                     "decode_steps": len(steps),
                     "tokens_per_s": round(batch * (prompt_len + generated) / total_s, 1)})
        print(f"batch {batch:3d}: TTFT {ttft:7.3f} ms   ITL {rows[-1]['itl_ms']:7.4f} ms   {rows[-1]['tokens_per_s']:10.1f} tok/s",
              file=sys.stderr)
        del engine
    print(json.dumps({"only": "serving", "model": "V32000 H1024 I4096 L8 nh16 nkv4 hd64, random weights", "dtype": "bf16",
                      "prompt": prompt_len, "generated": generated, "rows": rows}))
    return 0


# The reference's kernel benchmark (benchmarks/bench_kernels.py:7-27: CUDA events, the median of 100 launches after
# 25 warm-ups; 40-41 and 74-79: the grids): RMSNorm with the residual add over widths 2048, 4096, 8192 and 32 to
# 4,096 tokens; causal attention of one prompt of 512 to 4,096 tokens, 32 heads of 128 in 8 groups (here over the
# paged cache, pages of 16).  Each row carries the bytes or flops the kernel must move and the share of the measured
# peak that makes.  Every launch works on a fresh set of tensors until 256 MB have gone round (more than L2 holds).
def run_kernels(args):
    import torch

    from lyapunov_engine_b200 import ops

    pk = peaks()
    dev = "cuda:0"

    def median_us(launch, sets):
        for i in range(25):
            launch(i % sets)
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(100)]
        torch.cuda.synchronize()
        for i, (a, b) in enumerate(events):
            a.record()
            launch(i % sets)
            b.record()
        torch.cuda.synchronize()
        times = sorted(a.elapsed_time(b) * 1e3 for a, b in events)
        return times[len(times) // 2]

    rows = []
    for hidden in (2048, 4096, 8192):
        for tokens in (32, 256, 1024, 4096):
            nbytes = tokens * hidden * (4 + 2 + 4 + 2) + 4 * hidden       # residual in and out (float32), delta in, normed out
            sets = max(2, min(64, (256 << 20) // nbytes + 1))
            resid = [torch.randn(tokens, hidden, device=dev) for _ in range(sets)]
            delta = [torch.randn(tokens, hidden, device=dev).bfloat16() for _ in range(sets)]
            out = [torch.empty(tokens, hidden, device=dev, dtype=torch.bfloat16) for _ in range(sets)]
            weight = torch.ones(hidden, device=dev)
            us = median_us(lambda i: ops.rmsnorm(out[i], resid[i], delta[i], weight, 1e-5), sets)
            rows.append({"kernel": "rmsnorm + residual", "hidden": hidden, "tokens": tokens, "us": round(us, 2),
                         "gbs": round(nbytes / us / 1e3, 1), "hbm_frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)})
            del resid, delta, out
    nh, nkv, hd, page = 32, 8, 128, BLOCK_SIZE
    status = ops.new_status(dev)
    for seq in (512, 1024, 2048, 4096):
        pages = seq // page
        k = torch.randn(pages + 1, nkv, page, hd, device=dev).bfloat16()
        v = torch.randn(pages + 1, nkv, page, hd, device=dev).bfloat16()
        q = torch.randn(seq, (nh + 2 * nkv) * hd, device=dev).bfloat16()
        out = torch.empty(seq, nh * hd, device=dev, dtype=torch.bfloat16)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
        cu = torch.tensor([0, seq], dtype=torch.int32, device=dev)
        ctx = torch.zeros(1, dtype=torch.int32, device=dev)
        tiles = (seq + 127) // 128
        tile_request = torch.zeros(tiles, dtype=torch.int32, device=dev)
        tile_q0 = torch.arange(0, seq, 128, dtype=torch.int32, device=dev)
        us = median_us(lambda i: ops.attention_prefill_tc_bf16(out, q, q.stride(0), k, v, table, cu, ctx, tile_request, tile_q0,
                                                               tiles, nh, nkv, hd, page, 0, hd ** -0.5, status), 1)
        flops = 4 * nh * hd * seq * (seq + 1) // 2
        rows.append({"kernel": "prefill attention (tcgen05), 32 heads of 128 in 8 groups", "tokens": seq, "us": round(us, 2),
                     "tflops": round(flops / us / 1e6, 1), "bf16_frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3)})
    ops.check_status(status)
    for r in rows:
        print("  ".join(f"{k}={v}" for k, v in r.items()), file=sys.stderr)
    print(json.dumps({"only": "kernels", "peaks": pk["source"], "rows": rows}))
    return 0


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=256)
    p.add_argument("--warmup", type=int, default=16)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    p.add_argument("--only", choices=["decode", "prefill", "mixed", "serving", "kernels"], default=None,
                   help="run one kind of step and exit (for profilers and for further sizes); mixed = --batch decoding "
                        "requests beside one --tokens portion of a prompt in every step; serving = the reference's "
                        "serving benchmark (small model, prompts of 128 tokens, 32 generated: TTFT, ITL, tokens/s); "
                        "kernels = its kernel benchmark (RMSNorm and prefill attention over a grid of sizes)")
    p.add_argument("--batch-sizes", nargs="+", type=int, default=[1, 4, 8, 16], help="with --only serving")
    p.add_argument("--shapes", choices=sorted(SHAPES), default="1b", help="with --only: layer sizes of Llama-3.2-1B, 3.2-3B or 3.1-8B")
    p.add_argument("--batch", type=int, default=8, help="batch of --only decode")
    p.add_argument("--max-num-seqs", type=int, default=0,
                   help="with --only decode: the most requests the engine is set up for (0: --batch); a smaller batch "
                        "then runs as a partly filled step of the next power of two")
    p.add_argument("--page", type=int, default=BLOCK_SIZE, help="tokens per page of the cache")
    p.add_argument("--tokens", type=int, default=0, help="with --only prefill or mixed: tokens of the prompt or of its portion (at most the context and 8192)")
    p.add_argument("--context", type=int, default=0, help="with --only decode: the context the last step ends at")
    p.add_argument("--no-cuda-graphs", action="store_true", help="with --only decode: launch every kernel by itself")
    p.add_argument("--without", choices=["norms", "qkv", "attention", "o", "gate_up", "down", "head"], default=None,
                   help="with --only decode (batches up to 16): time the step with this kind of kernel left out")
    p.add_argument("--points", choices=["all", "1b"], default="all",
                   help="all: also decode, prefill and the mixed step at the 3B and 8B shapes (context 8192) in `points`")
    args = p.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if not args.only:
        args.warmup = max(args.warmup, 3)
    if args.only == "serving" and args.impl == "ours":
        return run_serving(args)
    if args.only == "kernels" and args.impl == "ours":
        return run_kernels(args)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
