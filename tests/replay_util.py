"""Drives bin/trace_run's program for the tests: builds traces for the ways of
cutting the work, runs them (in this process, or as a child process), gathers
the logits by (request, position) and compares them with the plain
implementation."""
from __future__ import annotations

import contextlib
import io
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Trace:
    def __init__(self):
        self.steps = []       # JSON objects
        self.wanted = []      # per step: list of (request, position)
        self._pos = {}

    def step(self, entries, end=()):
        """entries: list of (request id, tokens, want places or 'all' or None)."""
        js, wanted = [], []
        for rid, tokens, want in entries:
            start = self._pos.get(rid, 0)
            if want == "all":
                want = list(range(len(tokens)))
            want = list(want or [])
            js.append({"id": rid, "tokens": list(tokens), "want": want})
            wanted += [(rid, start + w) for w in want]
            self._pos[rid] = start + len(tokens)
        self.steps.append({"step": len(self.steps), "entries": js, "end": list(end)})
        self.wanted.append(wanted)
        for rid in end:
            self._pos.pop(rid, None)

    def lines(self):
        return [json.dumps(s) for s in self.steps]


def run_trace(trace: Trace, model_dir: str, dtype: str, out_dir: str, max_tokens: int, block_size: int,
              child: bool = False, extra=()):
    """Returns {(request, position): logits row (float32 numpy)}."""
    argv = ["--model", model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens),
            "--block-size", str(block_size), *extra]
    text = "\n".join(trace.lines()) + "\n"
    if child:
        proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), *argv], stdin=subprocess.PIPE,
                                stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        done = []
        for line, step in zip(trace.lines(), trace.steps):
            proc.stdin.write(line + "\n")
            proc.stdin.flush()
            answer = proc.stdout.readline().strip()
            if answer != f"done {step['step']}":
                err = proc.stderr.read()
                raise AssertionError(f"trace_run answered {answer!r} to step {step['step']}\n{err[-3000:]}")
            done.append(answer)
        proc.stdin.close()
        code = proc.wait(timeout=120)
        assert code == 0, proc.stderr.read()[-3000:]
    else:
        from lyapunov_engine_b200.replay import trace_run

        stdin, stdout = sys.stdin, io.StringIO()
        sys.stdin = io.StringIO(text)
        try:
            with contextlib.redirect_stdout(stdout):
                code = trace_run.main(argv)
        finally:
            sys.stdin = stdin
        assert code == 0
        assert stdout.getvalue().split("\n")[:-1] == [f"done {s['step']}" for s in trace.steps]
    out = {}
    for step, wanted in zip(trace.steps, trace.wanted):
        path = os.path.join(out_dir, f"{step['step']}.f32")
        if not wanted:
            assert not os.path.exists(path)
            continue
        data = np.fromfile(path, dtype="<f4")
        data = data.reshape(len(wanted), -1)
        for key, row in zip(wanted, data):
            out[key] = row
    return out


def peak_pool_tokens(trace: Trace, page: int) -> int:
    """The fewest tokens (a multiple of 64) whose pages hold what the trace's
    live requests hold at their peak, each request in whole pages."""
    held, peak = {}, 0
    for step in trace.steps:
        for e in step["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + page - 1) // page for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return (peak * page + 63) // 64 * 64


def read_pages(out_dir: str) -> dict:
    """What trace_run wrote about its page pool at exit."""
    with open(os.path.join(out_dir, "pages.json"), "r", encoding="utf-8") as f:
        return json.load(f)


def whole_trace(requests: dict) -> Trace:
    """Each request alone and whole, one step each."""
    t = Trace()
    for rid, ids in requests.items():
        t.step([(rid, ids, "all")], end=[rid])
    return t


def tail_trace(requests: dict, tail: int = 32) -> Trace:
    """Most of each request in one step, the last `tail` tokens one by one."""
    t = Trace()
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        t.step([(rid, ids[:head], "all")])
        for i in range(head, len(ids)):
            t.step([(rid, ids[i:i + 1], [0])], end=[rid] if i == len(ids) - 1 else [])
        if head == len(ids):
            t.step([], end=[rid])
    return t


def portions_trace(requests: dict, sizes=(7, 2, 16, 3, 2, 33, 5, 2, 64, 2, 11)) -> Trace:
    """Portions of changing size, down to two tokens."""
    t = Trace()
    for rid, ids in requests.items():
        pos, k = 0, 0
        while pos < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - pos)
            k += 1
            pos += n
            t.step([(rid, ids[pos - n:pos], "all")], end=[rid] if pos == len(ids) else [])
    return t


def mixed_trace(requests: dict, prompt_lens: dict, chunk: int = 16, max_live: int = 4, seed: int = 0) -> Trace:
    """Up to `max_live` live requests: portions of some prompts beside single
    decoded tokens of others; a request starts when another ends."""
    rng = np.random.RandomState(seed)
    t = Trace()
    waiting = list(requests)
    live, pos = [], {}
    while waiting or live:
        while waiting and len(live) < max_live:
            rid = waiting.pop(0)
            live.append(rid)
            pos[rid] = 0
            if rng.rand() < 0.5:
                break   # staggered starts
        entries, ended = [], []
        for rid in list(live):
            ids = requests[rid]
            p = pos[rid]
            if p < prompt_lens[rid]:
                n = min(prompt_lens[rid] - p, max(2, int(rng.randint(2, chunk + 1))))
                if prompt_lens[rid] - p - n == 1:
                    n += 1          # never leave a portion of one prompt token... keep portions >= 2 where possible
            else:
                if rng.rand() < 0.15:
                    continue        # left out of this step, goes on later
                n = 1
            n = min(n, len(ids) - p)
            entries.append((rid, ids[p:p + n], "all"))
            pos[rid] = p + n
            if pos[rid] == len(ids):
                ended.append(rid)
                live.remove(rid)
        t.step(entries, end=ended)
    return t


def compare(got: dict, reference: dict, atol: float, rtol: float, what: str):
    """reference: {request: logits [T, V] tensor}.  Reports the first wrong
    place in order of (request, position)."""
    worst = 0.0
    for (rid, p) in sorted(got):
        ref = reference[rid][p].numpy()
        row = got[(rid, p)]
        err = np.abs(row - ref)
        bound = atol + rtol * np.abs(ref)
        if not np.all(err <= bound) or not np.all(np.isfinite(row)):
            i = int(np.argmax(err - bound))
            raise AssertionError(f"{what}: request {rid!r} position {p}: logit {i} is {row[i]!r}, plain says {ref[i]!r} "
                                 f"(|diff| {err[i]:.3e} > {bound[i]:.3e}); max |diff| at this place {err.max():.3e}")
        worst = max(worst, float(err.max()))
    return worst


# --------------------------------------------------------------------------
# bfloat16: what "equal up to rounding" means, measured
# --------------------------------------------------------------------------
BF16_RMS_ALL = 1.25     # the root mean square of all differences, in units of the noise's
BF16_RMS_ROW = 2.5      # the root mean square over one place's logits
BF16_MAX_ABS = 1.6      # the largest single difference, in units of the noise's largest


def bf16_references(cfg, weights, requests, plain_forward):
    """The plain implementation with the pipeline's bfloat16 roundings (weights,
    activations between products, softmax numerators), and how far a second,
    equally valid evaluation of the same pipeline lies from it: sums in 64
    bits instead of 32, and the numerators scaled by exp(-0.5) before they are
    rounded (a kernel that keeps a running or lazy maximum rounds numerators
    that are scaled by another bound than the row's final maximum).  The two
    runs differ in nothing but which way roundings fall, as the engine does
    from either; their distance is the unit the engine's is measured in.
    Returns (reference logits per request, {"rms": ..., "max": ...})."""
    rounded = {k: v.to(torch.bfloat16).float() for k, v in weights.items()}
    wide = {k: v.double() for k, v in rounded.items()}
    bf = torch.bfloat16
    ref = {r: plain_forward(cfg, rounded, ids, act_dtype=bf, prob_dtype=bf) for r, ids in requests.items()}
    square, count, largest = 0.0, 0, 0.0
    for r, ids in requests.items():
        other = plain_forward(cfg, wide, ids, act_dtype=bf, prob_dtype=bf, prob_shift=0.5).float()
        d = (other - ref[r]).double()
        square += float(d.pow(2).sum())
        count += d.numel()
        largest = max(largest, float(d.abs().max()))
    return ref, {"rms": (square / max(count, 1)) ** 0.5, "max": largest}


def compare_bf16(got: dict, reference: dict, noise: dict, what: str):
    """Three bounds in units of the measured noise (see bf16_references): the
    root mean square of all differences (the float32 model's logits lie 1.6 to
    2.3 units from the bfloat16 model's and fail it), the root mean square at
    every single place (a wrong key, position or page moves one place's logits
    by 5 to 50 units), and the largest single difference."""
    square, count = 0.0, 0
    for (rid, p) in sorted(got):
        ref = reference[rid][p].numpy().astype(np.float64)
        row = got[(rid, p)].astype(np.float64)
        if not np.all(np.isfinite(row)):
            raise AssertionError(f"{what}: request {rid!r} position {p}: logits are not finite")
        d = row - ref
        row_rms = float(np.sqrt(np.mean(d * d)))
        if row_rms > BF16_RMS_ROW * noise["rms"]:
            raise AssertionError(f"{what}: request {rid!r} position {p}: the logits lie {row_rms:.3e} (rms) from the plain "
                                 f"implementation's, {row_rms / noise['rms']:.2f} units of rounding noise "
                                 f"(allowed {BF16_RMS_ROW})")
        worst = float(np.abs(d).max())
        if worst > BF16_MAX_ABS * noise["max"]:
            i = int(np.argmax(np.abs(d)))
            raise AssertionError(f"{what}: request {rid!r} position {p}: logit {i} is {row[i]!r}, plain says {ref[i]!r} "
                                 f"(|diff| {worst:.3e} > {BF16_MAX_ABS * noise['max']:.3e})")
        square += float(np.sum(d * d))
        count += d.size
    total = (square / max(count, 1)) ** 0.5
    if total > BF16_RMS_ALL * noise["rms"]:
        raise AssertionError(f"{what}: all logits together lie {total:.3e} (rms) from the plain implementation's, "
                             f"{total / noise['rms']:.2f} units of rounding noise (allowed {BF16_RMS_ALL})")
    return total / noise["rms"]
