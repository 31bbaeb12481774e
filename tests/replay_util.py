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
