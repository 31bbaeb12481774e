"""Trace replay: feeds given token ids through a model step by step and writes
the logits at the wanted places.  It samples nothing and has nothing of its
own: the model, the weights' loader, the cache manager, the step function and
the kernels are the ones generation uses.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input: one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
``entries`` gives each request's next tokens and the places among them whose
logits are wanted; all entries of a step run as one batch.  ``end`` lists the
requests that are finished after the step; their pages are given back.  For a
step with wanted places ``DIR/<step>.f32`` receives the logits [wanted, vocab]
as little-endian float32 in the order of the entries and of ``want``.  After
every step ``done <step>`` is printed and flushed.

The cache pool holds ``--max-tokens`` tokens (in pages of ``--block-size``),
so pages are used again as requests end.  At exit ``DIR/pages.json`` says how
the pool was used (pages in the pool, pages handed out in all, how many of
those had been used before, the most that were held at once) and how many
steps ran as captured graphs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def parse_args(argv=None):
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="tokens that live requests hold at most (each rounded up to a multiple of 64)")
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--max-num-seqs", type=int, default=8)
    p.add_argument("--no-cuda-graphs", action="store_true")
    return p.parse_args(argv)


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.block_size < 1 or 64 % args.block_size:
        print(f"trace_run: --block-size must divide 64, got {args.block_size}", file=sys.stderr)
        return 2
    import torch

    from lyapunov_engine_b200 import build
    from lyapunov_engine_b200.cache import DeviceCache
    from lyapunov_engine_b200.engine.llm_engine import load_model
    from lyapunov_engine_b200.engine.step import ModelRunner

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 1
    os.makedirs(args.out, exist_ok=True)
    host = build.load_host()
    max_tokens = (args.max_tokens + 63) // 64 * 64
    loaded = load_model(args.model, args.dtype, args.device, max_model_len=max_tokens)
    max_model_len = min(max_tokens, loaded.spec.max_positions)
    num_blocks = max_tokens // args.block_size
    with torch.cuda.device(loaded.runtime.device):
        cache = DeviceCache(loaded.model, loaded.runtime, num_blocks, args.block_size, args.max_num_seqs)
        runner = ModelRunner(loaded.model, cache, loaded.runtime, max_num_batched_tokens=max_tokens,
                             max_num_seqs=args.max_num_seqs, max_model_len=max_model_len,
                             use_cuda_graphs=not args.no_cuda_graphs, check_status=True)
        manager = cache.manager
        live: dict[str, object] = {}
        next_id = 0
        peak_used = 0
        vocab = loaded.spec.vocab_size
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            step = json.loads(line)
            number = step["step"]
            entries = []
            for e in step.get("entries", []):
                rid, tokens, want = str(e["id"]), [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]
                if not tokens:
                    raise SystemExit(f"trace_run: step {number}: request {rid!r} brings no token")
                bad = [t for t in tokens if not 0 <= t < vocab]
                if bad:
                    raise SystemExit(f"trace_run: step {number}: token id {bad[0]} is outside the vocabulary of {vocab}")
                seq = live.get(rid)
                if seq is None:
                    seq = host.Sequence(next_id, tokens, host.SamplingParams())
                    next_id += 1
                    live[rid] = seq
                else:
                    seq.extend_prompt(tokens)
                start = seq.get_num_computed_tokens()
                if start + len(tokens) > max_model_len:
                    raise SystemExit(f"trace_run: step {number}: request {rid!r} would hold {start + len(tokens)} tokens; "
                                     f"the limit is {max_model_len}")
                if not manager.grow(seq, start + len(tokens)):
                    raise SystemExit(f"trace_run: step {number}: no room for request {rid!r} "
                                     f"({manager.get_num_free_blocks()} free pages of {args.block_size} tokens); "
                                     f"raise --max-tokens")
                entries.append(host.StepEntry(seq, start, len(tokens), want))
            if loaded.model.groups:
                peak_used = max(peak_used, max(manager.get_num_used_blocks(g) for g in range(manager.get_num_groups())))
            logits = runner.step(entries) if entries else None
            if logits is not None:
                data = logits.detach().to("cpu", torch.float32).contiguous().numpy()
                if sys.byteorder != "little":
                    data = data.byteswap()
                tmp = os.path.join(args.out, f".{number}.f32.tmp")
                data.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{number}.f32"))
            else:
                torch.cuda.current_stream().synchronize()
            for e in entries:
                e.seq.set_num_computed_tokens(e.start + e.count)
                manager.release_passed(e.seq)
            for rid in step.get("end", []):
                seq = live.pop(str(rid), None)
                if seq is not None:
                    manager.free(seq)
            sys.stdout.write(f"done {number}\n")
            sys.stdout.flush()
        with open(os.path.join(args.out, "pages.json"), "w", encoding="utf-8") as f:
            json.dump({"pool_pages": num_blocks, "block_size": args.block_size,
                       "allocations": manager.get_num_allocations(), "reuses": manager.get_num_reuses(),
                       "peak_used_pages": peak_used, "steps": runner.num_steps, "graph_steps": runner.num_graph_steps,
                       "decode_graphs_captured": sum(g.graph is not None for g in runner._graphs.values()),
                       # (rows, width of the block tables, what the mixers launch differently in a partly filled step)
                       "decode_graph_shapes": sorted(([k[0], k[1], list(k[2])] for k, g in runner._graphs.items()
                                                      if g.graph is not None), key=repr),
                       "prompt_graphs_captured": sum(g.graph is not None for g in runner._prompt_graphs.values())}, f)
        problem = manager.audit()
        if problem:
            print(f"trace_run: cache audit failed: {problem}", file=sys.stderr)
            return 3
    return 0


if __name__ == "__main__":
    sys.exit(main())
