"""The ``lyapunov`` command line.

``lyapunov generate`` keeps the reference's options with their names, meanings
and defaults (python/lyapunov_engine/entrypoints/cli.py:82-98): --model,
--prompt, --max-tokens 64, --temperature 0.7, --top-p 1.0, --block-size 16,
--num-blocks 512, --max-num-seqs 16, --max-batched-tokens 2048.  Added:
--prompt-ids (token ids, no tokenizer needed), --top-k, --dtype, --seed,
--ignore-eos, --device, and --random-weights (``--model`` then names a
config.json, or a folder that holds one, and the weights are drawn from
--seed; nothing is read from or written to the folder).  The text tokenizer, as in the reference, is the one
``transformers.AutoTokenizer`` finds in the model folder; it is loaded only
when --prompt is given.

``lyapunov random-weights`` writes a model folder (config.json,
model.safetensors) from a config.json and a seed.  ``lyapunov replay`` is
bin/trace_run.  The reference's ``serve`` sub-command (an HTTP server) is not
part of this engine.
"""
from __future__ import annotations

import argparse
import json
import sys


def run_generate(args) -> int:
    import torch

    from ..engine.llm_engine import EngineConfig, LLMEngine, load_model
    from ..sampling import SamplingParams

    tokenizer = None
    if args.prompt_ids is not None:
        prompt_tokens = [int(x) for x in args.prompt_ids.replace(",", " ").split()]
    elif args.prompt is not None:
        from transformers import AutoTokenizer

        print(f"Loading tokenizer: {args.model}")
        tokenizer = AutoTokenizer.from_pretrained(args.model)
        prompt_tokens = tokenizer.encode(args.prompt)
    else:
        print("lyapunov generate: give --prompt or --prompt-ids", file=sys.stderr)
        return 2
    if not torch.cuda.is_available():
        print("lyapunov generate: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 1
    config = EngineConfig(block_size=args.block_size, num_gpu_blocks=args.num_blocks, max_num_seqs=args.max_num_seqs,
                          max_num_batched_tokens=args.max_batched_tokens, dtype=args.dtype, device=args.device)
    if args.random_weights:
        import os

        path = os.path.join(args.model, "config.json") if os.path.isdir(args.model) else args.model
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
        print(f"Random weights (seed {args.seed}) for {path}")
        loaded = load_model(config=raw, random_seed=args.seed, dtype=config.dtype, device=args.device)
    else:
        print(f"Loading weights: {args.model}")
        loaded = load_model(args.model, config.dtype, args.device)
    config.model_config = loaded.spec
    engine = LLMEngine(loaded, config)
    sampling = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                              max_tokens=args.max_tokens, ignore_eos=args.ignore_eos, seed=args.seed)
    engine.add_request("req-0", prompt_tokens, sampling)
    print("\n--- Output Generation ---")
    while engine.has_unfinished_requests():
        for out in engine.step():
            if out.is_finished:
                if out.finish_reason == "error":
                    print(f"request failed: {out.error}", file=sys.stderr)
                    return 1
                if tokenizer is not None:
                    print(tokenizer.decode(out.output_tokens, skip_special_tokens=True))
                else:
                    print(" ".join(str(t) for t in out.output_tokens))
    return 0


def run_random_weights(args) -> int:
    import torch

    from ..weights import write_random_model

    with open(args.config, "r", encoding="utf-8") as f:
        config = json.load(f)
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    write_random_model(args.out, config, args.seed, dtype, std=args.std, norm_jitter=args.norm_jitter)
    print(f"wrote {args.out}/config.json and {args.out}/model.safetensors")
    return 0


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="lyapunov", description="lyapunov_engine_b200: LLM inference on one B200")
    sub = parser.add_subparsers(dest="subcommand", required=True)

    gen = sub.add_parser("generate", help="Run text generation from prompt")
    gen.add_argument("--model", type=str, required=True, help="model folder (config.json, *.safetensors)")
    gen.add_argument("--prompt", type=str, default=None, help="Prompt text")
    gen.add_argument("--prompt-ids", type=str, default=None, help="prompt as token ids, e.g. 1,15,27")
    gen.add_argument("--max-tokens", type=int, default=64)
    gen.add_argument("--temperature", type=float, default=0.7)
    gen.add_argument("--top-p", type=float, default=1.0)
    gen.add_argument("--top-k", type=int, default=-1)
    gen.add_argument("--block-size", type=int, default=16)
    gen.add_argument("--num-blocks", type=int, default=512)
    gen.add_argument("--max-num-seqs", type=int, default=16)
    gen.add_argument("--max-batched-tokens", type=int, default=2048)
    gen.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    gen.add_argument("--seed", type=int, default=0)
    gen.add_argument("--ignore-eos", action="store_true")
    gen.add_argument("--random-weights", action="store_true",
                     help="--model names a config.json (or a folder with one); weights are drawn from --seed")
    gen.add_argument("--device", type=str, default="cuda:0")

    rnd = sub.add_parser("random-weights", help="Write a model folder with seeded random weights")
    rnd.add_argument("--config", required=True, help="a config.json naming the architecture and its sizes")
    rnd.add_argument("--out", required=True, help="folder to write")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    rnd.add_argument("--std", type=float, default=0.02)
    rnd.add_argument("--norm-jitter", type=float, default=0.0)

    sub.add_parser("replay", help="Trace replay (same as bin/trace_run)", add_help=False)
    return parser


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        from ..replay.trace_run import main as replay_main

        return replay_main(argv[1:])
    args = build_parser().parse_args(argv)
    if args.subcommand == "generate":
        return run_generate(args)
    if args.subcommand == "random-weights":
        return run_random_weights(args)
    return 2


if __name__ == "__main__":
    sys.exit(main())
