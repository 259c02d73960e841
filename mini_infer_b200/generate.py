"""Command line: generate tokens from a model folder.

    python -m mini_infer_b200.generate --model DIR --prompt-ids 1,2,3 --max-tokens 32

Option names mirror the keyword arguments of the Python entry point, which are the
reference's where it has them (``ModelRunner.from_pretrained``: ``--dtype``, ``--device``,
``--num-blocks``, ``--block-size``; ``ContinuousScheduler``: ``--max-concurrent``,
``--chunk-size``, ``--decode-headroom-blocks``, ``--trace-out``; request fields:
``--max-tokens``, ``--temperature``, ``--top-k``, ``--top-p``).  The reference's server
reads its settings from ``MINI_INFER_MODEL``, ``MINI_INFER_NUM_BLOCKS`` and
``MINI_INFER_BLOCK_SIZE`` (``api/server.py:74-126``); the same variables give this
program's defaults.  ``--random-weights`` writes a model folder from ``--config`` and
``--seed`` first (into ``--model``) and then runs from it.
"""

from __future__ import annotations

import argparse
import json
import os
import sys


def parse_ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv=None) -> int:
    env = os.environ
    ap = argparse.ArgumentParser(prog="python -m mini_infer_b200.generate",
                                 description="Generate tokens with the B200 engine.")
    ap.add_argument("--model", default=env.get("MINI_INFER_MODEL"), help="model folder (config.json + safetensors)")
    ap.add_argument("--config", help="config.json for --random-weights")
    ap.add_argument("--random-weights", action="store_true",
                    help="write seeded random weights for --config into --model first")
    ap.add_argument("--seed", type=int, default=0, help="seed of --random-weights")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="token ids of one prompt, comma or space separated (repeatable)")
    ap.add_argument("--prompt-file", help="JSON file: a list of prompts, each a list of token ids")
    ap.add_argument("--prompt", action="append", default=[],
                    help="text prompt (needs tokenizer files in the model folder)")
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--sampling-seed", type=int, default=None)
    ap.add_argument("--num-blocks", type=int, default=int(env.get("MINI_INFER_NUM_BLOCKS", 1024)))
    ap.add_argument("--block-size", type=int, default=int(env.get("MINI_INFER_BLOCK_SIZE", 16)))
    ap.add_argument("--max-concurrent", type=int, default=16)
    ap.add_argument("--chunk-size", type=int, default=None,
                    help="most prompt tokens one request feeds in a step (default: the step's token budget)")
    ap.add_argument("--max-tokens-per-step", type=int, default=2048)
    ap.add_argument("--decode-headroom-blocks", type=int, default=8)
    ap.add_argument("--eos-token-id", type=int, action="append", default=[])
    ap.add_argument("--cuda-graph", action="store_true", help="replay decode-only steps as CUDA graphs")
    ap.add_argument("--trace-out", help="write a Chrome trace of the engine steps here")
    args = ap.parse_args(argv)
    if not args.model:
        ap.error("--model (or MINI_INFER_MODEL) is required")

    if args.random_weights:
        if not args.config:
            ap.error("--random-weights needs --config")
        from .weights import write_random_model

        with open(args.config, "r", encoding="utf-8") as f:
            raw = json.load(f)
        write_random_model(raw, args.model, args.seed)

    from .engine import ContinuousScheduler, ModelRunner, Request
    from .sampling import SamplingParams

    runner = ModelRunner.from_pretrained(args.model, device=args.device, dtype=args.dtype,
                                         num_blocks=args.num_blocks, block_size=args.block_size,
                                         max_requests=args.max_concurrent, cuda_graph=args.cuda_graph)
    tokenizer = None
    if args.prompt:
        from .engine.tokenizer import Tokenizer

        tokenizer = Tokenizer.from_pretrained(args.model)
    prompts: list = [parse_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file, "r", encoding="utf-8") as f:
            prompts.extend(json.load(f))
    prompts.extend(args.prompt)
    if not prompts:
        ap.error("give at least one of --prompt-ids, --prompt-file, --prompt")
    eos = list(args.eos_token_id)
    if tokenizer is not None and tokenizer.eos_token_id is not None:
        eos.append(tokenizer.eos_token_id)
    scheduler = ContinuousScheduler(
        runner, max_concurrent=args.max_concurrent, chunk_size=args.chunk_size,
        max_tokens_per_step=args.max_tokens_per_step, decode_headroom_blocks=args.decode_headroom_blocks,
        eos_token_ids=eos, tokenizer=tokenizer, trace_out=args.trace_out,
    )
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            seed=args.sampling_seed)
    results = scheduler.generate([Request(p, params, args.max_tokens) for p in prompts])
    scheduler.stop()
    for r in results:
        print(json.dumps({"tokens": r.tokens, "text": r.text, "finish_reason": r.finish_reason,
                          "prompt_tokens": r.prompt_tokens}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
