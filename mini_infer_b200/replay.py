"""Trace replay: feed given token ids through the model step by step and write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps are read from standard input, one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch through the engine's own step function, cache
and kernels (nothing is sampled).  For a step that wants logits, ``<out>/<step>.f32``
receives them as little-endian float32 ``[wanted, vocab]`` in the order of the entries and
of ``want``.  After every step a line ``done <step>`` is printed and flushed.  Requests
listed under ``end`` give back what they hold after the step.  ``--max-tokens`` sizes the
page pool: the most tokens live requests hold at any time, each request's count rounded up
to a multiple of 64.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens held by live requests at any time (each rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-requests", type=int, default=8)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from .engine import ModelRunner, StepEntry

    os.makedirs(args.out, exist_ok=True)
    if args.block_size <= 0 or 64 % args.block_size:
        ap.error("--block-size must divide 64")
    num_blocks = max(1, -(-args.max_tokens // args.block_size))
    print(f"[trace_run] loading {args.model} ({args.dtype}), {num_blocks} pages of {args.block_size}",
          file=sys.stderr, flush=True)
    runner = ModelRunner.from_pretrained(
        args.model, device=args.device, dtype=args.dtype, num_blocks=num_blocks,
        block_size=args.block_size, max_requests=args.max_requests,
    )
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            if e["id"] not in runner.cache:
                runner.add_request(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        if entries:
            result = runner.step(entries)
            if result.rows:
                arr = result.logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            if rid in runner.cache:
                runner.free_request(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
