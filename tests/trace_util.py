"""Building replay traces (the JSON steps ``bin/trace_run`` reads) in several cuttings and
replaying them, in process through ``ModelRunner.step`` or through the program itself."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PORTIONS = [7, 2, 13, 5, 3, 11, 2, 29, 4, 17]


def ceil64(n: int) -> int:
    return -(-n // 64) * 64


def cut_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, one after the other."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def cut_last_decoded(requests: dict[str, list[int]], n_last: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``n_last`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - n_last) if len(toks) > 1 else 1
        pieces = [toks[:head]] + [[t] for t in toks[head:]]
        for i, piece in enumerate(pieces):
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": piece, "want": list(range(len(piece)))}],
                          "end": [rid] if i == len(pieces) - 1 else []})
    return steps


def cut_portions(requests: dict[str, list[int]], sizes=PORTIONS) -> list[dict]:
    """Portions of changing size, down to two tokens."""
    steps = []
    k = 0
    for rid, toks in requests.items():
        pos = 0
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            piece = toks[pos:pos + n]
            pos += n
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": piece, "want": list(range(len(piece)))}],
                          "end": [rid] if pos == len(toks) else []})
    return steps


def cut_mixed(requests: dict[str, list[int]], n_decode: int = 12, max_live: int = 4, sizes=PORTIONS,
              skip_every: int = 5) -> list[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of
    others; now and then a request sits a step out; a finished request ends and the next
    one comes in (so its pages are used again)."""
    pending = list(requests.items())
    live: list[list] = []     # [rid, tokens, pos]
    steps: list[dict] = []
    k = 0
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live.append([rid, toks, 0])
        entries, ended = [], []
        for idx, item in enumerate(list(live)):
            rid, toks, pos = item
            k += 1
            if len(live) > 1 and k % skip_every == 0 and entries:
                continue      # left out of this step, goes on later
            prefill_end = max(1, len(toks) - n_decode)
            if pos < prefill_end:
                n = min(sizes[k % len(sizes)], prefill_end - pos)
            else:
                n = 1
            piece = toks[pos:pos + n]
            item[2] = pos + n
            entries.append({"id": rid, "tokens": piece, "want": list(range(len(piece)))})
            if item[2] == len(toks):
                ended.append(rid)
        steps.append({"step": len(steps), "entries": entries, "end": ended})
        live = [it for it in live if it[0] not in ended]
    return steps


def max_tokens_needed(steps: list[dict]) -> int:
    """The most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    held: dict[str, int] = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(ceil64(n) for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


def collect(steps: list[dict], per_step: dict[int, np.ndarray], vocab: int) -> dict[str, np.ndarray]:
    """Per request, the logits of every fed position in feed order."""
    out: dict[str, list[np.ndarray]] = {}
    for s in steps:
        if not any(e["want"] for e in s["entries"]):
            continue
        arr = per_step[s["step"]].reshape(-1, vocab)
        row = 0
        for e in s["entries"]:
            n = len(e["want"])
            out.setdefault(e["id"], []).append(arr[row:row + n])
            row += n
        assert row == arr.shape[0]
    return {rid: np.concatenate(chunks, axis=0) for rid, chunks in out.items()}


def replay_in_process(runner, steps: list[dict]) -> dict[int, np.ndarray]:
    from mini_infer_b200.engine import StepEntry

    per_step = {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if e["id"] not in runner.cache:
                runner.add_request(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        res = runner.step(entries)
        if res.rows:
            per_step[s["step"]] = res.logits.float().cpu().numpy()
        for rid in s["end"]:
            runner.free_request(rid)
    return per_step


def replay_program(model_dir: str, dtype: str, steps: list[dict], out_dir: str, block_size: int = 16,
                   timeout: int = 900) -> dict[int, np.ndarray]:
    """Run ``bin/trace_run`` as a user would, feeding steps one at a time."""
    cmd = [os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens_needed(steps)), "--block-size", str(block_size)]
    env = dict(os.environ, MINI_INFER_PYTHON=sys.executable)
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"unexpected answer {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    per_step = {}
    for s in steps:
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if any(e["want"] for e in s["entries"]):
            per_step[s["step"]] = np.fromfile(path, dtype="<f4")
    return per_step


def plain_logits(state: dict[str, torch.Tensor], raw_config: dict, requests: dict[str, list[int]]):
    import plain_impl as P

    return {rid: P.llama_logits(state, raw_config, toks, dtype=torch.float64).numpy()
            for rid, toks in requests.items()}


def max_err(got: dict[str, np.ndarray], want: dict[str, np.ndarray]) -> tuple[float, float]:
    """``(largest absolute difference, largest |reference logit|)`` over all requests."""
    err = max(float(np.abs(got[r] - want[r]).max()) for r in want)
    scale = max(float(np.abs(want[r]).max()) for r in want)
    return err, scale


# What a row of logits may differ by from its reference.
#
# float32: rounding of a few hundred fp32 operations: 1e-4 of max(1, largest |reference logit|)
# (observed: 4e-6 and less).
#
# bfloat16, two bounds, both relative to the largest |reference logit| itself, with no floor:
# * no single logit further off than 3e-2 of it.  Activations are rounded to 8 bits of mantissa
#   about eight times per layer and attention that is peaked amplifies the rounding of its scores;
#   over the hundreds of thousands of logits of a test the largest error observed is 1.0 to
#   1.9e-2 of the scale for the tiny configurations;
# * no row whose root-mean-square error is above 1e-2 of it (observed over all rows: 1.4 to
#   2.6e-3 of the scale).  A wrong key, position or page moves a whole row by tens of percent.
class Bound(float):
    """The largest allowed |difference| (the float itself) and, optionally, the largest allowed
    root-mean-square difference of a row."""

    rms: float | None = None

    def __new__(cls, max_abs: float, rms: float | None = None):
        b = super().__new__(cls, max_abs)
        b.rms = rms
        return b


def tolerance(dtype: str, largest_logit: float) -> Bound:
    if dtype == "float32":
        return Bound(1e-4 * max(1.0, largest_logit))
    return Bound(3e-2 * largest_logit, rms=1e-2 * largest_logit)


def first_bad(got: np.ndarray, want: np.ndarray, tol: float) -> int | None:
    """The first row that is out of bounds (``tol`` a number or a ``Bound``)."""
    diff = got - want
    wrong = np.abs(diff).max(axis=1) > float(tol)
    rms = getattr(tol, "rms", None)
    if rms is not None:
        wrong |= np.sqrt((diff.astype(np.float64) ** 2).mean(axis=1)) > rms
    bad = np.nonzero(wrong)[0]
    return int(bad[0]) if bad.size else None
