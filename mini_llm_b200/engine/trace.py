"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: every
step goes through ``Engine.step``, the function generation uses.  The
reference's counterpart (scripts/golden_logits.py:33-54) replays a prompt and
40 teacher-forced single-token steps through its session API and saves every
row of logits; here the trace also says how the tokens are cut into steps and
batched.

Input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits
at the wanted places, in the order of the entries and of ``want``, as
little-endian float32 ``[wanted, vocab]``.  After every step ``done <step>`` is
printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def parse_args(argv=None):
    parser = argparse.ArgumentParser(prog="trace_run", description="Replay a trace of token ids through the engine")
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    parser.add_argument("--max-requests", type=int, default=8, help="most requests live at a time")
    parser.add_argument("--plain-kernels", action="store_true", help="run the plain kernel of every operation")
    return parser.parse_args(argv)


def replay(args, lines, out=sys.stdout):
    from .engine import Engine, StepEntry

    if args.page_size <= 0 or 64 % args.page_size != 0:
        raise SystemExit("--page-size must divide 64")
    os.makedirs(args.out, exist_ok=True)
    # a step of a trace may bring every token the cache holds at once
    engine = Engine(args.model, dtype=args.dtype, page_size=args.page_size, cache_tokens=args.max_tokens,
                    max_requests=args.max_requests, plain_kernels=args.plain_kernels,
                    max_tokens_per_step=max(int(args.max_tokens), 1))
    slots = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            name = item["id"]
            if name not in slots:
                slot = engine.open_request()
                if slot is None:
                    raise SystemExit(f"step {step}: no free slot for request '{name}' "
                                     f"(at most {args.max_requests} are live at a time)")
                slots[name] = slot
            entries.append(StepEntry(slots[name], list(item["tokens"]), list(item.get("want", []))))
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                host = logits.to("cpu", copy=True).numpy().astype("<f4", copy=False)
                engine.check_status()
                host.tofile(os.path.join(args.out, f"{step}.f32"))
        for name in record.get("end", []):
            if name in slots:
                engine.close_request(slots.pop(name))
        print(f"done {step}", file=out, flush=True)
    return 0


def main(argv=None):
    args = parse_args(argv)
    return replay(args, sys.stdin)
