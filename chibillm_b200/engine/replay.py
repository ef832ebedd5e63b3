"""Trace replay: feeds given token ids through a model step by step and writes
the logits that are asked for.  It samples nothing and has no model code of its
own: every step is one call of :meth:`ModelRunner.step`, the call that
generation makes, on the same model, cache and kernels.

Input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step that wants something, ``<out>/<step>.f32`` holds the logits of the
wanted places, in the order of the entries and of ``want``, as little-endian
float32 ``[wanted, vocab]``.  After every step a line ``done <step>`` is
printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Iterable, Optional

import numpy as np

from .batch import StepEntry
from .runner import ModelRunner


def replay_step(runner: ModelRunner, obj: dict, out_dir: Optional[str]):
    """Run one line of a trace; returns the logits as a numpy array or None."""
    entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in obj.get("entries", [])]
    result = None
    if entries:
        logits = runner.step(entries)
        if logits is not None:
            result = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            if out_dir is not None:
                result.tofile(os.path.join(out_dir, f"{obj['step']}.f32"))
    for request_id in obj.get("end", []):
        runner.end(request_id)
    return result


def replay(runner: ModelRunner, lines: Iterable[str], out_dir: str, report: IO = sys.stdout) -> int:
    os.makedirs(out_dir, exist_ok=True)
    steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        replay_step(runner, obj, out_dir)
        report.write(f"done {obj['step']}\n")
        report.flush()
        steps += 1
    return steps


def main(argv=None) -> int:
    import argparse

    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time (the cache pool's size)")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (default 16)")
    parser.add_argument("--max-requests", type=int, default=8, help="most live requests (default 8)")
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)
    if args.max_tokens <= 0 or args.page_size <= 0 or 64 % args.page_size != 0:
        parser.error("--max-tokens must be positive and --page-size must divide 64")
    runner = ModelRunner.from_folder(args.model, dtype=args.dtype, device=args.device,
                                     page_size=args.page_size, pool_tokens=args.max_tokens,
                                     max_requests=args.max_requests)
    replay(runner, iter(sys.stdin.readline, ""), args.out)
    return 0
