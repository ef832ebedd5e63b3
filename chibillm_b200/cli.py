"""The command line, in the manner of the reference's (src/cli_options.cc,
src/main.cpp, src/repl.cc): the same option names with the same meanings where
the reference has them, a read-eval-print loop on standard input, `[perf]` and
`[limits]` lines on standard error, one JSON record per request with
``--metrics-jsonl``.

The reference reads text and runs a tokenizer; tokenizers are outside this
engine, so a prompt here is a line of token ids (separated by blanks or commas)
and a reply is a line of token ids.  ``/reset`` forgets the history (the ids of
earlier turns are fed again before a new prompt, as the reference feeds its chat
history), ``/quit`` or ``/exit`` leaves.

Options the reference has and this engine does not build are refused by name:
``--serve`` and ``--kv-cache-tokens`` (HTTP server), ``--prompt-cache-mib``
other than 0 (prefix cache), ``--quantize q4`` (quantized weights).
"""
from __future__ import annotations

import json
import os
import sys
import time
from dataclasses import dataclass, field
from typing import List, Optional

KV_BLOCK_SIZE = 16          # src/cli_options.h:15

USAGE = """Usage: python -m chibillm_b200 [--context-length N] [--max-tokens N] [model-directory]
  --context-length N  Prompt + output capacity (default: 32768; multiple of 16)
  --max-tokens N      Reply limit (default: 8192)
  --quantize none     Only 'none': quantized weights are not built in this engine
  --prompt-cache-mib 0  Only 0: the prefix cache is not built in this engine
  --no-stream         Print replies only when complete
  --progress=auto|off  Prefill progress on terminals (default: auto)
  --metrics-jsonl PATH  Append request metrics, one JSON object a line
  --dtype bfloat16|float32  Arithmetic of the engine (default: bfloat16)
  --temperature T     0 = greedy (default); otherwise sample with softmax(logits / T)
  --seed S            Seed of the sampler (default: 0)
  --ignore-eos        Do not stop at the end-of-sequence token
  --prompt-ids IDS    Run one prompt (ids separated by commas) and exit; may be repeated
  --help              Show this help
"""


@dataclass
class CliOptions:
    model_directory: str = "qwen3_model"
    context_length: int = 32768
    max_tokens: int = 8192
    stream: bool = True
    progress: bool = True
    metrics_jsonl: str = ""
    dtype: str = "bfloat16"
    temperature: float = 0.0
    seed: int = 0
    ignore_eos: bool = False
    prompts: List[List[int]] = field(default_factory=list)
    help: bool = False


class CliError(ValueError):
    pass


def parse_ids(text: str) -> List[int]:
    parts = text.replace(",", " ").split()
    if not parts:
        raise CliError("a prompt needs at least one token id")
    try:
        ids = [int(p) for p in parts]
    except ValueError:
        raise CliError(f"token ids must be integers: {text!r}") from None
    if any(i < 0 for i in ids):
        raise CliError(f"token ids must not be negative: {text!r}")
    return ids


def parse_cli_options(argv: List[str]) -> CliOptions:
    """Same rules as src/cli_options.cc:28-101: a flag that takes a value takes
    the next argument; an unknown flag or a second model directory is an error."""
    o = CliOptions()
    has_directory = False
    i = 0

    def value(flag: str) -> str:
        nonlocal i
        i += 1
        if i >= len(argv):
            raise CliError(f"missing value for {flag}")
        return argv[i]

    while i < len(argv):
        arg = argv[i]
        if arg in ("--help", "-h"):
            o.help = True
        elif arg == "--no-stream":
            o.stream = False
        elif arg in ("--progress=auto", "--progress=off"):
            o.progress = arg == "--progress=auto"
        elif arg == "--metrics-jsonl":
            v = value(arg)
            if not v or v.startswith("-"):
                raise CliError("missing path for --metrics-jsonl")
            o.metrics_jsonl = v
        elif arg == "--quantize":
            v = value(arg)
            if v not in ("none", "q4"):
                raise CliError(f"invalid quantization: {v}")
            if v != "none":
                raise CliError("--quantize q4: quantized weights are not built in this engine")
        elif arg == "--serve":
            raise CliError("--serve: the HTTP server is not built in this engine")
        elif arg == "--kv-cache-tokens":
            value(arg)
            raise CliError("--kv-cache-tokens requires --serve, which is not built in this engine")
        elif arg == "--prompt-cache-mib":
            v = value(arg)
            if not v.isdigit():
                raise CliError(f"invalid prompt cache budget: {v}")
            if int(v) != 0:
                raise CliError("--prompt-cache-mib: the prefix cache is not built in this engine (use 0)")
        elif arg in ("--context-length", "--max-tokens"):
            v = value(arg)
            if not v.isdigit() or int(v) == 0 or (arg == "--context-length" and int(v) % KV_BLOCK_SIZE):
                raise CliError(f"invalid token limit for {arg}: {v}")
            if arg == "--context-length":
                o.context_length = int(v)
            else:
                o.max_tokens = int(v)
        elif arg == "--dtype":
            v = value(arg)
            if v not in ("bfloat16", "float32"):
                raise CliError(f"invalid dtype: {v}")
            o.dtype = v
        elif arg == "--temperature":
            v = value(arg)
            try:
                o.temperature = float(v)
            except ValueError:
                raise CliError(f"invalid temperature: {v}") from None
            if not (o.temperature >= 0.0):
                raise CliError(f"invalid temperature: {v}")
        elif arg == "--seed":
            v = value(arg)
            if not v.isdigit():
                raise CliError(f"invalid seed: {v}")
            o.seed = int(v)
        elif arg == "--ignore-eos":
            o.ignore_eos = True
        elif arg == "--prompt-ids":
            o.prompts.append(parse_ids(value(arg)))
        elif arg.startswith("-") or has_directory:
            raise CliError(f"unexpected argument: {arg}")
        else:
            o.model_directory = arg
            has_directory = True
        i += 1
    return o


def _perf_line(m: dict) -> str:
    parts = [f"{m['prompt_tokens']} prompt tok"]
    if m.get("prefill_tokens_per_second"):
        parts.append(f"prefill {m['prefill_tokens_per_second']:.1f} tok/s")
    parts.append(f"{m['output_tokens']} output tok")
    if m.get("decode_tokens_per_second"):
        parts.append(f"decode {m['decode_tokens_per_second']:.1f} tok/s")
    if m.get("time_to_first_token_seconds") is not None:
        parts.append(f"first token {m['time_to_first_token_seconds'] * 1e3:.1f} ms")
    return "[perf] " + " | ".join(parts)


def run(options: CliOptions, stdin=None, stdout=None, stderr=None) -> int:
    from .api import LLM
    from .config.base import ConfigError
    from .sampling.sampler import SamplingParams
    from .weights.loader import WeightError

    stdin, stdout, stderr = stdin or sys.stdin, stdout or sys.stdout, stderr or sys.stderr
    metrics_file = None
    if options.metrics_jsonl:
        try:
            metrics_file = open(options.metrics_jsonl, "a", encoding="utf-8")
        except OSError:
            print(f"failed to open metrics file: {options.metrics_jsonl}", file=stderr)
            return 1
    started = time.perf_counter()
    try:
        # one request at a time, large batches for its prompt (src/main.cpp:91-97)
        llm = LLM(options.model_directory, dtype=options.dtype, context_length=options.context_length,
                  kv_cache_tokens=options.context_length, max_sequences=1, max_batch_tokens=512)
    except ConfigError as e:
        what = ("unsupported model architecture in " if e.code == "unsupported_architecture"
                else "failed to load model from ")
        print(f"{what}{options.model_directory}: {e}", file=stderr)
        return 1
    except (WeightError, OSError, RuntimeError) as e:
        print(f"failed to load model from {options.model_directory}: {e}", file=stderr)
        return 1
    context = llm.context_length
    if context < 2:
        print("model context is too small for generation", file=stderr)
        return 1
    max_tokens = min(options.max_tokens, context - 1)
    print(f"[perf] model loaded in {time.perf_counter() - started:.2f} s", file=stderr)
    print(f"[limits] context {context} tok | max output {max_tokens} tok", file=stderr)

    engine = llm.engine
    request = 0

    def generate(prompt: List[int]) -> Optional[List[int]]:
        nonlocal request
        if len(prompt) >= context:
            print("conversation is too long; use /reset", file=stderr)
            return None
        request += 1
        budget = min(max_tokens, context - len(prompt))
        params = SamplingParams(max_new_tokens=budget, ignore_eos=options.ignore_eos,
                                temperature=options.temperature, seed=options.seed)
        try:
            engine.add(request, prompt, params)
            reply: List[int] = []
            while not engine.is_finished():
                for update in engine.step():
                    reply.append(update.token)
                    if options.stream:
                        stdout.write(("" if len(reply) == 1 else " ") + str(update.token))
                        stdout.flush()
        except Exception as e:                       # the engine left the sequences as they were
            print(f"generation failed: {e}", file=stderr)
            if engine.find_sequence(request) is not None and not engine.find_sequence(request).is_finished:
                engine.cancel(request)
            return None
        stdout.write("\n" if options.stream else " ".join(map(str, reply)) + "\n")
        stdout.flush()
        record = engine.metrics[request].as_dict()
        print(_perf_line(record), file=stderr)
        print(f"[stop] {record['finish_reason']}", file=stderr)
        if metrics_file is not None:
            record.update({"request_id": request, "model": os.path.basename(os.path.normpath(
                options.model_directory)), "context_length": context, "stream": options.stream})
            metrics_file.write(json.dumps(record) + "\n")
            metrics_file.flush()
        engine.remove(request)
        return reply

    if options.prompts:
        ok = all(generate(p) is not None for p in options.prompts)
        return 0 if ok else 1

    print("chibillm_b200 -- a prompt is a line of token ids; /reset clears history, /quit exits", file=stdout)
    history: List[int] = []
    while True:
        stdout.write("\nids> ")
        stdout.flush()
        line = stdin.readline()
        if not line or line.strip() in ("/quit", "/exit"):
            stdout.write("\n")
            break
        line = line.strip()
        if line == "/reset":
            history.clear()
            print("history cleared", file=stdout)
            continue
        if not line:
            continue
        try:
            ids = parse_ids(line)
        except CliError as e:
            print(str(e), file=stderr)
            continue
        reply = generate(history + ids)
        if reply is not None:
            history += ids + reply
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    try:
        options = parse_cli_options(argv)
    except CliError as e:
        print(str(e), file=sys.stderr)
        sys.stderr.write(USAGE)
        return 1
    if options.help:
        sys.stdout.write(USAGE)
        return 0
    return run(options)
