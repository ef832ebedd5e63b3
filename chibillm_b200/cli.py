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

Prompts given on the command line (``--prompt-ids``, ``--prompt-file``) are
run and the program exits; with ``--max-seqs`` above 1 they are submitted
together and the scheduler mixes their prompt portions and decoded tokens in
one batch.  The limits are derived as the reference derives them
(src/main.cpp:55-98): pages = context / page size (times the number of
sequences, unless ``--kv-blocks`` says otherwise), one sequence and batches of
512 tokens for a conversation.

Options the reference has and this engine does not build are refused by name:
``--serve`` and ``--kv-cache-tokens`` (HTTP server), ``--prompt-cache-mib``
other than 0 (prefix cache), ``--quantize q4`` (quantized weights).
"""
from __future__ import annotations

import json
import os
import sys
import time
from dataclasses import dataclass, field, replace
from typing import List, Optional

KV_BLOCK_SIZE = 16          # src/cli_options.h:15

USAGE = """Usage: python -m chibillm_b200 [--context-length N] [--max-tokens N] [model-directory]
  --context-length N  Prompt + output capacity (default: 32768; multiple of the page size)
  --max-tokens N      Reply limit (default: 8192)
  --quantize none     Only 'none': quantized weights are not built in this engine
  --prompt-cache-mib 0  Only 0: the prefix cache is not built in this engine
  --no-stream         Print replies only when complete
  --progress=auto|off  Prefill progress on terminals (default: auto)
  --metrics-jsonl PATH  Append request metrics, one JSON object a line
  --random CONFIG.json  Random weights for the architecture and sizes of this config.json
                      (instead of a model directory)
  --weights-seed S    Seed of the random weights (default: 0)
  --dtype bfloat16|float32  Arithmetic of the engine (default: bfloat16)
  --device cuda[:N]   Device to run on (default: cuda:0)
  --temperature T     0 = greedy (default); otherwise sample with softmax(logits / T)
  --seed S            Seed of the sampler (default: 0)
  --ignore-eos        Do not stop at the end-of-sequence token
  --prompt-ids IDS    Run one prompt (ids separated by commas) and exit; may be repeated
  --prompt-file PATH  Run the prompts of a file (one line of ids each) and exit
  --max-seqs N        Requests that run at the same time (default: 1)
  --max-batch-tokens N  Tokens of one step (default: 512 for one request, else 4096)
  --prefill-chunk N   Largest prompt portion while others wait or decode (default: 64 for one request, else 1024)
  --kv-block-size N   Tokens of a cache page (default: 16)
  --kv-blocks N       Pages of the cache pool (default: context / page size for each of --max-seqs)
  --profile           Time every kernel launch; print a table at the end
  --profile-passes    With --profile: one line per step (launches, device and wall milliseconds)
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
    device: str = "cuda:0"
    temperature: float = 0.0
    seed: int = 0
    ignore_eos: bool = False
    prompts: List[List[int]] = field(default_factory=list)
    random_config: str = ""
    weights_seed: int = 0
    max_seqs: int = 1
    max_batch_tokens: int = 0        # 0: derived from max_seqs
    prefill_chunk: int = 0           # 0: derived from max_seqs
    kv_block_size: int = KV_BLOCK_SIZE
    kv_blocks: int = 0               # 0: derived from the context length
    profile: bool = False
    profile_passes: bool = False
    help: bool = False

    def derived(self) -> "CliOptions":
        """The options with what was left open filled in (src/main.cpp:86-98: one
        sequence and 512 tokens a batch for a conversation; sizes for a B200
        when several requests run together)."""
        batch = self.max_batch_tokens or (512 if self.max_seqs == 1 else 4096)
        chunk = self.prefill_chunk or (64 if self.max_seqs == 1 else 1024)
        return replace(self, max_batch_tokens=batch, prefill_chunk=chunk)


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
            if not v.isdigit() or int(v) == 0:
                raise CliError(f"invalid token limit for {arg}: {v}")
            if arg == "--context-length":
                o.context_length = int(v)
            else:
                o.max_tokens = int(v)
        elif arg in ("--max-seqs", "--max-batch-tokens", "--prefill-chunk", "--kv-block-size", "--kv-blocks"):
            v = value(arg)
            if not v.isdigit() or int(v) == 0:
                raise CliError(f"invalid count for {arg}: {v}")
            setattr(o, arg[2:].replace("-", "_"), int(v))
        elif arg == "--random":
            v = value(arg)
            if not v or v.startswith("-"):
                raise CliError("missing path for --random")
            o.random_config = v
        elif arg == "--weights-seed":
            v = value(arg)
            if not v.isdigit():
                raise CliError(f"invalid seed: {v}")
            o.weights_seed = int(v)
        elif arg == "--device":
            v = value(arg)
            if not (v == "cuda" or (v.startswith("cuda:") and v[5:].isdigit())):
                raise CliError(f"invalid device: {v} (this engine runs on CUDA devices only)")
            o.device = v if ":" in v else "cuda:0"
        elif arg == "--prompt-file":
            v = value(arg)
            try:
                with open(v, encoding="utf-8") as f:
                    lines = [line.strip() for line in f]
            except OSError:
                raise CliError(f"failed to read prompt file: {v}") from None
            o.prompts += [parse_ids(line) for line in lines if line and not line.startswith("#")]
        elif arg == "--profile":
            o.profile = True
        elif arg == "--profile-passes":
            o.profile = o.profile_passes = True
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
    if o.context_length % o.kv_block_size:
        raise CliError(f"invalid token limit for --context-length: {o.context_length}")
    if o.random_config and has_directory:
        raise CliError("give a model directory or --random, not both")
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


def run(options: CliOptions, stdin=None, stdout=None, stderr=None, kernels=None, device=None) -> int:
    """``kernels`` and ``device``: a stand-in for the CUDA kernels and the device
    it works on (tests run the loop on a CPU with the plain restatements); None
    for the product's own kernels on ``options.device``."""
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
    options = options.derived()
    started = time.perf_counter()
    source = options.random_config or options.model_directory
    try:
        random_config = None
        if options.random_config:
            try:
                with open(options.random_config, encoding="utf-8") as f:
                    random_config = json.load(f)
            except (OSError, ValueError) as e:
                print(f"failed to read configuration {options.random_config}: {e}", file=stderr)
                return 1
        # pages: the context of every sequence unless told otherwise (src/main.cpp:55-61,86-88)
        pages = options.kv_blocks or (options.context_length // options.kv_block_size) * options.max_seqs
        llm = LLM(None if random_config is not None else options.model_directory, dtype=options.dtype,
                  device=device or options.device, context_length=options.context_length,
                  kv_cache_tokens=pages * options.kv_block_size, max_sequences=options.max_seqs,
                  max_batch_tokens=options.max_batch_tokens, prefill_chunk_tokens=options.prefill_chunk,
                  page_size=options.kv_block_size, kernels=kernels, random_config=random_config,
                  random_seed=options.weights_seed)
    except ConfigError as e:
        what = ("unsupported model architecture in " if e.code == "unsupported_architecture"
                else "failed to load model from ")
        print(f"{what}{source}: {e}", file=stderr)
        return 1
    except (WeightError, OSError, RuntimeError, ValueError) as e:
        print(f"failed to load model from {source}: {e}", file=stderr)
        return 1
    profiler = None
    if options.profile:
        enable = getattr(llm.runner.runtime.kernels, "enable_profiling", None)
        if enable is None:
            print("--profile: these kernels have no profiling mode", file=stderr)
            return 1
        profiler = enable()
        llm.engine.profile_passes = options.profile_passes
    context = llm.context_length
    if context < 2:
        print("model context is too small for generation", file=stderr)
        return 1
    max_tokens = min(options.max_tokens, context - 1)
    print(f"[perf] model loaded in {time.perf_counter() - started:.2f} s", file=stderr)
    print(f"[limits] context {context} tok | max output {max_tokens} tok | sequences {options.max_seqs} | "
          f"batch {options.max_batch_tokens} tok | prompt portion {options.prefill_chunk} tok | "
          f"pages {llm.runner.plan.groups[0].num_pages if llm.runner.plan.groups else 0} x {options.kv_block_size} tok",
          file=stderr)

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
            record.update({"request_id": request, "model": os.path.basename(os.path.normpath(source)),
                           "context_tokens": context, "stream": options.stream,
                           "max_batch_tokens": options.max_batch_tokens, "kv_block_size": options.kv_block_size})
            metrics_file.write(json.dumps(record) + "\n")
            metrics_file.flush()
        engine.remove(request)
        return reply

    def generate_together(prompts: List[List[int]]) -> bool:
        """All prompts submitted at once; the scheduler admits as many as fit and
        mixes prompt portions with decoded tokens.  Replies are printed in the
        order of the prompts once all are complete."""
        nonlocal request
        ids = []
        try:
            for prompt in prompts:
                if len(prompt) >= context:
                    print(f"a prompt of {len(prompt)} tokens does not fit a context of {context}", file=stderr)
                    return False
                request += 1
                ids.append(request)
                params = SamplingParams(max_new_tokens=min(max_tokens, context - len(prompt)),
                                        ignore_eos=options.ignore_eos, temperature=options.temperature,
                                        seed=options.seed)
                engine.add(request, prompt, params, sample_key=request - 1)
            while not engine.is_finished():
                engine.step()
        except Exception as e:
            print(f"generation failed: {e}", file=stderr)
            return False
        for rid in ids:
            reply = engine.remove(rid).completion
            stdout.write(" ".join(map(str, reply)) + "\n")
            record = engine.metrics[rid].as_dict()
            print(_perf_line(record), file=stderr)
            print(f"[stop] {record['finish_reason']}", file=stderr)
            if metrics_file is not None:
                record.update({"request_id": rid, "model": os.path.basename(os.path.normpath(source)),
                               "context_tokens": context, "stream": False,
                               "max_batch_tokens": options.max_batch_tokens,
                               "kv_block_size": options.kv_block_size})
                metrics_file.write(json.dumps(record) + "\n")
                metrics_file.flush()
        stdout.flush()
        return True

    def finish() -> None:
        if profiler is not None:
            profiler.dump(stderr)

    if options.prompts and options.max_seqs > 1:
        ok = generate_together(options.prompts)
        finish()
        return 0 if ok else 1
    if options.prompts:
        ok = all(generate(p) is not None for p in options.prompts)
        finish()
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
    finish()
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
