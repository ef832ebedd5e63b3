#!/usr/bin/env python3
"""Decode and prefill throughput of chibillm_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step.  The default run has the layer sizes of the
Qwen3-8B shape with random bfloat16 weights, a batch of 8 and a context capacity
of 4,096 tokens per request (2,048 held when decoding starts).  One JSON line is
printed: ``value`` is decoded tokens a second over K device-timed steps; ``e2e``
the same through the Python entry point (host token ids in, sampled ids out,
every step); ``prefill`` a 2,048-token prompt in one step; ``roofline`` the
decode step's bytes (every weight once, the cache of the live requests) over
its time, against the measured copy bandwidth; ``points`` decode at batch 1 and
64.  Token ids are uniform random; the caches that decoding starts from are
filled by real prefill steps for the end-to-end run and with random values for
the device-timed runs (the work of a decode step does not depend on the values).

``--timeline`` prints, instead of the record, when the CTAs of every kernel of one
decode step started, waited and ended.  ``--shape`` runs the same at the Qwen3-0.6B or
Qwen3-14B layer sizes, and
``--mixed-requests N`` replaces the record by a serving run: N requests with
prompts of 16 to 2,048 tokens and 256 new tokens each through ``LLM.generate``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "attention_bias": False,
    "hidden_act": "silu", "rope_scaling": None, "torch_dtype": "bfloat16",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 40960,
    "tie_word_embeddings": False, "use_sliding_window": False, "sliding_window": None,
}
# Other shapes of the same architecture (--shape); the default run and its record are the 8B shape.
SHAPES = {
    "qwen3-8b": {},
    "qwen3-0.6b": {"num_hidden_layers": 28, "hidden_size": 1024, "num_attention_heads": 16,
                   "num_key_value_heads": 8, "intermediate_size": 3072, "tie_word_embeddings": True},
    "qwen3-14b": {"num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40,
                  "num_key_value_heads": 8, "intermediate_size": 17408},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                obj = json.load(f)
            def number(v):
                return float(v["value"]) if isinstance(v, dict) else float(v)
            peaks = {k: number(obj[k]) for k in ("hbm_gbs", "bf16_tflops") if k in obj}
            peaks["bf16_tflops_sustained"] = number(obj.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
            if len(peaks) == 3 and all(v > 0 for v in peaks.values()):
                return peaks, "measured"
        except (OSError, ValueError, KeyError, TypeError, AttributeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed
    region runs (reading only; nothing is set)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------ accounting
def layer_weight_elements(c) -> int:
    H, I = c["hidden_size"], c["intermediate_size"]
    qw = c["num_attention_heads"] * c["head_dim"]
    kw = c["num_key_value_heads"] * c["head_dim"]
    return H * (qw + 2 * kw) + qw * H + 3 * H * I


def decode_step_bytes(c, layers, ctx_lens) -> float:
    """Bytes a decode step has to read: every weight it uses once (layers, norms,
    output matrix, the embedding rows of its tokens) and the cache of the live
    requests."""
    H = c["hidden_size"]
    weights = layers * (layer_weight_elements(c) + 2 * H + 2 * c["head_dim"]) + H + c["vocab_size"] * H
    weights += len(ctx_lens) * H
    kv_per_token = layers * 2 * c["num_key_value_heads"] * c["head_dim"]
    return 2.0 * (weights + kv_per_token * sum(ctx_lens))


def prefill_flops(c, layers, tokens, wanted_rows=1) -> float:
    linear = 2.0 * tokens * layers * layer_weight_elements(c)
    attention = layers * 2.0 * c["num_attention_heads"] * c["head_dim"] * float(tokens) * tokens
    head = 2.0 * wanted_rows * c["hidden_size"] * c["vocab_size"]
    return linear + attention + head


# ------------------------------------------------------------------ measurements
def fill_request(runner, request_id, tokens_held: int) -> None:
    """Give a request ``tokens_held`` tokens of context without running them:
    pages are reserved and hold whatever the pool was filled with."""
    runner.admit(request_id)
    runner.cache.reserve(request_id, tokens_held)
    runner.cache.commit(request_id, tokens_held)


def measure_decode(runner, sampler, batch, ctx_start, steps, warmup, vocab, tag):
    """K decode steps of ``batch`` requests, timed on the device."""
    import torch
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.sampling import SamplingParams

    ids = [f"{tag}{i}" for i in range(batch)]
    for rid in ids:
        fill_request(runner, rid, ctx_start)
    g = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, vocab, (batch,), generator=g).tolist()
    params = [SamplingParams()] * batch
    keys = list(range(batch))
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = 0
    ctx_lens = []
    for i in range(warmup + steps):
        if i == warmup:
            torch.cuda.synchronize()
            launches0 = runner.runtime.kernels.launches
            start.record()
        if i >= warmup:
            ctx_lens.append(ctx_start + i + 1)
        logits = runner.step([StepEntry(rid, [tok], [0]) for rid, tok in zip(ids, tokens)], check=False)
        pending = sampler.launch(logits, params, keys, [i] * batch)
        # as the engine does: the next step starts on the device while the tokens travel to the
        # host -- but not across the borders of the timed region, which holds exactly `steps` steps
        ahead = i != warmup - 1 and i != warmup + steps - 1 and runner.run_ahead(ids, pending.device_ids)
        tokens = pending.result()
        if ahead:
            runner.confirm_ahead(tokens)
    end.record()
    torch.cuda.synchronize()
    runner.runtime.kernels.check_error_word()
    ms = start.elapsed_time(end)
    launches = runner.runtime.kernels.launches - launches0
    for rid in ids:
        runner.end(rid)
    mean_ctx = sum(ctx_lens) / len(ctx_lens)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
            "mean_ctx": mean_ctx}


def measure_prefill(runner, tokens_n, vocab, repeats=7):
    """A prompt of ``tokens_n`` tokens in one step, timed on the device: the
    median of ``repeats`` runs after one that warms up (and the fastest, for the
    record).  Every run has other token ids; its weights (tens of GB) do not fit L2."""
    import torch
    from chibillm_b200.engine.batch import StepEntry

    g = torch.Generator().manual_seed(2)
    times = []
    for r in range(repeats + 1):
        ids = torch.randint(0, vocab, (tokens_n,), generator=g).tolist()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry("prefill", ids, [tokens_n - 1])], check=False)
        end.record()
        torch.cuda.synchronize()
        runner.end("prefill")
        if r > 0:                          # the first run warms up
            times.append(start.elapsed_time(end))
    runner.runtime.kernels.check_error_word()
    return statistics.median(times), min(times)


def measure_e2e(llm, batch, prompt_len, steps, warmup, vocab):
    """The same decode steps through the public entry point: every step takes
    host token ids (the packed batch goes to the device from pinned memory) and
    returns the sampled ids to the host.  The timed region holds the device work
    of exactly ``steps`` steps: the engine launches a step ahead of the host
    wherever the next step is foretold, so the last warm-up step is kept from
    doing that, and the requests' token limit ends them with the last timed step
    (a limit is foretold: nothing is launched past it)."""
    import torch
    from chibillm_b200.sampling import SamplingParams

    # The prompts of all requests run first (tens of milliseconds of dense work under the power
    # cap); the clocks need about five decode steps to settle after that, so this loop warms up
    # with at least 16 untimed steps whatever --warmup says.
    warmup = max(warmup, 16)
    g = torch.Generator().manual_seed(3)
    engine = llm.engine
    for i in range(batch):
        prompt = torch.randint(0, vocab, (prompt_len,), generator=g).tolist()
        # the prompt's last step yields token 1; then `warmup` and `steps` decode steps
        engine.add(("e2e", i), prompt, SamplingParams(max_new_tokens=1 + warmup + steps, ignore_eos=True))
    while any(s.status == "waiting" for s in engine.scheduler.sequences.values()):
        engine.step()
    for w in range(warmup):
        engine.run_ahead = w != warmup - 1
        engine.step()
    engine.run_ahead = True
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(engine.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert engine.is_finished() and produced == batch * steps
    h2d = llm.runner.last_meta_bytes
    ahead = llm.runner.steps_ahead_used
    for i in range(batch):
        engine.remove(("e2e", i))
    return {"tok_s": produced / dt, "h2d": h2d, "d2h": batch * 4 + 4, "steps_ahead": ahead, "warmup": warmup}


def measure_mixed(cfg, layers, full_layers, requests, shape, check_tokens=0):
    """Requests of mixed lengths through ``LLM.generate``: prompts of 16 to 2,048 uniform random
    tokens, 256 greedy tokens each (the end-of-sequence token ignored), all submitted at once, so
    that prompt portions run beside decoding requests.  Wall-clock time of the second of two runs."""
    import random
    import torch
    import chibillm_b200
    rng = random.Random(0)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(16, 2048))] for _ in range(requests)]
    new_tokens = 256
    llm = chibillm_b200.LLM(None, dtype="bfloat16", device="cuda:0", context_length=8192,
                            kv_cache_tokens=requests * (2048 + new_tokens + 64), max_sequences=requests,
                            max_batch_tokens=2048, prefill_chunk_tokens=2048, random_config=cfg, random_seed=0)
    seconds = None
    for _ in range(2):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, max_tokens=new_tokens, ignore_eos=True)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
    generated = sum(len(o) for o in outs)
    prompt_tokens = sum(len(p) for p in prompts)
    replays, ahead = llm.runner.graph_replays, llm.runner.steps_ahead_used
    del llm
    torch.cuda.empty_cache()
    check = None
    if check_tokens > 0:
        # What was timed is tied to correct output: the 32-bit engine generates the first tokens of
        # every request under two different budgets (other portions, other batches), which must
        # agree with one another; the timed bfloat16 run's tokens are counted against them.
        exact = []
        for budget, chunk in ((2048, 2048), (640, 96)):
            ref = chibillm_b200.LLM(None, dtype="float32", device="cuda:0", context_length=8192,
                                    kv_cache_tokens=requests * (2048 + check_tokens + 64), max_sequences=requests,
                                    max_batch_tokens=budget, prefill_chunk_tokens=chunk, random_config=cfg,
                                    random_seed=0)
            exact.append(ref.generate(prompts, max_tokens=check_tokens, ignore_eos=True))
            del ref
            torch.cuda.empty_cache()
        same = sum(a == b for x, y in zip(*exact) for a, b in zip(x, y))
        agree = sum(a == b for x, y in zip(outs, exact[0]) for a, b in zip(x, y))
        first = sum(x[0] == y[0] for x, y in zip(outs, exact[0]))
        total = requests * check_tokens
        check = {"tokens_per_request": check_tokens, "fp32_budgets_agree": round(same / total, 4),
                 "bf16_first_token_agrees": round(first / requests, 4), "bf16_tokens_agree": round(agree / total, 4)}
    return {"metric": f"generated tok/s, {requests} requests of mixed prompt lengths (Qwen3-{shape.split('-')[1].upper()} "
                      "shape, random bf16 weights)", "value": round(generated / seconds, 1), "unit": "tokens/s",
            "n_gpus": 1, "seconds": round(seconds, 3), "prompt_tokens": prompt_tokens, "generated_tokens": generated,
            "total_tok_s": round((prompt_tokens + generated) / seconds, 1), "layers": layers,
            "layers_full": full_layers, "dtype": "bf16", "data": "synthetic", "impl": "ours",
            "steps_from_graphs": replays, "steps_launched_ahead": ahead, "check": check}


def measure_products(cfg, rows, seconds=2.0):
    """The four matrix products of a layer at ``rows`` rows, plain (bfloat16 in and out, nothing
    folded in): this package's kernel beside the library's (torch.matmul) at the same shapes, each
    as a burst (best of 10 launches) and back to back for ``seconds`` (under the power cap)."""
    import torch
    from chibillm_b200.kernels.ops import CudaKernels

    k = CudaKernels(torch.device("cuda:0"))
    h, inter = cfg["hidden_size"], cfg["intermediate_size"]
    d = cfg.get("head_dim") or h // cfg["num_attention_heads"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * d
    shapes = {"qkv": (qkv, h), "o": (h, cfg["num_attention_heads"] * d), "gate_up": (2 * inter, h), "down": (h, inter)}

    def rate(fn, flops):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = None
        for _ in range(10):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            best = a.elapsed_time(b) if best is None else min(best, a.elapsed_time(b))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n, t0 = 0, time.perf_counter()
        a.record()
        while time.perf_counter() - t0 < seconds:
            for _ in range(20):
                fn()
            n += 20
            torch.cuda.synchronize()
        b.record()
        torch.cuda.synchronize()
        return round(flops / best / 1e9, 1), round(flops / (a.elapsed_time(b) / n) / 1e9, 1)

    out = {}
    for name, (n, kk) in shapes.items():
        x = torch.randn(rows, kk, device="cuda").bfloat16()
        w = (0.02 * torch.randn(n, kk, device="cuda")).bfloat16()
        y = torch.empty(rows, n, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * rows * n * kk
        ours = rate(lambda: k.linear(x, w, y), flops)
        lib = rate(lambda: torch.matmul(x, w.t(), out=y), flops)
        out[name] = {"n": n, "k": kk, "ours_burst": ours[0], "ours_sustained": ours[1], "library_burst": lib[0],
                     "library_sustained": lib[1]}
    k.check_error_word()
    return {"metric": f"TFLOP/s of a layer's four products at {rows} rows, this package's kernel and torch.matmul",
            "unit": "TFLOP/s", "rows": rows, "products": out, "n_gpus": 1, "dtype": "bf16", "data": "synthetic"}


def print_timeline(cfg, batch, held, prompt_tokens=0):
    """One decode step, replayed from its CUDA graph, as its CTAs saw it: for every launch when
    its first and last CTA started, when their wait for the launch before ended and when they
    left (microseconds from the step's start), and the points that kernels mark inside
    (chibillm_b200/kernels/timeline.py; the libraries are built with -DCHIBI_TIMELINE for this).
    With ``prompt_tokens`` the step is a prompt of so many tokens instead."""
    import torch
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.engine.runner import ModelRunner
    from chibillm_b200.kernels.ops import CudaKernels

    kernels = CudaKernels(torch.device("cuda:0"), timeline=True)
    pool = max(batch * (held + 128), prompt_tokens + 128)
    runner = ModelRunner.from_random(cfg, seed=0, dtype="bfloat16", page_size=16, pool_tokens=pool,
                                     max_requests=batch, kernels=kernels)
    for name in runner.storage.keys:
        runner.storage.keys[name].normal_()
        runner.storage.values[name].normal_()
    if prompt_tokens > 0:
        g = torch.Generator().manual_seed(2)
        for i in range(3):
            ids = torch.randint(0, cfg["vocab_size"], (prompt_tokens,), generator=g).tolist()
            torch.cuda.synchronize()
            kernels.timeline.reset()
            runner.step([StepEntry("prompt", ids, [prompt_tokens - 1])])
            torch.cuda.synchronize()
            runner.end("prompt")
        print(f"# prompt step of {prompt_tokens} tokens, {cfg['num_hidden_layers']} layers; times in us")
    else:
        ids = [f"r{i}" for i in range(batch)]
        for rid in ids:
            fill_request(runner, rid, held)
        for i in range(6):
            runner.step([StepEntry(rid, [5 + i], [0]) for rid in ids])
        torch.cuda.synchronize()
        kernels.timeline.reset()
        runner.step([StepEntry(rid, [77], [0]) for rid in ids])
        print(f"# decode step of {batch} x {held} tokens, {cfg['num_hidden_layers']} layers, from a graph: "
              f"{runner.graph_replays > 0}; times in us")
    launches = kernels.timeline.launches()
    cell = lambda v: "       -" if v is None else f"{v:8.2f}"
    print(f"{'kernel':42s} {'ctas':>5s} {'sms':>4s} {'start0':>8s} {'start1':>8s} {'wait0':>8s} {'wait1':>8s} "
          f"{'end0':>8s} {'end1':>8s}  marks (first..last CTA)")
    for l in launches:
        marks = "  ".join(f"{m[0]:.2f}..{m[1]:.2f}" for m in l["marks"] if m is not None)
        print(f"{l['kernel'][:42]:42s} {l['blocks']:5d} {l['sms']:4d} {cell(l['first_start'])} {cell(l['last_start'])} "
              f"{cell(l['first_waited'])} {cell(l['last_waited'])} {cell(l['first_end'])} {cell(l['last_end'])}  {marks}")


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None,
                    help="run only the first layers (each at full size); the JSON names both numbers")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=2048, help="tokens held when decoding starts")
    ap.add_argument("--context", type=int, default=4096, help="context capacity per request")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--point-steps", type=int, default=32)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--mixed-requests", type=int, default=0,
                    help="instead of the record: this many requests with prompts of 16 to 2,048 random tokens "
                         "and 256 new tokens each through the Python entry point; prints its own JSON line")
    ap.add_argument("--products", action="store_true",
                    help="instead of the record: the four matrix products of a layer at --prefill-tokens rows, "
                         "this package's kernel beside torch.matmul, burst and sustained")
    ap.add_argument("--timeline", action="store_true",
                    help="instead of the record: the timeline of one decode step (use with --layers 4 or so)")
    ap.add_argument("--timeline-prompt", type=int, default=0,
                    help="with --timeline: the step is a prompt of so many tokens instead of a decode step")
    ap.add_argument("--check-tokens", type=int, default=0,
                    help="with --mixed-requests: also generate this many tokens of every request with the 32-bit "
                         "engine under two budgets and report how the runs agree")
    ap.add_argument("--shape", default="qwen3-8b", choices=sorted(SHAPES),
                    help="layer sizes (random weights); the contract's record is the default")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "nireo/chibillm is an Apple-Metal C++ program without setup.py or pyproject.toml; "
                          "pip cannot install it and no machine here can run Metal"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this engine runs on a single GPU (--gpus {args.gpus} refused)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import chibillm_b200
    from chibillm_b200.sampling import Sampler

    cfg = dict(QWEN3_8B)
    cfg.update(SHAPES[args.shape])
    full_layers = cfg["num_hidden_layers"]
    layers = full_layers if args.layers is None else max(1, min(args.layers, full_layers))
    cfg["num_hidden_layers"] = layers
    vocab = cfg["vocab_size"]
    peaks, peaks_src = load_peaks()
    if args.products:
        print(json.dumps(measure_products(cfg, args.prefill_tokens)), flush=True)
        return 0
    if args.timeline:
        print_timeline(cfg, args.batch, args.prompt, args.timeline_prompt)
        return 0
    if args.mixed_requests > 0:
        print(json.dumps(measure_mixed(cfg, layers, full_layers, args.mixed_requests, args.shape,
                                       args.check_tokens)))
        return 0
    big = 64 if not args.skip_points else args.batch
    per_request = max(args.prompt + max(args.warmup, 16) + args.steps + 1, args.context) + 64
    pool = ((max(big, args.batch) * per_request + 63) // 64) * 64
    t_load = time.time()
    llm = chibillm_b200.LLM(None, dtype="bfloat16", device="cuda:0", context_length=args.context,
                            kv_cache_tokens=pool, max_sequences=max(big, args.batch),
                            max_batch_tokens=max(8192, args.prefill_tokens, args.batch * args.prompt),
                            prefill_chunk_tokens=max(2048, args.prompt),
                            random_config=cfg, random_seed=0)
    runner = llm.runner
    # the pool holds random values, so decoding from "filled" requests reads real numbers
    for name in runner.storage.keys:
        runner.storage.keys[name].normal_(0.0, 1.0)
        runner.storage.values[name].normal_(0.0, 1.0)
    sampler = Sampler(runner.runtime)
    torch.cuda.synchronize()
    load_s = time.time() - t_load

    prefill_ms, prefill_best_ms = measure_prefill(runner, args.prefill_tokens, vocab)
    flops = prefill_flops(cfg, layers, args.prefill_tokens)

    clocks = ClockSampler()
    clocks.start()
    main_run = measure_decode(runner, sampler, args.batch, args.prompt, args.steps, args.warmup, vocab, "d")
    clock_info = clocks.stop()

    points = {}
    if not args.skip_points:
        # batch 1 and 64 at the same context, and the default batch further along the 2,048 -> 4,096
        # range that the decoded tokens cross
        later = [c for c in (3072, 4032) if args.prompt < c <= args.context - args.point_steps - args.warmup]
        for b, held, key in [(1, args.prompt, "decode_b1"), (64, args.prompt, "decode_b64")] + \
                [(args.batch, c, f"decode_b{args.batch}_ctx{c}") for c in later]:
            r = measure_decode(runner, sampler, b, held, args.point_steps, args.warmup, vocab, key + "_")
            points[key] = round(r["tok_s"], 1)
            points[f"{key}_ms_per_step"] = round(r["ms_per_step"], 4)
            bytes_b = decode_step_bytes(cfg, layers, [r["mean_ctx"]] * b)
            points[f"{key}_hbm_frac"] = round(bytes_b / (r["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)

    e2e = None
    if not args.skip_e2e:
        e2e = measure_e2e(llm, args.batch, args.prompt, args.steps, args.warmup, vocab)

    shape_name = "Qwen3-" + args.shape.split("-")[1].upper()
    step_bytes = decode_step_bytes(cfg, layers, [main_run["mean_ctx"]] * args.batch)
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({shape_name} shape, random bf16 weights, KV bf16 paged, block 16)",
        "value": round(main_run["tok_s"], 2),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": f"{shape_name} shape, random weights", "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "single GPU", "layers": layers, "layers_full": full_layers,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": vocab, "kv_block": 16,
            "decode_ctx_start": args.prompt, "prefill_tokens": args.prefill_tokens,
            "l2": "inputs larger than L2: every step streams all weights",
            "peaks": peaks_src,
        },
        "prefill": {"value": round(args.prefill_tokens / (prefill_ms / 1e3), 1), "tokens": args.prefill_tokens,
                    "ms": round(prefill_ms, 3), "ms_best": round(prefill_best_ms, 3), "runs": 7, "stat": "median",
                    "frac": round(flops / (prefill_ms / 1e3) / 1e12 / peaks["bf16_tflops"], 4),
                    "frac_of_sustained": round(flops / (prefill_ms / 1e3) / 1e12 / peaks["bf16_tflops_sustained"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "gpu_launches": int(main_run["launches"]),
        "clocks": clock_info,
        "load_seconds": round(load_s, 1),
    }
    if e2e is not None:
        out["e2e"] = {"value": round(e2e["tok_s"], 2), "unit": "tokens/s",
                      "h2d_bytes_per_step": int(e2e["h2d"]), "d2h_bytes_per_step": int(e2e["d2h"]),
                      "warmup": int(e2e["warmup"]), "steps_launched_ahead": int(e2e["steps_ahead"])}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
