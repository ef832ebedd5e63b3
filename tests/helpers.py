"""Shared pieces of the tests: model folders in temporary places, traces in the
replay format for the different ways of cutting and batching, tolerances."""
from __future__ import annotations

import json
import os
import random
import tempfile
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

import plain_qwen3
import tiny_configs

# Largest allowed |engine - plain| as a fraction of the largest |plain logit| of
# the request.  32-bit: orders of summation differ, nothing else.  bfloat16:
# weights are exact (they are stored in bfloat16) but every activation between
# kernels is rounded to 8 bits of mantissa.  The limits are about twice the worst
# value that the suite measures on a B200 (the run prints every comparison's
# worst value next to its limit): 6.4e-6 in 32-bit (Qwen3-14B layer sizes) and
# 1.1e-2 in bfloat16 (the same sizes, portions against whole prompts).
TOL = {"float32": 1.5e-5, "bfloat16": 2.5e-2}
# bfloat16 runs against each other (same kernels, other batching)
TOL_SAME_DTYPE = {"float32": 1.5e-5, "bfloat16": 2.5e-2}


def make_model_dir(tmp_path, name: str, seed: int = 0, dtype=torch.bfloat16, **overrides) -> str:
    from chibillm_b200.weights import write_random_model

    cfg = tiny_configs.get(name)
    cfg.update(overrides)
    out = os.path.join(str(tmp_path), f"model_{name}_{seed}")
    write_random_model(cfg, out, seed=seed, dtype=dtype)
    return out


def random_requests(vocab: int, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def plain_logits(model_dir: str, requests: Dict[str, List[int]], dtype=torch.float32) -> Dict[str, torch.Tensor]:
    config, weights = plain_qwen3.read_model_folder(model_dir, dtype)
    return {rid: plain_qwen3.forward(config, weights, ids).float() for rid, ids in requests.items()}


# ------------------------------------------------------------------ traces
def round64(n: int) -> int:
    return (n + 63) // 64 * 64


def trace_whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole, every place wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}],
             "end": [rid]} for i, (rid, ids) in enumerate(requests.items())]


def trace_last_decoded(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:head],
                                                       "want": list(range(head))}], "end": []})
        for p in range(head, len(ids)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [ids[p]], "want": [0]}],
                          "end": [rid] if p == len(ids) - 1 else []})
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: Dict[str, List[int]], seed: int = 0) -> List[dict]:
    """Portions of changing size, down to two tokens (and single ones)."""
    rng = random.Random(seed)
    sizes = [2, 7, 3, 16, 2, 33, 1, 5, 17, 2, 64, 9, 1, 31]
    steps = []
    for rid, ids in requests.items():
        pos = 0
        k = rng.randrange(len(sizes))
        while pos < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - pos)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[pos:pos + n],
                                                           "want": list(range(n))}],
                          "end": [rid] if pos + n == len(ids) else []})
            pos += n
    return steps


PORTIONS = [2, 3, 5, 8, 13, 21, 40]      # sizes of the prompt portions of a mixed trace


def trace_mixed(requests: Dict[str, List[int]], max_tokens: int, seed: int = 0, max_live: int = 4,
                decode_tail: int = 12) -> List[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside single
    tokens of others, requests left out of a step now and then, and a pool so
    small that the pages of finished requests are used again."""
    rng = random.Random(seed)
    queue = list(requests.items())
    live: List[list] = []          # [rid, ids, pos, prompt_len]
    steps = []
    while queue or live:
        while queue and len(live) < max_live:
            held = sum(round64(len(r[1])) for r in live)
            if held + round64(len(queue[0][1])) > max_tokens:
                break
            rid, ids = queue.pop(0)
            live.append([rid, ids, 0, max(1, len(ids) - decode_tail)])
        assert live, "max_tokens is too small for the next request"
        entries, end = [], []
        chosen = [r for r in live if rng.random() > 0.2] or [live[0]]
        for r in chosen:
            rid, ids, pos, prompt_len = r
            if pos < prompt_len:
                n = min(rng.choice(PORTIONS), prompt_len - pos)
            else:
                n = 1
            entries.append({"id": rid, "tokens": ids[pos:pos + n], "want": list(range(n))})
            r[2] = pos + n
            if r[2] == len(ids):
                end.append(rid)
        live = [r for r in live if r[2] < len(r[1])]
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def peak_tokens(steps: List[dict]) -> int:
    """Most tokens (each request rounded up to 64) held at one time by a trace."""
    held: Dict[str, int] = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(round64(n) for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def run_trace(runner, steps: List[dict]) -> Dict[str, torch.Tensor]:
    """Replay in this process; returns the logits of every wanted place, per
    request, in position order."""
    from chibillm_b200.engine.replay import replay_step

    rows: Dict[str, List[Tuple[int, np.ndarray]]] = {}
    fed: Dict[str, int] = {}
    for obj in steps:
        out = replay_step(runner, obj, None)
        k = 0
        for e in obj["entries"]:
            base = fed.get(e["id"], 0)
            for w in e.get("want", []):
                rows.setdefault(e["id"], []).append((base + w, out[k].copy()))
                k += 1
            fed[e["id"]] = base + len(e["tokens"])
        for rid in obj["end"]:
            fed.pop(rid, None)
        assert out is None or k == out.shape[0]
    result = {}
    for rid, items in rows.items():
        items.sort(key=lambda x: x[0])
        assert [p for p, _ in items] == list(range(len(items))), f"{rid}: places are missing"
        result[rid] = torch.from_numpy(np.stack([a for _, a in items]))
    return result


# what every comparison of logits measured: name -> (worst |diff| / max |logit|, limit)
MEASURED: Dict[str, Tuple[float, float]] = {}


def assert_logits_close(actual: Dict[str, torch.Tensor], expected: Dict[str, torch.Tensor], tol: float,
                        what: str) -> None:
    for rid, ref in expected.items():
        got = actual[rid]
        assert got.shape == ref.shape, f"{what} {rid}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
        assert torch.isfinite(got).all(), f"{what} {rid}: logits are not finite"
        scale = float(ref.abs().max())
        diff = (got - ref).abs()
        worst = float(diff.max())
        MEASURED[what] = (max(MEASURED.get(what, (0.0, tol))[0], worst / max(scale, 1e-30)), tol)
        if worst > tol * scale:
            per_pos = diff.max(dim=1).values
            first = int(torch.nonzero(per_pos > tol * scale)[0, 0])
            raise AssertionError(
                f"{what} {rid}: max |diff| {worst:.3e} > {tol:.1e} * {scale:.3f}; first wrong position "
                f"{first} of {ref.shape[0]} (diff there {float(per_pos[first]):.3e}); positions over "
                f"the limit: {int((per_pos > tol * scale).sum())}")
