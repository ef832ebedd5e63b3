"""The engine against the plain implementation, in 32-bit and in bfloat16:
requests whole; most of a request in one step and its last 32 tokens one by
one; portions of changing size; mixed batches of up to four live requests with
so few pages that they are used again; the first tokens of a sequence; long
decoding.  Every run goes through ModelRunner.step, the call generation makes.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import tiny_configs

pytestmark = pytest.mark.gpu

CASES = {
    # name: (config, page size, request lengths)
    "A": ("A", 4, [5, 47, 100, 128]),
    "B": ("B", 16, [1, 40, 130, 250]),
    "C": ("C", 8, [3, 70, 200, 333]),
    # head sizes 64 and 128: the tensor-core attention kernels, and at 128 the decode attention that
    # finishes the q|k|v product itself (a window of 200 on the second layer)
    "D64": ("D64", 16, [2, 90, 260, 400]),
    "D128": ("D128", 16, [4, 65, 300, 520]),
    # sizes that the many-row products take with the norms folded in and the heads finished in the
    # q|k|v epilogue (prompts of more than 64 tokens), a window of 150 on the second layer
    "E128": ("E128", 8, [3, 70, 200, 410]),
}
MIXED_LENGTHS = {"A": [50, 100, 30, 128, 64, 90, 17], "B": [1, 200, 33, 250, 64, 129, 7],
                 "C": [300, 20, 150, 65, 333, 2, 180], "D64": [400, 31, 129, 64, 350, 3, 222],
                 "D128": [17, 520, 66, 250, 2, 480, 128], "E128": [410, 9, 130, 65, 300, 1, 222]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: helpers.make_model_dir(root, cfg, seed=i) for i, (name, (cfg, _, _)) in enumerate(CASES.items())}


def make_runner(folder, dtype, page_size, pool_tokens, max_requests=4):
    from chibillm_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", page_size=page_size,
                                     pool_tokens=pool_tokens, max_requests=max_requests)
    runner.storage.poison()      # a read of a slot that was never written gives NaN
    return runner


@pytest.fixture(scope="module")
def expected(folders):
    out = {}
    for name, (cfg, _, lengths) in CASES.items():
        vocab = tiny_configs.get(cfg)["vocab_size"]
        reqs = helpers.random_requests(vocab, lengths, seed=100)
        mixed = helpers.random_requests(vocab, MIXED_LENGTHS[name], seed=200)
        out[name] = (reqs, helpers.plain_logits(folders[name], reqs),
                     mixed, helpers.plain_logits(folders[name], mixed))
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(CASES))
def test_cutting_and_batching(folders, expected, case, dtype):
    cfg, page_size, lengths = CASES[case]
    reqs, ref, mixed_reqs, mixed_ref = expected[case]
    tol = helpers.TOL[dtype]
    runner = make_runner(folders[case], dtype, page_size, pool_tokens=helpers.round64(max(lengths)))

    whole = helpers.run_trace(runner, helpers.trace_whole(reqs))
    helpers.assert_logits_close(whole, ref, tol, f"{case} {dtype} whole")
    runner.cache.check_invariants()
    if case == "E128" and dtype == "bfloat16":
        # the prompts of more than 64 tokens went the way this case is here for: the q|k|v product
        # wrote q and the cache itself, from the per-step table of cache slots
        assert any(name.startswith("attn.slots") for name, _ in runner.workspace._buffers)

    tail = helpers.run_trace(runner, helpers.trace_last_decoded(reqs, 32))
    helpers.assert_logits_close(tail, ref, tol, f"{case} {dtype} last 32 decoded")
    helpers.assert_logits_close(tail, whole, helpers.TOL_SAME_DTYPE[dtype], f"{case} {dtype} decoded vs whole")

    parts = helpers.run_trace(runner, helpers.trace_portions(reqs, seed=3))
    helpers.assert_logits_close(parts, ref, tol, f"{case} {dtype} portions")
    helpers.assert_logits_close(parts, whole, helpers.TOL_SAME_DTYPE[dtype], f"{case} {dtype} portions vs whole")
    runner.cache.check_invariants()
    assert not runner.cache.requests, "requests are still held after their end"

    # mixed: a pool of 2.5 requests' worth, so later requests land on used pages
    pool = 2 * helpers.round64(max(MIXED_LENGTHS[case])) + 128
    trace = helpers.trace_mixed(mixed_reqs, pool, seed=5)
    assert helpers.peak_tokens(trace) <= pool
    assert max(len(s["entries"]) for s in trace) >= 3
    runner2 = make_runner(folders[case], dtype, page_size, pool_tokens=pool)
    total_pages = sum(helpers.round64(len(v)) for v in mixed_reqs.values()) // page_size
    assert total_pages > pool // page_size, "the trace would not reuse pages"
    mixed = helpers.run_trace(runner2, trace)
    helpers.assert_logits_close(mixed, mixed_ref, tol, f"{case} {dtype} mixed")
    runner2.cache.check_invariants()
    assert not runner2.cache.requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case,live", [("E128", 70), ("D128", 100), ("B", 130)])
def test_many_sequences_decoded_together(folders, case, live, dtype):
    """More than 64 sequences in one decode step (the products then run with 65 to
    128 rows, or as many-row products beyond): all prompts in one step, then six
    steps in which every sequence brings one token, against the plain implementation."""
    cfg, page_size, _ = CASES[case]
    vocab = tiny_configs.get(cfg)["vocab_size"]
    lengths = [9 + (7 * i) % 23 for i in range(live)]
    reqs = helpers.random_requests(vocab, lengths, seed=600)
    ref = helpers.plain_logits(folders[case], reqs)
    runner = make_runner(folders[case], dtype, page_size, pool_tokens=sum(helpers.round64(n) for n in lengths),
                         max_requests=live)
    tail = 6
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": ids[:-tail], "want": list(range(len(ids) - tail))}
                                     for rid, ids in reqs.items()], "end": []}]
    for j in range(tail):
        steps.append({"step": 1 + j, "entries": [{"id": rid, "tokens": [ids[len(ids) - tail + j]], "want": [0]}
                                                 for rid, ids in reqs.items()],
                      "end": list(reqs) if j == tail - 1 else []})
    got = helpers.run_trace(runner, steps)
    helpers.assert_logits_close(got, ref, helpers.TOL[dtype], f"{case} {dtype} {live} sequences together")
    runner.cache.check_invariants()
    assert not runner.cache.requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(folders, expected, dtype):
    """Position 0 alone, then every further token one by one up to the model's
    limit of positions."""
    case = "B"
    cfg, page_size, _ = CASES[case]
    vocab = tiny_configs.get(cfg)["vocab_size"]
    reqs = helpers.random_requests(vocab, [256], seed=300)
    ref = helpers.plain_logits(folders[case], reqs)
    runner = make_runner(folders[case], dtype, page_size, pool_tokens=256)
    trace = helpers.trace_last_decoded(reqs, tail=255)
    assert len(trace[0]["entries"][0]["tokens"]) == 1
    got = helpers.run_trace(runner, trace)
    helpers.assert_logits_close(got, ref, helpers.TOL[dtype], f"{dtype} decoded from the first token")


def test_window_frees_pages(folders):
    """Config C has a window of 24 on two layers: while a long request decodes,
    its windowed group holds only the pages the window still covers."""
    cfg, page_size, _ = CASES["C"]
    runner = make_runner(folders["C"], "float32", page_size, pool_tokens=512)
    vocab = tiny_configs.get(cfg)["vocab_size"]
    ids = helpers.random_requests(vocab, [300], seed=400)["r0"]
    from chibillm_b200.engine.batch import StepEntry
    runner.step([StepEntry("w", ids[:200], [])])
    windowed = [g for g in runner.cache.groups.values() if g.window is not None][0]
    full = [g for g in runner.cache.groups.values() if g.window is None][0]
    held = lambda g: g.num_pages - runner.cache.free_pages(g.name)
    assert held(full) == 200 // page_size
    assert held(windowed) <= 24 // page_size + 2
    for t in ids[200:]:
        runner.step([StepEntry("w", [t], [])])
        assert held(windowed) <= 24 // page_size + 2
    runner.cache.check_invariants()
    runner.end("w")
    assert held(full) == 0 and held(windowed) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folders, expected, tmp_path, dtype):
    """bin/trace_run as a user calls it: steps on standard input, a ``done`` line
    after each, <step>.f32 files with the wanted logits."""
    case = "A"
    reqs, ref, _, _ = expected[case]
    steps = helpers.trace_portions(reqs, seed=9)
    out_dir = tmp_path / f"out_{dtype}"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.Popen(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders[case], "--dtype", dtype,
         "--out", str(out_dir), "--max-tokens", str(helpers.peak_tokens(steps))],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    vocab = tiny_configs.get(case)["vocab_size"]
    rows = {}
    fed = {}
    for obj in steps:
        proc.stdin.write(json.dumps(obj) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {obj['step']}"
        data = np.fromfile(out_dir / f"{obj['step']}.f32", dtype="<f4").reshape(-1, vocab)
        k = 0
        for e in obj["entries"]:
            for w in e["want"]:
                rows.setdefault(e["id"], []).append(data[k])
                k += 1
        assert k == data.shape[0]
    proc.stdin.close()
    assert proc.wait(timeout=60) == 0
    got = {rid: torch.from_numpy(np.stack(v)) for rid, v in rows.items()}
    helpers.assert_logits_close(got, ref, helpers.TOL[dtype], f"trace_run {dtype}")
