"""The plain implementation and the engine against what nireo/chibillm's own
host code computed for the tiny models A and B (tests/golden/, made by
tests/golden/make_goldens.py from the reference's unmodified C++ behind a CPU
stand-in for its device layer): the logits of every position of prompt plus
generated tokens, and the greedy tokens that the reference's scheduler and
engine produced under a generous and a tight setting."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

import helpers
import plain_qwen3
import tiny_configs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL_FP32 = 2e-5


def load_golden(name):
    folder = os.path.join(GOLDEN, f"tiny_{name}")
    with open(os.path.join(folder, "golden.json")) as f:
        g = json.load(f)
    vocab = tiny_configs.get(name)["vocab_size"]
    g["logits"] = {rid: torch.from_numpy(np.fromfile(os.path.join(folder, f"whole_{rid}.f32"),
                                                     dtype="<f4").reshape(-1, vocab).copy())
                   for rid in g["prompts"]}
    first = next(iter(g["generate"].values()))
    g["tokens"] = first["tokens"]
    for setting in g["generate"].values():
        assert setting["tokens"] == g["tokens"]
    g["full"] = {rid: g["prompts"][rid] + g["tokens"][rid][:-1] for rid in g["prompts"]}
    return g


def golden_model_dir(tmp_path, g):
    """The model folder the goldens were made with, rebuilt from its seed."""
    folder = helpers.make_model_dir(tmp_path, g["config"], seed=g["weights_seed"], dtype=torch.bfloat16)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    assert digest == g["weights_sha256"], (
        "the random-weights generator no longer makes the weights the goldens belong to; "
        "run tests/golden/make_goldens.py again")
    return folder


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_implementation_matches_the_reference(tmp_path, name):
    g = load_golden(name)
    folder = golden_model_dir(tmp_path, g)
    config, weights = plain_qwen3.read_model_folder(folder)
    for rid, ids in g["full"].items():
        got = plain_qwen3.forward(config, weights, ids)
        ref = g["logits"][rid]
        assert got.shape == ref.shape
        worst = float((got - ref).abs().max()) / float(ref.abs().max())
        assert worst < TOL_FP32, f"tiny {name} request {rid}: {worst:.2e}"
        n = len(g["prompts"][rid])
        assert plain_qwen3.generate_greedy(config, weights, g["prompts"][rid], g["new_tokens"]) == g["tokens"][rid]
        assert [int(t) for t in ref[n - 1:].argmax(dim=1)] == g["tokens"][rid]


@pytest.mark.parametrize("name", ["A", "B"])
def test_engine_on_the_cpu_stand_in_matches_the_reference(tmp_path, name):
    """The step function, cache and scheduler with the PyTorch restatements of
    the kernels: logits of every position (whole and in portions), and greedy
    tokens under the reference's two scheduler settings."""
    import chibillm_b200
    from reference_ops import ReferenceKernels
    from chibillm_b200.engine.runner import ModelRunner

    g = load_golden(name)
    folder = golden_model_dir(tmp_path, g)
    runner = ModelRunner.from_folder(folder, dtype="float32", device="cpu", page_size=g["block_size"],
                                     pool_tokens=256, max_requests=4, kernels=ReferenceKernels())
    runner.storage.poison()
    for trace, what in ((helpers.trace_whole(g["full"]), "whole"),
                        (helpers.trace_portions(g["full"], seed=3), "portions")):
        got = helpers.run_trace(runner, trace)
        helpers.assert_logits_close(got, g["logits"], TOL_FP32, f"tiny {name} {what} vs reference")
    for setting in g["generate"].values():
        llm = chibillm_b200.LLM(folder, dtype="float32", device="cpu", context_length=128,
                                kv_cache_tokens=setting["kv_block_count"] * g["block_size"],
                                max_sequences=setting["max_sequences"],
                                max_batch_tokens=setting["max_batch_tokens"],
                                prefill_chunk_tokens=setting["prefill_chunk_tokens"],
                                page_size=g["block_size"], kernels=ReferenceKernels())
        got = llm.generate([g["prompts"][rid] for rid in g["prompts"]], max_tokens=g["new_tokens"])
        assert got == [g["tokens"][rid] for rid in g["prompts"]], setting["name"]
        llm.runner.cache.check_invariants()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_engine_matches_the_reference(tmp_path, name, dtype):
    """The CUDA engine against the reference's logits: whole, the last tokens
    one by one, in portions, and mixed with so few pages that they are reused;
    then greedy tokens through the entry point under the reference's settings."""
    import chibillm_b200
    from chibillm_b200.engine.runner import ModelRunner

    g = load_golden(name)
    folder = golden_model_dir(tmp_path, g)
    pool = 128
    runner = ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", page_size=g["block_size"],
                                     pool_tokens=pool, max_requests=4)
    runner.storage.poison()
    traces = ((helpers.trace_whole(g["full"]), "whole"),
              (helpers.trace_last_decoded(g["full"], 32), "last 32 decoded"),
              (helpers.trace_portions(g["full"], seed=3), "portions"),
              (helpers.trace_mixed(g["full"], pool, seed=5, max_live=3), "mixed"))
    for trace, what in traces:
        got = helpers.run_trace(runner, trace)
        helpers.assert_logits_close(got, g["logits"], helpers.TOL[dtype], f"tiny {name} {dtype} {what} vs reference")
    runner.cache.check_invariants()
    if dtype != "float32":
        return
    for setting in g["generate"].values():
        llm = chibillm_b200.LLM(folder, dtype=dtype, device="cuda:0", context_length=128,
                                kv_cache_tokens=setting["kv_block_count"] * g["block_size"],
                                max_sequences=setting["max_sequences"],
                                max_batch_tokens=setting["max_batch_tokens"],
                                prefill_chunk_tokens=setting["prefill_chunk_tokens"],
                                page_size=g["block_size"])
        got = llm.generate([g["prompts"][rid] for rid in g["prompts"]], max_tokens=g["new_tokens"])
        assert got == [g["tokens"][rid] for rid in g["prompts"]], setting["name"]
