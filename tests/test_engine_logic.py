"""The step function's logic without a GPU: the engine runs with the plain
PyTorch restatements of the kernels (tests/reference_ops.py) in place of the
CUDA ones, so what is tested here is batching, paging, windows and page reuse,
not the kernels.  Also the plain implementation against itself (32- vs 64-bit,
whole vs prefix)."""
import pytest
import torch

import helpers
import plain_qwen3
import tiny_configs
from reference_ops import ReferenceKernels


def cpu_runner(folder, page_size, pool_tokens, max_requests=4):
    from chibillm_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_folder(folder, dtype="float32", device="cpu", page_size=page_size,
                                     pool_tokens=pool_tokens, max_requests=max_requests,
                                     kernels=ReferenceKernels())
    runner.storage.poison()
    return runner


@pytest.mark.parametrize("name,page_size,lengths", [("A", 4, [5, 40, 70]), ("C", 8, [3, 50, 90])])
def test_cutting_and_batching_on_cpu(tmp_path, name, page_size, lengths):
    folder = helpers.make_model_dir(tmp_path, name, seed=3)
    vocab = tiny_configs.get(name)["vocab_size"]
    reqs = helpers.random_requests(vocab, lengths, seed=1)
    ref = helpers.plain_logits(folder, reqs)
    runner = cpu_runner(folder, page_size, helpers.round64(max(lengths)))
    for trace, what in ((helpers.trace_whole(reqs), "whole"),
                        (helpers.trace_last_decoded(reqs, 32), "last 32 decoded"),
                        (helpers.trace_portions(reqs, seed=2), "portions")):
        got = helpers.run_trace(runner, trace)
        helpers.assert_logits_close(got, ref, helpers.TOL["float32"], f"{name} {what}")
        runner.cache.check_invariants()
        assert not runner.cache.requests

    mixed_reqs = helpers.random_requests(vocab, [60, 90, 20, 70, 33, 64], seed=4)
    mixed_ref = helpers.plain_logits(folder, mixed_reqs)
    pool = 256
    trace = helpers.trace_mixed(mixed_reqs, pool, seed=6)
    assert helpers.peak_tokens(trace) <= pool
    assert sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > pool
    runner2 = cpu_runner(folder, page_size, pool)
    got = helpers.run_trace(runner2, trace)
    helpers.assert_logits_close(got, mixed_ref, helpers.TOL["float32"], f"{name} mixed")
    runner2.cache.check_invariants()
    assert not runner2.cache.requests


def test_plain_implementation_is_consistent(tmp_path):
    """32-bit against 64-bit arithmetic, and causality: the logits of a prefix
    do not change when tokens follow it."""
    for name in ("A", "B", "C"):
        folder = helpers.make_model_dir(tmp_path, name, seed=5)
        vocab = tiny_configs.get(name)["vocab_size"]
        ids = helpers.random_requests(vocab, [60], seed=7)["r0"]
        c32, w32 = plain_qwen3.read_model_folder(folder, torch.float32)
        c64, w64 = plain_qwen3.read_model_folder(folder, torch.float64)
        l32 = plain_qwen3.forward(c32, w32, ids)
        l64 = plain_qwen3.forward(c64, w64, ids)
        assert float((l32.double() - l64).abs().max()) < 2e-5 * float(l64.abs().max())
        prefix = plain_qwen3.forward(c32, w32, ids[:25])
        assert float((prefix - l32[:25]).abs().max()) < 1e-5


def test_plain_window_masks_far_keys():
    q = torch.zeros(10, 1, 4)
    k = torch.zeros(10, 1, 4)
    v = torch.arange(10, dtype=torch.float32).view(10, 1, 1).repeat(1, 1, 4)
    out_all = plain_qwen3.causal_attention(q, k, v, None)
    out_win = plain_qwen3.causal_attention(q, k, v, 3)
    assert torch.allclose(out_all[9, 0], torch.full((4,), 4.5))
    assert torch.allclose(out_win[9, 0], torch.full((4,), 8.0))   # mean of 7, 8, 9
    assert torch.allclose(out_win[1, 0], torch.full((4,), 0.5))


def test_plain_rope_and_norm_formulas():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])
    out = plain_qwen3.rope(x, torch.tensor([0]), 10000.0)
    assert torch.equal(out, x)                       # position 0 rotates nothing
    out = plain_qwen3.rope(x, torch.tensor([1]), 10000.0)
    inv = plain_qwen3.rope_inverse_frequencies(10000.0, 4)
    c, s = torch.cos(inv), torch.sin(inv)
    expect = torch.stack([1 * c[0] - 3 * s[0], 2 * c[1] - 4 * s[1], 3 * c[0] + 1 * s[0], 4 * c[1] + 2 * s[1]])
    assert torch.allclose(out[0, 0], expect, atol=1e-6)
    y = plain_qwen3.rms_norm(torch.tensor([[3.0, 4.0]]), torch.tensor([2.0, 0.5]), 0.0)
    rms = (12.5) ** 0.5
    assert torch.allclose(y, torch.tensor([[3.0 / rms * 2.0, 4.0 / rms * 0.5]]))


def test_generation_through_entry_point_on_cpu(tmp_path):
    """Scheduler, sampler and step function together: greedy tokens equal the
    plain implementation's for prompts that are cut into portions of 8 and mixed
    with decoding (the reference's own check is equality of tokens across batch
    budgets, tests/qwen_weights_test.cc:903-960)."""
    import chibillm_b200
    folder = helpers.make_model_dir(tmp_path, "B", seed=1)
    config, weights = plain_qwen3.read_model_folder(folder)
    prompts = list(helpers.random_requests(384, [1, 7, 23, 40], seed=1).values())
    expected = [plain_qwen3.generate_greedy(config, weights, p, 6) for p in prompts]
    for budget, chunk in ((16, 8), (512, 64), (7, 3)):
        llm = chibillm_b200.LLM(folder, dtype="float32", device="cpu", context_length=128,
                                kv_cache_tokens=256, max_sequences=3, max_batch_tokens=budget,
                                prefill_chunk_tokens=chunk, kernels=ReferenceKernels())
        got = llm.generate(prompts, max_tokens=6, ignore_eos=True)
        assert got == expected, f"budget {budget}"
        llm.runner.cache.check_invariants()
        assert not llm.runner.cache.requests


def test_a_step_refuses_what_it_cannot_run(tmp_path):
    """The checks of the batch packing (in the C++ runtime): a request twice, no
    tokens, an id outside the vocabulary, a position past the model's limit, a
    wanted place outside the entry; and a refused step changes no length."""
    from chibillm_b200.engine.batch import BatchError, StepEntry
    folder = helpers.make_model_dir(tmp_path, "A", seed=3)
    cfg = tiny_configs.get("A")
    runner = cpu_runner(folder, 4, 256)
    runner.step([StepEntry("a", [1, 2, 3], [2])])
    for entries, what in (
            ([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])], "twice"),
            ([StepEntry("a", [], [])], "no tokens"),
            ([StepEntry("a", [cfg["vocab_size"]], [0])], "vocabulary"),
            ([StepEntry("a", [-1], [0])], "vocabulary"),
            ([StepEntry("a", [1, 2], [2])], "wanted place"),
            ([StepEntry("a", [1] * cfg["max_position_embeddings"], [0])], "limit")):
        with pytest.raises(BatchError) as e:
            runner.step(entries)
        assert what in str(e.value), (what, str(e.value))
        assert runner.length("a") == 3
    logits = runner.step([StepEntry("a", [4], [0])])
    assert logits.shape == (1, cfg["vocab_size"]) and runner.length("a") == 4
    runner.cache.check_invariants()


def test_parts_at_the_decoders_ends_on_cpu(tmp_path):
    """A toy architecture with a learned table of absolute positions added to the
    (scaled) embeddings and soft-capped logits, both registered as adapters from
    outside the package: whole, in portions and mixed, against its plain restatement."""
    import toy_parts
    from chibillm_b200.config import unregister_architecture
    from chibillm_b200.weights import write_random_model
    toy_parts.register_absolute_toy()
    try:
        obj = dict(toy_parts.ABSOLUTE_TOY_CONFIG)
        folder = write_random_model(obj, str(tmp_path / "absolute"), seed=6, dtype=torch.float32)
        _, w = plain_qwen3.read_model_folder(folder)
        assert "positions.weight" in w and w["positions.weight"].shape == (96, 64)
        reqs = helpers.random_requests(113, [30, 8, 61, 17], seed=2)
        ref = {rid: toy_parts.absolute_toy_plain(obj, w, ids) for rid, ids in reqs.items()}
        assert float(max(r.abs().max() for r in ref.values())) <= obj["cap"]
        # the positions matter: the same tokens further along give other logits
        shifted = toy_parts.absolute_toy_plain(obj, w, reqs["r1"] + reqs["r1"])
        assert float((shifted[8:] - ref["r1"]).abs().max()) > 1e-3
        runner = cpu_runner(folder, 4, 128, max_requests=3)
        for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_portions(reqs, 3), "portions"),
                            (helpers.trace_mixed(reqs, 128, seed=4, max_live=3, decode_tail=5), "mixed")):
            got = helpers.run_trace(runner, trace)
            helpers.assert_logits_close(got, ref, 2e-5, f"absolute toy {what}")
            runner.cache.check_invariants()
    finally:
        unregister_architecture("ToyAbsoluteForCausalLM")
