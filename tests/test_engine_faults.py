"""Failures injected on the host into the generation loop: a step whose error
word reports a fault after the step has run, a sampler that returns too few
tokens, and the same for an architecture whose mixer keeps fixed-size state.
After the failure the same step is run again and generation ends with the
tokens of an undisturbed run (the reference tests this with a runner that
returns an error or a wrong count: tests/inference_engine_test.cc:150-179;
src/inference_engine.cc:140-151).  No GPU is involved or faulted."""
import pytest
import torch

import helpers
import plain_qwen3
import tiny_configs
import toy_parts
from reference_ops import ReferenceKernels


class InjectedFault(RuntimeError):
    pass


class FaultyKernels(ReferenceKernels):
    """The CPU stand-in with a device error word that reports a fault at the
    given (1-based) reads."""

    def __init__(self, fail_at):
        super().__init__()
        self.fail_at = set(fail_at)
        self.reads = 0

    def error_word_async(self):
        return None

    def check_error_copy(self):
        self.reads += 1
        if self.reads in self.fail_at:
            raise InjectedFault(f"error word at read {self.reads}")


def run_to_the_end(engine, faults_expected):
    seen = 0
    steps = 0
    while not engine.is_finished():
        steps += 1
        assert steps < 2000
        try:
            engine.step()
        except (InjectedFault, Exception) as e:     # noqa: B014
            if not isinstance(e, InjectedFault) and "result_count_mismatch" not in str(e):
                raise
            seen += 1
            assert not engine.scheduler.active, "the failed batch was not aborted"
    assert seen == faults_expected
    return seen


def make_llm(folder, kernels, page_size=16, **kw):
    import chibillm_b200
    args = dict(dtype="float32", device="cpu", context_length=128, kv_cache_tokens=256, max_sequences=3,
                max_batch_tokens=16, prefill_chunk_tokens=8, page_size=page_size, kernels=kernels)
    args.update(kw)
    return chibillm_b200.LLM(folder, **args)


def submit(llm, prompts, new_tokens):
    from chibillm_b200.sampling import SamplingParams
    ids = []
    for i, p in enumerate(prompts):
        ids.append(("r", i))
        llm.engine.add(("r", i), p, SamplingParams(max_new_tokens=new_tokens, ignore_eos=True), sample_key=i)
    return ids


def test_a_step_that_fails_after_it_ran_is_run_again(tmp_path):
    folder = helpers.make_model_dir(tmp_path, "B", seed=1)
    config, weights = plain_qwen3.read_model_folder(folder)
    prompts = list(helpers.random_requests(384, [1, 7, 23, 40], seed=1).values())
    expected = [plain_qwen3.generate_greedy(config, weights, p, 6) for p in prompts]
    # reads 2 and 3 are prompt portions (one of them twice in a row), 9 and 14 decode steps
    llm = make_llm(folder, FaultyKernels({2, 3, 9, 14}))
    ids = submit(llm, prompts, 6)
    run_to_the_end(llm.engine, 4)
    got = [llm.engine.remove(i).completion for i in ids]
    assert got == expected
    llm.runner.cache.check_invariants()
    assert not llm.runner.cache.requests


def test_a_wrong_number_of_samples_aborts_and_the_retry_is_identical(tmp_path):
    folder = helpers.make_model_dir(tmp_path, "A", seed=0)
    config, weights = plain_qwen3.read_model_folder(folder)
    prompts = list(helpers.random_requests(256, [5, 11, 17], seed=2).values())
    expected = [plain_qwen3.generate_greedy(config, weights, p, 8) for p in prompts]
    llm = make_llm(folder, ReferenceKernels(), page_size=4)
    launch = llm.engine.sampler.launch
    calls = {"n": 0}

    class Short:
        def __init__(self, inner):
            self.inner = inner
            self.device_ids = inner.device_ids

        def result(self):
            return self.inner.result()[:-1]

    def flaky(*args, **kw):
        calls["n"] += 1
        pending = launch(*args, **kw)
        return Short(pending) if calls["n"] in (1, 5) else pending

    llm.engine.sampler.launch = flaky
    ids = submit(llm, prompts, 8)
    run_to_the_end(llm.engine, 2)
    assert [llm.engine.remove(i).completion for i in ids] == expected
    llm.runner.cache.check_invariants()


def test_fixed_size_state_goes_back_when_a_step_fails(tmp_path):
    """The toy mixer advances a running state in place.  A step that fails after
    the mixer ran must leave the state where it was committed, or the retry
    would apply the same tokens twice."""
    from chibillm_b200.config import unregister_architecture
    from chibillm_b200.weights import write_random_model
    toy_parts.register_toy()
    try:
        obj = dict(toy_parts.TOY_CONFIG)
        folder = write_random_model(obj, str(tmp_path / "toy"), seed=3, dtype=torch.float32)
        _, w = plain_qwen3.read_model_folder(folder)
        prompts = list(helpers.random_requests(131, [9, 20, 3], seed=4).values())

        def greedy(prompt, n):
            ids = list(prompt)
            out = []
            for _ in range(n):
                tok = int(toy_parts.toy_plain(obj, w, ids)[-1].argmax())
                out.append(tok)
                ids.append(tok)
            return out

        expected = [greedy(p, 5) for p in prompts]
        clean = make_llm(folder, FaultyKernels(set()), page_size=4)
        ids = submit(clean, prompts, 5)
        run_to_the_end(clean.engine, 0)
        assert [clean.engine.remove(i).completion for i in ids] == expected

        llm = make_llm(folder, FaultyKernels({1, 3, 4, 8}), page_size=4)
        ids = submit(llm, prompts, 5)
        run_to_the_end(llm.engine, 4)
        assert [llm.engine.remove(i).completion for i in ids] == expected
        llm.runner.cache.check_invariants()
    finally:
        unregister_architecture("ToyHybridForCausalLM")


def test_a_retry_that_starts_elsewhere_than_the_cache_is_refused(tmp_path):
    """If the cache's length and the scheduler's count ever disagree, the step
    is refused before anything runs."""
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.engine.scheduler import SchedulerError
    folder = helpers.make_model_dir(tmp_path, "A", seed=0)
    llm = make_llm(folder, ReferenceKernels(), page_size=4)
    ids = submit(llm, [[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12]], 4)
    llm.engine.step()                                       # the first portion of 8
    llm.runner.step([StepEntry(ids[0], [9], [])])           # someone advances the cache behind the engine's back
    with pytest.raises(SchedulerError) as e:
        llm.engine.step()
    assert "inconsistent_batch" in str(e.value)


def test_the_runner_takes_a_provisional_step_back(tmp_path):
    from chibillm_b200.engine.batch import BatchError, StepEntry
    from chibillm_b200.engine.runner import ModelRunner
    folder = helpers.make_model_dir(tmp_path, "C", seed=2)       # windows on two layers: pages are given back
    runner = ModelRunner.from_folder(folder, dtype="float32", device="cpu", page_size=8, pool_tokens=256,
                                     max_requests=2, kernels=ReferenceKernels())
    ids = helpers.random_requests(301, [70], seed=3)["r0"]
    ref = helpers.plain_logits(folder, {"a": ids})["a"]
    runner.step([StepEntry("a", ids[:40], [])])
    free_before = {g: runner.cache.free_pages(g) for g in runner.cache.groups}
    first = runner.step([StepEntry("a", ids[40:64], [23])], provisional=True).clone()
    assert runner.length("a") == 64
    assert {g: runner.cache.free_pages(g) for g in runner.cache.groups} == \
        {g: free_before[g] - 3 for g in free_before}, "a held step must not give pages back yet"
    with pytest.raises(BatchError):
        runner.step([StepEntry("a", ids[64:66], [])], provisional=True)
    runner.rollback_step()
    assert runner.length("a") == 40
    again = runner.step([StepEntry("a", ids[40:64], [23])], provisional=True)
    assert torch.equal(first, again)
    runner.settle_step()
    assert any(runner.cache.free_pages(g) > free_before[g] - 3 for g in free_before), "settling frees window pages"
    last = runner.step([StepEntry("a", ids[64:], [5])])
    assert float((last[0] - ref[69]).abs().max()) < 2e-5 * float(ref.abs().max())
    runner.cache.check_invariants()
