"""The decode step that is launched before the host has the tokens of the step
before it: generation must give the same tokens with and without it, whether
requests end by their limit (foretold: nothing runs ahead then) or by an
end-of-sequence token (not foretold: the step that ran ahead is dropped), while
requests wait to be admitted, and with sampling at a temperature."""
import copy

import pytest
import torch

import tiny_configs

pytestmark = pytest.mark.gpu


def _generate(cfg, prompts, params, run_ahead, max_sequences=3):
    import chibillm_b200
    llm = chibillm_b200.LLM(None, random_config=cfg, dtype="bfloat16", context_length=256, kv_cache_tokens=1024,
                            max_sequences=max_sequences)
    llm.engine.run_ahead = run_ahead
    out = llm.engine.generate(prompts, params)
    runner = llm.runner
    runner.cache.check_invariants()
    for group in runner.cache.groups.values():
        assert runner.cache.free_pages(group.name) == group.num_pages, "pages were lost"
    return out, runner.steps_ahead_used, runner.steps_ahead_dropped


@pytest.mark.parametrize("name", ["D128", "B", "C"])
def test_running_ahead_gives_the_same_tokens(name):
    from chibillm_b200.sampling import SamplingParams
    cfg = copy.deepcopy(tiny_configs.get(name))
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (5, 33, 17, 64, 9, 21)]
    limits = ((40, 0.0), (25, 0.7), (60, 0.0), (33, 0.0), (50, 1.0), (12, 0.0))
    params = [SamplingParams(max_new_tokens=m, ignore_eos=True, temperature=t, seed=3) for m, t in limits]
    plain, used0, _ = _generate(cfg, prompts, params, run_ahead=False)
    ahead, used, dropped = _generate(cfg, prompts, params, run_ahead=True)
    assert used0 == 0 and used > 10, "no step ran ahead"
    assert ahead == plain
    assert [len(o) for o in ahead] == [m for m, _ in limits]
    assert dropped == 0, "a limit is foretold: no step should have been dropped"

    # An end-of-sequence token in the middle of a reply, with all requests running (nobody
    # waits, so steps do run ahead when it comes): a token that the reply has not used before.
    # Sampled at a temperature, so that replies of random weights do not just repeat a token.
    prompts = prompts[:3]
    params = [SamplingParams(max_new_tokens=60, ignore_eos=True, temperature=0.9, seed=3) for _ in prompts]
    free, _, _ = _generate(cfg, prompts, params, run_ahead=False)
    used_elsewhere = lambda r, tok, i: any(tok in free[o][:i + 2] for o in range(3) if o != r)
    r, at = next((r, i) for r in range(3) for i in range(10, 50)
                 if free[r][i] not in free[r][:i] and not used_elsewhere(r, free[r][i], i))
    cfg["eos_token_id"] = int(free[r][at])
    params = [SamplingParams(max_new_tokens=60, ignore_eos=False, temperature=0.9, seed=3) for _ in prompts]
    plain, _, _ = _generate(cfg, prompts, params, run_ahead=False)
    ahead, used, dropped = _generate(cfg, prompts, params, run_ahead=True)
    assert ahead == plain
    assert plain[r] == free[r][:at + 1]
    assert used >= 5 and dropped >= 1, "the step after an unforeseen end should have been dropped"


def test_a_failed_step_with_one_launched_ahead_is_run_again():
    """The error word is read after the next step has already been launched.  A
    fault reported then (injected on the host: the read of the copy raises once)
    takes both steps back, and generation ends with the tokens of a clean run."""
    import chibillm_b200
    from chibillm_b200.sampling import SamplingParams
    cfg = copy.deepcopy(tiny_configs.get("D128"))
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (12, 40, 7)]
    params = [SamplingParams(max_new_tokens=30, ignore_eos=True, temperature=0.8, seed=4) for _ in prompts]
    clean, used, _ = _generate(cfg, prompts, params, run_ahead=True)
    assert used > 10

    class Injected(RuntimeError):
        pass

    llm = chibillm_b200.LLM(None, random_config=cfg, dtype="bfloat16", context_length=256, kv_cache_tokens=1024,
                            max_sequences=3)
    kernels = llm.runner.runtime.kernels
    check = kernels.check_error_copy
    reads = {"n": 0, "ahead_at_fault": []}

    def flaky():
        reads["n"] += 1
        if reads["n"] in (1, 9, 10, 20):
            reads["ahead_at_fault"].append(llm.runner._ahead is not None)
            raise Injected()
        check()

    kernels.check_error_copy = flaky
    ids = []
    for i, (p, sp) in enumerate(zip(prompts, params)):
        ids.append(("r", i))
        llm.engine.add(("r", i), p, sp, sample_key=i)
    faults = 0
    while not llm.engine.is_finished():
        try:
            llm.engine.step()
        except Injected:
            faults += 1
    assert faults == 4 and any(reads["ahead_at_fault"]), "no fault came while a step was launched ahead"
    assert [llm.engine.remove(i).completion for i in ids] == clean
    llm.runner.cache.check_invariants()
