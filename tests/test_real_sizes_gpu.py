"""Layer sizes of real checkpoints (Qwen3-0.6B and slices of Qwen3-8B and Qwen3-14B: head size
128, vocabulary 151,936, tied or untied output) with random weights and one or
two layers, against the plain implementation run on the GPU in true 32-bit: the
32-bit engine and the bfloat16 engine, whole prompts, portions and decoded
tokens, four live requests with reused pages, and contexts of 8,200 and 16,400
tokens.  These sizes take the tensor-core kernels (tcgen05 products with split
K ranges, tensor-core attention, decode attention over many key ranges) that
the tiny configurations do not reach."""
import pytest
import torch

import helpers
import plain_qwen3

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")


def base(**kw):
    d = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "attention_bias": False,
         "hidden_act": "silu", "rope_scaling": None, "torch_dtype": "bfloat16", "head_dim": 128,
         "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 40960,
         "use_sliding_window": False, "sliding_window": None, "num_hidden_layers": 2}
    d.update(kw)
    return d


SHAPES = {
    "0.6B": base(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, intermediate_size=3072,
                 tie_word_embeddings=True),
    "8B": base(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, intermediate_size=12288,
               tie_word_embeddings=False),
    # five query heads per kv head, widths that are no multiple of 1,024
    "14B": base(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=17408,
                tie_word_embeddings=False),
}


@pytest.fixture(autouse=True)
def true_32_bit():
    """The plain implementation's products on the GPU are 32-bit FMA, no TF32."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = old


def plain_weights(cfg, seed):
    """name -> 32-bit tensor on the GPU: the values that the engine's
    ``from_random`` makes for this configuration and seed (stored as bfloat16)."""
    from chibillm_b200.config.registry import find_architecture
    from chibillm_b200.engine.model import DecoderModel
    from chibillm_b200.parts.base import Runtime
    from chibillm_b200.weights import random_tensors
    arch = find_architecture(cfg)
    model = DecoderModel(arch.model_spec(arch.read_config(cfg)), Runtime(DEV, torch.bfloat16, None))
    return {name: t.float() for name, t in random_tensors(model, seed, torch.bfloat16, DEV)}


def plain_rows(cfg, weights, reqs, want):
    return {rid: plain_qwen3.forward(cfg, weights, ids, rows=want[rid]).float().cpu() for rid, ids in reqs.items()}


def free():
    import gc
    gc.collect()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("shape", list(SHAPES))
def test_engines_against_the_plain_implementation(shape):
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.engine.runner import ModelRunner
    cfg = SHAPES[shape]
    reqs = helpers.random_requests(cfg["vocab_size"], [300, 70, 1, 129], seed=3)
    # only a few places are wanted: a row of logits is 600 KB
    want = {rid: sorted({0, len(ids) // 2, len(ids) - 1}) for rid, ids in reqs.items()}
    weights = plain_weights(cfg, 5)
    ref = plain_rows(cfg, weights, reqs, want)
    del weights
    free()

    def run(dtype, trace_fn):
        runner = ModelRunner.from_random(cfg, seed=5, dtype=dtype, page_size=16, pool_tokens=1024, max_requests=4)
        out = {}
        for rid, ids in reqs.items():
            rows = {}
            fed = 0
            for portion in trace_fn(ids):
                places = [w - fed for w in want[rid] if fed <= w < fed + len(portion)]
                logits = runner.step([StepEntry(rid, portion, places)])
                for k, w in enumerate(places):
                    rows[fed + w] = logits[k].float().cpu().clone()
                fed += len(portion)
            runner.end(rid)
            out[rid] = torch.stack([rows[w] for w in want[rid]])
        replays = runner.graph_replays
        del runner
        free()
        return out, replays

    whole = lambda ids: [ids]

    def cut(ids):          # a big portion, small ones, then the last 20 tokens one by one
        head = max(1, len(ids) - 20)
        parts = [ids[:head // 2], ids[head // 2:head]] if head > 1 else [ids[:head]]
        return [p for p in parts if p] + [[t] for t in ids[head:]]

    f32_whole, _ = run("float32", whole)
    helpers.assert_logits_close(f32_whole, ref, helpers.TOL["float32"], f"{shape} float32 whole vs plain")
    f32_cut, _ = run("float32", cut)
    helpers.assert_logits_close(f32_cut, ref, helpers.TOL["float32"], f"{shape} float32 cut vs plain")
    bf_whole, _ = run("bfloat16", whole)
    helpers.assert_logits_close(bf_whole, ref, helpers.TOL["bfloat16"], f"{shape} bfloat16 whole vs plain")
    bf_cut, replays = run("bfloat16", cut)
    assert replays > 0, "decode steps were not replayed from a graph"
    helpers.assert_logits_close(bf_cut, ref, helpers.TOL["bfloat16"], f"{shape} bfloat16 cut vs plain")
    helpers.assert_logits_close(bf_cut, bf_whole, helpers.TOL_SAME_DTYPE["bfloat16"], f"{shape} bfloat16 cut vs whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_at_the_8b_layer_sizes(dtype):
    """Four live requests at the Qwen3-8B layer sizes: portions of some beside
    decoded tokens of others, a pool so small that pages are used again, every
    position's logits against the plain implementation."""
    from chibillm_b200.engine.runner import ModelRunner
    cfg = dict(SHAPES["8B"], num_hidden_layers=1)
    reqs = helpers.random_requests(cfg["vocab_size"], [60, 50, 20, 90, 33, 64], seed=4)
    weights = plain_weights(cfg, 7)
    ref = {rid: plain_qwen3.forward(cfg, weights, ids).float().cpu() for rid, ids in reqs.items()}
    del weights
    free()
    pool = 320
    trace = helpers.trace_mixed(reqs, pool, seed=6)
    assert helpers.peak_tokens(trace) <= pool < sum(helpers.round64(len(v)) for v in reqs.values())
    assert any(len(s["entries"]) == 4 for s in trace)
    runner = ModelRunner.from_random(cfg, seed=7, dtype=dtype, page_size=16, pool_tokens=pool, max_requests=4)
    runner.storage.poison()
    got = helpers.run_trace(runner, trace)
    helpers.assert_logits_close(got, ref, helpers.TOL[dtype], f"8B sizes, mixed, {dtype}")
    runner.cache.check_invariants()
    assert not runner.cache.requests
    del runner
    free()


@pytest.mark.parametrize("shape,held,dtype", [("14B", 8200, "float32"), ("14B", 8200, "bfloat16"),
                                              ("8B", 16400, "bfloat16")])
def test_long_contexts_against_the_plain_implementation(shape, held, dtype):
    """One layer at the Qwen3-14B sizes (five query heads to a kv head) holding
    8,200 tokens, and at the 8B sizes holding 16,400, then eight decoded tokens:
    block tables of over a thousand pages and decode attention over dozens of key
    ranges, against the plain implementation."""
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.engine.runner import ModelRunner
    cfg = dict(SHAPES[shape], num_hidden_layers=1)
    ids = helpers.random_requests(cfg["vocab_size"], [held + 8], seed=21)["r0"]
    prompt_rows = [0, held // 2 + 3, held - 1]
    want = prompt_rows + list(range(held, held + 8))
    weights = plain_weights(cfg, 9)
    ref = {"a": plain_qwen3.forward(cfg, weights, ids, rows=want).float().cpu()}
    del weights
    free()
    runner = ModelRunner.from_random(cfg, seed=9, dtype=dtype, page_size=16, pool_tokens=held + 64, max_requests=2)
    runner.storage.poison()
    rows = [runner.step([StepEntry("a", ids[:held], prompt_rows)]).float().cpu().clone()]
    for t in ids[held:]:
        rows.append(runner.step([StepEntry("a", [t], [0])]).float().cpu().clone())
    runner.runtime.kernels.check_error_word()
    got = {"a": torch.cat(rows)}
    helpers.assert_logits_close(got, ref, helpers.TOL[dtype], f"{shape} sizes, {held} tokens held, {dtype}")
    del runner
    free()


def test_long_context_decode():
    """A context of 3,000 tokens at the 0.6B layer sizes, then 16 decoded tokens:
    the bfloat16 engine's logits stay close to the 32-bit engine's, so no key of
    the long context is lost by the split attention or at a page's edge."""
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.engine.runner import ModelRunner
    cfg = dict(SHAPES["0.6B"], num_hidden_layers=1)
    ids = helpers.random_requests(cfg["vocab_size"], [3016], seed=9)["r0"]
    outs = {}
    for dtype in ("float32", "bfloat16"):
        runner = ModelRunner.from_random(cfg, seed=6, dtype=dtype, page_size=16, pool_tokens=3072, max_requests=2)
        runner.step([StepEntry("a", ids[:3000], [])])
        rows = []
        for t in ids[3000:]:
            rows.append(runner.step([StepEntry("a", [t], [0])])[0].float().cpu().clone())
        outs[dtype] = {"a": torch.stack(rows)}
        del runner
        torch.cuda.empty_cache()
    helpers.assert_logits_close(outs["bfloat16"], outs["float32"], helpers.TOL["bfloat16"], "long context decode")


def test_long_prompt_takes_the_many_row_kernels():
    """A prompt of 1,600 tokens at the 8B layer sizes (one layer), whole and in two
    portions of which the second continues the first: the prompt attention with two
    query tiles per CTA, the per-token norm + rotation kernel and the persistent
    matrix product, against the 32-bit engine; then generation with and without
    steps that run ahead gives the same tokens."""
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.engine.runner import ModelRunner
    cfg = dict(SHAPES["8B"], num_hidden_layers=1)
    ids = helpers.random_requests(cfg["vocab_size"], [1600], seed=12)["r0"]
    want = [0, 511, 1100, 1599]
    outs = {}
    for dtype, cuts in (("float32", [1600]), ("bfloat16", [1600]), ("bfloat16", [900, 700])):
        runner = ModelRunner.from_random(cfg, seed=8, dtype=dtype, page_size=16, pool_tokens=2048, max_requests=2)
        rows, fed = {}, 0
        for n in cuts:
            places = [w - fed for w in want if fed <= w < fed + n]
            logits = runner.step([StepEntry("a", ids[fed:fed + n], places)])
            for k, w in enumerate(places):
                rows[fed + w] = logits[k].float().cpu().clone()
            fed += n
        outs[(dtype, len(cuts))] = {"a": torch.stack([rows[w] for w in want])}
        del runner
        torch.cuda.empty_cache()
    ref = outs[("float32", 1)]
    helpers.assert_logits_close(outs[("bfloat16", 1)], ref, helpers.TOL["bfloat16"], "long prompt, whole")
    helpers.assert_logits_close(outs[("bfloat16", 2)], ref, helpers.TOL["bfloat16"], "long prompt, two portions")
    helpers.assert_logits_close(outs[("bfloat16", 2)], outs[("bfloat16", 1)], helpers.TOL_SAME_DTYPE["bfloat16"],
                                "long prompt, portions vs whole")

    import chibillm_b200
    from chibillm_b200.sampling import SamplingParams
    tokens = {}
    for ahead in (False, True):
        llm = chibillm_b200.LLM(None, random_config=cfg, dtype="bfloat16", context_length=2048,
                                kv_cache_tokens=4096, max_sequences=2)
        llm.engine.run_ahead = ahead
        tokens[ahead] = llm.engine.generate([ids[:1300], ids[300:900]],
                                            [SamplingParams(max_new_tokens=24, ignore_eos=True)] * 2)
        assert (llm.runner.steps_ahead_used > 0) == ahead
        del llm
        torch.cuda.empty_cache()
    assert tokens[True] == tokens[False]


def test_many_sequences_decode_through_the_many_row_product():
    """80 sequences decode in step: more than 64 rows, so the products of the replayed decode
    graph are the many-row kernel, whose few tiles at this width are shared out by K blocks
    (partial sums through scratch and counters that every launch must leave at zero).  The
    bfloat16 engine against the 32-bit engine, step after step."""
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.engine.runner import ModelRunner
    cfg = base(hidden_size=1024, num_attention_heads=8, num_key_value_heads=2, intermediate_size=2048,
               vocab_size=4096, tie_word_embeddings=True)
    n, steps = 80, 6
    reqs = helpers.random_requests(cfg["vocab_size"], [3 + (i * 7) % 20 for i in range(n)], seed=9)
    follow = helpers.random_requests(cfg["vocab_size"], [steps] * n, seed=10)

    def run(dtype):
        runner = ModelRunner.from_random(cfg, seed=6, dtype=dtype, page_size=16, pool_tokens=64 * n, max_requests=n)
        rows = [runner.step([StepEntry(rid, ids, [len(ids) - 1]) for rid, ids in reqs.items()]).float().cpu().clone()]
        for s in range(steps):
            rows.append(runner.step([StepEntry(rid, [follow[rid][s]], [0]) for rid in reqs]).float().cpu().clone())
        runner.runtime.kernels.check_error_word()
        return torch.stack(rows), runner.graph_replays

    exact, _ = run("float32")
    got, replays = run("bfloat16")
    assert replays >= steps - 2, "the decode steps were not replayed from a graph"
    scale = float(exact.abs().max())
    worst = float((got - exact).abs().max())
    assert worst <= helpers.TOL["bfloat16"] * scale, f"bfloat16 against 32-bit: {worst} of {scale}"
    assert (got.argmax(-1) == exact.argmax(-1)).float().mean() > 0.9
