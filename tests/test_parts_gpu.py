"""Each part alone against the plain implementation's function for it, at sizes
other than the engine tests'; generation through the Python entry point; and a
toy architecture, defined in the tests (toy_parts.py), whose mixer keeps state
of its own: it is registered, built, loaded and stepped without a change to the
framework."""
import json
import math
import os
from dataclasses import dataclass

import pytest
import torch

import helpers
import plain_qwen3
import tiny_configs

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def runtime(dtype):
    from chibillm_b200.engine.runner import make_runtime
    return make_runtime(dtype, DEV)


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


class FakeCtx:
    """The least a feed-forward needs of a step's context."""

    def __init__(self):
        from chibillm_b200.engine.batch import Workspace
        self.workspace = Workspace(torch.device(DEV))


TOL = {"float32": 5e-6, "bfloat16": 2e-2}


def close(got, ref, dtype, what):
    scale = float(ref.abs().max())
    worst = float((got.float().cpu() - ref).abs().max())
    assert worst <= TOL[dtype] * scale, f"{what} ({dtype}): {worst:.3e} > {TOL[dtype]:.0e} * {scale:.3f}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from chibillm_b200.config import NormSpec
    from chibillm_b200.parts import make_norm
    rt = runtime(dtype)
    norm = make_norm(NormSpec("rmsnorm", 200, 2e-5, 0.0), "w", rt)
    assert [(t.name, t.shape) for t in norm.expected_tensors()] == [("w", (200,))]
    w = (1 + 0.1 * rnd(200, seed=1)).to(torch.bfloat16)
    norm.bind({"w": w.to(DEV).to(rt.dtype)})
    x = rnd(13, 200, seed=2, scale=4.0)
    out = torch.empty(13, 200, dtype=rt.dtype, device=DEV)
    norm.forward(x.to(DEV), out)
    close(out, plain_qwen3.rms_norm(x, w.float(), 2e-5), dtype, "norm")
    # per-head use: every run of 200 features of a wider row is one group
    wide = rnd(5, 600, seed=3)
    out = torch.empty(5, 600, dtype=rt.dtype, device=DEV)
    norm.forward(wide.to(DEV).to(rt.dtype), out)
    ref = plain_qwen3.rms_norm(wide.to(rt.dtype).float().view(5, 3, 200), w.float(), 2e-5).view(5, 600)
    close(out, ref, dtype, "grouped norm")


def test_position_part():
    from chibillm_b200.config import PositionSpec
    from chibillm_b200.parts import make_position
    rt = runtime("float32")
    rope = make_position(PositionSpec("rope", head_dim=48, rotary_dim=48, theta=5e5), rt)
    table, rot = rope.fused_rotation()
    assert rot == 48 and torch.equal(table.cpu(), plain_qwen3.rope_inverse_frequencies(5e5, 48))
    none = make_position(PositionSpec("none"), rt)
    assert none.fused_rotation() == (None, 0)
    with pytest.raises(ValueError):
        make_position(PositionSpec("rope", head_dim=48, rotary_dim=50, theta=1e4), rt)
    with pytest.raises(KeyError):
        make_position(PositionSpec("alibi"), rt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    from chibillm_b200.config import GatedMLPSpec
    from chibillm_b200.parts import make_feed_forward
    rt = runtime(dtype)
    H, I, T = 72, 200, 11
    names = {"gate_proj": "g", "up_proj": "u", "down_proj": "d"}
    ff = make_feed_forward(GatedMLPSpec("gated_mlp", hidden_size=H, intermediate_size=I, activation="silu"),
                           names, rt)
    assert sorted((t.name, t.shape) for t in ff.expected_tensors()) == [("d", (H, I)), ("g", (I, H)), ("u", (I, H))]
    w = {n: rnd(*s, seed=i, scale=0.1, dtype=torch.bfloat16) for i, (n, s) in
         enumerate([("g", (I, H)), ("u", (I, H)), ("d", (H, I))])}
    ff.bind({n: t.to(DEV).to(rt.dtype) for n, t in w.items()})
    x = rnd(T, H, seed=7).to(rt.dtype)
    residual = rnd(T, H, seed=8)
    res_dev = residual.to(DEV).clone()
    pending = ff.forward(x.to(DEV), res_dev, FakeCtx())
    if pending is not None:
        pending.add_into(res_dev)
    xf = x.float()
    gate, up = xf @ w["g"].float().t(), xf @ w["u"].float().t()
    ref = residual + ((gate / (1 + torch.exp(-gate))) * up) @ w["d"].float().t()
    close(res_dev, ref, dtype, "feed-forward")


def _one_layer_runner(dtype, tmp_path, window=None):
    """A runner over a one-layer model with sizes the engine tests do not use."""
    cfg = tiny_configs.get("A")
    cfg.update(num_hidden_layers=1, hidden_size=72, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
               intermediate_size=136, vocab_size=211, rope_theta=2e4, rms_norm_eps=1e-5,
               max_position_embeddings=256, tie_word_embeddings=False)
    if window:
        cfg.update(use_sliding_window=True, sliding_window=window, max_window_layers=0)
    from chibillm_b200.weights import write_random_model
    from chibillm_b200.engine.runner import ModelRunner
    folder = os.path.join(str(tmp_path), f"one_layer_{dtype}_{window}")
    write_random_model(cfg, folder, seed=11)
    runner = ModelRunner.from_folder(folder, dtype=dtype, device=DEV, page_size=8, pool_tokens=256)
    return cfg, folder, runner


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 20])
def test_mixer_and_block_parts(dtype, window, tmp_path):
    """The attention mixer alone (its output added to a zero residual) and the
    whole block, fed with hidden states of our own in two steps (40 tokens, then
    9 more) so that the second step reads the first one's pages."""
    from chibillm_b200.engine.batch import StepEntry
    cfg, folder, runner = _one_layer_runner(dtype, tmp_path, window)
    config, weights = plain_qwen3.read_model_folder(folder)
    config["head_dim"] = cfg["head_dim"]
    rt = runner.runtime
    block = runner.model.blocks[0]
    T0, T1, H = 40, 9, cfg["hidden_size"]
    hidden = rnd(T0 + T1, H, seed=21)
    prefix = "model.layers.0."
    # plain: mixer output = attention_block(h) - h, with the block's own input norm inside
    ref_attn = plain_qwen3.attention_block(hidden, weights, prefix, config, window) - hidden
    ref_block = plain_qwen3.mlp_block(plain_qwen3.attention_block(hidden, weights, prefix, config, window),
                                      weights, prefix, config)
    for what in ("mixer", "block"):
        rid = f"{what}-{dtype}"
        outs = []
        for lo, hi in ((0, T0), (T0, T0 + T1)):
            entries = [StepEntry(rid, [0] * (hi - lo), [])]
            if not runner.has(rid):
                runner.admit(rid)
            runner.cache.reserve(rid, hi)
            ctx, updates, _ = runner._build_context(entries, False)
            for name, (view, cap) in updates.items():
                if cap:
                    rt.kernels.apply_table_updates(runner.storage.tables[name], view, cap)
            h = hidden[lo:hi].to(DEV)
            if what == "mixer":
                x = torch.empty(hi - lo, H, dtype=rt.dtype, device=DEV)
                block.mixer_norm.forward(h, x)
                residual = torch.zeros(hi - lo, H, device=DEV)
                pending = block.mixer.forward(x, residual, ctx, runner.storage.views[0])
            else:
                residual = h.clone()
                pending = block.forward(residual, ctx, runner.storage.views[0])
            if pending is not None:          # a last product that was left for the next norm to add
                pending.add_into(residual)
            outs.append(residual.cpu())
            runner.cache.commit(rid, hi)
        rt.kernels.check_error_word()
        runner.end(rid)
        close(torch.cat(outs), ref_attn if what == "mixer" else ref_block, dtype, f"{what} window={window}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype, tmp_path):
    import chibillm_b200
    folder = helpers.make_model_dir(tmp_path, "B", seed=1)
    config, weights = plain_qwen3.read_model_folder(folder)
    prompts = list(helpers.random_requests(384, [1, 7, 23, 40], seed=1).values())
    expected = [plain_qwen3.generate_greedy(config, weights, p, 12) for p in prompts]
    llm = chibillm_b200.LLM(folder, dtype=dtype, context_length=128, kv_cache_tokens=256, max_sequences=3,
                            max_batch_tokens=16, prefill_chunk_tokens=8)
    got = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    if dtype == "float32":
        assert got == expected
    else:
        # bfloat16 may flip a near-tie; what follows a flip differs, so compare up to the first one
        same = sum(1 for g, e in zip(got, expected) if g == e)
        first = [next((i for i, (a, b) in enumerate(zip(g, e)) if a != b), 12) for g, e in zip(got, expected)]
        assert same >= 3 and min(first) >= 4, (got, expected)
    llm.runner.cache.check_invariants()
    assert not llm.runner.cache.requests
    # sampling with a temperature: the same seed gives the same tokens, whatever the batch budget
    a = llm.generate(prompts, max_tokens=8, temperature=0.7, seed=1, ignore_eos=True)
    llm2 = chibillm_b200.LLM(folder, dtype=dtype, context_length=128, kv_cache_tokens=512, max_sequences=4,
                             max_batch_tokens=512, prefill_chunk_tokens=64)
    b = llm2.generate(prompts, max_tokens=8, temperature=0.7, seed=1, ignore_eos=True)
    if dtype == "float32":
        assert a == b
    c = llm2.generate(prompts, max_tokens=8, temperature=0.7, seed=2, ignore_eos=True)
    assert c != b


# ------------------------------------------------------------------ a toy architecture
from toy_parts import ToyStateSpec, register_toy as _register_toy, toy_plain as _toy_plain  # noqa: E402


def test_toy_architecture_with_a_state_of_its_own(tmp_path):
    from chibillm_b200.config import unregister_architecture
    from chibillm_b200.engine.runner import ModelRunner
    from chibillm_b200.weights import write_random_model
    _register_toy()
    try:
        obj = {"architectures": ["ToyHybridForCausalLM"], "hidden_size": 64, "intermediate_size": 96,
               "vocab_size": 131, "eps": 1e-5, "decay": 0.6, "max_positions": 128}
        folder = write_random_model(obj, str(tmp_path / "toy"), seed=3, dtype=torch.float32)
        runner = ModelRunner.from_folder(folder, dtype="float32", device=DEV, page_size=4, pool_tokens=256,
                                         max_requests=3)
        # two run steps keep state, the two attention steps share one paged cache
        assert [type(v).__name__ for v in runner.storage.views] == \
               ["PagedKVView", "FixedStateView", "FixedStateView", "PagedKVView"]
        assert not runner.storage.views[3].writes and runner.plan.groups[0].num_entries == 1
        _, w = plain_qwen3.read_model_folder(folder)
        reqs = helpers.random_requests(131, [30, 17, 45, 8, 26], seed=9)
        ref = {rid: _toy_plain(obj, w, ids) for rid, ids in reqs.items()}
        for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_portions(reqs, 1), "portions"),
                            (helpers.trace_mixed(reqs, 192, seed=2, max_live=3, decode_tail=6), "mixed")):
            got = helpers.run_trace(runner, trace)
            helpers.assert_logits_close(got, ref, 2e-5, f"toy {what}")
            runner.cache.check_invariants()
        assert runner.graph_replays == 0        # a part that gives no launch key is never captured
    finally:
        unregister_architecture("ToyHybridForCausalLM")


# ------------------------------------------------------------------ a second toy: routing and another position encoding
@dataclass(frozen=True)
class ToyRoutedSpec:
    kind: str
    hidden_size: int = 0
    intermediate_size: int = 0
    experts: int = 0


def _register_routed_toy():
    """A feed-forward that sends every token to one of its experts (router logits
    and softmax in 32-bit, the chosen expert's output weighted by its
    probability), and a position encoding that the kernels do not know: it
    rotates neighbouring pairs (2i, 2i + 1) instead of split halves, so the
    attention part has to call ``apply`` before the keys are cached."""
    from chibillm_b200.config import (AttentionSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec, RunStep,
                                      register_architecture)
    from chibillm_b200.parts import (FeedForward, PositionEncoding, TensorSpec, register_feed_forward,
                                     register_position)

    class PairRotation(PositionEncoding):
        def __init__(self, spec, rt):
            self.spec = spec
            j = torch.arange(spec.rotary_dim // 2, dtype=torch.float32)
            self.inv_freq = torch.pow(torch.tensor(float(spec.theta)), -2.0 * j / spec.rotary_dim).to(rt.device)

        def fused_rotation(self):
            return None

        def apply(self, q, k, ctx):
            angle = ctx.positions.float()[:, None] * self.inv_freq[None, :]        # [T, d/2]
            c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            for t in (q, k):
                if t is None:
                    continue
                T = t.shape[0]
                x = t.float().reshape(T, -1, self.spec.head_dim // 2, 2)
                x0, x1 = x[..., 0], x[..., 1]
                y = torch.stack([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1)
                t.copy_(y.reshape(T, -1).to(t.dtype))

    class RoutedFeedForward(FeedForward):
        def __init__(self, spec, names, rt):
            self.spec, self.names, self.rt = spec, names, rt

        def expected_tensors(self):
            s = self.spec
            out = [TensorSpec(self.names["router"], (s.experts, s.hidden_size))]
            for e in range(s.experts):
                out += [TensorSpec(self.names[f"up_{e}"], (s.intermediate_size, s.hidden_size)),
                        TensorSpec(self.names[f"down_{e}"], (s.hidden_size, s.intermediate_size))]
            return out

        def bind(self, tensors):
            self.router = tensors[self.names["router"]].float()
            self.up = [tensors[self.names[f"up_{e}"]].float() for e in range(self.spec.experts)]
            self.down = [tensors[self.names[f"down_{e}"]].float() for e in range(self.spec.experts)]

        def forward(self, x, residual, ctx):
            xf = x.float()
            prob = torch.softmax(xf @ self.router.t(), dim=-1)
            chosen = prob.argmax(dim=-1)
            for e in range(self.spec.experts):
                rows = (chosen == e).nonzero().flatten()
                if rows.numel():
                    h = xf[rows] @ self.up[e].t()
                    h = h / (1 + torch.exp(-h))
                    residual[rows] += prob[rows, e, None] * (h @ self.down[e].t())

    register_position("toy_pairs", PairRotation, replace=True)
    register_feed_forward("toy_routed", RoutedFeedForward, replace=True)

    def model_spec(obj):
        H, E = obj["hidden_size"], obj["experts"]
        norm = NormSpec("rmsnorm", H, obj["eps"], 0.0)
        ff = ToyRoutedSpec("toy_routed", H, obj["intermediate_size"], E)
        attn = AttentionSpec(kind="attention", hidden_size=H, num_heads=6, num_kv_heads=3, head_dim=16,
                             scale=0.25, window=None, qk_norm=NormSpec("rmsnorm", 16, obj["eps"], 0.0),
                             position=PositionSpec("toy_pairs", head_dim=16, rotary_dim=16, theta=obj["theta"]))
        names = [("mixer_norm", "n1.weight"), ("feed_forward_norm", "n2.weight"), ("q_proj", "q.weight"),
                 ("k_proj", "k.weight"), ("v_proj", "v.weight"), ("o_proj", "o.weight"), ("q_norm", "qn.weight"),
                 ("k_norm", "kn.weight"), ("router", "router.weight")]
        for e in range(E):
            names += [(f"up_{e}", f"experts.{e}.up.weight"), (f"down_{e}", f"experts.{e}.down.weight")]
        layers = tuple(LayerSpec("prenorm", attn, ff, norm, norm, f"layers.{i}.", tuple(names)) for i in range(2))
        return ModelSpec(architecture="ToyRoutedForCausalLM", vocab_size=obj["vocab_size"], hidden_size=H,
                         max_positions=obj["max_positions"], layers=layers, run_order=(RunStep(0), RunStep(1)),
                         final_norm=norm, embedding_name="embed.weight", final_norm_name="norm.weight",
                         output_name="head.weight", tie_output_to_embedding=False)

    register_architecture("ToyRoutedForCausalLM", lambda obj: obj, model_spec, replace=True)


def _routed_toy_plain(obj, w, ids):
    """Whole sequence, no cache, token by token where that is simplest."""
    T, H, E, d = len(ids), obj["hidden_size"], obj["experts"], 16
    eps, theta = obj["eps"], obj["theta"]
    h = plain_qwen3.embedding(w["embed.weight"], ids)

    def pairs(x, pos):                     # x: [heads, d]
        out = x.clone()
        for i in range(d // 2):
            a = torch.tensor(float(pos), dtype=torch.float32) * torch.pow(torch.tensor(float(theta)),
                                                                        torch.tensor(-2.0 * i / d))
            c, s = torch.cos(a), torch.sin(a)
            out[:, 2 * i] = x[:, 2 * i] * c - x[:, 2 * i + 1] * s
            out[:, 2 * i + 1] = x[:, 2 * i + 1] * c + x[:, 2 * i] * s
        return out

    for layer in range(2):
        p = f"layers.{layer}."
        x = plain_qwen3.rms_norm(h, w[p + "n1.weight"], eps)
        q = plain_qwen3.rms_norm((x @ w[p + "q.weight"].t()).view(T, 6, d), w[p + "qn.weight"], eps)
        k = plain_qwen3.rms_norm((x @ w[p + "k.weight"].t()).view(T, 3, d), w[p + "kn.weight"], eps)
        v = (x @ w[p + "v.weight"].t()).view(T, 3, d)
        q = torch.stack([pairs(q[t], t) for t in range(T)])
        k = torch.stack([pairs(k[t], t) for t in range(T)])
        h = h + plain_qwen3.causal_attention(q, k, v, None).reshape(T, 6 * d) @ w[p + "o.weight"].t()
        x = plain_qwen3.rms_norm(h, w[p + "n2.weight"], eps)
        out = torch.zeros_like(h)
        for t in range(T):
            prob = torch.softmax(w[p + "router.weight"] @ x[t], dim=0)
            e = int(prob.argmax())
            u = w[p + f"experts.{e}.up.weight"] @ x[t]
            out[t] = prob[e] * (w[p + f"experts.{e}.down.weight"] @ (u / (1 + torch.exp(-u))))
        h = h + out
    return plain_qwen3.rms_norm(h, w["norm.weight"], eps) @ w["head.weight"].t()


def test_toy_architecture_with_routing_and_its_own_position_encoding(tmp_path):
    from chibillm_b200.config import unregister_architecture
    from chibillm_b200.engine.runner import ModelRunner
    from chibillm_b200.weights import write_random_model
    _register_routed_toy()
    try:
        obj = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 48, "intermediate_size": 40, "experts": 3,
               "vocab_size": 97, "eps": 1e-5, "theta": 5000.0, "max_positions": 96}
        folder = write_random_model(obj, str(tmp_path / "routed"), seed=4, dtype=torch.float32)
        runner = ModelRunner.from_folder(folder, dtype="float32", device=DEV, page_size=4, pool_tokens=192,
                                         max_requests=3)
        _, w = plain_qwen3.read_model_folder(folder)
        # wide router weights, so that the experts really take turns
        reqs = helpers.random_requests(97, [21, 9, 40, 14], seed=11)
        ref = {rid: _routed_toy_plain(obj, w, ids) for rid, ids in reqs.items()}
        for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_portions(reqs, 1), "portions"),
                            (helpers.trace_mixed(reqs, 128, seed=5, max_live=3, decode_tail=5), "mixed")):
            got = helpers.run_trace(runner, trace)
            helpers.assert_logits_close(got, ref, 2e-5, f"routed toy {what}")
            runner.cache.check_invariants()
        assert runner.graph_replays == 0
    finally:
        unregister_architecture("ToyRoutedForCausalLM")


def test_toy_architecture_with_parts_at_the_decoders_ends(tmp_path):
    """Learned absolute positions after the embedding and soft-capped logits as
    adapters registered from the tests: nothing in the decoder changes for them."""
    import toy_parts
    from chibillm_b200.config import unregister_architecture
    from chibillm_b200.engine.runner import ModelRunner
    from chibillm_b200.weights import write_random_model
    toy_parts.register_absolute_toy()
    try:
        obj = dict(toy_parts.ABSOLUTE_TOY_CONFIG)
        for dtype, tol in (("float32", 2e-5), ("bfloat16", helpers.TOL["bfloat16"])):
            folder = write_random_model(obj, str(tmp_path / f"absolute_{dtype}"), seed=6, dtype=torch.float32)
            _, w = plain_qwen3.read_model_folder(folder)
            reqs = helpers.random_requests(113, [30, 8, 61, 17], seed=2)
            ref = {rid: toy_parts.absolute_toy_plain(obj, w, ids) for rid, ids in reqs.items()}
            runner = ModelRunner.from_folder(folder, dtype=dtype, device=DEV, page_size=4, pool_tokens=128,
                                             max_requests=3)
            for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_portions(reqs, 3), "portions"),
                                (helpers.trace_mixed(reqs, 128, seed=4, max_live=3, decode_tail=5), "mixed")):
                got = helpers.run_trace(runner, trace)
                helpers.assert_logits_close(got, ref, tol, f"absolute toy {dtype} {what}")
                runner.cache.check_invariants()
            assert runner.graph_replays == 0        # the adapters give no launch key
    finally:
        unregister_architecture("ToyAbsoluteForCausalLM")
