"""A toy architecture defined outside the package, for tests: attention layers
around a mixer with a running state of its own per request (h <- decay * h +
x_t; out_t = W h), whose state lives in the cache manager's slots.  Registered
through the package's public registries; a plain whole-sequence restatement
stands beside it.  It is no model of anyone's."""
from dataclasses import dataclass

import torch

import plain_qwen3


@dataclass(frozen=True)
class ToyStateSpec:
    kind: str
    hidden_size: int = 0
    decay: float = 0.5


def register_toy():
    """A mixer with a running state h per request: h <- decay * h + x_t;
    out_t = W h.  Its state lives in the cache manager's slots."""
    from chibillm_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec,
                                      RunStep, register_architecture)
    from chibillm_b200.parts import FixedStateNeed, Mixer, TensorSpec, register_mixer

    class ToyStateMixer(Mixer):
        def __init__(self, spec, names, rt):
            self.spec, self.names, self.rt = spec, names, rt

        def expected_tensors(self):
            return [TensorSpec(self.names["mix"], (self.spec.hidden_size, self.spec.hidden_size))]

        def bind(self, tensors):
            self.w = tensors[self.names["mix"]].float()

        def cache_need(self):
            return FixedStateNeed((("h", (self.spec.hidden_size,), torch.float32),))

        def forward(self, x, residual, ctx, cache):
            h_all = cache.arrays["h"]
            start = 0
            for slot, n in zip(ctx.slot_list, ctx.q_lens):
                h = h_all[slot].clone()
                for t in range(start, start + n):
                    h = self.spec.decay * h + x[t].float()
                    residual[t] += self.w @ h
                h_all[slot] = h
                start += n

    register_mixer("toy_state", ToyStateMixer, replace=True)

    def read_config(obj):
        return obj

    def model_spec(obj):
        H = obj["hidden_size"]
        norm = NormSpec("rmsnorm", H, obj["eps"], 0.0)
        mlp = GatedMLPSpec("gated_mlp", hidden_size=H, intermediate_size=obj["intermediate_size"], activation="silu")
        attn = AttentionSpec(kind="attention", hidden_size=H, num_heads=4, num_kv_heads=2, head_dim=16,
                             scale=0.25, window=None, qk_norm=None,
                             position=PositionSpec("rope", head_dim=16, rotary_dim=16, theta=1e4))
        names_attn = (("mixer_norm", "n1.weight"), ("feed_forward_norm", "n2.weight"), ("q_proj", "q.weight"),
                      ("k_proj", "k.weight"), ("v_proj", "v.weight"), ("o_proj", "o.weight"),
                      ("gate_proj", "gate.weight"), ("up_proj", "up.weight"), ("down_proj", "down.weight"))
        names_toy = (("mixer_norm", "n1.weight"), ("feed_forward_norm", "n2.weight"), ("mix", "mix.weight"),
                     ("gate_proj", "gate.weight"), ("up_proj", "up.weight"), ("down_proj", "down.weight"))
        layers = (LayerSpec("prenorm", attn, mlp, norm, norm, "layers.0.", names_attn),
                  LayerSpec("prenorm", ToyStateSpec("toy_state", H, obj["decay"]), mlp, norm, norm, "layers.1.",
                            names_toy))
        # attention, toy, the toy layer again (shared weights, a state of its own), attention
        # once more reading the first step's cache
        order = (RunStep(0), RunStep(1), RunStep(1), RunStep(0, cache_of=0))
        return ModelSpec(architecture="ToyHybridForCausalLM", vocab_size=obj["vocab_size"], hidden_size=H,
                         max_positions=obj["max_positions"], layers=layers, run_order=order, final_norm=norm,
                         embedding_name="embed.weight", final_norm_name="norm.weight", output_name="head.weight",
                         tie_output_to_embedding=True)

    register_architecture("ToyHybridForCausalLM", read_config, model_spec, replace=True)


TOY_CONFIG = {"architectures": ["ToyHybridForCausalLM"], "hidden_size": 64, "intermediate_size": 96,
              "vocab_size": 131, "eps": 1e-5, "decay": 0.6, "max_positions": 128}


def toy_plain(obj, w, ids):
    """Whole sequence, no cache."""
    T = len(ids)
    h = plain_qwen3.embedding(w["embed.weight"], ids)
    eps = obj["eps"]

    def mlp(h, p):
        x = plain_qwen3.rms_norm(h, w[p + "n2.weight"], eps)
        gate, up = x @ w[p + "gate.weight"].t(), x @ w[p + "up.weight"].t()
        return h + ((gate / (1 + torch.exp(-gate))) * up) @ w[p + "down.weight"].t()

    def attn(h, p, kv_from=None):
        x = plain_qwen3.rms_norm(h, w[p + "n1.weight"], eps)
        pos = torch.arange(T)
        q = plain_qwen3.rope((x @ w[p + "q.weight"].t()).view(T, 4, 16), pos, 1e4)
        if kv_from is None:
            k = plain_qwen3.rope((x @ w[p + "k.weight"].t()).view(T, 2, 16), pos, 1e4)
            v = (x @ w[p + "v.weight"].t()).view(T, 2, 16)
        else:
            k, v = kv_from
        out = plain_qwen3.causal_attention(q, k, v, None).reshape(T, 64)
        return h + out @ w[p + "o.weight"].t(), (k, v)

    def toy(h, p):
        x = plain_qwen3.rms_norm(h, w[p + "n1.weight"], eps)
        state = torch.zeros(h.shape[1])
        out = torch.empty_like(h)
        for t in range(T):
            state = obj["decay"] * state + x[t]
            out[t] = w[p + "mix.weight"] @ state
        return h + out

    h, kv = attn(h, "layers.0.")
    h = mlp(h, "layers.0.")
    for _ in range(2):
        h = mlp(toy(h, "layers.1."), "layers.1.")
    h, _ = attn(h, "layers.0.", kv_from=kv)
    h = mlp(h, "layers.0.")
    return plain_qwen3.rms_norm(h, w["norm.weight"], eps) @ w["embed.weight"].t()


# ------------------------------------------------------------------ a toy with parts at the decoder's ends
def register_absolute_toy():
    """Attention without any position encoding inside the mixer; instead a
    learned table of absolute positions is added to the embeddings (an input
    adapter), the embeddings are scaled by a constant, and the logits are
    soft-capped, c * tanh(logits / c) (a logit adapter).  None of this needs a
    change to the decoder: the adapters are registered like any other part."""
    from chibillm_b200.config import (AdapterSpec, AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec,
                                      PositionSpec, RunStep, register_architecture)
    from chibillm_b200.parts import Adapter, TensorSpec, register_adapter

    class AbsolutePositions(Adapter):
        def __init__(self, spec, rt):
            self.spec, self.rt = spec, rt
            self.scale = spec.constants()["embedding_scale"]
            self.rows = int(spec.constants()["positions"])
            self.width = int(spec.constants()["width"])

        def expected_tensors(self):
            return [TensorSpec(self.spec.names()["table"], (self.rows, self.width))]

        def bind(self, tensors):
            self.table = tensors[self.spec.names()["table"]].float()

        def forward(self, x, ctx):
            x.mul_(self.scale).add_(self.table[ctx.positions.long()])

    class SoftCap(Adapter):
        def __init__(self, spec, rt):
            self.cap = spec.constants()["cap"]

        def forward(self, x, ctx):
            x.copy_(torch.tanh(x / self.cap) * self.cap)

    register_adapter("toy_absolute_positions", AbsolutePositions, replace=True)
    register_adapter("toy_soft_cap", SoftCap, replace=True)

    def model_spec(obj):
        H = obj["hidden_size"]
        norm = NormSpec("rmsnorm", H, obj["eps"], 0.0)
        mlp = GatedMLPSpec("gated_mlp", hidden_size=H, intermediate_size=obj["intermediate_size"], activation="silu")
        attn = AttentionSpec(kind="attention", hidden_size=H, num_heads=4, num_kv_heads=2, head_dim=16,
                             scale=0.25, window=None, qk_norm=None, position=PositionSpec("none"))
        names = (("mixer_norm", "n1.weight"), ("feed_forward_norm", "n2.weight"), ("q_proj", "q.weight"),
                 ("k_proj", "k.weight"), ("v_proj", "v.weight"), ("o_proj", "o.weight"),
                 ("gate_proj", "gate.weight"), ("up_proj", "up.weight"), ("down_proj", "down.weight"))
        layers = tuple(LayerSpec("prenorm", attn, mlp, norm, norm, f"layers.{i}.", names) for i in range(2))
        return ModelSpec(architecture="ToyAbsoluteForCausalLM", vocab_size=obj["vocab_size"], hidden_size=H,
                         max_positions=obj["max_positions"], layers=layers, run_order=(RunStep(0), RunStep(1)),
                         final_norm=norm, embedding_name="embed.weight", final_norm_name="norm.weight",
                         output_name="head.weight", tie_output_to_embedding=True,
                         input_adapters=(AdapterSpec("toy_absolute_positions", (("table", "positions.weight"),),
                                                     (("embedding_scale", obj["embedding_scale"]),
                                                      ("positions", obj["max_positions"]), ("width", H))),),
                         logit_adapters=(AdapterSpec("toy_soft_cap", (), (("cap", obj["cap"]),)),))

    register_architecture("ToyAbsoluteForCausalLM", lambda obj: obj, model_spec, replace=True)


ABSOLUTE_TOY_CONFIG = {"architectures": ["ToyAbsoluteForCausalLM"], "hidden_size": 64, "intermediate_size": 80,
                       "vocab_size": 113, "eps": 1e-5, "max_positions": 96, "embedding_scale": 8.0, "cap": 0.4}


def absolute_toy_plain(obj, w, ids):
    """Whole sequence, no cache."""
    T = len(ids)
    eps = obj["eps"]
    h = plain_qwen3.embedding(w["embed.weight"], ids) * obj["embedding_scale"] + w["positions.weight"][:T]
    for i in range(2):
        p = f"layers.{i}."
        x = plain_qwen3.rms_norm(h, w[p + "n1.weight"], eps)
        q = (x @ w[p + "q.weight"].t()).view(T, 4, 16)
        k = (x @ w[p + "k.weight"].t()).view(T, 2, 16)
        v = (x @ w[p + "v.weight"].t()).view(T, 2, 16)
        h = h + plain_qwen3.causal_attention(q, k, v, None).reshape(T, 64) @ w[p + "o.weight"].t()
        x = plain_qwen3.rms_norm(h, w[p + "n2.weight"], eps)
        gate, up = x @ w[p + "gate.weight"].t(), x @ w[p + "up.weight"].t()
        h = h + ((gate / (1 + torch.exp(-gate))) * up) @ w[p + "down.weight"].t()
    logits = plain_qwen3.rms_norm(h, w["norm.weight"], eps) @ w["embed.weight"].t()
    return torch.tanh(logits / obj["cap"]) * obj["cap"]
