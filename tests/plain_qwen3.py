"""A plain, slow implementation of Qwen3 dense for whole sequences.

No cache, no batching, no paging: one sequence of token ids in, the logits of
every position out.  One function per part, each written from the reference's
formulas (the file:line of the formula is cited in the function).  It shares no
code with the package ``chibillm_b200``; it reads config.json and the
safetensors file with the ``safetensors`` library.

The reference's kernels are Metal shaders, which nothing here can run; its host
model code is portable C++ and does run on a CPU behind a stand-in for the
device layer.  tests/golden/make_goldens.py does that once for the tiny models
A and B and keeps the logits and greedy tokens under tests/golden/;
tests/test_reference_goldens.py compares this file (and the engine) with them.
So the layer order, weight packing, head grouping, rotation convention, paging
and tie rule of this file are checked against the reference's own code; the
arithmetic inside each kernel rests on the formulas cited below.

All arithmetic is in the dtype given (float32 by default, float64 for a
tighter yardstick); weights are widened to it first.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------ loading
def read_model_folder(model_dir: str, dtype=torch.float32):
    """config.json as a dict and every tensor of model.safetensors widened to
    ``dtype``."""
    from safetensors import safe_open

    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return config, weights


def layer_windows(config: dict) -> List[Optional[int]]:
    """Per layer: None (all keys) or the number of most recent keys it sees."""
    layers = config["num_hidden_layers"]
    if not config.get("use_sliding_window", False):
        return [None] * layers
    window = config["sliding_window"]
    if config.get("layer_types"):
        return [window if t == "sliding_attention" else None for t in config["layer_types"]]
    first = config.get("max_window_layers", layers)
    return [None if i < first else window for i in range(layers)]


# ------------------------------------------------------------------ parts
def embedding(table: torch.Tensor, token_ids: List[int]) -> torch.Tensor:
    """h0[t, :] = float(E[token[t], :])  (src/metal/kernels/tensor_ops.metal:12-24)."""
    return table[torch.tensor(token_ids, dtype=torch.long, device=table.device)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Over the last dimension: s = sum x^2; inv = rsqrt(s / n + eps);
    y = (x * inv) * w, plain weight without an offset
    (src/metal/kernels/tensor_ops.metal:76-105; src/metal/metal_kernels.mm:42-43)."""
    n = x.shape[-1]
    s = (x * x).sum(dim=-1, keepdim=True)
    inv = torch.rsqrt(s / n + eps)
    return (x * inv) * weight


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = x . W^T with W stored [out, in]  (src/metal/kernels/linear.metal:136-156)."""
    return x @ weight.t()


def rope_inverse_frequencies(theta: float, rotary_dim: int) -> torch.Tensor:
    """inv_freq[j] = powf(theta, -2j / rotary_dim), computed in float
    (src/metal/metal_kernels.mm:186-191)."""
    j = torch.arange(rotary_dim // 2, dtype=torch.float32)
    return torch.pow(torch.tensor(float(theta), dtype=torch.float32), (-2.0 * j) / float(rotary_dim))


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x: [T, heads, d].  Split-half pairs (j, j + d/2): a = float(pos) * inv_freq[j];
    out[j] = x[j] cos a - x[j + d/2] sin a; out[j + d/2] = x[j + d/2] cos a + x[j] sin a
    (src/metal/kernels/tensor_ops.metal:168-197)."""
    d = x.shape[-1]
    half = d // 2
    inv_freq = rope_inverse_frequencies(theta, d).to(x.device)
    positions = positions.to(x.device)
    if x.dtype == torch.float64:
        angle = positions.to(torch.float64)[:, None] * inv_freq.to(torch.float64)[None, :]
    else:
        angle = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    c = torch.cos(angle).to(x.dtype)[:, None, :]
    s = torch.sin(angle).to(x.dtype)[:, None, :]
    lo, hi = x[..., :half], x[..., half:]
    return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int]) -> torch.Tensor:
    """q: [T, nq, d]; k, v: [T, nkv, d].  Query head i uses kv head i // (nq / nkv);
    the row at position p sees positions 0..p (with a window W: the W most recent,
    itself included); score = (q . k) * rsqrt(d), scaled after the dot product;
    softmax over the visible scores; output = sum p_u v_u
    (src/metal/kernels/attention.metal:81-158)."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = 1.0 / math.sqrt(float(d))
    out = torch.empty_like(q)
    pos = torch.arange(T, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > pos[:, None] - window
    for i in range(nq):
        g = i // group
        scores = (q[:, i, :] @ k[:, g, :].t()) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        p = torch.exp(scores - m)
        out[:, i, :] = (p @ v[:, g, :]) / p.sum(dim=-1, keepdim=True)
    return out


def attention_block(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, config: dict,
                    window: Optional[int]) -> torch.Tensor:
    """h + o_proj(attention(rope(norm_q(q)), rope(norm_k(k)), v)) with
    q, k, v = projections of RMSNorm(h, input_layernorm)
    (src/qwen/qwen_layer.cc:56-101 for projection and q/k norm, :20-30 rotation,
    :32-52 append, attention, output projection plus residual)."""
    T = h.shape[0]
    nq, nkv, d = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    eps = config["rms_norm_eps"]
    x = rms_norm(h, w[prefix + "input_layernorm.weight"], eps)
    q = linear(x, w[prefix + "self_attn.q_proj.weight"]).view(T, nq, d)
    k = linear(x, w[prefix + "self_attn.k_proj.weight"]).view(T, nkv, d)
    v = linear(x, w[prefix + "self_attn.v_proj.weight"]).view(T, nkv, d)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], eps)
    positions = torch.arange(T, device=h.device)
    q = rope(q, positions, config["rope_theta"])
    k = rope(k, positions, config["rope_theta"])
    att = causal_attention(q, k, v, window).reshape(T, nq * d)
    return h + linear(att, w[prefix + "self_attn.o_proj.weight"])


def mlp_block(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, config: dict) -> torch.Tensor:
    """h + down((gate / (1 + exp(-gate))) * up) on RMSNorm(h, post_attention_layernorm)
    (src/tensor/functions.cc:241-252; src/metal/kernels/tensor_ops.metal:120-123)."""
    x = rms_norm(h, w[prefix + "post_attention_layernorm.weight"], config["rms_norm_eps"])
    gate = linear(x, w[prefix + "mlp.gate_proj.weight"])
    up = linear(x, w[prefix + "mlp.up_proj.weight"])
    act = (gate / (1.0 + torch.exp(-gate))) * up
    return h + linear(act, w[prefix + "mlp.down_proj.weight"])


def final_logits(h: torch.Tensor, w: Dict[str, torch.Tensor], config: dict) -> torch.Tensor:
    """RMSNorm(h, model.norm) . W_vocab^T, W_vocab = lm_head.weight if the file has
    it, else the embedding table (src/tensor/functions.cc:338-358;
    src/qwen/qwen_weights.h:36-40)."""
    y = rms_norm(h, w["model.norm.weight"], config["rms_norm_eps"])
    vocab = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(y, vocab)


# ------------------------------------------------------------------ whole model
def forward(config: dict, weights: Dict[str, torch.Tensor], token_ids: List[int],
            rows: Optional[List[int]] = None) -> torch.Tensor:
    """Logits [T, vocab] of every position of one sequence, or of the positions
    ``rows`` only (layer order: src/qwen/qwen_layer.cc:124-146).  Runs on the
    device that holds the weights."""
    config = dict(config)
    config.setdefault("head_dim", config["hidden_size"] // config["num_attention_heads"])
    windows = layer_windows(config)
    h = embedding(weights["model.embed_tokens.weight"], token_ids)
    for layer in range(config["num_hidden_layers"]):
        prefix = f"model.layers.{layer}."
        h = attention_block(h, weights, prefix, config, windows[layer])
        h = mlp_block(h, weights, prefix, config)
    if rows is not None:
        h = h[torch.tensor(rows, dtype=torch.long, device=h.device)]
    return final_logits(h, weights, config)


def greedy(logits_row: torch.Tensor) -> int:
    """Arg max, ties to the lowest id (src/metal/kernels/sampling.metal:55-60,145-149)."""
    best = logits_row.max()
    return int(torch.nonzero(logits_row == best)[0, 0])


def generate_greedy(config: dict, weights: Dict[str, torch.Tensor], prompt: List[int], steps: int) -> List[int]:
    """Feed the whole sequence again for every new token."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        nxt = greedy(forward(config, weights, ids)[-1])
        out.append(nxt)
        ids.append(nxt)
    return out


# ------------------------------------------------------------------ sampling at a temperature
def sample_uniform(seed: int, request_key: int, index: int) -> float:
    """The number in [0, 1) that decides the ``index``-th generated token of a
    request: 24 bits of a SHA-256 over "seed/key/index".  The reference has no
    sampling at a temperature (src/server.cc:128-132 refuses one); this restates
    the engine's rule so that both draw the same number."""
    import hashlib
    digest = hashlib.sha256(f"{seed}/{request_key}/{index}".encode()).digest()
    return (int.from_bytes(digest[:8], "little") >> 40) / float(1 << 24)


def sample_at_temperature(logits_row: torch.Tensor, temperature: float, u: float) -> int:
    """p_i = exp((x_i - max) / T); the first id whose running sum of p, in id
    order, exceeds u * sum(p).  Sums in 64-bit so that this side adds no
    rounding of its own."""
    if not temperature > 0.0:
        return greedy(logits_row)
    x = logits_row.double()
    p = torch.exp((x - x.max()) / temperature)
    cdf = torch.cumsum(p, dim=0)
    target = u * float(cdf[-1])
    idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True))
    return min(idx, x.numel() - 1)


def generate_sampled(config: dict, weights: Dict[str, torch.Tensor], prompt: List[int], steps: int,
                     temperature: float, seed: int, request_key: int) -> List[int]:
    ids = list(prompt)
    out = []
    for index in range(steps):
        row = forward(config, weights, ids, rows=[len(ids) - 1])[0]
        tok = sample_at_temperature(row, temperature, sample_uniform(seed, request_key, index))
        out.append(tok)
        ids.append(tok)
    return out
