"""Causal grouped-query attention over the paged cache, as a mixer.

Order of operations (src/qwen/qwen_layer.cc:56-101, 20-52): one product gives
q | k | v (the three matrices are stacked, src/qwen/qwen_weights.cc:27-31);
every q and k head is RMS-normalised over its own features with one weight
shared by all heads; q and k are rotated; k and v are appended to the cache
before the scores are taken, so a token sees itself; softmax in 32-bit over
scale * (q . k); the output projection adds into the residual.

The part takes every size and constant from its spec: head counts, head size,
scale, window, the norm of q and k (or none), the position encoding (or none).
When its run step reads another step's cache, it computes q only and appends
nothing.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import (Mixer, PagedKVNeed, Runtime, TensorSpec, make_position, register_mixer)


class PagedAttention(Mixer):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        if spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.position = make_position(spec.position, runtime)
        self.qkv: torch.Tensor = None
        self.o_proj: torch.Tensor = None
        self.q_norm: torch.Tensor = None
        self.k_norm: torch.Tensor = None

    # ---- weights
    def expected_tensors(self) -> List[TensorSpec]:
        s = self.spec
        qw, kw = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        out = [TensorSpec(self.names["q_proj"], (qw, s.hidden_size)),
               TensorSpec(self.names["k_proj"], (kw, s.hidden_size)),
               TensorSpec(self.names["v_proj"], (kw, s.hidden_size)),
               TensorSpec(self.names["o_proj"], (s.hidden_size, qw))]
        if s.qk_norm is not None:
            out += [TensorSpec(self.names["q_norm"], (s.qk_norm.size,)),
                    TensorSpec(self.names["k_norm"], (s.qk_norm.size,))]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        q, k, v = (tensors[self.names[r]] for r in ("q_proj", "k_proj", "v_proj"))
        k, v = k.to(q.dtype), v.to(q.dtype)
        self.qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.o_proj = tensors[self.names["o_proj"]].contiguous()
        if self.spec.qk_norm is not None:
            self.q_norm = tensors[self.names["q_norm"]].contiguous()
            self.k_norm = tensors[self.names["k_norm"]].to(self.q_norm.dtype).contiguous()

    # ---- cache
    accepts_scaled_rows = True       # x goes to the q | k | v product and nowhere else

    def cache_need(self):
        s = self.spec
        return PagedKVNeed(num_kv_heads=s.num_kv_heads, head_dim=s.head_dim, window=s.window)

    def launch_key(self, ctx):
        if self.position.fused_rotation() is None:
            return None                      # an encoding of its own: nothing is promised
        k = self.runtime.kernels
        splits = getattr(k, "decode_attention_splits", None)
        if splits is None:
            return None
        s = self.spec
        return (splits(ctx.num_seqs, s.num_heads, s.num_kv_heads, ctx.max_ctx_len),)

    # ---- run
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache) -> None:
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T = x.shape[0]
        nq, nkv, d = s.num_heads, s.num_kv_heads, s.head_dim
        qw, kw = nq * d, nkv * d
        writes = cache.writes
        width = qw + 2 * kw if writes else qw
        fused = self.position.fused_rotation()
        if fused is not None and fused[0] is not None and self._heads_from_the_product(x, ctx, cache, fused):
            return self._attend(residual, ctx, cache)
        split = getattr(k, "linear_partial", None)
        pending = None
        if split is not None and fused is not None and d % 4 == 0:
            # the kernels that add these sums up (decode attention; norm + rotation + append) fetch
            # eight splits of a head in one go
            pending = split(x, self.qkv if writes else self.qkv[:qw], max_splits=8)
        if pending is None:
            qkv = ctx.workspace.get("attn.qkv", (T, width), rt.dtype)
            k.linear(x, self.qkv if writes else self.qkv[:qw], qkv)

        q = ctx.workspace.get("attn.q", (T, qw), rt.dtype)
        table = ctx.tables[cache.group]
        norm = s.qk_norm
        q_norm_w = self.q_norm if norm is not None else None
        k_norm_w = self.k_norm if norm is not None else None
        att = ctx.workspace.get("attn.out", (T, qw), rt.dtype)
        from_partial = getattr(k, "attention_decode_from_partial", None)
        if pending is not None and ctx.max_q_len == 1 and from_partial is not None and fused[0] is not None:
            # every sequence brings one token: the attention kernel finishes the product itself
            if from_partial(pending, cache.keys, cache.values, att, table, ctx.q_start, ctx.ctx_len, nq, nkv, d,
                            cache.page_size, s.scale, s.window, ctx.max_ctx_len, q_norm_w, k_norm_w, fused[0],
                            fused[1], norm.eps if norm is not None else 0.0,
                            norm.weight_offset if norm is not None else 0.0, writes, ctx.seq_rows):
                return k.linear(att, self.o_proj, residual, residual=residual, defer=True)
        if fused is None:
            # An encoding the kernels do not know: normalise head by head in
            # place, let the encoding transform q and k, then only copy and append.
            if norm is not None:
                heads = nq + (nkv if writes else 0)
                for h in range(heads):
                    view = qkv[:, h * d:(h + 1) * d]
                    k.rmsnorm(view, self.q_norm if h < nq else self.k_norm, norm.eps,
                              norm.weight_offset, view)
            self.position.apply(qkv[:, :qw], qkv[:, qw:qw + kw] if writes else None, ctx)
            q_norm_w = k_norm_w = None
            fused = (None, 0)
        inv_freq, rotary_dim = fused
        (k.qk_norm_rope_append_partial if pending is not None else k.qk_norm_rope_append)(
            pending if pending is not None else qkv, q, cache.keys if writes else None,
            cache.values if writes else None,
            q_norm_w, k_norm_w, inv_freq, rotary_dim, norm.eps if norm is not None else 0.0,
            norm.weight_offset if norm is not None else 0.0,
            ctx.positions, ctx.seq_of_token, table if writes else None, nq, nkv, d, cache.page_size,
            ctx.seq_rows)
        return self._attend(residual, ctx, cache)

    def _attend(self, residual, ctx, cache):
        """Attention over the cache from the step's q, then the output product, left
        for the next norm to add into the residual."""
        s, rt = self.spec, self.runtime
        k = rt.kernels
        nq, nkv, d = s.num_heads, s.num_kv_heads, s.head_dim
        T = ctx.num_tokens
        q = ctx.workspace.get("attn.q", (T, nq * d), rt.dtype)
        att = ctx.workspace.get("attn.out", (T, nq * d), rt.dtype)
        k.attention(q, cache.keys, cache.values, att, ctx.tables[cache.group], ctx.q_start, ctx.ctx_len,
                    ctx.seq_of_token, ctx.positions, nq, nkv, d, cache.page_size, s.scale,
                    s.window, ctx.max_q_len, ctx.max_ctx_len, ctx.min_q_len, ctx.seq_rows)
        return k.linear(att, self.o_proj, residual, residual=residual, defer=True)

    def _heads_from_the_product(self, x, ctx, cache, fused) -> bool:
        """Many rows on kernels that can do it: the q | k | v product normalises and
        rotates its heads itself and writes q and the cache entries; no q | k | v
        array exists.  The rotation table and the tokens' cache slots are made once
        per step and shared by the layers."""
        s, rt = self.spec, self.runtime
        k = rt.kernels
        takes = getattr(k, "finishes_heads", None)
        T = ctx.num_tokens
        nq, nkv, d = s.num_heads, s.num_kv_heads, s.head_dim
        if takes is None or not takes(T, d, fused[1], rt.dtype):
            return False
        cos_sin = self.position.step_table(ctx)
        if cos_sin is None:
            return False
        writes = cache.writes
        slots = None
        if writes:
            key = ("cache slots", cache.group, nkv, d, cache.page_size)
            slots = ctx.shared.get(key)
            if slots is None:
                slots = ctx.workspace.get(f"attn.slots.{cache.group}", (T,), torch.int64)
                k.cache_slots(ctx.positions, ctx.seq_of_token, ctx.seq_rows, ctx.tables[cache.group], nkv,
                              cache.page_size, cache.keys.shape[0], d, slots)
                ctx.shared[key] = slots
        norm = s.qk_norm
        q = ctx.workspace.get("attn.q", (T, nq * d), rt.dtype)
        return k.linear_heads(x, self.qkv if writes else self.qkv[:nq * d], q, cache.keys if writes else None,
                              cache.values if writes else None, self.q_norm if norm is not None else None,
                              self.k_norm if norm is not None else None, cos_sin, slots, nq, nkv, d,
                              cache.page_size, norm.eps if norm is not None else 0.0,
                              norm.weight_offset if norm is not None else 0.0)


register_mixer("attention", PagedAttention, replace=True)
