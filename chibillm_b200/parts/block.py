"""Block arrangements.  "prenorm": residual += mixer(norm(residual)), then
residual += feed_forward(norm(residual)); the residual itself is never
normalised in place (src/qwen/qwen_layer.cc:124-146)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import (Block, Runtime, TensorSpec, make_feed_forward, make_mixer, make_norm,
                   register_block)


class PreNormBlock(Block):
    def __init__(self, layer, runtime: Runtime):
        self.layer = layer
        self.runtime = runtime
        names = {role: layer.weight_prefix + name for role, name in layer.names().items()}
        self.mixer_norm = make_norm(layer.mixer_norm, names["mixer_norm"], runtime)
        self.feed_forward_norm = make_norm(layer.feed_forward_norm, names["feed_forward_norm"], runtime)
        self.mixer = make_mixer(layer.mixer, names, runtime)
        self.feed_forward = make_feed_forward(layer.feed_forward, names, runtime)
        self._parts = (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def expected_tensors(self) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for p in self._parts:
            out.extend(p.expected_tensors())
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.bind(tensors)

    def launch_key(self, ctx):
        a, b = self.mixer.launch_key(ctx), self.feed_forward.launch_key(ctx)
        return None if a is None or b is None else (a, b)

    def forward(self, residual: torch.Tensor, ctx, cache, pending=None):
        x = ctx.workspace.get("block.normed", tuple(residual.shape), self.runtime.dtype)
        normed = self.mixer_norm.forward_fused(residual, pending, x, self.mixer.accepts_scaled_rows)
        pending = self.mixer.forward(x if normed is None else normed, residual, ctx, cache)
        normed = self.feed_forward_norm.forward_fused(residual, pending, x, self.feed_forward.accepts_scaled_rows)
        return self.feed_forward.forward(x if normed is None else normed, residual, ctx)


register_block("prenorm", PreNormBlock, replace=True)
