"""Dense gated feed-forward (SwiGLU): residual += down(silu(gate(x)) * up(x))
(src/tensor/functions.cc:220-253).  gate and up are stacked into one matrix so
one product yields both (src/qwen/qwen_weights.cc:13-16)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FeedForward, Runtime, TensorSpec, register_feed_forward


class GatedMLP(FeedForward):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        if spec.activation != "silu":
            raise ValueError(f"activation '{spec.activation}' is not supported by gated_mlp")
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.gate_up: torch.Tensor = None
        self.gate_up_interleaved: torch.Tensor = None
        self.down: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        s = self.spec
        return [TensorSpec(self.names["gate_proj"], (s.intermediate_size, s.hidden_size)),
                TensorSpec(self.names["up_proj"], (s.intermediate_size, s.hidden_size)),
                TensorSpec(self.names["down_proj"], (s.hidden_size, s.intermediate_size))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        gate, up = tensors[self.names["gate_proj"]], tensors[self.names["up_proj"]]
        if gate.dtype != up.dtype:
            up = up.to(gate.dtype)
        interleave = getattr(self.runtime.kernels, "interleave_gate_up", None)
        self.gate_up_interleaved = interleave(gate, up) if interleave is not None else None
        # one of the two layouts is kept: blocks of 64 gate rows and their 64 up rows for the kernel
        # that applies SwiGLU itself, else gate rows followed by up rows
        self.gate_up = None if self.gate_up_interleaved is not None else torch.cat([gate, up], dim=0).contiguous()
        self.down = tensors[self.names["down_proj"]].contiguous()

    accepts_scaled_rows = True       # x goes to the gate | up product and nowhere else

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        k = self.runtime.kernels
        T = x.shape[0]
        inter = self.spec.intermediate_size
        act = ctx.workspace.get("mlp.act", (T, inter), self.runtime.dtype)
        if self.gate_up_interleaved is not None:
            if not k.linear_swiglu(x, self.gate_up_interleaved, act):
                raise RuntimeError("gated_mlp: the fused kernel refused a shape it was prepared for")
            return k.linear(act, self.down, residual, residual=residual, defer=True)
        split = getattr(k, "linear_partial", None)
        pending = split(x, self.gate_up) if split is not None else None
        if pending is not None:
            k.reduce_swiglu(pending, act)            # adds the partial sums and applies SwiGLU
        else:
            gate_up = ctx.workspace.get("mlp.gate_up", (T, 2 * inter), self.runtime.dtype)
            k.linear(x, self.gate_up, gate_up)
            k.swiglu(gate_up, act)
        return k.linear(act, self.down, residual, residual=residual, defer=True)


register_feed_forward("gated_mlp", GatedMLP, replace=True)
