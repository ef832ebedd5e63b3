"""Position encodings as parts.

"rope": split-half rotation of the first ``rotary_dim`` features of each head,
``inv_freq[j] = theta ** (-2j / rotary_dim)`` computed once in 32-bit on the
host, angle = float(position) * inv_freq[j] in 32-bit
(src/metal/metal_kernels.mm:186-191, src/metal/kernels/tensor_ops.metal:168-197).
The attention kernels apply it themselves from the table (``fused_rotation``).

"none": no position information inside the mixer.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding, Runtime, register_position


def rotary_inverse_frequencies(theta: float, rotary_dim: int) -> torch.Tensor:
    """The table shared by every user of one (theta, rotary_dim): float32 pow of
    float32 arguments, exponent -2j / rotary_dim."""
    j = torch.arange(rotary_dim // 2, dtype=torch.float32)
    exponent = (-2.0 * j) / float(rotary_dim)
    return torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, runtime: Runtime):
        if spec.rotary_dim % 2 != 0 or spec.rotary_dim > spec.head_dim or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and within head_dim {spec.head_dim}")
        self.spec = spec
        self.runtime = runtime
        self.inv_freq = rotary_inverse_frequencies(spec.theta, spec.rotary_dim).to(runtime.device)

    def fused_rotation(self):
        return self.inv_freq, self.spec.rotary_dim

    def step_table(self, ctx):
        table_of = getattr(self.runtime.kernels, "rope_table", None)
        if table_of is None:
            return None
        key = ("rope", float(self.spec.theta), int(self.spec.rotary_dim))
        table = ctx.shared.get(key)
        if table is None:
            table = ctx.workspace.get(f"rope.table.{key[1]}.{key[2]}", (ctx.num_tokens, self.spec.rotary_dim),
                                      torch.float32)
            table_of(ctx.positions, self.inv_freq, self.spec.rotary_dim, table)
            ctx.shared[key] = table
        return table


class NoPosition(PositionEncoding):
    def __init__(self, spec, runtime: Runtime):
        self.spec = spec

    def fused_rotation(self):
        return None, 0

    def apply(self, q, k, ctx) -> None:
        return None


register_position("rope", RotaryEncoding, replace=True)
register_position("none", NoPosition, replace=True)
