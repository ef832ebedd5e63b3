"""RMSNorm as a part: y = (x * rsqrt(mean(x^2) + eps)) * (w + offset), statistics
in 32-bit (src/metal/kernels/tensor_ops.metal:76-105)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import Norm, Runtime, TensorSpec, register_norm


class RMSNorm(Norm):
    def __init__(self, spec, weight_name: str, runtime: Runtime):
        self.spec = spec
        self.weight_name = weight_name
        self.runtime = runtime
        self.weight: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.spec.size,))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """x, out: [rows, k * size]; every run of ``size`` features is one group."""
        n = self.spec.size
        if x.shape[-1] == n:
            self.runtime.kernels.rmsnorm(x, self.weight, self.spec.eps, self.spec.weight_offset, out)
        else:
            if not x.is_contiguous() or not out.is_contiguous():
                raise ValueError("grouped norm needs contiguous rows")
            self.runtime.kernels.rmsnorm(x.view(-1, n), self.weight, self.spec.eps,
                                         self.spec.weight_offset, out.view(-1, n))


    def forward_fused(self, residual: torch.Tensor, pending, out: torch.Tensor, scaled_ok: bool = False):
        k = self.runtime.kernels
        if pending is not None and residual.shape[-1] == self.spec.size:
            if hasattr(pending, "finish_with_norm"):
                # a product of many rows that has not run yet: it writes the norm's output itself
                return pending.finish_with_norm(residual, self.weight, self.spec.eps, self.spec.weight_offset,
                                                out, scaled_ok)
            fused = getattr(k, "reduce_residual_rmsnorm", None)
            if fused is not None and hasattr(pending, "partial"):
                fused(pending, residual, self.weight, self.spec.eps, self.spec.weight_offset, out)
                return out
        return super().forward_fused(residual, pending, out, scaled_ok)


register_norm("rmsnorm", RMSNorm, replace=True)
