"""RMSNorm with the residual add fused in.

out = x * rsqrt(mean(x^2) + eps) * weight, eps inside the root, the weight used
as it is (crates/airun-cuda/kernels/ops.cu:12-41); with ``delta`` the sum
x + delta is formed first and, unless only some rows are wanted, stored back as
the new residual (ops.cu:47-78).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    device_driven = True

    def __init__(self, prefix: str, size: int, eps: float, dtype=None, device=None,
                 weight_name: str = "weight"):
        self.prefix, self.size, self.eps = prefix, int(size), float(eps)
        self.name = f"{prefix}.{weight_name}" if prefix else weight_name
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.size,), storage="float32", init="norm")]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]

    def forward(self, ctx, x, out, delta=None, rows=None) -> None:
        ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows)

    def fusable(self):
        """(weight, eps) for products that fold this norm in (out = x * rsqrt(mean x^2 + eps) * weight)."""
        return self.weight, self.eps


register_part("norm", "rmsnorm", RMSNorm)
