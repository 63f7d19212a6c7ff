"""SwiGLU feed-forward: down( silu(gate(h)) * up(h) ).

g = Wg h, u = Wu h, a = g / (1 + exp(-g)) * u, out = Wd a
(crates/airun-core/src/runtime.rs:688-747, crates/airun-cuda/kernels/ops.cu:191-200).
Gate and up run as one product over a matrix whose rows alternate between
blocks of ``group`` gate rows and ``group`` up rows, so a kernel that holds a
tile of the result has both factors of each output at hand.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import FeedForward, NormedActivations, register_part
from .linear import linear, linear_into_residual

INTERLEAVE = 16


class SwiGLU(FeedForward):
    device_driven = True

    fuses_norms = True        # takes NormedActivations as input and a ResidualSink for its output

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, names: Optional[Dict[str, str]] = None):
        self.prefix, self.H, self.I = prefix, int(hidden_size), int(intermediate_size)
        self.dtype, self.device = dtype, device
        self.group = INTERLEAVE if self.I % INTERLEAVE == 0 else self.I
        n = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_gu = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        nm = self.names
        return [WeightSpec(nm["gate"], (self.I, self.H)), WeightSpec(nm["up"], (self.I, self.H)),
                WeightSpec(nm["down"], (self.H, self.I))]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm, g = self.names, self.group
        gate, up = tensors.pop(nm["gate"]), tensors.pop(nm["up"])
        nb = self.I // g
        self.w_gu = torch.stack([gate.view(nb, g, self.H), up.view(nb, g, self.H)], dim=1) \
            .reshape(2 * self.I, self.H).contiguous()
        self.w_down = tensors.pop(nm["down"])

    def forward(self, ctx, h, sink=None):
        normed = h if isinstance(h, NormedActivations) else None
        hx = normed.h if normed is not None else h
        T, ws = hx.shape[0], ctx.ws
        act = ws.alloc((T, self.I), self.dtype)
        done = False
        if hx.dtype == torch.bfloat16:
            from ..kernels import fast
            done = fast.linear_swiglu_bf16(ctx, hx, self.w_gu, act, self.group, normed=normed)
        if not done:
            gu = ws.alloc((T, 2 * self.I), torch.float32)
            linear(ctx, h, self.w_gu, gu)
            ops.swiglu(gu, act, self.group)
        fused = linear_into_residual(ctx, act, self.w_down, sink)
        if fused is not None:
            return fused
        delta = ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_down, delta)
        return delta


register_part("feed_forward", "swiglu", SwiGLU)
