"""Rotary position encoding with the NeoX pairing.

Pair i couples dimensions i and i + r/2 of a head; the angle is
pos * inv_freq[i] with inv_freq[i] = theta^(-2i/r); dimensions >= r are left
alone (crates/airun-cuda/kernels/ops.cu:158-184,
crates/airun-cuda/kernels/airun.cuh:147-163).  inv_freq is computed once in
double precision and rounded to float32; the position is multiplied in float32
on the device, where the accurate sincosf is used.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..kernels import ops
from .base import PositionEncoding, register_part


class RotaryNeox(PositionEncoding):
    kind = ops.ROPE_NEOX

    def __init__(self, prefix: str = "", rotary_dim: int = 0, theta: float = 10000.0,
                 dtype=None, device=None):
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim must be a positive even number, found {rotary_dim}")
        self.rotary_dim, self.theta = int(rotary_dim), float(theta)
        i = torch.arange(0, rotary_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / rotary_dim)
        self.inv_freq = inv.to(torch.float32).to(device)

    def fused(self) -> Optional[Tuple[int, int, Optional[torch.Tensor]]]:
        return self.kind, self.rotary_dim, self.inv_freq


class RotaryInterleaved(RotaryNeox):
    """The same angles with the older pairing of neighbouring dimensions (2i, 2i + 1), which the reference
    keeps as a kernel parameter beside the NeoX pairing (crates/airun-cuda/kernels/ops.cu:154-157, :176-179).
    The dense Qwen3 decoder does not use it."""
    kind = ops.ROPE_INTERLEAVED


class NoPosition(PositionEncoding):
    def __init__(self, prefix: str = "", dtype=None, device=None):
        pass

    def fused(self):
        return ops.ROPE_NONE, 0, None


register_part("position", "rotary_neox", RotaryNeox)
register_part("position", "rotary_interleaved", RotaryInterleaved)
register_part("position", "none", NoPosition)
