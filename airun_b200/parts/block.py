"""Arrangement of a layer: norm -> mixer -> add -> norm -> feed-forward -> add.

The residual stream ``x`` is float32.  Each sub-layer returns a float32 delta;
the add is carried out by the NEXT norm (x += delta, then norm), as the
reference fuses every residual add with the norm that follows it
(crates/airun-core/src/runtime.rs:3564-3567, :3595-3599).  The block therefore
takes the delta still pending from the block before it and returns its own.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import WeightSpec
from .base import FeedForward, Mixer, Norm, Part, register_part


class PreNormBlock(Part):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward, dtype: torch.dtype):
        self.norm1, self.mixer, self.norm2, self.ffn, self.dtype = norm1, mixer, norm2, ffn, dtype

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.ffn)

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self.parts() for s in p.weight_specs()]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load_weights(tensors)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, x: torch.Tensor, delta: Optional[torch.Tensor], cache) -> torch.Tensor:
        T, H = x.shape
        h = ctx.ws.alloc((T, H), self.dtype)
        self.norm1.forward(ctx, x, h, delta=delta)
        a = self.mixer.forward(ctx, h, cache)
        h2 = ctx.ws.alloc((T, H), self.dtype)
        self.norm2.forward(ctx, x, h2, delta=a)
        return self.ffn.forward(ctx, h2)


register_part("arrangement", "pre_norm", PreNormBlock)
