"""Arrangement of a layer: norm -> mixer -> add -> norm -> feed-forward -> add.

The residual stream ``x`` is float32.  Each sub-layer returns a float32 delta;
the add is carried out by the NEXT norm (x += delta, then norm), as the
reference fuses every residual add with the norm that follows it
(crates/airun-core/src/runtime.rs:3564-3567, :3595-3599).  The block therefore
takes the delta still pending from the block before it and returns its own.

In the bfloat16 path, when the parts on both sides allow it (``fuses_norms``), a norm is not a
kernel of its own at all: the product that ends a sub-layer adds its result to x, writes
bfloat16(x * norm weight) and the sums of x^2 per token, and the product that starts the next
sub-layer scales each token's results by rsqrt(mean x^2 + eps) (parts/base.py NormedActivations).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import WeightSpec
from .base import FeedForward, Mixer, Norm, NormedActivations, Part, ResidualSink, register_part


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

    def device_driven(self) -> bool:
        """Do all parts of this block read the batch's layout from the device arrays only?"""
        return all(getattr(p, "device_driven", False) for p in self.parts())

    def graph_safe(self) -> bool:
        """May steps through this block be captured into CUDA graphs at all?"""
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def accepts_normed(self) -> bool:
        """Can this block start from NormedActivations (its first norm folded into the products)?"""
        return self.dtype == torch.bfloat16 and getattr(self.mixer, "fuses_norms", False) \
            and hasattr(self.norm1, "fusable")

    def forward(self, ctx, x: torch.Tensor, pending, cache, next_norm: Optional[Norm] = None):
        """``pending``: what the block before left: None, a float32 delta still to be added to x, or
        NormedActivations (x is up to date and this block's first norm is already folded in).
        ``next_norm``: the norm that will read x next, if it may be folded into this block's last
        product; the block then returns NormedActivations instead of a delta."""
        T, H = x.shape
        bf16 = self.dtype == torch.bfloat16
        if isinstance(pending, NormedActivations):
            h = pending
        else:
            h = ctx.ws.alloc((T, H), self.dtype)
            self.norm1.forward(ctx, x, h, delta=pending)
        if bf16 and getattr(self.mixer, "fuses_norms", False) and getattr(self.ffn, "fuses_norms", False) \
                and hasattr(self.norm2, "fusable"):
            a = self.mixer.forward(ctx, h, cache, sink=ResidualSink(x, *self.norm2.fusable()))
        else:
            a = self.mixer.forward(ctx, h, cache)
        if isinstance(a, NormedActivations):
            h2 = a
        else:
            h2 = ctx.ws.alloc((T, H), self.dtype)
            self.norm2.forward(ctx, x, h2, delta=a)
        if bf16 and next_norm is not None and getattr(self.ffn, "fuses_norms", False):
            return self.ffn.forward(ctx, h2, sink=ResidualSink(x, *next_norm.fusable()))
        return self.ffn.forward(ctx, h2)


register_part("arrangement", "pre_norm", PreNormBlock)
