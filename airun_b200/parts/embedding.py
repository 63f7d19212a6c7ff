"""Token embedding and the output head.

x[t] = E[token[t]] without scaling (crates/airun-cuda/kernels/ops.cu:227-252);
logits = W_out h for the wanted rows only, and with tied embeddings W_out is the
embedding table itself, not a copy (crates/airun-core/src/model.rs:781-796,
:1068-1074).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Part
from .linear import linear


class TokenEmbedding(Part):
    def __init__(self, name: str, vocab_size: int, hidden_size: int):
        self.name, self.V, self.H = name, int(vocab_size), int(hidden_size)
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.V, self.H))]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.name]

    def forward(self, ctx, token_ids: torch.Tensor, out: torch.Tensor) -> None:
        ops.embed(self.table, token_ids, out, ctx.err)


class LMHead(Part):
    def __init__(self, name: str, vocab_size: int, hidden_size: int, tied_to: Optional[TokenEmbedding]):
        self.name, self.V, self.H, self.tied_to = name, int(vocab_size), int(hidden_size), tied_to
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [] if self.tied_to is not None else [WeightSpec(self.name, (self.V, self.H))]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = self.tied_to.table if self.tied_to is not None else tensors[self.name]

    def forward(self, ctx, h: torch.Tensor, out: torch.Tensor) -> None:
        linear(ctx, h, self.weight, out)
