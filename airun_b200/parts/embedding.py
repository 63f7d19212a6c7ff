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
from .base import Embedding, Head, register_part
from .linear import linear


class TokenEmbedding(Embedding):
    """``scale``: every embedded row is multiplied by it (None or 1: no scaling, as the dense Qwen3
    decoder and the reference, crates/airun-cuda/kernels/ops.cu:241-252)."""

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, scale: Optional[float] = None,
                 dtype=None, device=None):
        """``prefix``: the full name of the table's tensor."""
        self.name, self.V, self.H = prefix, int(vocab_size), int(hidden_size)
        self.scale = 1.0 if scale is None else float(scale)
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.V, self.H))]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.name]

    def forward(self, ctx, token_ids: torch.Tensor, out: torch.Tensor) -> None:
        ops.embed(self.table, token_ids, out, ctx.err, self.scale)


class LMHead(Head):
    """logits = W h; ``tied_to``: an embedding part whose table is W.  ``soft_cap``: logits become
    cap * tanh(logits / cap) (None: no cap, as the dense Qwen3 decoder and the reference,
    crates/airun-core/src/runtime.rs:2632-2651)."""

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, tied_to: Optional[Embedding] = None,
                 soft_cap: Optional[float] = None, dtype=None, device=None):
        """``prefix``: the full name of the head's tensor (unused when tied)."""
        self.name, self.V, self.H, self.tied_to = prefix, int(vocab_size), int(hidden_size), tied_to
        self.soft_cap = None if soft_cap is None else float(soft_cap)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [] if self.tied_to is not None else [WeightSpec(self.name, (self.V, self.H))]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = self.tied_to.table if self.tied_to is not None else tensors[self.name]

    def forward(self, ctx, h: torch.Tensor, out: torch.Tensor) -> None:
        linear(ctx, h, self.weight, out)
        if self.soft_cap is not None:
            ops.soft_cap(out, self.soft_cap)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
