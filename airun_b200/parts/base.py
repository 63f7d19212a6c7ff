"""Interfaces of the parts a model is put together from, and their registries.

A layer is an arrangement (``Block``) of a mixer, a feed-forward and norms; the
mixer may use a position encoding.  Each part takes its sizes and constants as
constructor parameters, declares the weight tensors it needs by name, and, if it
keeps something between tokens, declares that as a cache spec.  No part knows
which model it belongs to.  The reference switches mixer and feed-forward per
layer through two enums around shared norm/residual code
(crates/airun-core/src/model.rs:446-464, crates/airun-core/src/runtime.rs:3537-3589);
here the choice is a name looked up in a registry, so that a new part needs no
change to existing files.

Interfaces
----------
Part            weight_specs() -> [WeightSpec];  load_weights(tensors: dict) -> None
Norm            forward(ctx, x, out, delta=None, rows=None)
                  out = norm(x [+ delta]); with delta and no rows, x += delta in place
PositionEncoding fused() -> (kind, rotary_dim, inv_freq) the attention prologue
                  kernel understands (none, NeoX pairing, interleaved pairing);
                rotation_positions(ctx) -> int32 [T] or None (None: the cache positions)
Embedding       forward(ctx, token_ids, out float32 [T, hidden]); .table for a tied head
Head            forward(ctx, h [rows, hidden], out float32 [rows, vocab])
Mixer           cache_spec() -> PagedKVSpec | StateSpec | None
                forward(ctx, h, cache) -> float32 [T, hidden] (the residual delta)
FeedForward     forward(ctx, h) -> float32 [T, hidden]
                Optional, for both: ``fuses_norms = True`` says that forward also takes
                ``sink=ResidualSink`` (then it adds its result to the residual itself and returns
                NormedActivations for the next sub-layer, or ignores the sink and returns a delta)
                and accepts NormedActivations as ``h``.
                Optional, for every part: ``device_driven = True`` promises that forward launches the
                same kernels with the same arguments for every batch of ctx.num_tokens rows, i.e. that
                it reads which rows belong to which request, their positions and lengths from the
                device arrays of ctx only (never from ctx.query_lens and the other host lists), and
                that rows of request -1 are padding it skips.  Steps of a model whose parts all promise
                this are replayed from CUDA graphs, prompt portions included.
                ``graph_safe = False`` on a part says the opposite of the least a graph needs: its
                forward reads values back to the host and launches accordingly (a routed feed-forward
                that loops over the experts that got tokens, say); a model with such a part runs
                every step kernel by kernel.
Block           forward(ctx, x, delta, cache) -> delta of the block's last sub-layer,
                  still to be added to x by whoever norms x next
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..weights.loader import WeightSpec


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every (or the last ``window``) token(s), in pages."""
    num_kv_heads: int
    head_dim: int
    window: int = 0          # 0: all tokens are kept


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, zero when a request starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class NormedActivations:
    """The input of a sub-layer whose RMSNorm has been folded into the products around it:
    ``h`` = bfloat16(x * norm weight) without the 1/rms factor, and the sums of x^2 per token in
    ``ssq`` [parts, T]; the product that reads ``h`` multiplies each token's results by
    rsqrt(sum of parts / size + eps), which is the same as norming first."""
    h: torch.Tensor
    ssq: torch.Tensor
    eps: float
    size: int


@dataclass
class ResidualSink:
    """Handed to the last product of a sub-layer that may fold the residual add and the norm that
    follows: the residual stream ``x`` and that norm's weight and eps."""
    x: torch.Tensor
    norm_weight: torch.Tensor
    eps: float


class Part:
    """Something with weights.  ``prefix`` is its tensor-name prefix in the model file."""

    prefix: str = ""

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor,
                delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    def fused(self) -> Optional[Tuple[int, int, Optional[torch.Tensor]]]:
        """(kind, rotary_dim, inv_freq) for the q/k prologue kernel: kind is ops.ROPE_NONE, ops.ROPE_NEOX
        (pair i couples dims i and i + r/2) or ops.ROPE_INTERLEAVED (dims 2i and 2i + 1)."""
        return None

    def rotation_positions(self, ctx) -> Optional[torch.Tensor]:
        """int32 [T] on the device: the position every row of the step is rotated by, when that is not
        its place in the cache (positions that restart after an inserted block, say); None: the cache
        positions ``ctx.positions``.  To stay replayable from a CUDA graph the tensor must be made from
        device arrays of ``ctx`` by kernels, at the same address for every step of a shape."""
        return None


class Embedding(Part):
    """forward(ctx, token_ids int32 [T], out float32 [T, hidden]); ``table`` is the [vocab, hidden]
    matrix a tied head may use."""
    table: Optional[torch.Tensor] = None

    def forward(self, ctx, token_ids: torch.Tensor, out: torch.Tensor) -> None:
        raise NotImplementedError


class Head(Part):
    """forward(ctx, h [rows, hidden] in the compute type, out float32 [rows, vocab])."""

    def forward(self, ctx, h: torch.Tensor, out: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward(self, ctx, h: torch.Tensor, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "arrangement": {}, "embedding": {}, "head": {}}


def register_part(kind: str, name: str, factory: Callable) -> None:
    """Registers ``factory(prefix=..., dtype=..., device=..., **args)`` under ``name``."""
    if kind not in _REGISTRIES:
        raise KeyError(f"unknown kind of part {kind!r}; kinds: {sorted(_REGISTRIES)}")
    _REGISTRIES[kind][name] = factory


def make_part(kind: str, name: str, **kwargs):
    reg = _REGISTRIES[kind]
    if name not in reg:
        raise KeyError(f"no {kind} named {name!r} is registered; registered: {sorted(reg)}")
    return reg[name](**kwargs)


def registered_parts(kind: str) -> List[str]:
    return sorted(_REGISTRIES[kind])
