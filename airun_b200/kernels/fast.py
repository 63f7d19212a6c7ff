"""Dispatch to the tensor-core kernels of the bfloat16 path.

Each function returns True when a fast kernel took the call and False when the
sizes are outside what the fast kernels accept, in which case the caller runs
the plain kernel.
"""
from __future__ import annotations

import torch


def linear_bf16(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    return False


def linear_swiglu_bf16(ctx, x: torch.Tensor, w_gu: torch.Tensor, out: torch.Tensor, group: int) -> bool:
    return False


def attention_bf16(ctx, q, out, cache, nh: int, nkv: int, hd: int, scale: float, window: int) -> bool:
    return False
