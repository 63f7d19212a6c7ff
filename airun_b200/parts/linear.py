"""Matrix products y = x W^T of the projections.

``linear`` picks the kernel by operand type and shape: float32 operands always
run on the CUDA cores with float32 accumulation (the true 32-bit path);
bfloat16 operands use the tensor-core kernels where one takes the sizes, and the
plain CUDA-core kernel otherwise.  Both accumulate in float32.  Every projection is
y = W x over row-major rows of length K, without a bias, as in the reference
(crates/airun-cuda/src/ops.rs:290-293; crates/airun-core/src/model.rs:906-912).
"""
from __future__ import annotations

import torch

from ..kernels import ops


def linear(ctx, x, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[T, N] = x[T, K] @ w[N, K]^T.  ``x`` may be NormedActivations (see parts/base.py)."""
    from .base import NormedActivations
    if isinstance(x, NormedActivations):
        from ..kernels import fast
        if not fast.linear_bf16(ctx, x.h, w, out, normed=x):
            raise RuntimeError("a folded norm reached a product the tensor-core kernel does not take")
        return out
    if x.dtype == torch.bfloat16:
        from ..kernels import fast
        if fast.linear_bf16(ctx, x, w, out):
            return out
    ops.gemm_simt(x, w, out)
    return out


def linear_into_residual(ctx, x: torch.Tensor, w: torch.Tensor, sink):
    """The last product of a sub-layer with the residual add and the next norm folded in:
    sink.x += x @ w^T, and the un-normalised input of the next sub-layer is returned as
    NormedActivations.  Returns None when the tensor-core kernel does not take the sizes (the
    caller then returns a plain delta)."""
    from .base import NormedActivations
    from ..kernels import fast
    if sink is None or x.dtype != torch.bfloat16 or not fast.fusion_usable(x, w):
        return None
    T, N = x.shape[0], w.shape[0]
    h = ctx.ws.alloc((T, N), torch.bfloat16)
    ssq = ctx.ws.alloc((fast.max_resid_parts(N), T), torch.float32)
    parts = fast.linear_resid_norm_bf16(ctx, x, w, sink.x[:T], sink.norm_weight, h, ssq)
    return NormedActivations(h, ssq[:parts], sink.eps, N)
