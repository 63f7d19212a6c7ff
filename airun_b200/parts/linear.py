"""Matrix products y = x W^T of the projections.

``linear`` picks the kernel by operand type and shape: float32 operands always
run on the CUDA cores with float32 accumulation (the true 32-bit path);
bfloat16 operands use the tensor-core kernels where one takes the sizes, and the
plain CUDA-core kernel otherwise.  Both accumulate in float32.
"""
from __future__ import annotations

import torch

from ..kernels import ops


def linear(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[T, N] = x[T, K] @ w[N, K]^T."""
    if x.dtype == torch.bfloat16:
        from ..kernels import fast
        if fast.linear_bf16(ctx, x, w, out):
            return out
    ops.gemm_simt(x, w, out)
    return out
