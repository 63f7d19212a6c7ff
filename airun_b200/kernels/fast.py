"""Dispatch to the tensor-core kernels of the bfloat16 path.

Each ``*_bf16`` function returns True when a fast kernel took the call and False
when the sizes are outside what the fast kernels accept, in which case the
caller runs the plain kernel.  ``gemm_tcgen05`` is the raw entry.
"""
from __future__ import annotations

import os
from ctypes import c_int, c_longlong, c_void_p
from typing import Dict, Optional, Tuple

import torch

from . import ops
from .ops import _check, _cuda, _fn, _need, _p, _stream

EPI_F32, EPI_BF16, EPI_SWIGLU = 0, 1, 2
TARGET_CTAS = 296                      # two waves of 148 SMs

_SCRATCH: Dict[torch.device, Tuple[torch.Tensor, torch.Tensor]] = {}
SCRATCH_FLOATS = 16 << 20              # 64 MiB of partial tiles
SCRATCH_COUNTERS = 1 << 16

DISABLED = set(filter(None, os.environ.get("AIRUN_DISABLE_FAST", "").split(",")))


def all_libraries():
    return [("gemm_tcgen05", None)]


def scratch_for(device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Partial-tile buffer and tile counters shared by the split-K launches of one device.
    Launches on one stream run one after the other, so they can share it."""
    s = _SCRATCH.get(device)
    if s is None:
        s = (torch.empty(SCRATCH_FLOATS, dtype=torch.float32, device=device),
             torch.zeros(SCRATCH_COUNTERS, dtype=torch.int32, device=device))
        _SCRATCH[device] = s
    return s


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, swap: bool, bn: int,
                 ksplit: int, err: torch.Tensor, scratch: Optional[torch.Tensor] = None,
                 counters: Optional[torch.Tensor] = None) -> None:
    """out = x @ w^T on tcgen05 (see csrc/gemm_tcgen05.cu for the modes)."""
    _cuda(x, w, out, err, scratch, counters)
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "tcgen05 gemm takes bfloat16 operands")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "operands must be row-major")
    _need(K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
          and w.data_ptr() % 16 == 0, "tcgen05 gemm needs K and row strides in multiples of 8 and 16-byte aligned rows")
    if epi == EPI_SWIGLU:
        _need(N % 32 == 0 and tuple(out.shape) == (M, N // 2) and out.dtype == torch.bfloat16,
              "SwiGLU epilogue writes bfloat16 [M, N/2]")
    else:
        _need(tuple(out.shape) == (M, N), "output must be [M, N]")
        _need(out.dtype == (torch.float32 if epi == EPI_F32 else torch.bfloat16), "output type does not match the epilogue")
    if swap:
        _need(bn in (16, 32, 64, 128), "swapped mode takes bn in 16, 32, 64, 128")
    else:
        _need(bn in (128, 256), "normal mode takes bn 128 or 256")
    if ksplit > 1:
        if scratch is None:
            scratch, counters = scratch_for(x.device)
        f = _fn("gemm_tcgen05", "airun_gemm_tcgen05_scratch_floats", [c_int, c_int, c_int, c_int, c_int])
        f.restype = c_longlong
        need = f(M, N, 1 if swap else 0, bn, ksplit)
        a_rows, b_rows = (N, M) if swap else (M, N)
        tiles = ((a_rows + 127) // 128) * ((b_rows + bn - 1) // bn)
        _need(need <= scratch.numel() and tiles <= counters.numel(), "split-K scratch is too small for this launch")
    f = _fn("gemm_tcgen05", "airun_gemm_tcgen05",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
             c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(x), _p(w), _p(out), M, N, K, x.stride(0) if M > 1 else max(K, x.stride(0)),
             w.stride(0), out.stride(0) if M > 1 else max(out.shape[1], out.stride(0)),
             epi, 1 if swap else 0, bn, ksplit, _p(scratch), _p(counters), _p(err), _stream()), "gemm_tcgen05")


def plan_gemm(M: int, N: int, K: int) -> Tuple[bool, int, int]:
    """(swap, bn, ksplit) for a product of M tokens with an [N, K] weight."""
    if M <= 128:
        swap = True
        bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
        tiles = (N + 127) // 128
    else:
        swap, bn = False, (256 if N >= 256 else 128)
        tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
    kb = (K + 63) // 64
    ksplit = 1
    if tiles < TARGET_CTAS:
        ksplit = max(1, min(TARGET_CTAS // tiles, kb // 4))
    return swap, bn, ksplit


def _usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    K = x.shape[1]
    return ("gemm" not in DISABLED and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x.shape[0] > 0)


def linear_bf16(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    if not _usable(x, w) or out.dtype not in (torch.float32, torch.bfloat16):
        return False
    swap, bn, ksplit = plan_gemm(x.shape[0], w.shape[0], x.shape[1])
    gemm_tcgen05(x, w, out, EPI_F32 if out.dtype == torch.float32 else EPI_BF16, swap, bn, ksplit, ctx.err)
    return True


def linear_swiglu_bf16(ctx, x: torch.Tensor, w_gu: torch.Tensor, out: torch.Tensor, group: int) -> bool:
    if group != 16 or not _usable(x, w_gu) or w_gu.shape[0] % 32 != 0:
        return False
    swap, bn, ksplit = plan_gemm(x.shape[0], w_gu.shape[0], x.shape[1])
    gemm_tcgen05(x, w_gu, out, EPI_SWIGLU, swap, bn, ksplit, ctx.err)
    return True


def attention_bf16(ctx, q, out, cache, nh: int, nkv: int, hd: int, scale: float, window: int) -> bool:
    return False
