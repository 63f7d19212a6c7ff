"""Dispatch to the tensor-core kernels of the bfloat16 path.

Each ``*_bf16`` function returns True when a fast kernel took the call and False
when the sizes are outside what the fast kernels accept, in which case the
caller runs the plain kernel.  ``gemm_tcgen05`` is the raw entry.

The reference chooses between its kernels the same way, by operand type and row
count, in one place (``matvec``, crates/airun-core/src/runtime.rs:5531-5625: the
half-precision matvec for a few rows, the wmma product for many; its attention
runs the flash kernel from 16 tokens on and the plain or split kernels below,
crates/airun-cuda/kernels/ops.cu:2130-2142, crates/airun-cuda/src/ops.rs:1207-1318).
"""
from __future__ import annotations

import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, Optional, Tuple

import torch

from . import ops
from .ops import _check, _cuda, _fn, _need, _p, _stream

EPI_F32, EPI_BF16, EPI_SWIGLU, EPI_RESID = 0, 1, 2, 3
B200_SMS = 148                         # the SM count the plans are sized for when no GPU can be asked


class Machine:
    """How many CTAs of each kernel the GPU holds at once: the SM count read from the device, times the
    CTAs of that kernel one SM holds (fixed by the kernels' shared memory and registers)."""

    def __init__(self, sms: int):
        self.sms = int(sms)
        self.stream_ctas = 2 * self.sms                   # streaming product: two CTAs per SM
        # CTAs a split product may use: its clusters (of up to 8) must all be resident together, so a
        # margin is left below the 2-per-SM slots: the multiples of 32 that fit in nine tenths of them
        self.split_ctas = max(32, (2 * self.sms * 9 // 10) // 32 * 32)
        self.decode_slots = 3 * self.sms                  # cp.async decode attention: three CTAs per SM
        self.decode_slots_tma = 2 * self.sms              # its TMA variant keeps three stages per warp: two per SM
        self.wide_min_ctas = self.sms * 128 // B200_SMS   # fewest CTAs the two-tile prefill attention is used for


_MACHINES: Dict[object, Machine] = {}


def machine(device=None) -> Machine:
    """The Machine of ``device`` (default: the current CUDA device; without a GPU, a B200's numbers)."""
    if not torch.cuda.is_available():
        return _MACHINES.setdefault(None, Machine(B200_SMS))
    idx = torch.device(device).index if device is not None and torch.device(device).index is not None \
        else torch.cuda.current_device()
    m = _MACHINES.get(idx)
    if m is None:
        m = _MACHINES[idx] = Machine(torch.cuda.get_device_properties(idx).multi_processor_count)
    return m


STREAM_CTAS = Machine(B200_SMS).stream_ctas    # the B200's figures, for callers that plan without a device
SPLIT_CTAS = Machine(B200_SMS).split_ctas

_SCRATCH: Dict[torch.device, Tuple[torch.Tensor, torch.Tensor]] = {}
SCRATCH_FLOATS = 16 << 20              # 64 MiB of partial tiles
SCRATCH_COUNTERS = 1 << 16

DISABLED = set(filter(None, os.environ.get("AIRUN_DISABLE_FAST", "").split(",")))


def all_libraries():
    return [("gemm_tcgen05", None), ("gemm_tcgen05", {"AIRUN_FOLD_NORM": 1}), ("attention_plan", None), ("attention_mma", {"HD": 128}), ("attention_mma", {"HD": 64}),
            ("attention_tcgen05", {"HD": 128}), ("attention_tcgen05", {"HD": 64})]


def scratch_for(device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Partial-tile buffer and tile counters shared by the split-K launches of one device.
    Launches on one stream run one after the other, so they can share it."""
    s = _SCRATCH.get(device)
    if s is None:
        s = (torch.empty(SCRATCH_FLOATS, dtype=torch.float32, device=device),
             torch.zeros(SCRATCH_COUNTERS, dtype=torch.int32, device=device))
        _SCRATCH[device] = s
    return s


def resid_parts(N: int, swap: bool, bn: int) -> int:
    """Parts the residual + norm epilogue writes the sums of squares in."""
    return (N + 127) // 128 if swap else (N + bn - 1) // bn


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, swap: bool, bn: int,
                 ksplit: int, err: torch.Tensor, scratch: Optional[torch.Tensor] = None,
                 counters: Optional[torch.Tensor] = None, ssq_in: Optional[torch.Tensor] = None,
                 eps_in: float = 0.0, norm_size: int = 0, resid: Optional[torch.Tensor] = None,
                 norm_w: Optional[torch.Tensor] = None, ssq_out: Optional[torch.Tensor] = None) -> None:
    """out = x @ w^T on tcgen05 (see csrc/gemm_tcgen05.cu for the modes).

    ``ssq_in`` [parts, M] float32: x is bfloat16(residual * norm weight) and each token's results are
    scaled by rsqrt(sum of its parts / norm_size + eps_in).  ``epi == EPI_RESID``: ``resid`` [M, N]
    float32 += result, out = bfloat16(resid * norm_w), ssq_out [resid_parts, M] = sums of resid^2."""
    _cuda(x, w, out, err, scratch, counters, ssq_in, resid, norm_w, ssq_out)
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "tcgen05 gemm takes bfloat16 operands")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "operands must be row-major")
    _need(K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
          and w.data_ptr() % 16 == 0, "tcgen05 gemm needs K and row strides in multiples of 8 and 16-byte aligned rows")
    if epi == EPI_SWIGLU:
        _need(N % 32 == 0 and tuple(out.shape) == (M, N // 2) and out.dtype == torch.bfloat16,
              "SwiGLU epilogue writes bfloat16 [M, N/2]")
    elif epi == EPI_RESID:
        _need(tuple(out.shape) == (M, N) and out.dtype == torch.bfloat16, "residual epilogue writes bfloat16 [M, N]")
        _need(resid is not None and resid.dtype == torch.float32 and tuple(resid.shape) == (M, N) and resid.stride(1) == 1,
              "resid must be float32 [M, N]")
        _need(norm_w is not None and norm_w.dtype == torch.float32 and tuple(norm_w.shape) == (N,), "norm_w must be float32 [N]")
        _need(ssq_out is not None and ssq_out.dtype == torch.float32 and ssq_out.dim() == 2 and ssq_out.is_contiguous()
              and ssq_out.shape[0] >= resid_parts(N, swap, bn) and ssq_out.shape[1] >= M, "ssq_out must be float32 [parts, M]")
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
    if ssq_in is not None:
        _need(ssq_in.dtype == torch.float32 and ssq_in.dim() == 2 and ssq_in.is_contiguous() and ssq_in.shape[1] >= M
              and norm_size > 0, "ssq_in must be float32 [parts, M]")
    # the build with the folded norm only where it is asked for; the plain one is leaner
    fold = {"AIRUN_FOLD_NORM": 1} if (ssq_in is not None or epi == EPI_RESID) else None
    f = _fn("gemm_tcgen05", "airun_gemm_tcgen05_ex",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
             c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_float, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int], fold)
    _check(f(_p(x), _p(w), _p(out), M, N, K, x.stride(0) if M > 1 else max(K, x.stride(0)),
             w.stride(0), out.stride(0) if M > 1 else max(out.shape[1], out.stride(0)),
             epi, 1 if swap else 0, bn, ksplit, _p(scratch), _p(counters), _p(err), _stream(),
             _p(ssq_in), ssq_in.shape[0] if ssq_in is not None else 0, ssq_in.shape[1] if ssq_in is not None else 0,
             float(eps_in), int(norm_size), _p(resid), resid.stride(0) if resid is not None and M > 1 else N,
             _p(norm_w), _p(ssq_out), ssq_out.shape[1] if ssq_out is not None else 0), "gemm_tcgen05")


def plan_gemm(M: int, N: int, K: int, mach: Optional[Machine] = None) -> Tuple[bool, int, int]:
    """(swap, bn, ksplit) for a product of M tokens with an [N, K] weight.

    Up to 128 tokens the weights are the 128-row operand (swap), except for the widest products from 65 tokens on.  Up to 16 tokens the K range is cut
    until about STREAM_CTAS CTAs stream the weights (a slice keeping 10 K-steps) and the slices add
    up through a scratch in memory.  From 17 tokens on, where the partial tiles are larger, it is cut
    into up to 8 slices that run as one thread-block cluster and add up through distributed shared
    memory: as many as keep the CTAs within SPLIT_CTAS (all clusters must be resident at once; 288
    CTAs in clusters of 6 were not and took half as long again) and a slice at 8 K-steps or more.  Above
    128 tokens, tiles of 128 x 256 on the persistent kernel once there are 96 of them; fewer tiles
    leave SMs idle, so the tile narrows to 128 x 128, and only if that still fills less than one
    wave and a slice keeps 32 K-steps is K cut as well.  Both rules come from sweeps over the
    Qwen3-1.7B and -8B shapes, 1 to 2048 tokens, timed inside CUDA graphs."""
    mach = mach or machine()
    kb = (K + 63) // 64
    if 64 < M <= 128 and N >= 256 and (N + 255) // 256 >= mach.sms * 96 // B200_SMS:
        # Above 64 tokens a swapped CTA reads as many activation bytes from the L2 cache as weight bytes, and the
        # two together, not the weights alone, meet the limit of what the SMs take in (about 7 TB/s here): tiles
        # of 128 tokens x 256 weight rows read half the activations per weight byte (gate/up at 128 tokens: 46
        # against 55 us; at 64 tokens the two orientations take the same time)
        return False, 256, 1
    if M <= 128:
        bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
        tiles = (N + 127) // 128
        if M <= 16:
            return True, bn, max(1, min(mach.stream_ctas // tiles, kb // 10))
        return True, bn, max(1, min(mach.split_ctas // tiles, kb // 8, 8))
    mt = (M + 127) // 128
    if N >= 256 and mt * ((N + 255) // 256) >= mach.sms * 96 // B200_SMS:
        return False, 256, 1
    tiles = mt * ((N + 127) // 128)
    return False, 128, max(1, min(mach.sms // tiles, kb // 32))


def _usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    K = x.shape[1]
    return ("gemm" not in DISABLED and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x.shape[0] > 0)


def _normed_args(normed) -> dict:
    return {} if normed is None else dict(ssq_in=normed.ssq, eps_in=normed.eps, norm_size=normed.size)


def linear_bf16(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, normed=None) -> bool:
    """``normed``: x is the un-normalised activation of a NormedActivations; its token scales are
    applied in the epilogue."""
    if not _usable(x, w) or out.dtype not in (torch.float32, torch.bfloat16):
        return False
    swap, bn, ksplit = plan_gemm(x.shape[0], w.shape[0], x.shape[1])
    gemm_tcgen05(x, w, out, EPI_F32 if out.dtype == torch.float32 else EPI_BF16, swap, bn, ksplit, ctx.err,
                 **_normed_args(normed))
    return True


def linear_swiglu_bf16(ctx, x: torch.Tensor, w_gu: torch.Tensor, out: torch.Tensor, group: int, normed=None) -> bool:
    if group != 16 or not _usable(x, w_gu) or w_gu.shape[0] % 32 != 0:
        return False
    swap, bn, ksplit = plan_gemm(x.shape[0], w_gu.shape[0], x.shape[1])
    gemm_tcgen05(x, w_gu, out, EPI_SWIGLU, swap, bn, ksplit, ctx.err, **_normed_args(normed))
    return True


# Folding the residual add and the RMSNorm into the products around them (EPI_RESID + token scales)
# removes two launches per layer, but as measured on the Qwen3-8B shape the heavier epilogues cost
# what the launches saved (decode) or more (prompt portions, whose epilogue accesses are strided),
# so it is off unless AIRUN_NORM_FUSION=1; tests exercise it either way.
NORM_FUSION = os.environ.get("AIRUN_NORM_FUSION", "") not in ("", "0")


def fusion_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Can the product x @ w^T end a sub-layer with the residual add and the next norm folded in?"""
    return NORM_FUSION and _usable(x, w) and w.shape[0] % 8 == 0


def linear_resid_norm_bf16(ctx, x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, norm_w: torch.Tensor,
                           h_out: torch.Tensor, ssq_out: torch.Tensor) -> int:
    """resid += x @ w^T; h_out = bfloat16(resid * norm_w); ssq_out[:parts] = sums of resid^2 per token.
    Returns the number of parts written."""
    M, K = x.shape
    N = w.shape[0]
    swap, bn, ksplit = plan_gemm(M, N, K)
    gemm_tcgen05(x, w, h_out, EPI_RESID, swap, bn, ksplit, ctx.err, resid=resid, norm_w=norm_w, ssq_out=ssq_out)
    return resid_parts(N, swap, bn)


def max_resid_parts(N: int) -> int:
    return (N + 127) // 128


# ---------------------------------------------------------------- attention
_ARANGE: Dict[torch.device, torch.Tensor] = {}
DECODE_MIN_KEYS_PER_SPLIT = 128
PREFILL_ROWS = 128                     # packed rows (tokens x heads of a KV group) of one prefill CTA
PREFILL_ROWS_WIDE = 256                # of the tcgen05 kernel with two Q tiles
WIDE_MIN_CTAS = None                   # fewest CTAs the wide kernel is used for; None: the machine's (one CTA per SM)


def _arange(device: torch.device, n: int) -> torch.Tensor:
    a = _ARANGE.get(device)
    if a is None or a.numel() < n:
        a = torch.arange(max(n, 4096), dtype=torch.int32, device=device)
        _ARANGE[device] = a
    return a


def attention_supported(hd: int, nh: int, nkv: int) -> bool:
    return "attention" not in DISABLED and hd % 16 == 0 and 16 <= hd <= 256 and nh % nkv == 0 and nh // nkv <= PREFILL_ROWS


def _attn_common_args(q, out, cache, ctx, nh, nkv, scale, window):
    pool, bt = cache.pool, cache.block_table
    return [_p(q), _p(out), _p(pool), _p(bt), bt.stride(0), _p(ctx.positions), _p(ctx.req_of_token),
            int(ctx.num_reqs), pool.shape[0], pool.shape[3], nh, nkv, float(scale), int(window)]


_COMMON_SIG = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
               c_float, c_int]


def attn_prefill(ctx, q, out, cache, nh, nkv, hd, scale, window, tiles: torch.Tensor, n_tiles: int,
                 n_tiles_dev: Optional[torch.Tensor] = None) -> None:
    """Flash attention of prompt portions; ``tiles`` is int32 [n, 4] = (request, first row, tokens, 0).
    With ``n_tiles_dev`` (int32 on the device) the launch is made for ``n_tiles`` and runs that many."""
    _cuda(q, out, cache.pool, cache.block_table, tiles)
    _need(q.dtype == torch.bfloat16 and cache.pool.dtype == torch.bfloat16 and q.is_contiguous() and out.is_contiguous(),
          "tensor-core attention takes contiguous bfloat16 q, out and pages")
    _need(tiles.dtype == torch.int32 and tiles.is_contiguous() and tiles.numel() >= 4 * n_tiles, "tiles must be int32 [n, 4]")
    f = _fn("attention_mma", "airun_attn_prefill", _COMMON_SIG + [c_void_p, c_int, c_void_p, c_void_p, c_void_p], {"HD": hd})
    _check(f(*_attn_common_args(q, out, cache, ctx, nh, nkv, scale, window), _p(tiles), n_tiles, _p(n_tiles_dev),
             _p(ctx.err), _stream()), "attn_prefill")


def prefill_tc_supported(hd: int, page_size: int) -> bool:
    """The tcgen05 prefill kernel takes head sizes 64 and 128 and pages of 16, 32, 64, ... tokens."""
    return ("attention_tc" not in DISABLED and hd in (64, 128) and page_size >= 16
            and (page_size & (page_size - 1)) == 0)


def attn_prefill_tc(ctx, q, out, cache, nh, nkv, hd, scale, window, tiles: torch.Tensor, n_tiles: int,
                    n_tiles_dev: Optional[torch.Tensor] = None, wide: bool = False) -> None:
    """Flash attention of prompt portions on tcgen05 (csrc/attention_tcgen05.cu); same tiles as attn_prefill.
    ``wide``: the tiles hold up to PREFILL_ROWS_WIDE // G tokens (the kernel with two Q tiles to a CTA)."""
    _cuda(q, out, cache.pool, cache.block_table, tiles)
    _need(q.dtype == torch.bfloat16 and cache.pool.dtype == torch.bfloat16 and q.is_contiguous() and out.is_contiguous(),
          "tensor-core attention takes contiguous bfloat16 q, out and pages")
    _need(prefill_tc_supported(hd, cache.pool.shape[3]), "head size or page size not taken by the tcgen05 attention")
    _need(tiles.dtype == torch.int32 and tiles.is_contiguous() and tiles.numel() >= 4 * n_tiles, "tiles must be int32 [n, 4]")
    pool, bt = cache.pool, cache.block_table
    f = _fn("attention_tcgen05", "airun_attn_prefill_wide" if wide else "airun_attn_prefill_tc",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int,
             c_void_p, c_int, c_void_p, c_void_p, c_void_p], {"HD": hd})
    _check(f(_p(q), _p(out), _p(pool), _p(bt), bt.stride(0), _p(ctx.positions), pool.shape[0], pool.shape[3],
             nh, nkv, float(scale), int(window), _p(tiles), n_tiles, _p(n_tiles_dev), _p(ctx.err), _stream()),
           "attn_prefill_tc")


def attn_decode(ctx, q, out, cache, nh, nkv, hd, scale, window, rows: torch.Tensor, n_rows: int, n_splits: int,
                n_rows_dev: Optional[torch.Tensor] = None, dyn_slots: int = 0,
                k_begin_dev: Optional[torch.Tensor] = None, extra_slices: int = 0, early: Optional[bool] = None) -> None:
    """Attention of single decoded tokens (batch rows ``rows``; None: rows 0..n_rows-1), the keys cut
    into ``n_splits`` slices.  With ``n_rows_dev`` (int32 on the device) the launch is made for ``n_rows``
    rows and ``n_splits`` slices, runs the rows counted there, and every row picks its slices itself so
    that about ``dyn_slots`` CTAs run.  With ``k_begin_dev`` (int32 on the device) the keys below that
    position are left out and the ``extra_slices`` results another kernel (``attn_shared_prefix``) has
    put into the scratch for them are merged in.  ``early``: the kernel may ask for keys and values
    before the kernel in front of it has finished, which holds when all but each token's newest key were
    written before this chain of launches began; by default, when the launch is being captured into a
    graph (a whole step, bounded by the graph's own launch)."""
    if early is None:
        early = torch.cuda.is_current_stream_capturing()
    _cuda(q, out, cache.pool, cache.block_table, rows)
    _need(q.dtype == torch.bfloat16 and cache.pool.dtype == torch.bfloat16 and q.is_contiguous() and out.is_contiguous(),
          "tensor-core attention takes contiguous bfloat16 q, out and pages")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.is_contiguous() and rows.numel() >= n_rows, "rows must be int32 [n]")
    scratch, counters = scratch_for(q.device)
    hgroups = (nh // nkv + 15) // 16
    if n_splits + extra_slices > 1:
        # rows picking their own slices use at most max(dyn_slots, rows x head groups) slices together
        units = n_rows * nkv * hgroups
        need = (units * (n_splits + extra_slices) if n_rows_dev is None else max(dyn_slots, units)) * 16 * (hd + 2)
        _need(need <= scratch.numel() and n_rows * nkv * hgroups <= counters.numel(),
              "split-K scratch is too small for this decode launch")
    f = _fn("attention_mma", "airun_attn_decode",
            _COMMON_SIG + [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                           c_void_p], {"HD": hd})
    _check(f(*_attn_common_args(q, out, cache, ctx, nh, nkv, scale, window), _p(rows), n_rows, n_splits,
             _p(scratch), _p(counters), _p(n_rows_dev), int(dyn_slots), _p(k_begin_dev), int(extra_slices),
             1 if early else 0, _p(ctx.err), _stream()), "attn_decode")


def attn_shared_prefix(ctx, q, cache, nh, nkv, hd, scale, n_rows: int, k_end_dev: torch.Tensor, slices: int,
                       n_splits: int) -> None:
    """First half of the attention of decoded tokens whose requests begin with the same pages: the keys
    [0, k_end) once for all of them (rows 0..n_rows-1 of the batch), in ``slices`` slices whose results go
    to the decode kernel's scratch; ``attn_decode(..., k_begin_dev=k_end_dev, extra_slices=slices)`` with
    the same ``n_splits`` must follow on the same stream."""
    _cuda(q, cache.pool, cache.block_table, k_end_dev)
    _need(q.dtype == torch.bfloat16 and cache.pool.dtype == torch.bfloat16 and q.is_contiguous(),
          "tensor-core attention takes contiguous bfloat16 q and pages")
    _need(k_end_dev.dtype == torch.int32 and k_end_dev.numel() >= 1, "k_end_dev must be int32 [1]")
    scratch, _ = scratch_for(q.device)
    hgroups = (nh // nkv + 15) // 16
    _need(n_rows * nkv * hgroups * (n_splits + slices) * 16 * (hd + 2) <= scratch.numel(),
          "split-K scratch is too small for this shared-prefix launch")
    pool, bt = cache.pool, cache.block_table
    if prefill_tc_supported(hd, cache.page_size):
        f = _fn("attention_tcgen05", "airun_attn_shared_prefix_tc",
                [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                 c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p], {"HD": hd})
        _check(f(_p(q), _p(pool), _p(bt), bt.stride(0), _p(ctx.req_of_token), int(ctx.num_reqs), pool.shape[0],
                 pool.shape[3], nh, nkv, float(scale), int(n_rows), _p(k_end_dev), int(slices), int(n_splits),
                 _p(scratch), _p(ctx.err), _stream()), "attn_shared_prefix_tc")
        return
    f = _fn("attention_mma", "airun_attn_shared_prefix",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
             c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p], {"HD": hd})
    _check(f(_p(q), _p(pool), _p(bt), bt.stride(0), _p(ctx.positions), _p(ctx.req_of_token), int(ctx.num_reqs),
             pool.shape[0], pool.shape[3], nh, nkv, float(scale), int(n_rows), _p(k_end_dev), int(slices), int(n_splits),
             _p(scratch), _p(ctx.err), _stream()), "attn_shared_prefix")


def attn_plan(ctx, per_tile: int, tiles: torch.Tensor, rows: torch.Tensor, counts: torch.Tensor) -> None:
    """The attention work lists of the batch, made on the device (csrc/attention_plan.cu): tiles of
    ``per_tile`` tokens of every portion, the rows of single tokens, and how many of each."""
    _cuda(ctx.cu_tokens, ctx.context_lens, tiles, rows, counts)
    for t in (tiles, rows, counts):
        _need(t.dtype == torch.int32 and t.is_contiguous(), "the plan's lists are contiguous int32")
    _need(ctx.cu_tokens.numel() >= ctx.num_reqs + 1 and ctx.context_lens.numel() >= ctx.num_reqs and counts.numel() >= 2,
          "the batch's layout arrays are shorter than its number of requests")
    f = _fn("attention_plan", "airun_attn_plan",
            [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_p(ctx.cu_tokens), _p(ctx.context_lens), int(ctx.num_reqs), int(per_tile), _p(tiles), tiles.shape[0],
             _p(rows), rows.numel(), _p(counts), _p(ctx.err), _stream()), "attn_plan")


def plan_decode_splits(n_rows: int, nkv: int, hgroups: int, context_len: int, hd: int, slots: Optional[int] = None) -> int:
    """Slices of the keys per (token, KV head).  A CTA costs a fixed part (set-up, merge of its warps,
    its share of the merge of the slices) plus a part per key; CTAs run in waves of ``slots``.  The
    constants come from timing the kernel at batch 1, 8 and 64 with 4096 keys."""
    slots = slots or machine().decode_slots
    units = max(1, n_rows * nkv * hgroups)
    most = max(1, min(64, (context_len + DECODE_MIN_KEYS_PER_SPLIT - 1) // DECODE_MIN_KEYS_PER_SPLIT))
    best, best_cost = 1, None
    for s in range(1, most + 1):
        if s > 1 and units * s * 16 * (hd + 2) > SCRATCH_FLOATS:
            break
        waves = -(-units * s // slots)
        cost = waves * (context_len / s * 0.02 + 9.0) + (1.0 if s > 1 else 0.0) + 0.15 * s
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def _wide_tiles(ctx, G: int, nkv: int) -> bool:
    """Whether the step's portions go to tiles of PREFILL_ROWS_WIDE rows: when those tiles still fill
    the machine (a CTA per tile and KV head).  They read every key once for twice as many rows, which is
    what bounds a long prompt; a step with few tiles is better spread over more, narrower ones."""
    shape = ctx.extras.get("device_plan")
    if shape:
        # a padded batch: what the shape allows at least
        if not shape["max_portions"]:
            return False
        tiles = (ctx.num_tokens - min(shape["max_rows"], ctx.num_tokens)) * G // PREFILL_ROWS_WIDE
    else:
        tiles = sum(-(-n * G // PREFILL_ROWS_WIDE) for n in ctx.query_lens if n > 1)
    return tiles * nkv >= (WIDE_MIN_CTAS if WIDE_MIN_CTAS is not None else machine().wide_min_ctas)


def _attention_plan(ctx, G: int, tile_rows: int = PREFILL_ROWS):
    """Which rows are single decoded tokens and how the prompt portions are cut into tiles
    of tile_rows // G tokens; made once per step, group size and tile size."""
    key = ("attn_plan", G, tile_rows)
    plan = ctx.extras.get(key)
    if plan is not None:
        return plan
    dev = ctx.token_ids.device
    shape = ctx.extras.get("device_plan")
    if shape:
        # the batch is padded and its layout is only on the device: lists long enough for any batch
        # of this shape (``shape`` bounds its single tokens and portions), filled by a kernel, the
        # counts read by the attention kernels themselves
        per = max(1, tile_rows // G)
        T = ctx.num_tokens
        max_rows, max_portions = min(shape["max_rows"], T), min(shape["max_portions"], T // 2)
        max_tiles = (T // per + max_portions + 1) if max_portions else 0
        buf = ctx.ws_main.alloc((4 + 4 * max(max_tiles, 1) + max(max_rows, 1),), torch.int32)
        counts, tiles = buf[:4], buf[4:4 + 4 * max(max_tiles, 1)].view(max(max_tiles, 1), 4)
        rows = buf[4 + 4 * max(max_tiles, 1):]
        attn_plan(ctx, per, tiles, rows, counts)
        plan = dict(rows=rows, n_rows=max_rows, tiles=tiles, n_tiles=max_tiles,
                    n_tiles_dev=counts[0:1], n_rows_dev=counts[1:2], min_rows=max(1, shape["min_rows"]))
    elif ctx.decode_only:
        plan = dict(rows=None, n_rows=ctx.num_tokens, tiles=None, n_tiles=0)
    else:
        per = max(1, tile_rows // G)
        rows, tiles, t = [], [], 0
        for r, (n, c) in enumerate(zip(ctx.query_lens, ctx.context_lens_host)):
            if n == 1:
                rows.append(t)
            else:
                for s in range(0, n, per):
                    k = min(per, n - s)
                    tiles.append((r, t + s, k, c - n + s + k))     # last field: keys its last token sees
            t += n
        # the tiles with the most keys first: CTAs are handed out in order, and the longest
        # ones must not be the last to start
        tiles.sort(key=lambda x: -x[3])
        plan = dict(
            rows=torch.tensor(rows, dtype=torch.int32).to(dev, non_blocking=True) if rows else None, n_rows=len(rows),
            tiles=torch.tensor(tiles, dtype=torch.int32).to(dev, non_blocking=True) if tiles else None, n_tiles=len(tiles))
    ctx.extras[key] = plan
    return plan


def attention_bf16(ctx, q, out, cache, nh: int, nkv: int, hd: int, scale: float, window: int) -> bool:
    if not attention_supported(hd, nh, nkv) or q.dtype != torch.bfloat16:
        return False
    G = nh // nkv
    tc = prefill_tc_supported(hd, cache.page_size)
    wide = tc and "attention_wide" not in DISABLED and _wide_tiles(ctx, G, nkv)
    plan = _attention_plan(ctx, G, PREFILL_ROWS_WIDE if wide else PREFILL_ROWS)
    n_tiles_dev, n_rows_dev = plan.get("n_tiles_dev"), plan.get("n_rows_dev")
    if plan["n_tiles"]:
        if tc:
            attn_prefill_tc(ctx, q, out, cache, nh, nkv, hd, scale, window, plan["tiles"], plan["n_tiles"], n_tiles_dev, wide)
        else:
            attn_prefill(ctx, q, out, cache, nh, nkv, hd, scale, window, plan["tiles"], plan["n_tiles"], n_tiles_dev)
    if plan["n_rows"]:
        context = ctx.extras.get("planning_context_len", ctx.max_context_len)
        if window > 0:
            context = min(context, window)
        tma = hd % 64 == 0 and cache.page_size % 16 == 0 and (cache.page_size & (cache.page_size - 1)) == 0
        mach = machine(q.device)
        slots = mach.decode_slots_tma if tma else mach.decode_slots
        if n_rows_dev is not None:
            # no row takes more slices than fit when the fewest rows of this shape are there
            fit = max(1, slots // (plan["min_rows"] * nkv * ((G + 15) // 16)))
            most = max(1, min(64, (context + DECODE_MIN_KEYS_PER_SPLIT - 1) // DECODE_MIN_KEYS_PER_SPLIT, fit))
            attn_decode(ctx, q, out, cache, nh, nkv, hd, scale, window, plan["rows"], plan["n_rows"], most,
                        n_rows_dev, slots)
        elif (ctx.extras.get("use_shared_prefix") and plan["rows"] is None and window == 0
              and getattr(cache, "shared_prefix", None) is not None and _shared_prefix_slices(plan["n_rows"], nkv, G, hd) > 0):
            # the requests of the batch begin with the same pages: those keys once for all tokens (in
            # slices of their own), each token's later keys as usual, one merge
            splits = plan_decode_splits(plan["n_rows"], nkv, (G + 15) // 16, min(context, SHARED_SUFFIX_PLAN), hd, slots)
            slices = _shared_prefix_slices(plan["n_rows"], nkv, G, hd, splits,
                                           mach.sms if prefill_tc_supported(hd, cache.page_size) else 2 * mach.sms)
            attn_shared_prefix(ctx, q, cache, nh, nkv, hd, scale, plan["n_rows"], cache.shared_prefix, slices, splits)
            attn_decode(ctx, q, out, cache, nh, nkv, hd, scale, window, None, plan["n_rows"], splits,
                        k_begin_dev=cache.shared_prefix, extra_slices=slices)
        else:
            splits = plan_decode_splits(plan["n_rows"], nkv, (G + 15) // 16, context, hd, slots)
            attn_decode(ctx, q, out, cache, nh, nkv, hd, scale, window, plan["rows"], plan["n_rows"], splits)
    return True


SHARED_SUFFIX_PLAN = 2048              # keys after the shared prefix the slice count of such a step is chosen for


def _shared_prefix_slices(n_rows: int, nkv: int, G: int, hd: int, splits: int = 8, slots: Optional[int] = None) -> int:
    """Slices of the shared keys: about one CTA per SM slot (``slots``: the SM count for the tcgen05 kernel,
    one CTA to an SM; twice that for the mma.sync one), as many as the scratch has room for beside the
    ``splits`` slices of the tokens' own keys, at most 64 of both together."""
    slots = slots or 2 * machine().sms
    groups = -(-n_rows * G // PREFILL_ROWS)
    want = max(1, min(37, slots // max(1, nkv * groups)))
    room = SCRATCH_FLOATS // (n_rows * nkv * ((G + 15) // 16) * 16 * (hd + 2)) - splits
    return max(0, min(want, room, 64 - splits))
