"""Python entry to the hand-written sm_100a kernels.

Each function checks shapes, types and contiguity, refuses what its kernel does
not take with a clear error, and launches on torch's current CUDA stream through
the library's C entry point.  Nothing here computes on the CPU and nothing falls
back to a library routine: a missing or failing extension raises.

The reference has the same layer: safe wrappers that check sizes before they hand
raw pointers to ``extern "C"`` launchers (crates/airun-cuda/src/ops.rs:1-6, :290-330;
the launchers at crates/airun-cuda/kernels/ops.cu:2222-2578).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_float, c_void_p
from typing import Optional

import torch

from ..csrc import build

DT_F32, DT_BF16 = 0, 1
ROPE_NONE, ROPE_NEOX, ROPE_INTERLEAVED = 0, 1, 2
_DT = {torch.float32: DT_F32, torch.bfloat16: DT_BF16}

DEV_ERR_BITS = {1: "a block-table entry outside the page pool", 2: "a token naming a request outside the batch",
                4: "a token id outside the vocabulary", 8: "a bounded device-side wait ran out"}


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        raise KernelError(f"dtype {t.dtype} is not handled by the kernels (float32 and bfloat16 are)")
    return _DT[t.dtype]


def _p(t: Optional[torch.Tensor]):
    return None if t is None else c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None:
            _need(t.is_cuda, "kernel arguments must live on the GPU (there is no CPU path)")


LAUNCHES = [0]          # kernels launched through this module (CUDA-graph replays are counted by their owner)


def _check(status: int, what: str) -> None:
    if status == 0:
        LAUNCHES[0] += 1
        return
    if status == 1000:
        raise KernelError(f"{what}: the kernel refuses these sizes or pointers")
    if status == 1001:
        raise KernelError(f"{what}: this combination of types is not supported")
    raise KernelError(f"{what}: CUDA error {status} at launch")


_SIGS = {}


def _fn(lib_name: str, fn_name: str, argtypes, defines=None):
    key = (lib_name, fn_name, tuple(sorted((defines or {}).items())))
    f = _SIGS.get(key)
    if f is None:
        lib = build.load(lib_name, defines)
        f = getattr(lib, fn_name)
        f.argtypes = argtypes
        f.restype = c_int
        _SIGS[key] = f
    return f


def required_libraries(dtype: torch.dtype, head_dim: int):
    """(name, defines) of every library a model of this dtype and head size uses."""
    libs = [("elementwise", None), ("gemm_simt", None), ("qkv_post", None),
            ("attention_generic", None), ("sampling", None)]
    return libs


# ---------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None,
          scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] widened to float32 (times ``scale``; 1 leaves the values as they are)."""
    _cuda(table, ids, out, err)
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be a contiguous [V, H] tensor")
    _need(ids.dtype == torch.int32 and ids.dim() == 1 and ids.is_contiguous(), "ids must be int32 [T]")
    T, (V, H) = ids.shape[0], table.shape
    _need(out.dtype == torch.float32 and tuple(out.shape) == (T, H) and out.is_contiguous(),
          "embedding output must be float32 [T, H]")
    f = _fn("elementwise", "airun_embed",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(f(_p(table), _dt(table), _p(ids), _p(out), T, H, V, float(scale), _p(err), _stream()), "embed")


def soft_cap(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap), in place."""
    _cuda(x)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "soft_cap takes a contiguous float32 tensor")
    _need(cap > 0.0, "the cap must be positive")
    f = _fn("elementwise", "airun_soft_cap", [c_void_p, c_longlong, c_float, c_void_p])
    _check(f(_p(x), x.numel(), float(cap), _stream()), "soft_cap")


def copy_pages(pool: torch.Tensor, pairs: torch.Tensor, err: Optional[torch.Tensor] = None) -> None:
    """pool: [owners, pages, ...] cache pages of one group; pairs: int32 [n, 2] (source page, destination page) on
    the device.  Every owner layer's page ``dst`` becomes a copy of its page ``src``."""
    _cuda(pool, pairs, err)
    _need(pool.dim() >= 3 and pool.is_contiguous(), "pool must be contiguous [owners, pages, ...]")
    _need(pairs.dtype == torch.int32 and pairs.dim() == 2 and pairs.shape[1] == 2 and pairs.is_contiguous(),
          "pairs must be int32 [n, 2]")
    page_bytes = pool[0, 0].numel() * pool.element_size()
    _need(page_bytes % 16 == 0, "a page must be a multiple of 16 bytes")
    f = _fn("elementwise", "airun_copy_pages", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_p(pool), pool.shape[0], pool.shape[1], page_bytes, _p(pairs), pairs.shape[0], _p(err), _stream()), "copy_pages")


def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """out = rmsnorm(x [+ delta]) * weight.

    With ``delta`` and no ``rows`` the sum is written back into ``x`` (the
    residual stream).  With ``rows`` only those rows are normed, into
    out[0..len(rows)), and ``x`` is left as it is.
    """
    _cuda(x, weight, out, delta, rows)
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "x must be float32 [T, n]")
    n = x.shape[1]
    if weight is not None:
        _need(weight.dtype == torch.float32 and tuple(weight.shape) == (n,) and weight.is_contiguous(),
              "norm weight must be float32 [n]")
    if delta is not None:
        _need(delta.dtype == torch.float32 and delta.shape == x.shape and delta.is_contiguous(),
              "delta must match x")
    n_rows = x.shape[0]
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), "rows must be int32 [R]")
        n_rows = rows.shape[0]
    _need(out.dim() == 2 and out.shape[0] >= n_rows and out.shape[1] == n and out.is_contiguous(),
          "norm output must be [rows, n]")
    f = _fn("elementwise", "airun_rmsnorm",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    write_back = 1 if (delta is not None and rows is None) else 0
    _check(f(_p(x), _p(delta), _p(weight), _p(out), _dt(out), _p(rows), n_rows, n, float(eps), write_back,
             _stream()), "rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, group: int) -> None:
    """out[t, i] = silu(g) * u where gate and up columns alternate in blocks of ``group``."""
    _cuda(gate_up, out)
    _need(gate_up.dim() == 2 and out.dim() == 2 and gate_up.is_contiguous() and out.is_contiguous(),
          "swiglu takes contiguous [T, 2I] and [T, I]")
    T, I = out.shape
    _need(gate_up.shape[0] == T and gate_up.shape[1] == 2 * I, "swiglu input must be [T, 2I]")
    f = _fn("elementwise", "airun_swiglu", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_p(gate_up), _dt(gate_up), _p(out), _dt(out), T, I, int(group), _stream()), "swiglu")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(src, rows, out)
    _need(src.dim() == 2 and src.is_contiguous() and out.is_contiguous() and out.dtype == src.dtype,
          "gather_rows takes contiguous 2-d tensors of one type")
    _need(rows.dtype == torch.int32 and rows.is_contiguous(), "rows must be int32")
    rb = src.shape[1] * src.element_size()
    _need(rb % 4 == 0, "row size must be a multiple of 4 bytes")
    _need(out.shape[0] >= rows.shape[0] and out.shape[1] == src.shape[1], "gather output too small")
    f = _fn("elementwise", "airun_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(src), _p(out), _p(rows), rows.shape[0], rb, _stream()), "gather_rows")


# ---------------------------------------------------------------- matrix products
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on the CUDA cores, float32 accumulation."""
    _cuda(a, w, out)
    _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "gemm takes 2-d tensors")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(out.shape) == (M, N), f"gemm shapes do not agree: {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _need(a.dtype == w.dtype, "gemm operands must share a type")
    f = _fn("gemm_simt", "airun_gemm_simt",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
             c_longlong, c_longlong, c_longlong, c_void_p])
    _check(f(_p(a), _dt(a), _p(w), _dt(w), _p(out), _dt(out), M, N, K,
             a.stride(0) if M > 1 else max(K, a.stride(0)), w.stride(0) if N > 1 else max(K, w.stride(0)),
             out.stride(0) if M > 1 else max(N, out.stride(0)), _stream()), "gemm_simt")


# ---------------------------------------------------------------- attention
def qkv_post(qkv: torch.Tensor, q_out: torch.Tensor, q_norm_w: Optional[torch.Tensor],
             k_norm_w: Optional[torch.Tensor], eps: float, positions: torch.Tensor,
             req_of_token: torch.Tensor, rope_kind: int, rotary_dim: int, inv_freq: Optional[torch.Tensor],
             pool: Optional[torch.Tensor], block_table: Optional[torch.Tensor], num_reqs: int,
             page_size: int, nh: int, nkv: int, hd: int, err: torch.Tensor,
             store: bool = True, kv_in_row: bool = True, rope_positions: Optional[torch.Tensor] = None) -> None:
    """Per-head norm, rotary encoding, q out, k/v into their pages (see csrc/qkv_post.cu).

    ``pool`` is one layer's pages [num_pages, 2, nkv, page_size, hd].  ``rope_kind``: ROPE_NONE, ROPE_NEOX
    (pair i couples dims i and i + r/2) or ROPE_INTERLEAVED (dims 2i and 2i + 1).  ``rope_positions``
    (int32 [T]): the position each row is rotated by, when that is not its place in the cache."""
    _cuda(qkv, q_out, q_norm_w, k_norm_w, positions, req_of_token, inv_freq, pool, block_table, err, rope_positions)
    if rope_positions is not None:
        _need(rope_positions.dtype == torch.int32 and rope_positions.is_contiguous() and rope_positions.shape[0] >= qkv.shape[0],
              "rope_positions must be int32 [T]")
    T = qkv.shape[0]
    width = (nh + 2 * nkv) * hd if kv_in_row else nh * hd
    _need(qkv.dtype == torch.float32 and qkv.dim() == 2 and qkv.shape[1] == width and qkv.stride(1) == 1,
          f"qkv must be float32 [T, {width}]")
    _need(tuple(q_out.shape) == (T, nh * hd) and q_out.is_contiguous(), "q_out must be [T, nh*hd]")
    _need(hd <= 256, f"head_dim {hd} is above the kernel's limit of 256")
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            _need(w.dtype == torch.float32 and tuple(w.shape) == (hd,), "q/k norm weights must be float32 [head_dim]")
    _need(positions.dtype == torch.int32 and req_of_token.dtype == torch.int32
          and positions.shape[0] >= T and req_of_token.shape[0] >= T, "positions / req_of_token must be int32 [T]")
    if rope_kind != ROPE_NONE:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.shape[0] == rotary_dim // 2,
              "inv_freq must be float32 [rotary_dim/2]")
    num_pages, max_blocks = 0, 0
    do_store = bool(store and kv_in_row)
    if do_store:
        _need(pool is not None and pool.is_contiguous() and pool.dim() == 5
              and tuple(pool.shape[1:]) == (2, nkv, page_size, hd), "pool must be [pages, 2, nkv, page_size, hd]")
        _need(pool.dtype == q_out.dtype, "q and the cache pages must share a type")
        _need(block_table is not None and block_table.dtype == torch.int32 and block_table.dim() == 2
              and block_table.stride(1) == 1, "block_table must be int32 [R, max_blocks]")
        num_pages, max_blocks = pool.shape[0], block_table.stride(0)
    f = _fn("qkv_post", "airun_qkv_post",
            [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
             c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(qkv), qkv.stride(0), _p(q_out), _dt(q_out), _p(q_norm_w), _p(k_norm_w), float(eps),
             _p(positions), _p(req_of_token), T, int(rope_kind), int(rotary_dim), _p(inv_freq), _p(rope_positions),
             _p(pool), _dt(q_out), _p(block_table), max_blocks, int(num_reqs), num_pages, int(page_size),
             1 if do_store else 0, 1 if kv_in_row else 0, nh, nkv, hd, _p(err), _stream()), "qkv_post")


def attention_generic(q: torch.Tensor, out: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor,
                      positions: torch.Tensor, req_of_token: torch.Tensor, num_reqs: int,
                      nh: int, nkv: int, hd: int, scale: float, window: int, err: torch.Tensor) -> None:
    """Causal attention of every token over its request's pages, float32 arithmetic."""
    _cuda(q, out, pool, block_table, positions, req_of_token, err)
    T = q.shape[0]
    _need(tuple(q.shape) == (T, nh * hd) and q.is_contiguous() and out.shape == q.shape and out.is_contiguous()
          and out.dtype == q.dtype, "q and out must be contiguous [T, nh*hd] of one type")
    _need(hd <= 256, f"head_dim {hd} is above the kernel's limit of 256")
    _need(nh % nkv == 0, "query heads must be a multiple of KV heads")
    _need(pool.is_contiguous() and pool.dim() == 5 and pool.shape[1] == 2 and pool.shape[2] == nkv
          and pool.shape[4] == hd and pool.dtype == q.dtype, "pool must be [pages, 2, nkv, page_size, hd] of q's type")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1,
          "block_table must be int32 [R, max_blocks]")
    f = _fn("attention_generic", "airun_attention_generic",
            [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _dt(q), _p(pool), _dt(pool), _p(block_table), block_table.stride(0),
             _p(positions), _p(req_of_token), T, int(num_reqs), pool.shape[0], pool.shape[3],
             nh, nkv, hd, float(scale), int(window), _p(err), _stream()), "attention_generic")


# ---------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None) -> None:
    """out[r] = first argmax of logits[r], or a draw at temperature[r] > 0 using uniform[r]."""
    _cuda(logits, out, temperature, uniform)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be float32 [R, V]")
    R, V = logits.shape
    _need(out.dtype == torch.int32 and out.shape[0] >= R and out.is_contiguous(), "sample output must be int32 [R]")
    for t in (temperature, uniform):
        if t is not None:
            _need(t.dtype == torch.float32 and t.shape[0] >= R and t.is_contiguous(), "temperature / uniform must be float32 [R]")
    scratch = None
    if V >= 8192:
        scratch = _SAMPLE_SCRATCH.get(logits.device)
        if scratch is None or scratch.numel() < R * 128:
            scratch = torch.empty(max(R, 256) * 128, dtype=torch.int32, device=logits.device)
            _SAMPLE_SCRATCH[logits.device] = scratch
    f = _fn("sampling", "airun_sample",
            [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(logits), logits.stride(0) if R > 1 else max(V, logits.stride(0)), R, V,
             _p(temperature), _p(uniform), _p(out), _p(scratch), _stream()), "sample")


_SAMPLE_SCRATCH = {}

LARGEST_LOGITS_MAX = 512


def largest_logits(logits: torch.Tensor, rows: torch.Tensor, n: int, n_cand: int, out_ids: torch.Tensor,
                   out_vals: torch.Tensor, out_flags: torch.Tensor) -> None:
    """For the ``n`` rows ``rows[i]`` of ``logits``: out_ids[i], out_vals[i] = the ``n_cand`` largest logits with
    their ids, the largest first, equal values by ascending id (-1 / -inf beyond the row's size); out_flags[i] != 0
    when the kernel cannot vouch for the list (the caller then takes the whole row)."""
    _cuda(logits, rows, out_ids, out_vals, out_flags)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be float32 [R, V]")
    _need(1 <= n_cand <= LARGEST_LOGITS_MAX, f"1 to {LARGEST_LOGITS_MAX} candidates a row")
    _need(rows.dtype == torch.int32 and rows.numel() >= n and rows.is_contiguous(), "rows must be int32 [n]")
    _need(out_ids.dtype == torch.int32 and out_ids.is_contiguous() and out_ids.numel() >= n * n_cand
          and out_vals.dtype == torch.float32 and out_vals.is_contiguous() and out_vals.numel() >= n * n_cand
          and out_flags.dtype == torch.int32 and out_flags.numel() >= n, "candidate outputs are [n, n_cand] and [n]")
    R, V = logits.shape
    f = _fn("sampling", "airun_largest_logits",
            [c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(logits), logits.stride(0) if R > 1 else max(V, logits.stride(0)), V, _p(rows), int(n), int(n_cand),
             _p(out_ids), _p(out_vals), _p(out_flags), _stream()), "largest_logits")


def describe_device_error(bits: int) -> str:
    return "; ".join(msg for b, msg in DEV_ERR_BITS.items() if bits & b) or f"unknown error bits {bits}"
