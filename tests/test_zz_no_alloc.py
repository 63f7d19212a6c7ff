"""The matrix product for callers that cannot allocate device memory
(airun_gemm_tcgen05_static, declared in airun_b200/csrc/gemm_tcgen05_static.h).

Who needs it: code that runs where cudaMalloc is not allowed or not wanted, for example
inside a CUDA-graph capture, under a framework that hands out all device memory once, or
in a plug-in that only ever receives input and output buffers.  The regular entry point
asks such a caller for split-K scratch it has no way to provide; this one keeps the scratch
in arrays that belong to the library.

The test calls the new entry point through its exported C symbol, twice in a row (the
arrays keep what the first call left), and holds its output to the regular entry point's.
This file sorts last on purpose: a run that stops at the first failure has by then run
every other test.
"""
import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_STATIC_TOO_LARGE = 1002


def _lib():
    from airun_b200.csrc import build
    lib = build.load("gemm_tcgen05")
    fn = lib.airun_gemm_tcgen05_static
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                   c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    fn.restype = c_int
    return fn


def _call(fn, x, w, out, epi, swap, bn, ksplit, err):
    M, K = x.shape
    N = w.shape[0]
    return fn(c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), M, N, K,
              x.stride(0), w.stride(0), out.stride(0), epi, 1 if swap else 0, bn, ksplit,
              c_void_p(err.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("M,N,K,epi,swap,bn,ksplit", [
    (8, 512, 4096, 0, True, 16, 8),          # a decode-sized product cut into 8 slices
    (40, 384, 2048, 2, True, 64, 4),         # SwiGLU epilogue after the slices are added
    (300, 256, 1024, 0, False, 128, 2),      # prompt-sized, normal mode
])
def test_static_scratch_entry_point_matches_the_regular_one(M, N, K, epi, swap, bn, ksplit):
    from airun_b200.kernels import fast
    fn = _lib()
    dev = "cuda"
    torch.manual_seed(21)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) * 0.1).to(torch.bfloat16)
    shape = (M, N // 2) if epi == 2 else (M, N)
    dtype = torch.float32 if epi == 0 else torch.bfloat16
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    want = torch.empty(shape, dtype=dtype, device=dev)
    fast.gemm_tcgen05(x, w, want, epi, swap, bn, ksplit, err)            # the existing entry point
    torch.cuda.synchronize()
    for call in range(2):                                               # two calls in a row share the arrays
        got = torch.full(shape, 5.0, dtype=dtype, device=dev)
        rc = _call(fn, x, w, got, epi, swap, bn, ksplit, err)
        assert rc == 0, f"call {call}: status {rc}"
        torch.cuda.synchronize()
        assert err.item() == 0
        assert torch.allclose(got.float(), want.float(), rtol=1e-2, atol=1e-2), f"call {call}"
        # the slices are added in the same order by both, so float32 results agree to the bit
        if epi == 0:
            assert torch.equal(got, want)
        x = x.flip(0).contiguous()                                      # other inputs on the second call
        fast.gemm_tcgen05(x, w, want, epi, swap, bn, ksplit, err)
        torch.cuda.synchronize()


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    fn = _lib()
    dev = "cuda"
    x = torch.zeros(64, 8192, device=dev, dtype=torch.bfloat16)
    w = torch.zeros(16384, 8192, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(64, 16384, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    # 128 tiles x 32 slices x 64 x 128 floats = 32 Mi floats, more than the 4 Mi the library holds
    assert _call(fn, x, w, out, 0, True, 64, 32, err) == ERR_STATIC_TOO_LARGE
    assert _call(fn, x, w, out, 0, True, 64, 1, err) == 0               # without slices no scratch is needed
    torch.cuda.synchronize()
    assert err.item() == 0
