"""Each kernel alone against its plain reference, at sizes other than the engine's."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


class Ctx:
    """The few fields of a step context the attention wrappers read."""

    def __init__(self, positions, req_of_token, num_reqs, query_lens, context_lens):
        self.positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
        self.req_of_token = torch.tensor(req_of_token, dtype=torch.int32, device=DEV)
        self.token_ids = self.positions
        self.num_reqs, self.num_tokens = num_reqs, len(positions)
        self.query_lens, self.context_lens_host = query_lens, context_lens
        self.max_context_len = max(context_lens)
        self.max_query_len = max(query_lens)
        self.decode_only = all(q == 1 for q in query_lens)
        self.err = _err()
        self.extras = {}


class Cache:
    def __init__(self, pool, block_table, page_size):
        self.pool, self.block_table, self.page_size, self.shared = pool, block_table, page_size, False


def paged_from_dense(ks, vs, page_size, dtype, extra_pages=5, seed=0):
    """ks, vs: per request [n_i, nkv, hd] float tensors.  Scatters them into a pool through a
    shuffled block table, and fills unused pages with large values that must never be read."""
    nkv, hd = ks[0].shape[1:]
    blocks = [(k.shape[0] + page_size - 1) // page_size for k in ks]
    n_pages = sum(blocks) + extra_pages
    g = np.random.default_rng(seed)
    perm = g.permutation(n_pages)
    pool = torch.full((n_pages, 2, nkv, page_size, hd), 1e4, dtype=torch.float32)
    bt = torch.full((len(ks), max(blocks) + 2), -1, dtype=torch.int32)
    p = 0
    for r, (k, v) in enumerate(zip(ks, vs)):
        for b in range(blocks[r]):
            page = int(perm[p]); p += 1
            bt[r, b] = page
            n = min(page_size, k.shape[0] - b * page_size)
            pool[page, 0, :, :n] = k[b * page_size:b * page_size + n].transpose(0, 1)
            pool[page, 1, :, :n] = v[b * page_size:b * page_size + n].transpose(0, 1)
    return pool.to(dtype).to(DEV), bt.to(DEV)


# ----------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("T,H,out_dtype", [(5, 100, torch.float32), (3, 4096, torch.bfloat16), (1, 36, torch.float32),
                                          (7, 1500, torch.bfloat16), (600, 1024, torch.bfloat16), (515, 2560, torch.float32),
                                          (1300, 516, torch.float32), (2400, 2048, torch.bfloat16)])
def test_rmsnorm_and_fused_add(T, H, out_dtype):
    from airun_b200.kernels import ops
    torch.manual_seed(1)
    x = torch.randn(T, H) * 3
    d = torch.randn(T, H)
    w = 1 + 0.5 * torch.rand(H)
    eps = 3e-5
    tol = 1e-4 if out_dtype == torch.float32 else 1e-2
    xd, out = x.to(DEV), torch.empty(T, H, dtype=out_dtype, device=DEV)
    ops.rmsnorm(xd, w.to(DEV), eps, out)
    want = P.plain_rmsnorm(x.double(), w.double(), eps)
    assert torch.allclose(out.cpu().double(), want, rtol=tol, atol=tol * 1e-1)
    ops.rmsnorm(xd, w.to(DEV), eps, out, delta=d.to(DEV))              # x += d, then the norm
    assert torch.allclose(xd.cpu(), x + d, rtol=0, atol=1e-6)
    want = P.plain_rmsnorm((x + d).double(), w.double(), eps)
    assert torch.allclose(out.cpu().double(), want, rtol=tol, atol=tol * 1e-1)
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)     # gathered rows leave x alone
    x2 = x.to(DEV)
    out2 = torch.empty(2, H, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x2, w.to(DEV), eps, out2, delta=d.to(DEV), rows=rows)
    assert torch.equal(x2.cpu(), x)
    assert torch.allclose(out2.cpu().double(), want[[T - 1, 0]], rtol=tol, atol=tol * 1e-1)


def test_embedding_and_bad_token_flag():
    from airun_b200.kernels import ops
    torch.manual_seed(2)
    for dt in (torch.float32, torch.bfloat16):
        table = torch.randn(37, 52).to(dt)
        ids = [3, 36, 0, 36, 17]
        out = torch.empty(5, 52, device=DEV)
        err = _err()
        ops.embed(table.to(DEV), torch.tensor(ids, dtype=torch.int32, device=DEV), out, err)
        assert torch.equal(out.cpu(), P.plain_embedding(table, ids, torch.float32))
        assert err.item() == 0
        ops.embed(table.to(DEV), torch.tensor([1, 99], dtype=torch.int32, device=DEV), out[:2], err)
        assert err.item() == 4 and torch.equal(out[1].cpu(), table[0].float())    # out of range reads row 0


@pytest.mark.parametrize("group", [16, 8, 48])
def test_swiglu_interleaved(group):
    from airun_b200.kernels import ops
    torch.manual_seed(3)
    T, I = 6, 96
    g, u = torch.randn(T, I) * 4, torch.randn(T, I)
    gu = torch.stack([g.view(T, I // group, group), u.view(T, I // group, group)], dim=2).reshape(T, 2 * I)
    want = g.double() / (1 + torch.exp(-g.double())) * u.double()
    out = torch.empty(T, I, device=DEV)
    ops.swiglu(gu.to(DEV), out, group)
    assert torch.allclose(out.cpu().double(), want, rtol=1e-5, atol=1e-6)
    outb = torch.empty(T, I, dtype=torch.bfloat16, device=DEV)
    ops.swiglu(gu.to(DEV), outb, group)
    assert torch.allclose(outb.cpu().double(), want, rtol=1e-2, atol=1e-2)


# ----------------------------------------------------------------------------- matrix products
@pytest.mark.parametrize("M,N,K", [(1, 70, 33), (65, 129, 100), (130, 64, 257), (7, 1000, 64)])
def test_gemm_simt_float32_is_true_32_bit(M, N, K):
    """Backward-error bound of a float32 dot product: |err| <= eps * sqrt(K) * 4 * sum|a*w|
    (the reference's matvec test uses this bound, crates/airun-cli/src/selftest.rs:382-409)."""
    from airun_b200.kernels import ops
    torch.manual_seed(4)
    a, w = torch.randn(M, K), torch.randn(N, K)
    out = torch.empty(M, N, device=DEV)
    ops.gemm_simt(a.to(DEV), w.to(DEV), out)
    want = a.double() @ w.double().T
    bound = np.finfo(np.float32).eps * math.sqrt(K) * 4 * (a.abs().double() @ w.abs().double().T)
    assert bool(((out.cpu().double() - want).abs() <= bound).all())
    # tf32 would miss this: float32 keeps 2^-20 next to 1
    a2 = torch.zeros(1, 8); a2[0, 0] = 1.0; a2[0, 1] = 1.0
    w2 = torch.zeros(1, 8); w2[0, 0] = 1.0; w2[0, 1] = 2.0 ** -20
    o2 = torch.empty(1, 1, device=DEV)
    ops.gemm_simt(a2.to(DEV), w2.to(DEV), o2)
    assert o2.item() == 1.0 + 2.0 ** -20


CASES_TC = [  # M, N, K, epi, swap, bn, ksplit
    (128, 128, 64, 0, False, 128, 1), (200, 384, 520, 0, False, 128, 1), (130, 300, 72, 0, False, 128, 1),
    (300, 520, 1000, 0, False, 256, 1), (257, 256, 2048, 0, False, 256, 3), (8, 256, 512, 0, True, 16, 1),
    (5, 300, 72, 0, True, 16, 1), (33, 392, 1024, 0, True, 64, 4), (64, 520, 4096, 0, True, 64, 8),
    (100, 264, 2048, 1, True, 128, 3), (256, 448, 512, 2, False, 128, 1), (7, 448, 512, 2, True, 16, 1),
    (20, 4128, 1024, 2, True, 32, 2), (1, 96, 8, 0, True, 16, 1),
    # the persistent kernel: more tiles than SMs (each CTA walks several), ragged edges, every epilogue
    (2048, 4096, 256, 0, False, 256, 1), (1100, 2336, 200, 2, False, 256, 1), (513, 1000, 320, 1, False, 256, 1),
    (300, 576, 512, 2, False, 256, 1)]


@pytest.mark.parametrize("M,N,K,epi,swap,bn,ksplit", CASES_TC)
def test_gemm_tcgen05_against_the_plain_kernel(M, N, K, epi, swap, bn, ksplit):
    from airun_b200.kernels import fast, ops
    torch.manual_seed(5)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.1).to(torch.bfloat16)
    ref = torch.empty(M, N, device=DEV)
    ops.gemm_simt(x, w, ref)                                   # float32 accumulation of the same operands
    err = _err()
    if epi == 2:
        g = ref.view(M, N // 32, 2, 16)
        want = (g[:, :, 0] / (1 + torch.exp(-g[:, :, 0])) * g[:, :, 1]).reshape(M, N // 2)
        out = torch.full((M, N // 2), 7.0, dtype=torch.bfloat16, device=DEV)
    else:
        want = ref
        out = torch.full((M, N), 7.0, dtype=torch.float32 if epi == 0 else torch.bfloat16, device=DEV)
    for _ in range(2):                                         # twice: the tile counters must come back to zero
        fast.gemm_tcgen05(x, w, out, epi, swap, bn, ksplit, err)
        torch.cuda.synchronize()
        assert err.item() == 0
        if epi == 0:
            # same operands, float32 sums in another order
            bound = 1e-5 * math.sqrt(K) * (x.float().abs() @ w.float().abs().T) + 1e-6
            assert bool(((out - want).abs() <= bound).all())
        else:
            assert torch.allclose(out.float(), want, rtol=1e-2, atol=1e-2)
        out.fill_(7.0)
    want64 = x.cpu().double() @ w.cpu().double().T              # and the plain kernel itself is right
    assert torch.allclose(ref.cpu().double(), want64, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("M,N,K,swap,bn,ksplit", [(8, 256, 512, True, 16, 1), (5, 328, 1024, True, 16, 4),
                                                   (40, 1024, 2048, True, 64, 3), (100, 264, 512, True, 128, 2),
                                                   (300, 520, 256, False, 256, 1), (1000, 2304, 320, False, 256, 1),
                                                   (200, 392, 512, False, 128, 2), (8, 16640, 256, True, 16, 1)])
def test_gemm_tcgen05_folded_norm(M, N, K, swap, bn, ksplit):
    """The product that ends a sub-layer adds into the residual and prepares the next norm; the
    product that starts the next sub-layer applies the token scales: together they equal
    add -> RMSNorm -> product."""
    from airun_b200.kernels import fast
    torch.manual_seed(8)
    eps = 1e-5
    act = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w1 = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    resid0 = torch.randn(M, N, device=DEV)
    norm_w = (1 + 0.3 * torch.randn(N, device=DEV)).contiguous()
    err = _err()
    resid = resid0.clone()
    h = torch.full((M, N), 3.0, dtype=torch.bfloat16, device=DEV)
    ssq = torch.zeros(fast.max_resid_parts(N), M, device=DEV)
    parts = fast.resid_parts(N, swap, bn)
    for _ in range(2):                                           # counters come back to zero
        resid.copy_(resid0)
        fast.gemm_tcgen05(act, w1, h, fast.EPI_RESID, swap, bn, ksplit, err, resid=resid, norm_w=norm_w, ssq_out=ssq)
        torch.cuda.synchronize()
        assert err.item() == 0
    want_resid = resid0.double() + act.double() @ w1.double().T
    assert torch.allclose(resid.double(), want_resid, rtol=1e-4, atol=1e-4)
    assert torch.allclose(h.double(), (resid.double() * norm_w.double()), rtol=1e-2, atol=1e-2)
    assert torch.allclose(ssq[:parts].sum(0).double(), (want_resid ** 2).sum(1), rtol=1e-4)
    # the consumer: scales from the parts, float32 and SwiGLU epilogues, both modes
    N2 = 320
    w2 = (torch.randn(N2, N, device=DEV) * 0.05).to(torch.bfloat16)
    normed = want_resid * torch.rsqrt((want_resid ** 2).mean(1, keepdim=True) + eps) * norm_w.double()
    want = normed @ w2.double().T
    for (swap2, bn2, ks2) in ((True, 128 if M > 64 else 64 if M > 16 else 16, 2), (False, 256, 1), (False, 128, 1)):
        if swap2 and M > 128:
            continue
        out = torch.zeros(M, N2, device=DEV)
        fast.gemm_tcgen05(h, w2, out, fast.EPI_F32, swap2, bn2, ks2, err, ssq_in=ssq[:parts], eps_in=eps, norm_size=N)
        torch.cuda.synchronize()
        assert err.item() == 0
        assert torch.allclose(out.double(), want, rtol=2e-2, atol=2e-2 * float(want.abs().max())), (swap2, bn2)
        g = want.view(M, N2 // 32, 2, 16)
        want_act = (g[:, :, 0] / (1 + torch.exp(-g[:, :, 0])) * g[:, :, 1]).reshape(M, N2 // 2)
        out2 = torch.zeros(M, N2 // 2, dtype=torch.bfloat16, device=DEV)
        fast.gemm_tcgen05(h, w2, out2, fast.EPI_SWIGLU, swap2, bn2, ks2, err, ssq_in=ssq[:parts], eps_in=eps, norm_size=N)
        torch.cuda.synchronize()
        assert torch.allclose(out2.double(), want_act, rtol=3e-2, atol=3e-2 * float(want_act.abs().max())), (swap2, bn2)


def test_gemm_tcgen05_refuses_what_it_cannot_take():
    from airun_b200.kernels import fast
    from airun_b200.kernels.ops import KernelError
    x = torch.zeros(4, 12, device=DEV, dtype=torch.bfloat16)          # K not a multiple of 8
    w = torch.zeros(16, 12, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(KernelError):
        fast.gemm_tcgen05(x, w, torch.zeros(4, 16, device=DEV), 0, True, 16, 1, _err())
    x = torch.zeros(4, 16, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(24, 16, device=DEV, dtype=torch.bfloat16)          # SwiGLU needs N % 32 == 0
    with pytest.raises(KernelError):
        fast.gemm_tcgen05(x, w, torch.zeros(4, 12, device=DEV, dtype=torch.bfloat16), 2, True, 16, 1, _err())


# ----------------------------------------------------------------------------- q/k norm + rope + cache write
@pytest.mark.parametrize("nh,nkv,hd,page,dtype", [(4, 2, 16, 4, torch.float32), (6, 3, 48, 16, torch.bfloat16),
                                                  (8, 1, 128, 8, torch.float32), (3, 3, 80, 32, torch.float32),
                                                  (8, 2, 128, 16, torch.bfloat16)])
def test_qkv_post_against_the_plain_parts(nh, nkv, hd, page, dtype):
    from airun_b200.kernels import ops
    from airun_b200.parts.rope import RotaryNeox
    torch.manual_seed(6)
    positions = [3, 17, 40, 41, 63, 0, 1, 2]                     # two requests; the first at scattered places
    req = [0, 0, 0, 0, 0, 1, 1, 1]
    T = len(positions)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd) * 2
    qw, kw = 1 + 0.5 * torch.rand(hd), 1 + 0.5 * torch.rand(hd)
    eps, theta = 1e-5, 1e6
    rope = RotaryNeox(rotary_dim=hd, theta=theta, device=DEV)
    n_pages = 40
    pool = torch.zeros(n_pages, 2, nkv, page, hd, dtype=dtype, device=DEV)
    bt = torch.full((2, 20), -1, dtype=torch.int32)
    perm = np.random.default_rng(0).permutation(n_pages)
    bt[0, :17] = torch.tensor(perm[:17].astype(np.int32))
    bt[1, :3] = torch.tensor(perm[17:20].astype(np.int32))
    q_out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    err = _err()
    kind, rdim, inv = rope.fused()
    ops.qkv_post(qkv.to(DEV), q_out, qw.to(DEV), kw.to(DEV), eps, torch.tensor(positions, dtype=torch.int32, device=DEV),
                 torch.tensor(req, dtype=torch.int32, device=DEV), kind, rdim, inv, pool, bt.to(DEV), 2, page,
                 nh, nkv, hd, err)
    assert err.item() == 0
    q = qkv[:, :nh * hd].view(T, nh, hd)
    k = qkv[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
    want_q = P.plain_rope_neox(P.plain_rmsnorm(q, qw, eps), positions, theta, hd)
    want_k = P.plain_rope_neox(P.plain_rmsnorm(k, kw, eps), positions, theta, hd)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(q_out.cpu().float().view(T, nh, hd), want_q, rtol=tol, atol=tol)
    poolc = pool.cpu().float()
    for t in range(T):
        pg, row = int(bt[req[t], positions[t] // page]), positions[t] % page
        assert torch.allclose(poolc[pg, 0, :, row], want_k[t], rtol=tol, atol=tol)
        assert torch.allclose(poolc[pg, 1, :, row], v[t].to(dtype).float(), rtol=0, atol=0)
    written = sum(1 for _ in range(T)) * 2 * nkv * hd
    assert int((poolc != 0).sum()) <= written                     # nothing else was touched
    # a block-table entry outside the pool sets the flag and writes nothing
    bad = bt.clone(); bad[1, 0] = n_pages + 3
    pool2 = torch.zeros_like(pool)
    ops.qkv_post(qkv.to(DEV), q_out, qw.to(DEV), kw.to(DEV), eps, torch.tensor(positions, dtype=torch.int32, device=DEV),
                 torch.tensor(req, dtype=torch.int32, device=DEV), kind, rdim, inv, pool2, bad.to(DEV), 2, page,
                 nh, nkv, hd, err)
    assert err.item() == 1


@pytest.mark.parametrize("hd,rdim", [(128, 128), (48, 32), (16, 16)])
def test_qkv_post_interleaved_pairing_and_rotation_positions(hd, rdim):
    """The other pairing (dims 2i, 2i + 1), a partial rotation, and rows rotated by positions that are not
    their places in the cache: keys still land at the cache positions."""
    from airun_b200.kernels import ops
    from airun_b200.parts.rope import RotaryInterleaved
    torch.manual_seed(8)
    nh, nkv, page = 4, 2, 8
    positions, rpos = [5, 6, 7, 30], [100, 3, 0, 4095]
    T = len(positions)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd)
    qw, kw = 1 + 0.5 * torch.rand(hd), 1 + 0.5 * torch.rand(hd)
    eps, theta = 1e-6, 1e4
    kind, r, inv = RotaryInterleaved(rotary_dim=rdim, theta=theta, device=DEV).fused()
    assert kind == ops.ROPE_INTERLEAVED
    pool = torch.zeros(6, 2, nkv, page, hd, device=DEV)
    bt = torch.tensor([[4, 2, 0, 5, 1]], dtype=torch.int32, device=DEV)
    q_out = torch.empty(T, nh * hd, device=DEV)
    err = _err()
    ops.qkv_post(qkv.to(DEV), q_out, qw.to(DEV), kw.to(DEV), eps, torch.tensor(positions, dtype=torch.int32, device=DEV),
                 torch.zeros(T, dtype=torch.int32, device=DEV), kind, r, inv, pool, bt, 1, page, nh, nkv, hd, err,
                 rope_positions=torch.tensor(rpos, dtype=torch.int32, device=DEV))
    assert err.item() == 0
    q = qkv[:, :nh * hd].view(T, nh, hd)
    k = qkv[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    want_q = P.plain_rope_interleaved(P.plain_rmsnorm(q, qw, eps), rpos, theta, rdim)
    want_k = P.plain_rope_interleaved(P.plain_rmsnorm(k, kw, eps), rpos, theta, rdim)
    assert torch.allclose(q_out.cpu().view(T, nh, hd), want_q, rtol=2e-5, atol=2e-5)
    for t in range(T):
        pg, row = int(bt[0, positions[t] // page]), positions[t] % page
        assert torch.allclose(pool[pg, 0, :, row].cpu(), want_k[t], rtol=2e-5, atol=2e-5)


def test_copy_pages_and_soft_cap():
    from airun_b200.kernels import ops
    torch.manual_seed(9)
    pool = torch.randn(3, 10, 2, 2, 8, 16, device=DEV).to(torch.bfloat16)      # owners, pages, K/V, heads, page, head size
    before = pool.clone()
    err = _err()
    ops.copy_pages(pool, torch.tensor([[1, 7], [4, 0], [1, 9]], dtype=torch.int32, device=DEV), err)
    torch.cuda.synchronize()
    want = before.clone()
    for s_, d_ in ((1, 7), (4, 0), (1, 9)):
        want[:, d_] = before[:, s_]
    assert torch.equal(pool, want) and err.item() == 0
    ops.copy_pages(pool, torch.tensor([[1, 10]], dtype=torch.int32, device=DEV), err)       # outside the pool: flagged, skipped
    torch.cuda.synchronize()
    assert torch.equal(pool, want) and err.item() == 1
    x = torch.randn(7, 333, device=DEV) * 20
    y = x.clone()
    ops.soft_cap(y, 30.0)
    assert torch.allclose(y.cpu(), 30.0 * torch.tanh(x.cpu().double() / 30.0).float(), rtol=1e-5, atol=1e-5)
    table = torch.randn(11, 64).to(torch.bfloat16).to(DEV)
    ids = torch.tensor([3, 10, 0], dtype=torch.int32, device=DEV)
    out = torch.empty(3, 64, device=DEV)
    ops.embed(table, ids, out, err, scale=8.0)
    assert torch.equal(out.cpu(), table.float().cpu()[[3, 10, 0]] * 8.0)


# ----------------------------------------------------------------------------- attention
def attention_case(nh, nkv, hd, page, window, lens, qlens, dtype, seed, peaked=True):
    """Requests with contexts ``lens``; the last ``qlens[i]`` tokens of each are this step's queries.
    With ``peaked`` one far key per (request, head) is made to dominate, so a kernel that loses
    it (a page's edge, a slice's edge, the window's edge) gives a visibly different row."""
    torch.manual_seed(seed)
    g = nh // nkv
    ks = [torch.randn(n, nkv, hd) for n in lens]
    vs = [torch.randn(n, nkv, hd) for n in lens]
    qs, positions, req = [], [], []
    for r, (n, ql) in enumerate(zip(lens, qlens)):
        q = torch.randn(ql, nh, hd)
        if peaked:
            for i in range(ql):
                pos = n - ql + i
                lo = max(0, pos - window + 1) if window else 0
                for h in range(nh):
                    far = lo if (h + i) % 2 == 0 else (lo + pos) // 2     # the window's first key, or a middle one
                    q[i, h] = q[i, h] * 0.3 + ks[r][far, h // g] * (6.0 / math.sqrt(hd))
        qs.append(q)
        positions += list(range(n - ql, n))
        req += [r] * ql
    scale = hd ** -0.5
    ks = [k.to(dtype).float() for k in ks]
    vs = [v.to(dtype).float() for v in vs]
    qs = [q.to(dtype).float() for q in qs]
    want = []
    for r, (n, ql) in enumerate(zip(lens, qlens)):
        # plain attention of the whole request, then the rows of this step's queries
        full_q = torch.zeros(n, nh, hd)
        full_q[n - ql:] = qs[r]
        want.append(P.plain_attention(full_q, ks[r], vs[r], list(range(n)), scale, window)[n - ql:])
    want = torch.cat(want).reshape(len(positions), nh * hd)
    pool, bt = paged_from_dense(ks, vs, page, dtype, seed=seed)
    q = torch.cat(qs).reshape(len(positions), nh * hd).to(dtype).to(DEV)
    ctx = Ctx(positions, req, len(lens), list(qlens), list(lens))
    return ctx, Cache(pool, bt, page), q, want, scale


ATT = [  # nh, nkv, hd, page, window, context lengths, query lengths
    (4, 2, 16, 4, 0, [5, 33, 70], [5, 1, 50]),            # a whole short prompt, one decoded token, a portion at 20..69
    (8, 1, 32, 8, 0, [130, 17], [2, 17]),                 # MQA, a two-token portion
    (6, 3, 48, 16, 24, [90, 25, 64], [1, 25, 40]),        # window 24, head size 48
    (4, 4, 64, 32, 0, [300], [1]),                        # a far key among hundreds
    (16, 2, 128, 16, 0, [257, 129], [1, 129]),            # page edge + 1
    (2, 1, 128, 16, 100, [1000], [1]),                    # window in a long context
    (20, 1, 16, 8, 0, [40, 9], [1, 9]),                   # more than 16 heads in a group
    (8, 2, 128, 16, 0, [700, 300, 131], [700, 45, 3]),    # long prompts: several 128-key tiles, ragged ends
    (8, 2, 128, 32, 200, [900, 260], [400, 260]),         # window across tiles, pages of 32
    (12, 4, 64, 16, 0, [513, 64], [513, 2]),              # head size 64, three heads in a group
    (5, 1, 128, 64, 0, [260], [260]),                     # a group of 5: 25 tokens per tile, rows left over
    (8, 2, 64, 24, 0, [100, 49, 75], [1, 49, 3]),         # pages of 24 tokens: no power of two, no divisor of 64
    (4, 2, 128, 24, 30, [200, 48], [1, 48]),              # the same with a window and head size 128
]


@pytest.mark.parametrize("case", ATT)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_generic(case, dtype):
    from airun_b200.kernels import ops
    nh, nkv, hd, page, window, lens, qlens = case
    ctx, cache, q, want, scale = attention_case(nh, nkv, hd, page, window, lens, qlens, dtype, seed=11)
    out = torch.empty_like(q)
    ops.attention_generic(q, out, cache.pool, cache.block_table, ctx.positions, ctx.req_of_token, ctx.num_reqs,
                          nh, nkv, hd, scale, window, ctx.err)
    assert ctx.err.item() == 0
    tol = 1e-3 if dtype == torch.float32 else 2e-2           # 1e-3: the reference's float32 attention bound
    assert torch.allclose(out.cpu().float(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("wide", [True, False])
@pytest.mark.parametrize("case", ATT)
def test_attention_tensor_core(case, wide, monkeypatch):
    """``wide``: prompts with more than 128 packed rows go to the tcgen05 kernel with two Q tiles to a CTA
    (256 rows), else all go to the one with 128 rows."""
    from airun_b200.kernels import fast
    if wide:
        monkeypatch.setattr(fast, "WIDE_MIN_CTAS", 1)
    else:
        monkeypatch.setattr(fast, "DISABLED", fast.DISABLED | {"attention_wide"})
    nh, nkv, hd, page, window, lens, qlens = case
    ctx, cache, q, want, scale = attention_case(nh, nkv, hd, page, window, lens, qlens, torch.bfloat16, seed=12)
    out = torch.full_like(q, 9.0)
    assert fast.attention_bf16(ctx, q, out, cache, nh, nkv, hd, scale, window)
    torch.cuda.synchronize()
    assert ctx.err.item() == 0
    assert torch.allclose(out.cpu().float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
def test_decode_attention_slices_agree(splits):
    """Cutting the keys into slices changes nothing beyond rounding; empty slices are harmless."""
    from airun_b200.kernels import fast
    nh, nkv, hd, page, window = 8, 2, 64, 16, 0
    lens = [1, 15, 16, 17, 100, 1000]
    ctx, cache, q, want, scale = attention_case(nh, nkv, hd, page, window, lens, [1] * len(lens), torch.bfloat16, seed=13)
    out = torch.full_like(q, 9.0)
    rows = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    for early in (False, True):                               # twice: the counters return to zero; the second time
        # the first tiles are requested before the dependency wait, as inside a captured step
        fast.attn_decode(ctx, q, out, cache, nh, nkv, hd, scale, window, rows, len(lens), splits, early=early)
        torch.cuda.synchronize()
        assert ctx.err.item() == 0
        assert torch.allclose(out.cpu().float(), want, rtol=2e-2, atol=2e-2)
        out.fill_(9.0)


def test_decode_attention_over_32768_keys():
    """One decoded token of each of five requests at positions 0, 15, 16, 4095 and 32767, one KV head, the far
    key of every head made to dominate (the first key for even heads, a middle one for odd heads): against a
    float64 softmax over all keys.  The reference checks its split attention the same way at 6,000 and 212,992
    keys (crates/airun-cli/src/selftest.rs:2748-2861)."""
    from airun_b200.kernels import fast, ops
    torch.manual_seed(31)
    nh, nkv, hd, page = 4, 1, 128, 16
    lens = [1, 16, 17, 4096, 32768]
    ks = [torch.randn(n, nkv, hd) for n in lens]
    vs = [torch.randn(n, nkv, hd) for n in lens]
    q = torch.randn(len(lens), nh, hd) * 0.3
    for r, n in enumerate(lens):
        for h in range(nh):
            far = 0 if h % 2 == 0 else (n - 1) // 2
            q[r, h] += ks[r][far, 0] * (16.0 / math.sqrt(hd))
    for dtype in (torch.bfloat16, torch.float32):
        kd = [k.to(dtype).float() for k in ks]
        vd = [v.to(dtype).float() for v in vs]
        qd = q.to(dtype).float()
        want = torch.zeros(len(lens), nh, hd, dtype=torch.float64)
        for r in range(len(lens)):
            for h in range(nh):
                sc = (kd[r][:, 0].double() @ qd[r, h].double()) * hd ** -0.5
                want[r, h] = torch.softmax(sc, 0) @ vd[r][:, 0].double()
        want = want.reshape(len(lens), nh * hd).float()
        assert float(want[-1].abs().max()) > 1.0                  # the far keys do dominate, among 32768 too
        pool, bt = paged_from_dense(kd, vd, page, dtype, seed=31)
        ctx = Ctx([n - 1 for n in lens], list(range(len(lens))), len(lens), [1] * len(lens), lens)
        cache = Cache(pool, bt, page)
        qdev = qd.reshape(len(lens), nh * hd).to(dtype).to(DEV)
        out = torch.full_like(qdev, 9.0)
        if dtype == torch.float32:
            ops.attention_generic(qdev, out, pool, bt, ctx.positions, ctx.req_of_token, ctx.num_reqs, nh, nkv, hd,
                                  hd ** -0.5, 0, ctx.err)
            torch.cuda.synchronize()
            assert ctx.err.item() == 0
            assert torch.allclose(out.cpu(), want, rtol=1e-3, atol=1e-3)
            continue
        assert fast.attention_bf16(ctx, qdev, out, cache, nh, nkv, hd, hd ** -0.5, 0)     # the slices its cost model picks
        torch.cuda.synchronize()
        assert ctx.err.item() == 0
        assert torch.allclose(out.float().cpu(), want, rtol=2e-2, atol=2e-2)
        for splits in (1, 37, 64):
            out.fill_(9.0)
            fast.attn_decode(ctx, qdev, out, cache, nh, nkv, hd, hd ** -0.5, 0, None, len(lens), splits)
            torch.cuda.synchronize()
            assert ctx.err.item() == 0
            assert torch.allclose(out.float().cpu(), want, rtol=2e-2, atol=2e-2), splits


def test_window_of_one_returns_the_value_at_its_own_place():
    from airun_b200.kernels import fast, ops
    nh, nkv, hd, page = 4, 2, 32, 8
    for dtype in (torch.float32, torch.bfloat16):
        ctx, cache, q, want, scale = attention_case(nh, nkv, hd, page, 1, [37, 50], [1, 20], dtype, seed=14, peaked=False)
        out = torch.empty_like(q)
        ops.attention_generic(q, out, cache.pool, cache.block_table, ctx.positions, ctx.req_of_token, 2,
                              nh, nkv, hd, scale, 1, ctx.err)
        assert torch.allclose(out.cpu().float(), want, rtol=1e-6, atol=1e-6)
        if dtype == torch.bfloat16:
            out2 = torch.empty_like(q)
            assert fast.attention_bf16(ctx, q, out2, cache, nh, nkv, hd, scale, 1)
            assert torch.allclose(out2.cpu().float(), want, rtol=1e-2, atol=1e-2)


def test_attention_flags_a_bad_page():
    from airun_b200.kernels import fast, ops
    nh, nkv, hd, page = 4, 2, 64, 16
    ctx, cache, q, want, scale = attention_case(nh, nkv, hd, page, 0, [40, 40], [1, 40], torch.bfloat16, seed=15)
    cache.block_table[0, 1] = cache.pool.shape[0] + 7
    out = torch.empty_like(q)
    ops.attention_generic(q, out, cache.pool, cache.block_table, ctx.positions, ctx.req_of_token, 2,
                          nh, nkv, hd, scale, 0, ctx.err)
    assert ctx.err.item() == 1
    ctx.err.zero_()
    fast.attention_bf16(ctx, q, out, cache, nh, nkv, hd, scale, 0)
    torch.cuda.synchronize()
    assert ctx.err.item() == 1


# ----------------------------------------------------------------------------- sampling
def test_sample_kernel_first_maximum_and_temperature():
    from airun_b200.kernels import ops
    torch.manual_seed(7)
    V = 151936
    logits = torch.randn(6, V)
    logits[0, 777] = logits[0, 90000] = 50.0                  # a tie: the first wins
    logits[1] = float("-inf")                                 # all -inf gives 0
    logits[2, :5] = float("nan"); logits[2, 9] = 40.0         # NaN never wins
    logits[3, V - 1] = 60.0
    picked = torch.zeros(6, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), picked)
    got = picked.cpu().tolist()
    assert got[:4] == [777, 0, 9, V - 1]
    assert got[4] == P.plain_argmax(logits[4].tolist()) and got[5] == int(torch.argmax(logits[5]))
    # temperature: the draw inverts the cumulative sum in vocabulary order at u * total
    small = torch.log(torch.tensor([[0.5, 0.25, 0.125, 0.125]] * 4))
    temp = torch.tensor([1.0, 1.0, 1.0, 0.0], device=DEV)
    u = torch.tensor([0.1, 0.6, 0.99, 0.99], device=DEV)
    out = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.sample(small.to(DEV), out, temp, u)
    assert out.cpu().tolist() == [0, 1, 3, 0]
    # a large vocabulary: the picked index brackets the target in the host's cumulative sum
    big = (torch.randn(3, 50000) * 2).to(DEV)
    temp = torch.tensor([0.8, 1.3, 0.2], device=DEV)
    u = torch.tensor([0.3, 0.77, 0.5], device=DEV)
    out = torch.zeros(3, dtype=torch.int32, device=DEV)
    ops.sample(big, out, temp, u)
    for r in range(3):
        l = big[r].cpu().double()
        p = torch.exp((l - l.max()) / float(temp[r]))
        cdf = torch.cumsum(p, 0) / p.sum()
        i = int(out[r])
        lo = float(cdf[i - 1]) if i > 0 else 0.0
        assert lo - 1e-4 <= float(u[r]) <= float(cdf[i]) + 1e-4


@pytest.mark.parametrize("V,n_cand", [(151936, 105), (300, 41), (20000, 512), (5000, 8), (37, 64)])
def test_largest_logits_kernel_against_a_sort(V, n_cand):
    """The rows' n largest logits with their ids, the largest first and equal values by ascending id, as
    ``np.lexsort`` gives them: random rows, a row of few distinct values (ties everywhere, also at the cut), a row
    with NaN and infinities, a row whose largest values all fall to one thread's share (the kernel must either list
    them or raise the row's flag), and rows picked out of order."""
    from airun_b200.kernels import ops
    rng = np.random.default_rng(V + n_cand)
    R = 6
    rows = (rng.standard_normal((R, V)) * 4).astype(np.float32)
    rows[1] = np.round(rows[1])
    rows[2, rng.integers(0, V, max(1, V // 50))] = np.nan
    rows[2, rng.integers(0, V, 3)] = np.inf
    rows[2, rng.integers(0, V, 3)] = -np.inf
    rows[3, ::1024] += 100.0                                   # one thread's share holds all the largest values
    pick = np.array([4, 1, 2, 3, 0, 1], dtype=np.int32)
    logits = torch.from_numpy(rows).to(DEV)
    ids = torch.full((len(pick) * n_cand,), -7, dtype=torch.int32, device=DEV)
    vals = torch.zeros(len(pick) * n_cand, dtype=torch.float32, device=DEV)
    flags = torch.full((len(pick),), -1, dtype=torch.int32, device=DEV)
    ops.largest_logits(logits, torch.from_numpy(pick).to(DEV), len(pick), n_cand, ids, vals, flags)
    ids, vals, flags = ids.cpu().numpy().reshape(len(pick), n_cand), vals.cpu().numpy().reshape(len(pick), n_cand), flags.cpu().numpy()
    flagged = 0
    for j, r in enumerate(pick):
        real = np.nonzero(~np.isnan(rows[r]))[0]                # NaN never wins: it is not listed at all
        order = real[np.lexsort((real, -rows[r][real]))]
        want = order[:n_cand]
        if flags[j]:                                            # the kernel cannot vouch for this list: the caller takes the row
            flagged += 1
            assert V > 4 * 1024 and n_cand > 4                  # never where a thread's share is at most what it keeps
            assert r == 3 or n_cand > 256                       # at the engine's sizes only the planted row
            continue
        got = ids[j][:len(want)]
        assert np.array_equal(got, want), (V, n_cand, r)
        assert np.array_equal(vals[j][:len(want)], rows[r][want])
        assert (ids[j][len(real):] == -1).all() and np.isneginf(vals[j][len(real):]).all()      # beyond the row's values
    if V > 4 * 1024 and n_cand > 4:
        assert flagged >= 1                                     # 149 values of one thread's share cannot all be listed


def test_sample_kernel_distribution():
    from airun_b200.kernels import ops
    probs = torch.tensor([0.4, 0.3, 0.2, 0.1])
    n = 4000
    logits = torch.log(probs).repeat(n, 1).to(DEV)
    from airun_b200.sampling.sampler import XorShift64
    rng = XorShift64(123)
    u = torch.tensor([rng.next_f32() for _ in range(n)], device=DEV)
    out = torch.zeros(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, torch.ones(n, device=DEV), u)
    counts = np.bincount(out.cpu().numpy(), minlength=4)
    chi2 = float(((counts - n * probs.numpy()) ** 2 / (n * probs.numpy())).sum())
    assert chi2 < 16.3


@pytest.mark.parametrize("R,G,S,page", [(16, 8, 1040, 16), (5, 4, 272, 16), (40, 4, 128, 32), (3, 2, 64, 8),
                                        (3, 4, 32768, 16)])
def test_shared_prefix_attention(R, G, S, page):
    """Decoded tokens whose requests begin with the same pages: the shared keys once for all of them
    (several slices), each token's own later keys by the decode kernel, one merge; against plain
    attention over each request's whole context."""
    from airun_b200.kernels import fast
    torch.manual_seed(11)
    nkv, hd = 2, 128
    nh = nkv * G
    own = [int(x) for x in torch.randint(1, 90, (R,))]
    shared_k, shared_v = torch.randn(S, nkv, hd), torch.randn(S, nkv, hd)
    ks = [torch.cat([shared_k, torch.randn(n, nkv, hd)]).to(torch.bfloat16).float() for n in own]
    vs = [torch.cat([shared_v, torch.randn(n, nkv, hd)]).to(torch.bfloat16).float() for n in own]
    lens = [S + n for n in own]
    # pages: the first S / page of every block table are the same pages
    n_shared = S // page
    blocks = [(n + page - 1) // page for n in lens]
    n_pages = n_shared + sum(b - n_shared for b in blocks) + 3
    perm = np.random.default_rng(3).permutation(n_pages)
    pool = torch.full((n_pages, 2, nkv, page, hd), 1e4)
    bt = torch.full((R, max(blocks) + 1), -1, dtype=torch.int32)
    nxt = n_shared
    for r in range(R):
        for b in range(blocks[r]):
            if b < n_shared:
                pg = int(perm[b])
            else:
                pg = int(perm[nxt]); nxt += 1
            bt[r, b] = pg
            n = min(page, lens[r] - b * page)
            pool[pg, 0, :, :n] = ks[r][b * page:b * page + n].transpose(0, 1)
            pool[pg, 1, :, :n] = vs[r][b * page:b * page + n].transpose(0, 1)
    pool, bt = pool.to(torch.bfloat16).to(DEV), bt.to(DEV)
    pos = [n - 1 for n in lens]
    ctx = Ctx(pos, list(range(R)), R, [1] * R, lens)
    q = torch.randn(R, nh, hd) * 0.3
    for r in range(R):                                   # one key dominates: a shared one (even heads), an own one (odd)
        for h in range(nh):
            far = (S // 3 + 7 * r) % S if h % 2 == 0 else S + (own[r] - 1) // 2
            q[r, h] += ks[r][far, h // G] * (16.0 / math.sqrt(hd))
    q = q.to(torch.bfloat16).float()
    want = torch.zeros(R, nh, hd, dtype=torch.float64)
    for r in range(R):                                   # softmax(q K^T / sqrt(d)) V over the request's whole context
        for h in range(nh):
            sc = (ks[r][:, h // G].double() @ q[r, h].double()) * hd ** -0.5
            want[r, h] = torch.softmax(sc, 0) @ vs[r][:, h // G].double()
    want = want.reshape(R, nh * hd)
    assert float(want.abs().max()) > 1.0
    qd = q.to(torch.bfloat16).to(DEV).view(R, nh * hd)
    out = torch.zeros_like(qd)
    cache = Cache(pool, bt, page)
    k_end = torch.tensor([S], dtype=torch.int32, device=DEV)
    for splits, slices in ((1, 3), (2, 7)):
        out.zero_()
        fast.attn_shared_prefix(ctx, qd, cache, nh, nkv, hd, hd ** -0.5, R, k_end, slices, splits)
        fast.attn_decode(ctx, qd, out, cache, nh, nkv, hd, hd ** -0.5, 0, None, R, splits,
                         k_begin_dev=k_end, extra_slices=slices)
        torch.cuda.synchronize()
        assert ctx.err.item() == 0
        assert torch.allclose(out.float().cpu(), want.float(), atol=2e-2, rtol=2e-2), (splits, slices)


@pytest.mark.parametrize("kind,dtype", [("normal", torch.bfloat16), ("normal", torch.float32), ("norm", torch.float32),
                                        ("int", torch.int32)])
def test_random_fill_is_the_same_on_the_device_and_on_the_host(kind, dtype):
    """A tensor filled by the kernel equals the host's fill of the same (seed, name) bit for bit, and
    both equal the tests' own statement of the generator."""
    from airun_b200.weights.loader import WeightSpec, random_tensors
    from helpers import plain_random_tensor
    specs = [WeightSpec("model.layers.7.mlp.up_proj.weight", (37, 1001), "compute" if dtype == torch.bfloat16 else "as_stored",
                        kind if kind != "normal" else "normal"),
             WeightSpec("x", (5,), "compute" if dtype == torch.bfloat16 else "as_stored", kind)]
    host = random_tensors(specs, 1234, "cpu", torch.bfloat16)
    dev = random_tensors(specs, 1234, "cuda:0", torch.bfloat16)
    torch.cuda.synchronize()
    for s in specs:
        h, d = host[s.name], dev[s.name].cpu()
        assert h.dtype == d.dtype == dtype and h.shape == d.shape
        assert torch.equal(h.view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                           d.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)), s.name
        if kind != "int":
            mine = plain_random_tensor(1234, s.name, s.shape, kind == "norm")
            if dtype == torch.float32 and kind == "normal":
                mine = plain_random_tensor(1234, s.name, s.shape, False).float()   # bfloat16 of the same value
                assert torch.equal(h.to(torch.bfloat16).float(), mine)
            else:
                assert torch.equal(h, mine), s.name
