"""Each part of a layer alone, built with its own sizes and constants and stepped through
the real step context and cache, against the plain function of the same part."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda"


class Harness:
    """A cache manager, storage and step context around ONE part."""

    def __init__(self, cache_spec, dtype, page_size=8, pages=24, reqs=3):
        from airun_b200.cache import CacheManager, CacheStorage
        from airun_b200.engine.step import StepRunner

        class Stub:                      # the runner only asks its model for the device
            device = torch.device(DEV)

        self.manager = CacheManager([cache_spec], [None], page_size, pages, reqs)
        self.storage = CacheStorage(self.manager, dtype, DEV)
        self.runner = StepRunner(Stub(), self.manager, self.storage, 256, reqs, pages * page_size)

    def context(self, entries):
        from airun_b200.engine.step import StepEntry
        es = [StepEntry(r, [0] * n, ()) for r, n in entries]
        for r, _ in entries:
            if r not in self.manager.requests:
                self.manager.add_request(r)
        self.runner.reserve(es)
        ctx, _ = self.runner.build_context(es)
        ctx.ws = ctx.ws_pair[0]
        ctx.ws.reset()
        return ctx

    def commit(self, entries):
        for r, n in entries:
            self.manager.commit(r, n)


def weights_for(part, seed, dtype):
    from airun_b200.weights.loader import load_tensors, random_tensors, DictSource
    t = random_tensors(part.weight_specs(), seed, "cpu")
    for n in t:
        if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
            t[n] = t[n] * 2.0
    loaded = load_tensors(part.weight_specs(), DictSource(t), dtype, DEV)
    part.load_weights(dict(loaded))
    return {k: v.float() for k, v in t.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from airun_b200.parts.base import make_part
    norm = make_part("norm", "rmsnorm", prefix="n", size=72, eps=2e-5, dtype=dtype, device=DEV)
    W = weights_for(norm, 1, dtype)
    x = torch.randn(9, 72)
    d = torch.randn(9, 72)
    xd, out = x.to(DEV), torch.empty(9, 72, dtype=dtype, device=DEV)
    norm.forward(None, xd, out, delta=d.to(DEV))
    want = P.plain_rmsnorm(x + d, W["n.weight"], 2e-5)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(out.cpu().float(), want, rtol=tol, atol=tol)
    assert torch.allclose(xd.cpu(), x + d, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from airun_b200.parts.base import make_part
    H, I = 40, 112
    ffn = make_part("feed_forward", "swiglu", prefix="f", hidden_size=H, intermediate_size=I, dtype=dtype, device=DEV)
    W = weights_for(ffn, 2, dtype)
    from airun_b200.parts.base import PagedKVSpec
    hz = Harness(PagedKVSpec(1, 16, 0), dtype)
    ctx = hz.context([("a", 11)])
    h = (torch.randn(11, H) * 3).to(dtype)
    out = ffn.forward(ctx, h.to(DEV))
    want = P.plain_swiglu_ffn(h.float(), W["f.gate_proj.weight"], W["f.up_proj.weight"], W["f.down_proj.weight"],
                              round_to=None if dtype == torch.float32 else torch.bfloat16)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert out.dtype == torch.float32 and torch.allclose(out.cpu(), want, rtol=tol, atol=tol * float(want.abs().max()))


@pytest.mark.parametrize("dtype,nh,nkv,hd,window", [(torch.float32, 6, 2, 16, 0), (torch.bfloat16, 4, 4, 32, 0),
                                                     (torch.float32, 8, 1, 48, 10), (torch.bfloat16, 4, 2, 64, 12)])
def test_attention_part_over_steps(dtype, nh, nkv, hd, window):
    """The mixer alone: a prompt in two portions, then single tokens, next to another request;
    its output equals the plain attention layer over the whole sequence."""
    from airun_b200.parts.base import make_part
    H, eps, theta = 56, 1e-5, 50000.0
    att = make_part("mixer", "gqa_attention", prefix="a", hidden_size=H, num_heads=nh, num_kv_heads=nkv,
                    head_dim=hd, scale=hd ** -0.5, window=window, qk_norm=True, qk_norm_eps=eps,
                    position="rotary_neox", position_args=dict(rotary_dim=hd, theta=theta), dtype=dtype, device=DEV)
    W = weights_for(att, 3, dtype)
    Wp = {k.replace("a.", "x.self_attn."): v for k, v in W.items()}
    c = dict(nh=nh, nkv=nkv, hd=hd, eps=eps, theta=theta)
    rt = None if dtype == torch.float32 else torch.bfloat16
    torch.manual_seed(4)
    hs = {r: (torch.randn(n, H) * 2).to(dtype) for r, n in (("a", 29), ("b", 13))}
    want = {r: P.plain_attention_layer(h.float(), Wp, "x.self_attn", c, list(range(h.shape[0])), window, rt)[0]
            for r, h in hs.items()}
    hz = Harness(att.cache_spec(), dtype, page_size=8, pages=16, reqs=3)
    got = {"a": [], "b": []}
    done = {"a": 0, "b": 0}
    plan = [[("a", 17)], [("a", 2), ("b", 13)], [("a", 1)], [("a", 1)], [("a", 8)]]
    for step in plan:
        ctx = hz.context(step)
        h = torch.cat([hs[r][done[r]:done[r] + n] for r, n in step]).to(DEV)
        out = att.forward(ctx, h, ctx.caches[0]).cpu()
        assert ctx.err.item() == 0
        o = 0
        for r, n in step:
            got[r].append(out[o:o + n]); o += n; done[r] += n
        hz.commit(step)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for r in got:
        g = torch.cat(got[r])
        assert torch.allclose(g, want[r], rtol=tol, atol=tol * float(want[r].abs().max())), r


def test_block_embedding_and_head_parts():
    from airun_b200.parts.base import PagedKVSpec, make_part
    from airun_b200.parts.embedding import LMHead, TokenEmbedding
    dtype = torch.float32
    H, V = 48, 77
    emb = TokenEmbedding("e.weight", V, H)
    head = LMHead("h.weight", V, H, tied_to=emb)
    W = weights_for(emb, 5, dtype)
    head.load_weights({})
    hz = Harness(PagedKVSpec(1, 16, 0), dtype)
    ctx = hz.context([("a", 6)])
    ids = torch.tensor([3, 76, 0, 5, 5, 41], dtype=torch.int32, device=DEV)
    x = torch.empty(6, H, device=DEV)
    emb.forward(ctx, ids, x)
    assert torch.equal(x.cpu(), P.plain_embedding(W["e.weight"], ids.tolist(), torch.float32))
    logits = torch.empty(6, V, device=DEV)
    head.forward(ctx, x, logits)
    assert torch.allclose(logits.cpu(), x.cpu() @ W["e.weight"].T, rtol=1e-5, atol=1e-6)
    # a whole block: norm -> attention -> add -> norm -> feed-forward, delta returned for the next norm
    nh, nkv, hd, I, eps = 4, 2, 16, 96, 1e-6
    norm_args = dict(size=H, eps=eps)
    blk = make_part("arrangement", "pre_norm",
                    norm1=make_part("norm", "rmsnorm", prefix="b.input_layernorm", dtype=dtype, device=DEV, **norm_args),
                    mixer=make_part("mixer", "gqa_attention", prefix="b.self_attn", hidden_size=H, num_heads=nh,
                                    num_kv_heads=nkv, head_dim=hd, scale=hd ** -0.5, qk_norm_eps=eps,
                                    position_args=dict(rotary_dim=hd, theta=1e4), dtype=dtype, device=DEV),
                    norm2=make_part("norm", "rmsnorm", prefix="b.post_attention_layernorm", dtype=dtype, device=DEV, **norm_args),
                    ffn=make_part("feed_forward", "swiglu", prefix="b.mlp", hidden_size=H, intermediate_size=I,
                                  dtype=dtype, device=DEV), dtype=dtype)
    Wb = weights_for(blk, 6, dtype)
    hz2 = Harness(blk.cache_spec(), dtype)
    ctx = hz2.context([("a", 10)])
    x0, d0 = torch.randn(10, H), torch.randn(10, H) * 0.1
    xd = x0.to(DEV)
    delta = blk.forward(ctx, xd, d0.to(DEV), ctx.caches[0]).cpu()
    c = dict(nh=nh, nkv=nkv, hd=hd, eps=eps, theta=1e4)
    xr = x0 + d0
    a, _ = P.plain_attention_layer(P.plain_rmsnorm(xr, Wb["b.input_layernorm.weight"], eps), Wb, "b.self_attn", c,
                                   list(range(10)), 0)
    xr = xr + a
    f = P.plain_swiglu_ffn(P.plain_rmsnorm(xr, Wb["b.post_attention_layernorm.weight"], eps),
                           Wb["b.mlp.gate_proj.weight"], Wb["b.mlp.up_proj.weight"], Wb["b.mlp.down_proj.weight"])
    assert torch.allclose(xd.cpu(), xr, rtol=1e-5, atol=1e-5)            # the residual holds x + d0 + attention
    assert torch.allclose(delta, f, rtol=1e-4, atol=1e-5)                # the feed-forward's delta is still pending
