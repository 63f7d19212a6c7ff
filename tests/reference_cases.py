"""Cases that pin the plain implementation (tests/plain_qwen3.py) on the reference's own kernels.

Each case makes its inputs from a seed, computes the expected values with the plain
functions on the CPU (``plain``), and computes the same on a GPU with the reference's
kernels through their C entry points (``reference``; baseline/reference_kernels.py).
Shapes, positions and bounds are the reference's own where it states them: the attention
shapes (8 heads / 2 KV heads / 64, 16 / 2 / 128), the scattered positions 40, 55, 70 and
the 50-token portion at 20..69 with their 1e-3 / 3e-3 bounds
(crates/airun-cli/src/selftest.rs:2300-2316, :2863-2876), the fused prologue's case (8 / 2 /
128, rotary base 1e6, positions 3, 17, 40, 41, 63, norm weights 1 + 0.5 u; :2374-2426), the
argmax cases (:2328-2357), the rmsnorm bound of 1e-4 relative (:886).

The same cases serve twice: ``tests/test_reference_kernels.py`` runs both sides on a GPU;
``tests/golden/make_reference_kernel_outputs.py`` stores the reference side's outputs, which
``tests/test_reference_golden.py`` compares with the plain side on any machine.

The reference refuses head sizes that are not a multiple of 32 (ops.cu:2496, :2522), so the
tiny configuration with head size 16 has no case here and rests on the formulas alone.
"""
from __future__ import annotations

import math
import os
import sys
from typing import Callable, Dict, List

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import plain_qwen3 as P                                   # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rk():
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_kernels
    return reference_kernels


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to("cuda:0")
    return t if dtype is None else t.to(dtype)


def _f16(a: np.ndarray) -> np.ndarray:
    return a.astype(np.float16).astype(np.float32)


class Case:
    def __init__(self, name: str, make: Callable[[], dict], plain: Callable[[dict], Dict[str, np.ndarray]],
                 reference: Callable[[dict], Dict[str, np.ndarray]], atol: float, rtol: float = 0.0):
        self.name, self.make, self.plain, self.reference, self.atol, self.rtol = name, make, plain, reference, atol, rtol

    def check(self, got: Dict[str, np.ndarray], want: Dict[str, np.ndarray]) -> None:
        assert set(got) == set(want), f"{self.name}: outputs {sorted(got)} vs {sorted(want)}"
        for k in want:
            g, w = np.asarray(got[k]), np.asarray(want[k])
            assert g.shape == w.shape, f"{self.name}.{k}: shape {g.shape} vs {w.shape}"
            if w.dtype.kind in "iu":
                assert (g == w).all(), f"{self.name}.{k}: {g.tolist()} vs {w.tolist()}"
                continue
            assert np.isfinite(g).all(), f"{self.name}.{k}: non-finite values"
            err = np.abs(g.astype(np.float64) - w.astype(np.float64))
            bound = self.atol + self.rtol * np.abs(w)
            if not (err <= bound).all():
                i = np.unravel_index(np.argmax(err - bound), err.shape)
                raise AssertionError(f"{self.name}.{k}{list(i)}: reference kernel {g[i]:.7g}, plain {w[i]:.7g} "
                                     f"(err {err[i]:.3e}, bound {float(np.broadcast_to(bound, err.shape)[i]):.3e})")


# ----------------------------------------------------------------------------- norms
def _norm_case(n: int, rows: int, eps: float, seed: int) -> Case:
    def make():
        g = np.random.default_rng(seed)
        return dict(x=g.standard_normal((rows, n)).astype(np.float32) * 3.0,
                    b=g.standard_normal((rows, n)).astype(np.float32),
                    w=(1.0 + 0.1 * g.standard_normal(n)).astype(np.float32))

    def plain(d):
        x, b, w = (torch.from_numpy(d[k]) for k in "xbw")
        s = x + b
        return dict(norm=P.plain_rmsnorm(x, w, eps).numpy(), sum=s.numpy(), add_norm=P.plain_rmsnorm(s, w, eps).numpy())

    def reference(d):
        rk = _rk()
        x, b, w = _dev(d["x"]), _dev(d["b"]), _dev(d["w"])
        out = torch.empty_like(x)
        rk.rmsnorm(out, x, w, n, rows, eps)
        out2 = torch.empty_like(x)
        x2 = x.clone()
        rk.add_rmsnorm(out2, x2, b, w, n, rows, eps)
        torch.cuda.synchronize()
        return dict(norm=out.cpu().numpy(), sum=x2.cpu().numpy(), add_norm=out2.cpu().numpy())

    return Case(f"rmsnorm_n{n}", make, plain, reference, atol=2e-6, rtol=1e-4)


# ----------------------------------------------------------------------------- q/k norm + rotation + cache write
def _prologue_case(nh: int, nkv: int, hd: int, positions: List[int], theta: float, eps: float, seed: int,
                   interleaved: bool = False) -> Case:
    max_seq = 64
    T = len(positions)
    rope = P.plain_rope_interleaved if interleaved else P.plain_rope_neox

    def make():
        g = np.random.default_rng(seed)
        f = lambda *s: (2.0 * g.random(s) - 1.0).astype(np.float32)
        return dict(q=f(T, nh, hd), k=f(T, nkv, hd), v=f(T, nkv, hd),
                    qn=(1.0 + 0.5 * g.random(hd)).astype(np.float32), kn=(1.0 + 0.5 * g.random(hd)).astype(np.float32))

    def plain(d):
        q, k, v, qn, kn = (torch.from_numpy(d[n]) for n in ("q", "k", "v", "qn", "kn"))
        qo = rope(P.plain_rmsnorm(q, qn, eps), positions, theta, hd)
        ko = rope(P.plain_rmsnorm(k, kn, eps), positions, theta, hd)
        return dict(q=qo.numpy(), k_rows=_f16(ko.numpy()), v_rows=_f16(v.numpy()))

    def reference(d):
        rk = _rk()
        q, k, v, qn, kn = (_dev(d[n]) for n in ("q", "k", "v", "qn", "kn"))
        kc = torch.zeros(nkv, max_seq, hd, dtype=torch.float16, device="cuda:0")
        vc = torch.zeros_like(kc)
        pos = _dev(np.asarray(positions, dtype=np.int32))
        rk.qk_norm_rope_store(q, k, v, qn, kn, kc, vc, pos, T, nh, nkv, hd, max_seq, eps, hd, theta,
                              interleaved=interleaved)
        torch.cuda.synchronize()
        rows = torch.tensor(positions, device="cuda:0")
        untouched = torch.ones(max_seq, dtype=torch.bool, device="cuda:0")
        untouched[rows] = False
        assert float(kc[:, untouched].abs().max()) == 0.0 and float(vc[:, untouched].abs().max()) == 0.0, \
            "the reference kernel wrote cache rows of other positions"
        return dict(q=q.cpu().numpy(), k_rows=kc[:, rows].permute(1, 0, 2).float().cpu().numpy(),
                    v_rows=vc[:, rows].permute(1, 0, 2).float().cpu().numpy())

    # float16 storage of values up to ~2: half an ulp is 5e-4; the rotation's sincosf and powf are accurate
    return Case(f"qk_norm_rope_store_{nh}_{nkv}_{hd}" + ("_interleaved" if interleaved else ""), make, plain, reference,
                atol=1.2e-3, rtol=0.0)


def _rope_case(hd: int, rotary: int, theta: float, seed: int) -> Case:
    """The rotation alone in float32 (no float16 storage in the way): pairs, angle, untouched dims."""
    T, heads = 6, 3
    positions = [0, 1, 7, 100, 4095, 32767]

    def make():
        g = np.random.default_rng(seed)
        return dict(x=g.standard_normal((T, heads, hd)).astype(np.float32))

    def plain(d):
        return dict(x=P.plain_rope_neox(torch.from_numpy(d["x"]), positions, theta, rotary).numpy())

    def reference(d):
        rk = _rk()
        x = _dev(d["x"])
        rk.rope(x, _dev(np.asarray(positions, dtype=np.int32)), T, heads, hd, rotary, theta)
        torch.cuda.synchronize()
        return dict(x=x.cpu().numpy())

    # the reference forms the frequency with powf in float32, the plain code in double rounded once: at
    # position 32767 a relative 1e-7 of the angle is 3e-3 rad
    return Case(f"rope_hd{hd}_r{rotary}", make, plain, reference, atol=2e-2, rtol=0.0)


# ----------------------------------------------------------------------------- attention
def _attention_case(nh: int, nkv: int, hd: int, positions: List[int], window: int, seed: int, label: str,
                    keep: List[int] = None, splits: int = 0) -> Case:
    max_seq = 96
    T = len(positions)
    keep = list(range(T)) if keep is None else keep
    tol = 3e-3 if T >= 16 else 1e-3

    def make():
        g = np.random.default_rng(seed)
        f = lambda *s: (2.0 * g.random(s) - 1.0).astype(np.float32)
        return dict(q=f(T, nh, hd), k=_f16(f(nkv, max_seq, hd)), v=_f16(f(nkv, max_seq, hd)))

    def plain(d):
        # the plain attention takes one whole sequence: queries at every position, of which the case's are read
        n = max(positions) + 1
        qf = torch.zeros(n, nh, hd)
        qf[positions] = torch.from_numpy(d["q"])
        k = torch.from_numpy(d["k"])[:, :n].permute(1, 0, 2).contiguous()
        v = torch.from_numpy(d["v"])[:, :n].permute(1, 0, 2).contiguous()
        o = P.plain_attention(qf, k, v, list(range(n)), hd ** -0.5, window)
        return dict(out=o[positions][keep].numpy())

    def reference(d):
        rk = _rk()
        q = _dev(d["q"])
        kc, vc = _dev(d["k"], torch.float16), _dev(d["v"], torch.float16)
        pos = _dev(np.asarray(positions, dtype=np.int32))
        out = torch.zeros_like(q)
        if splits:
            partial = torch.zeros(nh * splits * (hd + 2), device="cuda:0")
            for t in range(T):
                rk.attention_split(out[t:t + 1], partial, q[t:t + 1], kc, vc, pos[t:t + 1], nh, nkv, hd, max_seq,
                                   hd ** -0.5, window, splits)
        else:
            rk.attention(out, q, kc, vc, pos, T, nh, nkv, hd, max_seq, hd ** -0.5, window, max(positions) + 1)
        torch.cuda.synchronize()
        return dict(out=out[keep].cpu().numpy())

    return Case(f"attention_{label}", make, plain, reference, atol=tol)


# ----------------------------------------------------------------------------- activation, argmax, embedding, products
def _swiglu_case() -> Case:
    def make():
        g = np.random.default_rng(5)
        gate = np.concatenate([g.standard_normal(500) * 4.0, [0.0, -30.0, 30.0, 1e-4]]).astype(np.float32)
        return dict(gate=gate, up=g.standard_normal(gate.shape[0]).astype(np.float32))

    def plain(d):
        g, u = torch.from_numpy(d["gate"]), torch.from_numpy(d["up"])
        eye = torch.eye(1)
        # the activation of plain_swiglu_ffn with 1 x 1 identity products around it
        a = torch.stack([P.plain_swiglu_ffn(torch.ones(1, 1), g[i].view(1, 1), u[i].view(1, 1), eye)[0, 0]
                         for i in range(g.shape[0])])
        return dict(a=a.numpy())

    def reference(d):
        rk = _rk()
        g, u = _dev(d["gate"]), _dev(d["up"])
        rk.swiglu(g, u, g.shape[0])
        torch.cuda.synchronize()
        return dict(a=g.cpu().numpy())

    return Case("swiglu", make, plain, reference, atol=1e-5, rtol=1e-4)      # __expf under fast math


def _argmax_case() -> Case:
    def make():
        g = np.random.default_rng(0xA76)
        f = lambda n: (2.0 * g.random(n) - 1.0).astype(np.float32)
        tie = f(100_000)
        tie[[777, 50_001, 99_999]] = 5.0
        nan = f(4097)
        nan[10], nan[11] = np.nan, 3.0
        last = f(151_936)
        last[-1] = 9.0
        first = f(70_000)
        first[0] = 9.0
        rows = [f(151_936), tie, nan, np.full(300, -np.inf, dtype=np.float32), np.asarray([-1.0], dtype=np.float32),
                last, first]
        return {f"row{i}": r for i, r in enumerate(rows)}

    def plain(d):
        return dict(picks=np.asarray([P.plain_argmax(d[f"row{i}"].tolist()) for i in range(len(d))], dtype=np.int32))

    def reference(d):
        rk = _rk()
        out = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        scratch = torch.zeros(256, dtype=torch.int32, device="cuda:0")
        picks = []
        for i in range(len(d)):
            x = _dev(d[f"row{i}"])
            rk.argmax(x, x.shape[0], out, scratch)
            picks.append(int(out.cpu()[0]))
        return dict(picks=np.asarray(picks, dtype=np.int32))

    return Case("argmax", make, plain, reference, atol=0.0)


def _embed_case() -> Case:
    V, H = 50, 64

    def make():
        g = np.random.default_rng(9)
        table = torch.from_numpy(g.standard_normal((V, H)).astype(np.float32)).to(torch.bfloat16)
        return dict(table=table.float().numpy(), ids=np.asarray([0, 49, 7, 7, 23], dtype=np.int32))

    def plain(d):
        return dict(x=P.plain_embedding(torch.from_numpy(d["table"]).to(torch.bfloat16), d["ids"].tolist(), torch.float32).numpy())

    def reference(d):
        rk = _rk()
        table = _dev(d["table"], torch.bfloat16)
        ids = _dev(d["ids"])
        out = torch.zeros(ids.shape[0], H, device="cuda:0")
        rk.embed(out, table, ids, ids.shape[0], H, V)
        torch.cuda.synchronize()
        return dict(x=out.cpu().numpy())

    return Case("embed", make, plain, reference, atol=0.0)


def _matvec_case(n_rows: int, k: int, n_tokens: int, seed: int) -> Case:
    """y[t] = W x[t] with W [rows, k] row-major in bfloat16: what every projection is (ops.rs:290-293)."""
    def make():
        g = np.random.default_rng(seed)
        w = torch.from_numpy((0.05 * g.standard_normal((n_rows, k))).astype(np.float32)).to(torch.bfloat16)
        return dict(w=w.float().numpy(), x=g.standard_normal((n_tokens, k)).astype(np.float32))

    def plain(d):
        return dict(y=(torch.from_numpy(d["x"]).double() @ torch.from_numpy(d["w"]).double().T).float().numpy())

    def reference(d):
        rk = _rk()
        w, x = _dev(d["w"], torch.bfloat16), _dev(d["x"])
        y = torch.zeros(n_tokens, n_rows, device="cuda:0")
        rk.matvec(w, x, y, k, n_rows, n_tokens)
        torch.cuda.synchronize()
        return dict(y=y.cpu().numpy())

    # 64 tokens and more go to the wmma kernel, which rounds x to float16 (matmul.cu:545-579)
    return Case(f"matvec_{n_rows}x{k}_t{n_tokens}", make, plain, reference,
                atol=(4e-3 if n_tokens >= 64 else 2e-5) * math.sqrt(k / 256), rtol=1e-4)


def _glu_case() -> Case:
    rows, k = 96, 256

    def make():
        g = np.random.default_rng(12)
        mk = lambda: torch.from_numpy((0.1 * g.standard_normal((rows, k))).astype(np.float32)).to(torch.bfloat16).float().numpy()
        return dict(wg=mk(), wu=mk(), x=g.standard_normal((1, k)).astype(np.float32))

    def plain(d):
        wg, wu, x = (torch.from_numpy(d[n]) for n in ("wg", "wu", "x"))
        return dict(a=P.plain_swiglu_ffn(x, wg, wu, torch.eye(rows)).numpy())

    def reference(d):
        rk = _rk()
        wg, wu, x = _dev(d["wg"], torch.bfloat16), _dev(d["wu"], torch.bfloat16), _dev(d["x"])
        y = torch.zeros(1, rows, device="cuda:0")
        rk.matvec_glu(wg, wu, x, y, k, rows)
        torch.cuda.synchronize()
        return dict(a=y.cpu().numpy())

    return Case("matvec_glu", make, plain, reference, atol=2e-5, rtol=2e-4)


# ----------------------------------------------------------------------------- a whole model on the reference's kernels
WHOLE = {
    # multi-query, head size 32 (the generic attention kernel), heads x head size != width, untied head
    "mqa32": dict(num_hidden_layers=3, hidden_size=96, num_attention_heads=8, num_key_value_heads=1, head_dim=32,
                  intermediate_size=224, vocab_size=384, rms_norm_eps=1e-5, rope_theta=1e6, tie_word_embeddings=False),
    # grouped, head size 64 (the flash kernel from 16 tokens on, the grouped split kernel for single tokens), tied head
    "gqa64": dict(num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                  intermediate_size=256, vocab_size=320, rms_norm_eps=1e-6, rope_theta=1e4, tie_word_embeddings=True),
}


def whole_model_weights(cfg: dict, seed: int, sharpen: float = 2.5) -> Dict[str, torch.Tensor]:
    """Random weights by the HF names: matrices N(0, 0.05) in bfloat16, norm vectors 1 + N(0, 0.1) in float32,
    the q/k norm weights scaled so that attention is peaked and a wrong key or pairing shows."""
    g = torch.Generator().manual_seed(seed)
    H, nh, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    I, V = cfg["intermediate_size"], cfg["vocab_size"]
    mat = lambda r, c: (0.05 * torch.randn(r, c, generator=g)).to(torch.bfloat16)
    vec = lambda n, s=1.0: ((1.0 + 0.1 * torch.randn(n, generator=g)) * s).float()
    W = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": vec(H)}
    if not cfg["tie_word_embeddings"]:
        W["lm_head.weight"] = mat(V, H)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}"
        W[f"{p}.input_layernorm.weight"] = vec(H)
        W[f"{p}.post_attention_layernorm.weight"] = vec(H)
        W[f"{p}.self_attn.q_proj.weight"] = mat(nh * hd, H)
        W[f"{p}.self_attn.k_proj.weight"] = mat(nkv * hd, H)
        W[f"{p}.self_attn.v_proj.weight"] = mat(nkv * hd, H)
        W[f"{p}.self_attn.o_proj.weight"] = mat(H, nh * hd)
        W[f"{p}.self_attn.q_norm.weight"] = vec(hd, sharpen)
        W[f"{p}.self_attn.k_norm.weight"] = vec(hd, sharpen)
        W[f"{p}.mlp.gate_proj.weight"] = mat(I, H)
        W[f"{p}.mlp.up_proj.weight"] = mat(I, H)
        W[f"{p}.mlp.down_proj.weight"] = mat(H, I)
    return W


def _whole_case(name: str, seed: int, T: int = 24, tail: int = 5) -> Case:
    """A whole prompt in one pass (every row's logits), then ``tail`` more tokens one by one, through the
    reference's kernels in its runtime's order, against plain_forward.  The reference keeps K and V in
    float16 and, from 16 tokens on, rounds Q and the probabilities to float16 too; the bound is how far
    float16 rounding of the activations moves the plain implementation's logits."""
    cfg = WHOLE[name]

    def make():
        g = np.random.default_rng(seed)
        return dict(tokens=g.integers(0, cfg["vocab_size"], size=T + tail).astype(np.int32))

    def plain(d):
        W = whole_model_weights(cfg, seed)
        return dict(logits=P.plain_forward(cfg, W, d["tokens"].tolist()).numpy())

    def reference(d):
        rk = _rk()
        W = {k: v.to("cuda:0") for k, v in whole_model_weights(cfg, seed).items()}
        dec = rk.ReferenceDecoder(cfg, W, ctx=64, slots=1, max_batch=64)
        toks = d["tokens"].tolist()
        rows = [dec.forward(0, toks[:T], all_logits=True)]
        for t in toks[T:]:
            rows.append(dec.forward(0, [t])[None].clone())
        torch.cuda.synchronize()
        return dict(logits=torch.cat(rows).cpu().numpy())

    c = Case(f"whole_model_{name}", make, plain, reference, atol=0.0)

    def check(got, want, _self=c):
        d = make()
        W = whole_model_weights(cfg, seed)
        rounded = P.plain_forward(cfg, W, d["tokens"].tolist(), round_to=torch.float16).numpy()
        noise = np.abs(rounded - want["logits"]).max(axis=-1, keepdims=True)
        g, w = got["logits"], want["logits"]
        assert g.shape == w.shape and np.isfinite(g).all()
        err = np.abs(g - w)
        bound = 2.0 * noise + 2e-4 * np.abs(w).max(axis=-1, keepdims=True) + 1e-4
        if not (err <= bound).all():
            r = int(np.argmax((err > bound).any(axis=1)))
            raise AssertionError(f"{_self.name}: first bad row {r}: err {err[r].max():.3e}, bound {bound[r, 0]:.3e}, "
                                 f"largest logit {np.abs(w[r]).max():.3f}")
        assert (g.argmax(-1) == w.argmax(-1)).mean() > 0.9
    c.check = check
    return c


def all_cases() -> List[Case]:
    few, chunk = [40, 55, 70], list(range(20, 70))
    edge = [0, 1, 15, 16, 17, 31, 32, 48, 49]
    return [
        _norm_case(96, 5, 1e-5, 1), _norm_case(2080, 2, 1e-6, 2), _norm_case(100, 2, 3e-6, 3),
        _prologue_case(8, 2, 128, [3, 17, 40, 41, 63], 1e6, 1e-6, 4),
        _prologue_case(8, 1, 32, [0, 1, 2, 31, 62], 1e6, 1e-5, 5),
        _prologue_case(4, 2, 64, [5, 6, 7, 8, 9, 10], 1e4, 1e-6, 6),
        _prologue_case(4, 2, 64, [0, 9, 33, 63], 1e4, 1e-6, 9, interleaved=True),
        _rope_case(128, 128, 1e6, 7), _rope_case(64, 32, 1e4, 8),
        _attention_case(8, 2, 64, few, 0, 10, "8_2_64_few"),
        _attention_case(16, 2, 128, few, 0, 11, "16_2_128_few"),
        _attention_case(8, 1, 32, few, 0, 12, "8_1_32_few"),
        _attention_case(8, 2, 64, chunk, 0, 13, "8_2_64_portion", keep=edge),
        _attention_case(16, 2, 128, chunk, 0, 14, "16_2_128_portion", keep=edge),
        _attention_case(8, 2, 64, few, 24, 15, "8_2_64_few_window24"),
        _attention_case(8, 2, 64, chunk, 24, 16, "8_2_64_portion_window24", keep=edge),
        _attention_case(8, 2, 64, few, 0, 17, "8_2_64_split16", splits=16),
        _attention_case(16, 2, 128, few, 24, 18, "16_2_128_split4_window24", splits=4),
        _swiglu_case(), _argmax_case(), _embed_case(),
        _matvec_case(100, 256, 1, 20), _matvec_case(96, 512, 8, 21), _matvec_case(128, 256, 64, 22),
        _matvec_case(40, 96, 5, 23), _glu_case(),
        _whole_case("mqa32", 31), _whole_case("gqa64", 32),
    ]
