"""The plain implementation checked against itself: each part in float32 against float64
and against hand-worked cases (no GPU)."""
import math

import pytest
import torch

import plain_qwen3 as P
from helpers import TINY, make_model_folder, random_tokens


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    out = P.plain_rmsnorm(x, w, 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]]))
    assert float(P.plain_rmsnorm(torch.zeros(1, 4), torch.ones(4), 1e-6).abs().sum()) == 0.0


def test_rope_pairs_and_position_zero():
    x = torch.randn(3, 2, 8, dtype=torch.float64)
    assert torch.equal(P.plain_rope_neox(x, [0, 0, 0], 10000.0, 8), x)           # angle 0 leaves x alone
    y = P.plain_rope_neox(x, [5, 6, 7], 10000.0, 4)                               # partial: dims >= 4 untouched
    assert torch.equal(y[..., 4:], x[..., 4:])
    # pair i couples dims i and i + r/2 and is a rotation by pos * theta^(-2i/r)
    for i in range(2):
        ang = 5 * 10000.0 ** (-2 * i / 4)
        assert float(y[0, 0, i]) == pytest.approx(float(x[0, 0, i]) * math.cos(ang) - float(x[0, 0, i + 2]) * math.sin(ang))
        assert float(y[0, 0, i + 2]) == pytest.approx(float(x[0, 0, i]) * math.sin(ang) + float(x[0, 0, i + 2]) * math.cos(ang))
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # relative property: the score of rotated q and k depends on the distance only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    s1 = (P.plain_rope_neox(q, [9], 1e6, 8) * P.plain_rope_neox(k, [4], 1e6, 8)).sum()
    s2 = (P.plain_rope_neox(q, [105], 1e6, 8) * P.plain_rope_neox(k, [100], 1e6, 8)).sum()
    assert float(s1) == pytest.approx(float(s2), abs=1e-9)


def test_attention_mask_window_and_groups():
    torch.manual_seed(0)
    T, nh, nkv, hd = 6, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, dtype=torch.float64) for n in (nh, nkv, nkv))
    pos = list(range(T))
    o = P.plain_attention(q, k, v, pos, hd ** -0.5, 0)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 3], v[0, 1])   # first token sees itself only
    one = P.plain_attention(q, k, v, pos, hd ** -0.5, 1)                            # window 1: V at its own place
    for t in range(T):
        assert torch.allclose(one[t, 1], v[t, 0]) and torch.allclose(one[t, 2], v[t, 1])
    w3 = P.plain_attention(q, k, v, pos, hd ** -0.5, 3)
    s = (k[3:6, 0] @ q[5, 0]) * hd ** -0.5
    assert torch.allclose(w3[5, 0], torch.softmax(s, 0) @ v[3:6, 0])
    big = q.clone()
    big[5, 2] = 50 * k[1, 1]                                                        # one far key dominates
    assert torch.allclose(P.plain_attention(big, k, v, pos, 1.0, 0)[5, 2], v[1, 1], atol=1e-6)


def test_swiglu_by_hand():
    h = torch.tensor([[1.0, -2.0]])
    wg, wu, wd = torch.tensor([[1.0, 0.0]]), torch.tensor([[0.0, 1.0]]), torch.tensor([[2.0], [3.0]])
    a = (1.0 / (1.0 + math.exp(-1.0))) * -2.0
    assert torch.allclose(P.plain_swiglu_ffn(h, wg, wu, wd), torch.tensor([[2 * a, 3 * a]]))


@pytest.mark.parametrize("name", list(TINY))
def test_float32_agrees_with_float64(name, tmp_path):
    d = make_model_folder(name, str(tmp_path))
    cfg, W = P.read_model_folder(d)
    toks = random_tokens(40, cfg["vocab_size"], 3)
    a = P.plain_forward(cfg, W, toks, torch.float32)
    b = P.plain_forward(cfg, W, toks, torch.float64)
    assert float((a.double() - b).abs().max()) < 2e-5 * float(b.abs().max()) + 1e-6
    # a prefix gives the same logits: the model is causal
    c = P.plain_forward(cfg, W, toks[:17], torch.float64)
    assert torch.allclose(c, b[:17], atol=1e-10)


def test_window_changes_only_far_positions(tmp_path):
    d = make_model_folder("C", str(tmp_path))
    cfg, W = P.read_model_folder(d)
    toks = random_tokens(60, cfg["vocab_size"], 4)
    full_cfg = dict(cfg, use_sliding_window=False)
    a = P.plain_forward(cfg, W, toks, torch.float64)
    b = P.plain_forward(full_cfg, W, toks, torch.float64)
    assert torch.allclose(a[:24], b[:24], atol=1e-12)          # within the window nothing is hidden yet
    assert float((a[24:] - b[24:]).abs().max()) > 1e-4         # beyond it the window shows


def test_shared_cache_entry_and_repeated_layer(tmp_path):
    d = make_model_folder("A", str(tmp_path))
    cfg, W = P.read_model_folder(d)
    toks = random_tokens(12, cfg["vocab_size"], 5)
    base = P.plain_forward(cfg, W, toks, torch.float64)
    same = P.plain_forward(cfg, W, toks, torch.float64, order=[(0, None), (1, None)])
    assert torch.equal(base, same)
    twice = P.plain_forward(cfg, W, toks, torch.float64, order=[(0, None), (1, None), (1, 1)])
    assert float((twice - base).abs().max()) > 1e-6
