"""A plain, slow implementation of the dense Qwen3 decoder for the tests.

Whole sequences, no cache, no batching, one function for each part, torch on
the CPU.  It shares no code with the package: it reads config.json with the
json module and model.safetensors with the ``safetensors`` library, and every
function is written from the formulas the reference computes (file:line below,
paths within the reference project).

The reference's model code is Rust calling CUDA kernels and has no CPU forward
pass; neither cargo nor rustc is installed here, so it can be neither imported
nor compiled on the CPU.  Its CUDA kernels, however, compile unmodified for a
B200 behind their C entry points, and this file is pinned on them: the outputs
of the reference's own kernels for 28 cases (every part, and two whole tiny
models run in the order its runtime calls the kernels) are stored in
``tests/golden/reference_kernel_outputs.npz`` by
``tests/golden/make_reference_kernel_outputs.py`` (run once on a B200), and
``tests/test_reference_golden.py`` compares the functions below with them on
any machine; ``tests/test_reference_kernels.py`` runs both sides on a GPU.
Head sizes below 32 (not accepted by the reference's kernels) rest on the
formulas alone.

``round_to`` emulates where the engine's bfloat16 path rounds activations
(normed hidden states, q, cached k and v, the attention output, the SwiGLU
product); with ``round_to=None`` nothing is rounded.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# ----------------------------------------------------------------------------- loading
def read_model_folder(model_dir: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights = load_file(os.path.join(model_dir, "model.safetensors"))
    return cfg, weights


def config_values(cfg: dict) -> dict:
    """Defaults as crates/airun-cli/src/convert.rs:48-91 applies them."""
    nh = cfg["num_attention_heads"]
    L = cfg["num_hidden_layers"]
    c = dict(L=L, H=cfg["hidden_size"], nh=nh,
             nkv=cfg.get("num_key_value_heads") or nh,
             hd=cfg.get("head_dim") or cfg["hidden_size"] // nh,
             I=cfg["intermediate_size"], V=cfg["vocab_size"],
             eps=cfg.get("rms_norm_eps") or 1e-6,
             theta=cfg.get("rope_theta") or 10000.0,
             tied=bool(cfg.get("tie_word_embeddings", False)))
    windows = [0] * L
    if cfg.get("use_sliding_window"):
        w = cfg["sliding_window"]
        if cfg.get("layer_types") is not None:
            windows = [w if t == "sliding_attention" else 0 for t in cfg["layer_types"]]
        else:
            first = cfg.get("max_window_layers", L)
            windows = [w if i >= first else 0 for i in range(L)]
    c["windows"] = windows
    return c


def _r(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(x.dtype)


# ----------------------------------------------------------------------------- parts
def plain_embedding(table: torch.Tensor, ids: Sequence[int], dtype) -> torch.Tensor:
    """x[t] = E[token[t]], no scaling (crates/airun-cuda/kernels/ops.cu:227-252)."""
    return torch.stack([table[int(i)].to(dtype) for i in ids])


def plain_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """out = x * rsqrt(sum(x^2)/n + eps) * w, eps inside the root
    (crates/airun-cuda/kernels/ops.cu:12-41)."""
    n = x.shape[-1]
    inv = torch.rsqrt((x * x).sum(-1, keepdim=True) / n + eps)
    return x * inv * w.to(x.dtype)


def plain_rope_neox(x: torch.Tensor, positions: Sequence[int], theta: float, rotary_dim: int) -> torch.Tensor:
    """x: [T, heads, hd].  Pair i couples dims i and i + r/2; angle = pos * theta^(-2i/r);
    x'_i = x_i cos - x_{i+r/2} sin, x'_{i+r/2} = x_i sin + x_{i+r/2} cos; dims >= r untouched
    (crates/airun-cuda/kernels/ops.cu:158-184, crates/airun-cuda/kernels/airun.cuh:147-163).
    The frequency is formed in double precision and rounded once to float32; the angle is
    the float32 product position * frequency (for a float64 run everything stays double)."""
    T, heads, hd = x.shape
    half = rotary_dim // 2
    out = x.clone()
    fdt = torch.float32 if x.dtype == torch.float32 else torch.float64
    pos = torch.tensor([float(p) for p in positions], dtype=fdt)
    for i in range(half):
        inv_freq = torch.tensor(float(theta) ** (-2.0 * i / rotary_dim), dtype=torch.float64).to(fdt)
        ang = pos * inv_freq                                  # [T], one rounding in float32
        c, s = torch.cos(ang).to(x.dtype)[:, None], torch.sin(ang).to(x.dtype)[:, None]
        x0, x1 = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = x0 * c - x1 * s
        out[:, :, i + half] = x0 * s + x1 * c
    return out


def plain_rope_interleaved(x: torch.Tensor, positions: Sequence[int], theta: float, rotary_dim: int) -> torch.Tensor:
    """The same angles with the older pairing: pair i couples dims 2i and 2i + 1
    (crates/airun-cuda/kernels/ops.cu:154-157, :176-183).  Not used by the dense Qwen3 decoder; here for
    parts that ask the fused prologue for it."""
    T, heads, hd = x.shape
    out = x.clone()
    fdt = torch.float32 if x.dtype == torch.float32 else torch.float64
    pos = torch.tensor([float(p) for p in positions], dtype=fdt)
    for i in range(rotary_dim // 2):
        inv_freq = torch.tensor(float(theta) ** (-2.0 * i / rotary_dim), dtype=torch.float64).to(fdt)
        ang = pos * inv_freq
        c, s = torch.cos(ang).to(x.dtype)[:, None], torch.sin(ang).to(x.dtype)[:, None]
        x0, x1 = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = x0 * c - x1 * s
        out[:, :, 2 * i + 1] = x0 * s + x1 * c
    return out


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: Sequence[int],
                    scale: float, window: int) -> torch.Tensor:
    """q: [T, nh, hd]; k, v: [T, nkv, hd] of one whole sequence.  Head h reads KV head
    h // (nh // nkv); s_j = scale * q.K_j; key j visible iff j <= pos and (window == 0 or
    pos - j < window); softmax over the visible keys; o = sum_j p_j V_j
    (crates/airun-cuda/kernels/ops.cu:524-645, mask rule :573-576)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.zeros_like(q)
    for t in range(T):
        pos = positions[t]
        keys = [j for j in range(T) if positions[j] <= pos and (window == 0 or pos - positions[j] < window)]
        for h in range(nh):
            kh = h // g
            s = (k[keys, kh] @ q[t, h]) * scale               # one score per visible key
            p = torch.softmax(s, dim=0)
            out[t, h] = p @ v[keys, kh]
    return out


def plain_swiglu_ffn(h: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor,
                     round_to=None) -> torch.Tensor:
    """g = Wg h, u = Wu h, a = g / (1 + exp(-g)) * u, out = Wd a
    (crates/airun-cuda/kernels/ops.cu:191-200, crates/airun-core/src/runtime.rs:688-747)."""
    g = h @ wg.T
    u = h @ wu.T
    a = g / (1.0 + torch.exp(-g)) * u
    return _r(a, round_to) @ wd.T


def plain_attention_layer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, c: dict,
                          positions: Sequence[int], window: int, round_to=None,
                          kv_override=None):
    """Projections without bias, per-head q/k RMSNorm (shared weight, the layer eps) BEFORE
    the rotation, rotation of q and k, attention, output projection
    (crates/airun-core/src/runtime.rs:3848-4120, crates/airun-cuda/kernels/ops.cu:422-501).
    Returns (output, (k, v)) so that another entry can read this one's keys and values."""
    dt = h.dtype
    T = h.shape[0]
    nh, nkv, hd = c["nh"], c["nkv"], c["hd"]
    q = (h @ W[f"{p}.q_proj.weight"].to(dt).T).view(T, nh, hd)
    q = plain_rmsnorm(q, W[f"{p}.q_norm.weight"], c["eps"])
    q = _r(plain_rope_neox(q, positions, c["theta"], hd), round_to)
    if kv_override is None:
        k = (h @ W[f"{p}.k_proj.weight"].to(dt).T).view(T, nkv, hd)
        v = (h @ W[f"{p}.v_proj.weight"].to(dt).T).view(T, nkv, hd)
        k = plain_rmsnorm(k, W[f"{p}.k_norm.weight"], c["eps"])
        k = _r(plain_rope_neox(k, positions, c["theta"], hd), round_to)
        v = _r(v, round_to)
    else:
        k, v = kv_override
    o = plain_attention(q, k, v, positions, hd ** -0.5, window)
    o = _r(o, round_to).reshape(T, nh * hd)
    return o @ W[f"{p}.o_proj.weight"].to(dt).T, (k, v)


# ----------------------------------------------------------------------------- whole model
def plain_forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: Sequence[int],
                  dtype=torch.float32, round_to: Optional[torch.dtype] = None,
                  order: Optional[List[Tuple[int, Optional[int]]]] = None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence at positions 0..T-1.

    Pre-norm residual blocks: x += attn(norm(x)); x += ffn(norm(x)); final norm; head
    (crates/airun-core/src/runtime.rs:3507-3602, :2601-2655); a tied head is the embedding
    table (crates/airun-core/src/model.rs:1068-1074).  ``order`` is a list of
    (layer, cache_from) entries; default: every layer once, in turn."""
    c = config_values(cfg)
    T = len(tokens)
    positions = list(range(T))
    x = plain_embedding(W["model.embed_tokens.weight"], tokens, dtype)
    order = order if order is not None else [(i, None) for i in range(c["L"])]
    kvs = []
    for (l, src) in order:
        p = f"model.layers.{l}"
        h = _r(plain_rmsnorm(x, W[f"{p}.input_layernorm.weight"], c["eps"]), round_to)
        a, kv = plain_attention_layer(h, W, f"{p}.self_attn", c, positions, c["windows"][l], round_to,
                                      kv_override=None if src is None else kvs[src])
        kvs.append(kv)
        x = x + a
        h = _r(plain_rmsnorm(x, W[f"{p}.post_attention_layernorm.weight"], c["eps"]), round_to)
        x = x + plain_swiglu_ffn(h, W[f"{p}.mlp.gate_proj.weight"].to(dtype), W[f"{p}.mlp.up_proj.weight"].to(dtype),
                                 W[f"{p}.mlp.down_proj.weight"].to(dtype), round_to)
    h = _r(plain_rmsnorm(x, W["model.norm.weight"], c["eps"]), round_to)
    head = W["model.embed_tokens.weight"] if c["tied"] else W["lm_head.weight"]
    return h @ head.to(dtype).T


# ----------------------------------------------------------------------------- sampling
def plain_argmax(logits: Sequence[float]) -> int:
    """First maximum, strictly greater replaces, NaN never wins, all -inf gives 0
    (crates/airun-core/src/sample.rs:639-649)."""
    best, best_val = 0, -math.inf
    for i, l in enumerate(logits):
        if l > best_val:
            best, best_val = i, l
    return best


class PlainRng:
    """xorshift64 with state seed|1; u = (x >> 40) / 2^24 (crates/airun-core/src/sample.rs:778-798)."""

    def __init__(self, seed: int):
        self.s = (seed | 1) & 0xFFFFFFFFFFFFFFFF

    def next_u64(self) -> int:
        x = self.s
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        self.s = x
        return x

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)


def plain_greedy_generate(cfg: dict, W: Dict[str, torch.Tensor], prompt: Sequence[int], n_new: int,
                          dtype=torch.float32) -> List[int]:
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        logits = plain_forward(cfg, W, toks, dtype)[-1]
        t = plain_argmax(logits.tolist())
        out.append(t)
        toks.append(t)
    return out
