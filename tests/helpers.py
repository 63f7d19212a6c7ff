"""Shared by the tests: the tiny configurations, model folders, replay driver, tolerances."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Tiny configurations that differ in every size and option.
TINY = {
    # 2 layers, GQA 2x, head_dim 16, tied head, page 16
    "A": dict(cfg=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       intermediate_size=128, max_position_embeddings=128, rms_norm_eps=1e-6,
                       rope_theta=10000.0, tie_word_embeddings=True),
              page_size=16, seed=11),
    # 3 layers, MQA (one KV head, 8 query heads), heads*head_dim != hidden, untied head, page 8
    "B": dict(cfg=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=384, hidden_size=96,
                       num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1, head_dim=32,
                       intermediate_size=224, max_position_embeddings=256, rms_norm_eps=1e-5,
                       rope_theta=1000000.0, tie_word_embeddings=False),
              page_size=8, seed=22),
    # 4 layers, head_dim 48, odd vocabulary, two layers with a window of 24 (two cache groups), page 16
    "C": dict(cfg=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=300, hidden_size=80,
                       num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
                       intermediate_size=176, max_position_embeddings=512, rms_norm_eps=3e-6,
                       rope_theta=500000.0, tie_word_embeddings=False, use_sliding_window=True,
                       sliding_window=24,
                       layer_types=["full_attention", "sliding_attention", "full_attention", "sliding_attention"]),
              page_size=16, seed=33),
    # head size 128, the size of the benchmark's model: prompt portions on the tcgen05 attention, single tokens
    # on the TMA decode attention, inside the engine; 2 layers, untied head
    "D": dict(cfg=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=512, hidden_size=256,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                       intermediate_size=384, max_position_embeddings=512, rms_norm_eps=1e-6,
                       rope_theta=1000000.0, tie_word_embeddings=False),
              page_size=16, seed=44),
}
# Sizes the tensor-core kernels refuse, so that the plain kernels run inside the bfloat16 engine: a width of 100
# (not a multiple of 8: no TMA rows), an intermediate size of 180 (no fused SwiGLU tile), one layer, as many KV
# heads as heads (groups of 1), head size 80, a prime vocabulary, tied head, page 32
TINY["E"] = dict(cfg=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=257, hidden_size=100,
                          num_hidden_layers=1, num_attention_heads=3, num_key_value_heads=3, head_dim=80,
                          intermediate_size=180, max_position_embeddings=256, rms_norm_eps=2e-5,
                          rope_theta=20000.0, tie_word_embeddings=True),
                 page_size=32, seed=55)
# A again with pages of 24 tokens: a page size that is no power of two and does not divide 64
TINY["A24"] = dict(TINY["A"], page_size=24)


def make_model_folder(name: str, root: str, sharpen: float = 2.5) -> str:
    """Writes the tiny model ``name`` under ``root``.  The per-head q/k norm weights are
    scaled by ``sharpen`` so that attention is peaked: a wrong or missing key then moves
    the logits far more than rounding does."""
    from airun_b200.config import Qwen3Config
    from airun_b200.engine.model import DecoderModel
    from airun_b200.weights.loader import random_tensors
    from airun_b200.weights.safetensors_io import write_safetensors
    spec = TINY[name]
    cfg = Qwen3Config.from_dict(spec["cfg"])
    model = DecoderModel(cfg, torch.float32, "cpu")
    tensors = random_tensors(model.weight_specs(), spec["seed"], "cpu", torch.bfloat16)
    for n in tensors:
        if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
            tensors[n] = tensors[n] * sharpen
    d = os.path.join(root, f"tiny_{name}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d


def _plain_mix(z):
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def plain_random_tensor(seed: int, name: str, shape, norm: bool) -> torch.Tensor:
    """The tests' own statement of the seeded random weights (the package's is weights/loader.py and
    csrc/elementwise.cu): element i of tensor ``name`` is a function of (seed, name, i).  The key is
    the FNV-1a hash of the name mixed with the seed; three hashes of the counter give twelve 16-bit
    fields whose sum, centred and divided by 65536, is z; a matrix is bfloat16(0.02 z), a norm weight
    float32(1 + 0.1 z)."""
    M = (1 << 64) - 1
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & M
    k = (h ^ ((seed * 0x9E3779B97F4A7C15) & M)) & M
    k = ((k ^ (k >> 30)) * 0xBF58476D1CE4E5B9) & M
    k = ((k ^ (k >> 27)) * 0x94D049BB133111EB) & M
    k ^= k >> 31
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        c = np.arange(n, dtype=np.uint64) * np.uint64(3)
        total = np.zeros(n, dtype=np.int64)
        for j in range(3):
            hj = _plain_mix(np.uint64(k) + (c + np.uint64(j)) * np.uint64(0x9E3779B97F4A7C15))
            for f in range(4):
                total += ((hj >> np.uint64(16 * f)) & np.uint64(0xFFFF)).astype(np.int64)
    z = (total - 393210).astype(np.float32) / np.float32(65536.0)
    if norm:
        return torch.from_numpy(np.float32(1.0) + z * np.float32(0.1)).view(*shape)
    return torch.from_numpy(z * np.float32(0.02)).view(*shape).to(torch.bfloat16)


_PLAIN_WEIGHTS: Dict[str, Dict[str, torch.Tensor]] = {}


def plain_random_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """The weights ``Engine.from_config(config, seed)`` fills a dense Qwen3 model with, by their HF names."""
    key = json.dumps(cfg, sort_keys=True) + f"#{seed}"
    if key not in _PLAIN_WEIGHTS:
        _PLAIN_WEIGHTS.clear()                      # one model's weights at a time
        _PLAIN_WEIGHTS[key] = _plain_random_weights(cfg, seed)
    return _PLAIN_WEIGHTS[key]


def _plain_random_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    H, nh = cfg["hidden_size"], cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    hd = cfg.get("head_dim") or H // nh
    I, V = cfg["intermediate_size"], cfg["vocab_size"]
    W = {}

    def mat(name, r, c):
        W[name] = plain_random_tensor(seed, name, (r, c), False)

    def vec(name, n):
        W[name] = plain_random_tensor(seed, name, (n,), True)

    mat("model.embed_tokens.weight", V, H)
    vec("model.norm.weight", H)
    if not cfg.get("tie_word_embeddings", False):
        mat("lm_head.weight", V, H)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}"
        vec(f"{p}.input_layernorm.weight", H)
        vec(f"{p}.post_attention_layernorm.weight", H)
        mat(f"{p}.self_attn.q_proj.weight", nh * hd, H)
        mat(f"{p}.self_attn.k_proj.weight", nkv * hd, H)
        mat(f"{p}.self_attn.v_proj.weight", nkv * hd, H)
        mat(f"{p}.self_attn.o_proj.weight", H, nh * hd)
        vec(f"{p}.self_attn.q_norm.weight", hd)
        vec(f"{p}.self_attn.k_norm.weight", hd)
        mat(f"{p}.mlp.gate_proj.weight", I, H)
        mat(f"{p}.mlp.up_proj.weight", I, H)
        mat(f"{p}.mlp.down_proj.weight", H, I)
    return W


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = np.random.default_rng(seed)
    return [int(t) for t in g.integers(0, vocab, size=n)]


class Replay:
    """Drives bin/trace_run as a child process, one step at a time."""

    def __init__(self, model_dir: str, dtype: str, out_dir: str, max_tokens: int, page_size: int = 16,
                 env: Optional[dict] = None):
        self.out_dir = out_dir
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
               "--out", out_dir, "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
        self.step_no = 0
        self.vocab = None

    def step(self, entries: Sequence[dict], end: Sequence[str] = ()) -> Optional[np.ndarray]:
        """entries: [{"id", "tokens", "want"}].  Returns logits [wanted, vocab] or None."""
        rec = {"step": self.step_no, "entries": list(entries), "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {self.step_no}":
            rest = self.proc.stdout.read()
            raise RuntimeError(f"trace_run did not finish step {self.step_no}: {line!r} {rest!r} "
                               f"(exit {self.proc.poll()})")
        n_want = sum(len(e.get("want", ())) for e in entries)
        out = None
        if n_want:
            raw = np.fromfile(os.path.join(self.out_dir, f"{self.step_no}.f32"), dtype="<f4")
            out = raw.reshape(n_want, -1)
        self.step_no += 1
        return out

    def close(self) -> int:
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        return rc


def tolerance(dtype: str):
    """(rtol on the row's largest |logit|, floor) for float32: sums in another order and
    rsqrt / exp / sincos within a few ulp."""
    assert dtype == "float32"
    return (2e-4, 2e-5)


def bf16_noise(plain_rounded: np.ndarray, plain_exact: np.ndarray) -> np.ndarray:
    """How far bfloat16 rounding of the activations alone moves the logits of each position of a
    sequence: per row, the largest difference between the plain implementation with the bfloat16
    path's rounding places and the plain implementation without rounding, [T, 1].  The engine's
    bfloat16 logits of a row are held to the rounded plain logits within that row's own noise
    (times two: the engine's sums run in another order and a last-place flip of an activation
    moves the result as rounding itself does) plus a small floor; an early row, whose noise is
    small, is not held to a late row's."""
    return np.abs(plain_rounded - plain_exact).max(axis=-1, keepdims=True)


def assert_close(got: np.ndarray, want: np.ndarray, dtype: str, what: str, noise: float = None) -> None:
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - want)
    if dtype == "float32":
        rtol, floor = tolerance(dtype)
        bound = rtol * np.abs(want).max(axis=-1, keepdims=True) + floor
    else:
        assert noise is not None, "bfloat16 comparisons need the sequence's rounding noise"
        noise = np.asarray(noise, dtype=np.float32)
        if noise.ndim == 0:
            noise = np.full((got.shape[0], 1), float(noise), dtype=np.float32)
        assert noise.shape == (got.shape[0], 1), f"{what}: noise rows {noise.shape} for {got.shape[0]} logit rows"
        # a row's own noise can be accidentally small; no row is held tighter than a quarter of the median row's
        bound = 2.0 * np.maximum(noise, 0.25 * np.median(noise)) + 1e-3
    if not (err <= bound).all():
        r, c = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{what}: row {r} col {c}: got {got[r, c]:.6f} want {want[r, c]:.6f} "
                             f"(err {err[r, c]:.3e}, bound {bound[r, 0]:.3e}); first bad row "
                             f"{int(np.argmax((err > bound).any(axis=1)))}")
