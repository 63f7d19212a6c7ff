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
}


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


def bf16_noise(plain_rounded: np.ndarray, plain_exact: np.ndarray) -> float:
    """How far bfloat16 rounding of the activations alone moves the logits of a sequence:
    the largest difference between the plain implementation with the bfloat16 path's
    rounding places and the plain implementation without rounding.  The engine's bfloat16
    logits are held to the rounded plain logits within this much (plus a small floor):
    it may differ in the order of sums and in last-place flips, which move the result as
    rounding itself does, but not more."""
    return float(np.abs(plain_rounded - plain_exact).max())


def assert_close(got: np.ndarray, want: np.ndarray, dtype: str, what: str, noise: float = None) -> None:
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - want)
    if dtype == "float32":
        rtol, floor = tolerance(dtype)
        bound = rtol * np.abs(want).max(axis=-1, keepdims=True) + floor
    else:
        assert noise is not None, "bfloat16 comparisons need the sequence's rounding noise"
        bound = np.full((got.shape[0], 1), noise + 1e-3, dtype=np.float32)
    if not (err <= bound).all():
        r, c = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{what}: row {r} col {c}: got {got[r, c]:.6f} want {want[r, c]:.6f} "
                             f"(err {err[r, c]:.3e}, bound {bound[r, 0]:.3e}); first bad row "
                             f"{int(np.argmax((err > bound).any(axis=1)))}")
