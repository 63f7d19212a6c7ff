"""Long decoding, and the first tokens of a sequence, through the trace replay."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from helpers import TINY, Replay, assert_close, bf16_noise, make_model_folder, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("long_models")
    return {n: make_model_folder(n, str(root)) for n in ("B", "C")}


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("B", "bfloat16"), ("C", "float32"), ("C", "bfloat16")])
def test_long_decoding(name, dtype, folders, tmp_path):
    """A short prompt, then 230 tokens one by one (B) or 300 (C: far beyond its window of 24,
    so pages behind the window are given back and used again while decoding)."""
    cfg, W = P.read_model_folder(folders[name])
    n_prompt, n_decode = (9, 230) if name == "B" else (20, 300)
    seq = random_tokens(n_prompt + n_decode, cfg["vocab_size"], 77)
    exact = P.plain_forward(cfg, W, seq, torch.float32).numpy()
    want = exact if dtype == "float32" else P.plain_forward(cfg, W, seq, torch.float32, round_to=torch.bfloat16).numpy()
    noise = bf16_noise(want, exact)
    # C's window groups need few pages once the window has passed; the pool is sized for the whole sequence
    rp = Replay(folders[name], dtype, str(tmp_path), (len(seq) + 63) // 64 * 64, TINY[name]["page_size"])
    try:
        rows = [rp.step([dict(id="r", tokens=seq[:n_prompt], want=list(range(n_prompt)))])]
        for t in seq[n_prompt:]:
            rows.append(rp.step([dict(id="r", tokens=[t], want=[0])]))
        rp.step([], end=["r"])
        assert rp.close() == 0
    finally:
        if rp.proc.poll() is None:
            rp.proc.kill()
    assert_close(np.concatenate(rows), want, dtype, f"{name} {dtype} long decode", noise)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(dtype, folders, tmp_path):
    """Positions 0, 1, 2, ...: a request that starts with one token, requests of one and two
    tokens, and a request whose first step brings two tokens."""
    name = "B"
    cfg, W = P.read_model_folder(folders[name])
    seq = random_tokens(12, cfg["vocab_size"], 78)
    exact = P.plain_forward(cfg, W, seq, torch.float32).numpy()
    want = exact if dtype == "float32" else P.plain_forward(cfg, W, seq, torch.float32, round_to=torch.bfloat16).numpy()
    noise = bf16_noise(want, exact)
    rp = Replay(folders[name], dtype, str(tmp_path), 256, TINY[name]["page_size"])
    try:
        one = [rp.step([dict(id="a", tokens=[t], want=[0])]) for t in seq]          # from position 0, one by one
        rp.step([], end=["a"])
        single = rp.step([dict(id="b", tokens=seq[:1], want=[0])], end=["b"])         # a request of one token
        pair = rp.step([dict(id="c", tokens=seq[:2], want=[0, 1])], end=["c"])        # and of two
        two = [rp.step([dict(id="d", tokens=seq[:2], want=[0, 1])]), rp.step([dict(id="d", tokens=seq[2:4], want=[0, 1])]),
               rp.step([dict(id="d", tokens=seq[4:], want=list(range(8)))], end=["d"])]
        assert rp.close() == 0
    finally:
        if rp.proc.poll() is None:
            rp.proc.kill()
    assert_close(np.concatenate(one), want, dtype, "one by one from position 0", noise)
    assert_close(single, want[:1], dtype, "request of one token", noise[:1])
    assert_close(pair, want[:2], dtype, "request of two tokens", noise[:2])
    assert_close(np.concatenate(two), want, dtype, "two tokens at a time, then the rest", noise)
