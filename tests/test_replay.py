"""Trace replay against the plain implementation: the same requests whole, with the last
32 tokens one by one, in portions of changing size, and mixed with other requests in a
pool so small that pages are used again; float32 and bfloat16; three tiny configurations."""
from __future__ import annotations

import random

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from helpers import TINY, Replay, assert_close, bf16_noise, make_model_folder, random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 100], "B": [70, 40, 9, 121], "C": [90, 50, 130, 37], "D": [150, 16, 129, 45],
           "A24": [5, 17, 33, 100], "E": [41, 100, 12, 66]}
CHUNKS = [7, 2, 13, 3, 2, 24, 5, 2, 31, 4]


def ceil64(n: int) -> int:
    return (n + 63) // 64 * 64


def mixed_schedule(seqs, seed):
    """Steps for six requests (the four sequences, then the first two again under new ids),
    at most four live at a time: portions of 2..20 tokens until the last 8 tokens of a
    request, which come one by one; a live request sometimes sits a step out.
    Returns (steps, peak) where peak is the most tokens live requests hold, each rounded
    up to a multiple of 64."""
    rng = random.Random(seed)
    jobs = [(f"m{i}", seqs[i % len(seqs)]) for i in range(len(seqs) + 2)]
    done_at = {}
    pos = {}
    live = []
    waiting = list(jobs)
    steps = []
    peak = 0
    start_gap = 0
    while waiting or live:
        if waiting and len(live) < 4 and start_gap <= 0:
            rid, toks = waiting.pop(0)
            live.append((rid, toks))
            pos[rid] = 0
            start_gap = rng.choice([0, 1, 2])
        start_gap -= 1
        peak = max(peak, sum(ceil64(len(t)) for _, t in live))
        entries, end = [], []
        for rid, toks in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # sits this step out
            left = len(toks) - pos[rid]
            n = 1 if left <= 8 else min(left - 8, rng.randint(2, 20))
            entries.append(dict(id=rid, tokens=toks[pos[rid]:pos[rid] + n], want=list(range(n)),
                                first=pos[rid]))
            pos[rid] += n
            if pos[rid] == len(toks):
                end.append(rid)
                live.remove((rid, toks))
        if entries:
            steps.append((entries, end))
    return steps, peak


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: make_model_folder(name, str(root)) for name in TINY}


@pytest.fixture(scope="module")
def plain_logits(folders):
    """Logits of every sequence by the plain implementation: float32, and float32 with
    the bfloat16 path's rounding places."""
    out = {}
    for name, d in folders.items():
        cfg, W = P.read_model_folder(d)
        seqs = [random_tokens(n, cfg["vocab_size"], 1000 + i) for i, n in enumerate(LENGTHS[name])]
        out[name] = dict(
            seqs=seqs,
            float32=[P.plain_forward(cfg, W, s, torch.float32).numpy() for s in seqs],
            bfloat16=[P.plain_forward(cfg, W, s, torch.float32, round_to=torch.bfloat16).numpy() for s in seqs])
    return out


_CACHE = {}


def run_all_modes(name, dtype, folders, plain_logits, tmp_path_factory):
    key = (name, dtype)
    if key in _CACHE:
        return _CACHE[key]
    seqs = plain_logits[name]["seqs"]
    steps, peak = mixed_schedule(seqs, seed=7)
    max_tokens = max(peak, max(ceil64(len(s)) for s in seqs))
    out_dir = tmp_path_factory.mktemp(f"replay_{name}_{dtype}")
    rp = Replay(folders[name], dtype, str(out_dir), max_tokens, TINY[name]["page_size"])
    res = dict(whole=[], tail=[], chunks=[], mixed={})
    try:
        for i, s in enumerate(seqs):                      # whole
            res["whole"].append(rp.step([dict(id=f"w{i}", tokens=s, want=list(range(len(s))))], end=[f"w{i}"]))
        for i, s in enumerate(seqs):                      # most in one step, the last 32 one by one
            head = max(1, len(s) - 32)
            rows = [rp.step([dict(id=f"t{i}", tokens=s[:head], want=list(range(head)))])]
            for j in range(head, len(s)):
                rows.append(rp.step([dict(id=f"t{i}", tokens=[s[j]], want=[0])],
                                    end=[f"t{i}"] if j == len(s) - 1 else []))
            if head == len(s):
                rp.step([], end=[f"t{i}"])
            res["tail"].append(np.concatenate(rows))
        for i, s in enumerate(seqs):                      # portions of changing size, down to two
            rows, p, k = [], 0, i
            while p < len(s):
                n = min(CHUNKS[k % len(CHUNKS)], len(s) - p)
                k += 1
                rows.append(rp.step([dict(id=f"c{i}", tokens=s[p:p + n], want=list(range(n)))],
                                    end=[f"c{i}"] if p + n == len(s) else []))
                p += n
            res["chunks"].append(np.concatenate(rows))
        got = {}
        for entries, end in steps:                        # mixed, pages used again
            logits = rp.step([dict(id=e["id"], tokens=e["tokens"], want=e["want"]) for e in entries], end=end)
            r = 0
            for e in entries:
                n = len(e["tokens"])
                got.setdefault(e["id"], []).append(logits[r:r + n])
                r += n
        res["mixed"] = {rid: np.concatenate(v) for rid, v in got.items()}
        res["exit"] = rp.close()
    finally:
        if rp.proc.poll() is None:
            rp.proc.kill()
    _CACHE[key] = res
    return res


CASES = [(n, d) for n in TINY for d in ("float32", "bfloat16")]


def noise_of(plain_logits, name, i):
    return bf16_noise(plain_logits[name]["bfloat16"][i], plain_logits[name]["float32"][i])


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole(name, dtype, folders, plain_logits, tmp_path_factory):
    res = run_all_modes(name, dtype, folders, plain_logits, tmp_path_factory)
    assert res["exit"] == 0
    for i, want in enumerate(plain_logits[name][dtype]):
        assert_close(res["whole"][i], want, dtype, f"{name} {dtype} whole seq {i}", noise_of(plain_logits, name, i))


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_one_by_one(name, dtype, folders, plain_logits, tmp_path_factory):
    res = run_all_modes(name, dtype, folders, plain_logits, tmp_path_factory)
    for i, want in enumerate(plain_logits[name][dtype]):
        assert_close(res["tail"][i], want, dtype, f"{name} {dtype} tail seq {i}", noise_of(plain_logits, name, i))


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions(name, dtype, folders, plain_logits, tmp_path_factory):
    res = run_all_modes(name, dtype, folders, plain_logits, tmp_path_factory)
    for i, want in enumerate(plain_logits[name][dtype]):
        assert_close(res["chunks"][i], want, dtype, f"{name} {dtype} portions seq {i}", noise_of(plain_logits, name, i))


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_pages_reused(name, dtype, folders, plain_logits, tmp_path_factory):
    res = run_all_modes(name, dtype, folders, plain_logits, tmp_path_factory)
    wants = plain_logits[name][dtype]
    assert len(res["mixed"]) == len(wants) + 2
    for rid, got in res["mixed"].items():
        i = int(rid[1:]) % len(wants)
        assert_close(got, wants[i], dtype, f"{name} {dtype} mixed request {rid}", noise_of(plain_logits, name, i))


@pytest.mark.parametrize("name,dtype", CASES)
def test_modes_agree(name, dtype, folders, plain_logits, tmp_path_factory):
    """The logits at a position do not depend on how the tokens were cut into steps."""
    res = run_all_modes(name, dtype, folders, plain_logits, tmp_path_factory)
    for i in range(len(plain_logits[name]["seqs"])):
        assert_close(res["tail"][i], res["whole"][i], dtype, f"{name} {dtype} tail vs whole seq {i}", noise_of(plain_logits, name, i))
        assert_close(res["chunks"][i], res["whole"][i], dtype, f"{name} {dtype} portions vs whole seq {i}", noise_of(plain_logits, name, i))
