"""Sampling: parameters with the reference's names, meanings and defaults, the
host chain, and the choice between the device kernel and the host chain.

Chain order, as the reference's (crates/airun-core/src/sample.rs:1-13, pick at
:348-486): logit bias -> repetition / presence / frequency penalties ->
top-n-sigma -> [temperature <= 0: first argmax] -> top-k -> softmax at
temperature -> typical -> min-p -> top-p -> draw.  Every filter keeps at least
one candidate.  The draw walks the candidates in descending probability with
``target = u * total`` (sample.rs:478-485); ``u`` comes from xorshift64 seeded
with ``seed | 1``, ``u = (x >> 40) / 2^24`` (sample.rs:778-798); seed 0 means
"pick one from the clock" (sample.rs:233-242).

Not built: grammar constraints, DRY, XTC, dynamic temperature, mirostat.

A request whose parameters reduce to "argmax of the raw logits" (the
reference's ``is_pure_greedy``, sample.rs:292-298) or to a plain temperature
draw is sampled by the device kernel, which walks the cumulative sum in
vocabulary order; anything else copies the row's logits to the host and runs
this chain.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np


@dataclass
class SamplingParams:
    temperature: float = 0.8        # 0 means greedy
    top_k: int = 40                 # 0 disables
    top_p: float = 0.95             # 1.0 disables
    min_p: float = 0.05             # 0 disables
    typical_p: float = 1.0          # 1.0 disables
    top_n_sigma: float = 0.0        # <= 0 disables
    repeat_penalty: float = 1.1     # 1.0 disables
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repeat_last_n: int = 64
    logit_bias: Tuple[Tuple[int, float], ...] = ()
    seed: int = 0

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, typical_p=1.0, top_n_sigma=0.0,
                   repeat_penalty=1.0, presence_penalty=0.0, frequency_penalty=0.0, repeat_last_n=0)

    @classmethod
    def temperature_only(cls, temperature: float, seed: int = 0) -> "SamplingParams":
        p = cls.greedy()
        p.temperature, p.seed = float(temperature), int(seed)
        return p

    @property
    def penalizing(self) -> bool:
        return (self.repeat_penalty != 1.0 or self.presence_penalty != 0.0
                or self.frequency_penalty != 0.0) and self.repeat_last_n > 0

    @property
    def changes_logits(self) -> bool:
        return bool(self.logit_bias) or self.penalizing or self.top_n_sigma > 0.0

    @property
    def is_pure_greedy(self) -> bool:
        return self.temperature <= 0.0 and not self.logit_bias and not self.penalizing

    @property
    def device_ok(self) -> bool:
        """True when the device kernel alone gives this request's draw."""
        if self.is_pure_greedy:
            return True
        return (self.temperature > 0.0 and not self.changes_logits and self.top_k == 0
                and self.top_p >= 1.0 and self.min_p <= 0.0 and self.typical_p >= 1.0)


class XorShift64:
    def __init__(self, seed: int):
        if seed == 0:
            seed = time.time_ns() or 0x2545F4914F6CDD1D
        self.state = (seed | 1) & 0xFFFFFFFFFFFFFFFF

    def next_u64(self) -> int:
        x = self.state
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        self.state = x
        return x

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)


def first_argmax(logits: np.ndarray) -> int:
    """First maximum; NaN never wins; all -inf gives 0."""
    l = np.where(np.isnan(logits), -np.inf, logits)
    i = int(np.argmax(l))                      # numpy returns the first maximum
    return i if l[i] > -np.inf else 0


def apply_penalties(logits: np.ndarray, history: Sequence[int], last_n: int, repeat: float,
                    presence: float, frequency: float) -> None:
    window = list(history)[max(0, len(history) - last_n):]
    counts = {}
    for t in window:
        if 0 <= t < logits.shape[0]:
            counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        l = float(logits[t])
        if repeat != 1.0:
            l = l / repeat if l > 0.0 else l * repeat
        logits[t] = np.float32(l - (c * frequency + presence))


def apply_top_n_sigma(logits: np.ndarray, n: float) -> None:
    if logits.shape[0] < 2:
        return
    mx = np.max(logits)
    std = float(np.std(logits.astype(np.float64)))
    logits[logits < np.float32(mx - n * np.float32(std))] = -np.inf


class Sampler:
    """One request's sampler: its parameters and its generator."""

    def __init__(self, params: SamplingParams):
        self.params = params
        self.rng = XorShift64(params.seed)

    def next_uniform(self) -> float:
        return self.rng.next_f32()

    def sample(self, logits: np.ndarray, history: Sequence[int]) -> int:
        """The full chain on the host; ``logits`` (float32 [V]) is modified in place."""
        p = self.params
        for tok, bias in p.logit_bias:
            if 0 <= tok < logits.shape[0]:
                logits[tok] += np.float32(bias)
        if p.penalizing:
            apply_penalties(logits, history, p.repeat_last_n, p.repeat_penalty,
                            p.presence_penalty, p.frequency_penalty)
        if p.top_n_sigma > 0.0:
            apply_top_n_sigma(logits, p.top_n_sigma)
        if p.temperature <= 0.0:
            return first_argmax(logits)
        V = logits.shape[0]
        keep = min(max(p.top_k, 1), V) if p.top_k > 0 else V
        clean = np.where(np.isnan(logits), -np.inf, logits)
        if keep < V:
            idx = np.argpartition(-clean, keep - 1)[:keep]
        else:
            idx = np.arange(V)
        order = idx[np.argsort(-clean[idx], kind="stable")]
        vals = clean[order].astype(np.float32)
        mx = vals[0]
        probs = np.exp(((vals - mx) / np.float32(p.temperature)).astype(np.float64)).astype(np.float32)
        s = np.float32(probs.sum(dtype=np.float32))
        probs = probs / s
        ids = order
        if p.typical_p < 1.0:
            ids, probs = _typical(ids, probs, p.typical_p)
        if p.min_p > 0.0:
            k = int(np.count_nonzero(probs >= np.float32(p.min_p) * probs[0]))
            ids, probs = ids[:max(k, 1)], probs[:max(k, 1)]
        if p.top_p < 1.0:
            cum = np.cumsum(probs, dtype=np.float32)
            hit = np.nonzero(cum >= np.float32(p.top_p))[0]
            cut = int(hit[0]) + 1 if hit.size else len(ids)
            ids, probs = ids[:max(cut, 1)], probs[:max(cut, 1)]
        total = float(probs.sum(dtype=np.float32))
        if total <= 0.0:
            return int(ids[0])
        target = self.rng.next_f32() * total
        for i, pr in zip(ids, probs):
            target -= float(pr)
            if target <= 0.0:
                return int(i)
        return int(ids[-1])


def _typical(ids: np.ndarray, probs: np.ndarray, typical_p: float):
    pos = probs > 0
    entropy = -float(np.sum(probs[pos] * np.log(probs[pos])))
    surprise = np.where(pos, -np.log(np.where(pos, probs, 1.0)), np.inf)
    order = np.argsort(np.abs(surprise - entropy), kind="stable")
    cum = np.cumsum(probs[order], dtype=np.float32)
    hit = np.nonzero(cum >= np.float32(typical_p))[0]
    cut = int(hit[0]) + 1 if hit.size else len(order)
    sel = order[:max(cut, 1)]
    back = sel[np.argsort(-probs[sel], kind="stable")]
    return ids[back], probs[back]
