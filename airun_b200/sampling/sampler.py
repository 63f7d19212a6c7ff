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

DRY stands behind the penalties, XTC behind top-p, the dynamic temperature takes
the place of the fixed one in the softmax, and mirostat 1 / 2, when on, replaces
everything after DRY and top-n-sigma (sample.rs:386-388, :520-596).  Grammar
constraints and the reasoning budget belong to the reference's server and are not
built.

A request whose parameters reduce to "argmax of the raw logits" (the
reference's ``is_pure_greedy``, sample.rs:292-298) or to a plain temperature
draw is sampled by the device kernel, which walks the cumulative sum in
vocabulary order; anything else copies the row's logits to the host and runs
this chain.
"""
from __future__ import annotations

import ctypes
import itertools
import math
import time
from dataclasses import dataclass
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
    # The samplers beyond the classic chain, all off at their usual settings (sample.rs:96-111).
    dynatemp_range: float = 0.0     # temperature moves within +-range with the candidates' entropy; 0 disables
    dynatemp_exponent: float = 1.0
    xtc_probability: float = 0.0    # with this probability drop every candidate >= threshold but the least likely of them
    xtc_threshold: float = 0.1
    dry_multiplier: float = 0.0     # 0 disables
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_penalty_last_n: int = 0     # 0: the whole history
    dry_breakers: Tuple[int, ...] = ()   # token ids that end any repeated sequence
    mirostat: int = 0               # 1 or 2; 0 disables
    mirostat_tau: float = 5.0
    mirostat_eta: float = 0.1
    # None: off.  n >= 0: record every sampled token's log-probability under the raw logits and the n
    # likeliest alternatives (the reference's with_probs, sample.rs:128-140, :280-284).
    logprobs: Optional[int] = None

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
        return bool(self.logit_bias) or self.penalizing or self.top_n_sigma > 0.0 or self.dry_multiplier > 0.0

    @property
    def is_pure_greedy(self) -> bool:
        return (self.temperature <= 0.0 and not self.logit_bias and not self.penalizing
                and self.dry_multiplier <= 0.0 and self.logprobs is None)

    def candidates_needed(self, limit: int) -> int:
        """How many of a row's largest RAW logits (with their ids) are enough to run this request's chain exactly, or 0
        when the chain needs the whole row.  The chain cuts to the ``top_k`` largest after stages that can only lower
        logits, of at most ``repeat_last_n`` distinct tokens (the penalties): the k largest afterwards are among the
        k + n largest before.  A bias may raise any token, top-n-sigma and mirostat read the whole row's statistics,
        log-probabilities its normaliser, and DRY's reach is the whole history: those take the whole row."""
        if self.logit_bias or self.top_n_sigma > 0.0 or self.dry_multiplier > 0.0 or self.mirostat != 0 \
                or self.logprobs is not None:
            return 0
        k = 1 if self.temperature <= 0.0 else self.top_k
        if k <= 0:
            return 0
        n = k + (self.repeat_last_n if self.penalizing else 0) + 1
        return n if n <= limit else 0

    @property
    def device_ok(self) -> bool:
        """True when the device kernel alone gives this request's draw."""
        if self.is_pure_greedy:
            return True
        return (self.temperature > 0.0 and not self.changes_logits and self.top_k == 0
                and self.top_p >= 1.0 and self.min_p <= 0.0 and self.typical_p >= 1.0
                and self.dynatemp_range <= 0.0 and self.xtc_probability <= 0.0 and self.mirostat == 0
                and self.logprobs is None)


@dataclass
class TokenProbs:
    """One sampled token's log-probability under softmax(raw logits), before any sampler touched
    them, and the likeliest alternatives, the best first (sample.rs:128-137, :489-503)."""
    token: int
    logprob: float
    top: List[Tuple[int, float]]


def token_probs(logits: np.ndarray, token: int, n: int) -> TokenProbs:
    clean = np.where(np.isnan(logits), -np.inf, logits).astype(np.float32, copy=False)
    mx = np.float32(clean.max())
    lse = np.float32(mx + np.float32(math.log(float(np.exp((clean - mx).astype(np.float64)).sum()))))
    n = min(max(int(n), 0), clean.shape[0])
    top: List[Tuple[int, float]] = []
    if n > 0:
        ids, vals = largest_logits(clean, n)
        top = [(int(i), float(np.float32(v - lse))) for i, v in zip(ids, vals)]
    logprob = float(np.float32(clean[token] - lse)) if 0 <= token < clean.shape[0] else float("-inf")
    return TokenProbs(int(token), logprob, top)


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
    """Repetition, presence and frequency penalties over the last ``last_n`` tokens, once per distinct
    token however often it occurs (sample.rs:651-705): a positive logit is divided by ``repeat``, a
    negative one multiplied; then ``count * frequency + presence`` is taken off."""
    n = len(history)
    window = np.asarray(history[max(0, n - last_n):] if last_n > 0 else [], dtype=np.int64)
    if window.size == 0:
        return
    ids, counts = np.unique(window, return_counts=True)
    inside = (ids >= 0) & (ids < logits.shape[0])
    ids, counts = ids[inside], counts[inside]
    l = logits[ids].astype(np.float64)
    if repeat != 1.0:
        l = np.where(l > 0.0, l / repeat, l * repeat)
    logits[ids] = (l - (counts * frequency + presence)).astype(np.float32)


def apply_top_n_sigma(logits: np.ndarray, n: float) -> None:
    if logits.shape[0] < 2:
        return
    mx = np.max(logits)
    std = float(np.std(logits.astype(np.float64)))
    logits[logits < np.float32(mx - n * np.float32(std))] = -np.inf


def apply_dry(logits: np.ndarray, history: Sequence[int], multiplier: float, base: float, allowed_length: int,
              last_n: int, breakers: Sequence[int] = ()) -> None:
    """DRY ("don't repeat yourself", sample.rs:598-637).  Wherever an earlier position j holds the
    newest token, the run of tokens ending at j that equals the run ending at the newest token is a
    repeat in the making, and the token behind j would make it longer.  Once such a run is
    ``allowed_length`` long that token loses ``multiplier * base ** (length - allowed_length)``; the
    longest run counts.  A breaker token ends a run and is itself never punished; only the last
    ``last_n`` tokens are searched (0: all of them)."""
    h = list(history)
    n = len(h)
    if n < 2:
        return
    start = n - (n if last_n <= 0 else min(last_n, n))
    stop = set(breakers)
    newest = h[n - 1]
    if newest in stop:
        return
    longest = {}
    for j in range(start, n - 1):
        if h[j] != newest:
            continue
        length = 0
        while j - length >= start and h[j - length] == h[n - 1 - length] and h[j - length] not in stop:
            length += 1
        follower = h[j + 1]
        if length >= allowed_length and follower not in stop:
            longest[follower] = max(longest.get(follower, 0), length)
    for tok, length in longest.items():
        if 0 <= tok < logits.shape[0]:
            logits[tok] -= np.float32(np.float32(multiplier) * np.float32(base) ** np.float32(length - allowed_length))


def dynamic_temperature(values: np.ndarray, temperature: float, rng_range: float, exponent: float) -> float:
    """The temperature between ``temperature - range`` and ``temperature + range`` (not below 0)
    that the candidates' normalised entropy at temperature 1 calls for (sample.rs:503-518);
    ``values``: the candidates' logits, the largest first."""
    if rng_range <= 0.0 or values.shape[0] < 2:
        return temperature
    ps = np.exp((values - values[0]).astype(np.float64))
    ps = ps / ps.sum()
    pos = ps[ps > 0.0]
    entropy = -float(np.sum(pos * np.log(pos)))
    norm = min(max(entropy / math.log(values.shape[0]), 0.0), 1.0)
    lo, hi = max(temperature - rng_range, 0.0), temperature + rng_range
    return max(float(np.float32(lo + (hi - lo) * np.float32(norm ** exponent))), 1e-6)


class Sampler:
    """One request's sampler: its parameters, its generator and mirostat's running ``mu``."""

    def __init__(self, params: SamplingParams):
        self.params = params
        self.rng = XorShift64(params.seed)
        self.mu = 2.0 * params.mirostat_tau           # sample.rs:259-262
        self.probs: List[TokenProbs] = []             # one per sampled token when params.logprobs is set
        self._packed = None                           # the parameters as a record of the native core (packed_params)
        # what the engine asks every step, worked out once (the parameters of a live request do not change)
        self.device_ok = params.device_ok
        self.candidates_needed = params.candidates_needed(512)

    def _draw(self, ids: np.ndarray, probs: np.ndarray) -> int:
        """Index into ``ids`` / ``probs`` (descending) of the inverse-CDF draw (sample.rs:478-485)."""
        total = float(np.cumsum(probs, dtype=np.float32)[-1])
        target = self.rng.next_f32() * total
        for i, pr in enumerate(probs):
            target -= float(pr)
            if target <= 0.0:
                return i
        return len(ids) - 1

    def _mirostat(self, logits: np.ndarray) -> int:
        """Mirostat 1 or 2 over the whole vocabulary at the temperature; ``mu`` follows the surprise
        of the token picked (sample.rs:520-596)."""
        p = self.params
        scaled = np.where(np.isnan(logits), -np.inf, logits).astype(np.float32) * np.float32(1.0 / p.temperature)
        e = np.exp((scaled - scaled.max()).astype(np.float64)).astype(np.float32)
        probs = (e.astype(np.float64) / float(e.astype(np.float64).sum())).astype(np.float32)
        order = np.argsort(-probs, kind="stable")
        V = probs.shape[0]
        if p.mirostat == 1:
            # Zipf exponent from the 100 likeliest tokens, then the k that mu asks for
            top = probs[order[:101]]
            m = min(100, top.shape[0] - 1)
            i = np.arange(m, dtype=np.float64)
            t = np.log((i + 2.0) / (i + 1.0))
            tiny = float(np.finfo(np.float32).tiny)
            b = np.log(top[:m].astype(np.float64) / np.maximum(top[1:m + 1].astype(np.float64), tiny))
            den = float(np.sum(t * t))
            s_hat = float(np.sum(t * b)) / den if den > 0.0 else 1.0
            eps = s_hat - 1.0
            with np.errstate(all="ignore"):
                k = np.float64(eps * 2.0 ** self.mu) / (1.0 - np.float64(V) ** (-eps))
                k = np.power(k, 1.0 / s_hat) if s_hat != 0.0 else np.inf
            k = int(k) if np.isfinite(k) else V
            keep = order[:min(max(k, 1), V)]
        else:
            floor = np.float32(2.0) ** np.float32(-self.mu)          # surprise at most mu
            keep = order[probs[order] >= floor]
            if keep.shape[0] == 0:
                keep = order[:1]
        kp = probs[keep]
        total = float(np.cumsum(kp, dtype=np.float32)[-1])
        j = self._draw(keep, kp)
        tiny32 = float(np.finfo(np.float32).tiny)
        surprise = -math.log2(max(float(kp[j]) / total, tiny32))
        self.mu -= p.mirostat_eta * (surprise - p.mirostat_tau)
        return int(keep[j])

    def next_uniform(self) -> float:
        return self.rng.next_f32()

    def packed_params(self) -> np.ndarray:
        """This request's parameters as one ChainParams record of the native core (made once)."""
        if self._packed is None:
            p = self.params
            self._packed = np.array([(p.temperature, p.top_p, p.min_p, p.repeat_penalty, p.presence_penalty, p.frequency_penalty,
                                      p.top_k, 1 if p.penalizing else 0, 0, 0, 0)], dtype=_CAND_PARAMS)[0]
        return self._packed

    def sample(self, logits: np.ndarray, history: Sequence[int]) -> int:
        """The full chain on the host for one row; ``logits`` (float32 [V]) is modified in place."""
        return sample_rows([self], logits.reshape(1, -1), [history])[0]

    # The chain in three stages, so that several rows share one call of the native top-k.
    def _before_candidates(self, logits: np.ndarray, history: Sequence[int]) -> Optional[int]:
        """Everything that works on the whole row.  Returns the token when the chain ends here (greedy,
        mirostat), else None: the row then goes on with its ``candidate_count`` largest logits."""
        p = self.params
        for tok, bias in p.logit_bias:
            if 0 <= tok < logits.shape[0]:
                logits[tok] += np.float32(bias)
        if p.penalizing:
            apply_penalties(logits, history, p.repeat_last_n, p.repeat_penalty,
                            p.presence_penalty, p.frequency_penalty)
        if p.dry_multiplier > 0.0:
            apply_dry(logits, history, p.dry_multiplier, p.dry_base, p.dry_allowed_length, p.dry_penalty_last_n,
                      p.dry_breakers)
        if p.top_n_sigma > 0.0:
            apply_top_n_sigma(logits, p.top_n_sigma)
        if p.temperature <= 0.0:
            return first_argmax(logits)
        if p.mirostat != 0:
            return self._mirostat(logits)
        return None

    def candidate_count(self, vocab: int) -> int:
        """top-k first: it is the cheapest cut, and everything behind it sorts (sample.rs:390-403)."""
        k = self.params.top_k
        return min(max(k, 1), vocab) if k > 0 else vocab

    def _from_candidates(self, ids: np.ndarray, vals: np.ndarray) -> int:
        """Softmax over the candidates (``vals`` float32, the largest first), the filters on
        probabilities, the draw."""
        p = self.params
        mx = vals[0]
        temperature = dynamic_temperature(vals, p.temperature, p.dynatemp_range, p.dynatemp_exponent)
        with np.errstate(invalid="ignore"):               # a row of nothing but -inf gives NaN, as in the reference
            probs = np.exp(((vals - mx) / np.float32(temperature)).astype(np.float64)).astype(np.float32)
        s = np.cumsum(probs, dtype=np.float32)[-1]        # float32, one after the other (sample.rs:409-418)
        probs = probs / s
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
        if p.xtc_probability > 0.0 and self.rng.next_f32() < p.xtc_probability:
            # XTC (sample.rs:436-443): of the leading candidates at or above the threshold only the
            # least likely stays
            above = int(np.count_nonzero(np.cumprod(probs >= np.float32(p.xtc_threshold))))
            if above >= 2:
                ids, probs = ids[above - 1:], probs[above - 1:]
        if float(np.cumsum(probs, dtype=np.float32)[-1]) <= 0.0:
            return int(ids[0])
        return int(ids[self._draw(ids, probs)])


def largest_logits(row: np.ndarray, k: int) -> Tuple[np.ndarray, np.ndarray]:
    """(ids, values) of the ``k`` largest entries of a float32 row, the largest first, with numpy: the
    plain twin of the native top-k, and what serves when every logit is a candidate (top-k off).
    NaN counts as -inf; which of several equal values at the cut stays is numpy's choice."""
    clean = np.where(np.isnan(row), -np.inf, row).astype(np.float32, copy=False)
    n = clean.shape[0]
    idx = np.argpartition(-clean, k - 1)[:k] if k < n else np.arange(n)
    order = idx[np.argsort(-clean[idx], kind="stable")]
    return order, clean[order]


NATIVE_TOPK_MAX = 4096        # candidates up to which the one-pass heap of csrc/sampler_core.cpp is used
_TOPK_THREADS = 8


def _native_topk():
    """``airun_topk_rows`` of csrc/sampler_core.cpp, compiled with the C++ compiler at first use."""
    global _TOPK_FN
    if _TOPK_FN is None:
        import ctypes
        from ..csrc import build
        f = build.load("sampler_core").airun_topk_rows
        f.restype = ctypes.c_int
        f.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p,
                      ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int]
        _TOPK_FN = f
    return _TOPK_FN


_TOPK_FN = None


def largest_logits_rows(rows: np.ndarray, ks: Sequence[int]) -> List[Tuple[np.ndarray, np.ndarray]]:
    """The ``ks[r]`` largest logits of every row of ``rows`` (float32 [R, V], rows contiguous), the rows
    side by side on threads of the native core.  Equal values come by ascending id."""
    R, V = rows.shape
    if rows.dtype != np.float32 or rows.strides[1] != 4 or rows.strides[0] % 4 != 0 or rows.strides[0] < 4 * V:
        raise ValueError("largest_logits_rows wants float32 rows that are contiguous")
    kmax = max(ks)
    ks_arr = np.asarray(ks, dtype=np.int32)
    idx = np.empty((R, kmax), dtype=np.int32)
    val = np.empty((R, kmax), dtype=np.float32)
    status = _native_topk()(rows.ctypes.data, rows.strides[0] // 4, R, V, ks_arr.ctypes.data, idx.ctypes.data,
                            val.ctypes.data, kmax, _TOPK_THREADS)
    if status != 0:
        raise ValueError("the native top-k refused its arguments")
    return [(idx[r, :ks[r]], val[r, :ks[r]]) for r in range(R)]


class _ChainParams(ctypes.Structure):           # ChainParams of csrc/sampler_core.cpp
    _fields_ = [("temperature", ctypes.c_double), ("top_p", ctypes.c_double), ("min_p", ctypes.c_double),
                ("repeat", ctypes.c_double), ("presence", ctypes.c_double), ("frequency", ctypes.c_double),
                ("top_k", ctypes.c_int), ("penalize", ctypes.c_int), ("n_bias", ctypes.c_int),
                ("bias_ids", ctypes.c_void_p), ("bias_vals", ctypes.c_void_p)]


class _ChainRow(ctypes.Structure):              # ChainRow of csrc/sampler_core.cpp
    _fields_ = [("logits", ctypes.c_void_p), ("window", ctypes.c_void_p), ("n_window", ctypes.c_longlong),
                ("params", ctypes.c_void_p), ("rng_state", ctypes.c_void_p), ("out", ctypes.c_int)]


_CHAIN_FN = None


def _native_chain():
    """``airun_sample_chain_rows`` of csrc/sampler_core.cpp."""
    global _CHAIN_FN
    if _CHAIN_FN is None:
        from ..csrc import build
        f = build.load("sampler_core").airun_sample_chain_rows
        f.restype = ctypes.c_int
        f.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int]
        _CHAIN_FN = f
    return _CHAIN_FN


def usual_chain(p: SamplingParams, vocab: int) -> bool:
    """Whether the native chain takes these parameters: bias, penalties, top-k (on, and small enough for
    the one-pass heap), a fixed temperature, min-p, top-p, and nothing else."""
    return (p.temperature > 0.0 and 0 < p.top_k < vocab and p.top_k <= NATIVE_TOPK_MAX and p.typical_p >= 1.0
            and p.top_n_sigma <= 0.0 and p.dry_multiplier <= 0.0 and p.dynatemp_range <= 0.0
            and p.xtc_probability <= 0.0 and p.mirostat == 0 and p.logprobs is None)


def _sample_rows_native(samplers: Sequence["Sampler"], rows: np.ndarray, histories: Sequence[Sequence[int]],
                        which: Sequence[int]) -> List[int]:
    """The rows ``which`` through the native chain, side by side on threads; the samplers' generators
    move on as if the Python chain had drawn."""
    n, V = len(which), rows.shape[1]
    c_rows = (_ChainRow * n)()
    c_params = (_ChainParams * n)()
    states = np.empty(n, dtype=np.uint64)
    keep = []                                                     # arrays the structures point into
    for j, r in enumerate(which):
        p = samplers[r].params
        last_n = p.repeat_last_n if p.penalizing else 0
        h = histories[r]
        window = np.asarray(h[max(0, len(h) - last_n):] if last_n > 0 else [], dtype=np.int64)
        bias_ids = np.asarray([t for t, _ in p.logit_bias], dtype=np.int32)
        bias_vals = np.asarray([b for _, b in p.logit_bias], dtype=np.float32)
        keep += [window, bias_ids, bias_vals]
        c_params[j] = _ChainParams(p.temperature, p.top_p, p.min_p, p.repeat_penalty, p.presence_penalty,
                                   p.frequency_penalty, p.top_k, 1 if p.penalizing else 0, len(p.logit_bias),
                                   bias_ids.ctypes.data, bias_vals.ctypes.data)
        states[j] = samplers[r].rng.state
        c_rows[j] = _ChainRow(rows[r].ctypes.data, window.ctypes.data, window.shape[0],
                              ctypes.addressof(c_params) + j * ctypes.sizeof(_ChainParams),
                              states.ctypes.data + 8 * j, -1)
    if _native_chain()(ctypes.addressof(c_rows), n, V, _TOPK_THREADS) != 0:
        raise ValueError("the native sampling chain refused its arguments")
    for j, r in enumerate(which):
        samplers[r].rng.state = int(states[j])
    return [int(c_rows[j].out) for j in range(n)]


def sample_rows(samplers: Sequence["Sampler"], rows: np.ndarray, histories: Sequence[Sequence[int]],
                native: bool = True) -> List[int]:
    """One token for every row: ``rows[r]`` (float32 [V], modified in place) goes through the chain of
    ``samplers[r]`` with the tokens of its request so far, ``histories[r]``.  Rows with the usual
    parameters (``usual_chain``) run in the native core, all in one call; the others run the chain
    below, sharing one native top-k call.  ``native=False``: everything in Python (the plain twin)."""
    V = rows.shape[1]
    fast = [r for r, s in enumerate(samplers) if usual_chain(s.params, V)] if native else []
    if fast and rows.dtype == np.float32 and rows.strides[1] == 4:
        picked = _sample_rows_native(samplers, rows, histories, fast)
        if len(fast) == len(samplers):
            return picked
        rest = [r for r in range(len(samplers)) if r not in set(fast)]
        others = sample_rows([samplers[r] for r in rest], rows[rest], [histories[r] for r in rest], native=False)
        out_all: List[int] = [0] * len(samplers)
        for r, t in zip(fast, picked):
            out_all[r] = t
        for r, t in zip(rest, others):
            out_all[r] = t
        return out_all
    out: List[Optional[int]] = []
    raw = {r: rows[r].copy() for r, s in enumerate(samplers) if s.params.logprobs is not None}
    for s, row, h in zip(samplers, rows, histories):
        out.append(s._before_candidates(row, h))
    V = rows.shape[1]
    pending = [r for r, t in enumerate(out) if t is None]
    native = [r for r in pending if samplers[r].candidate_count(V) < V and samplers[r].candidate_count(V) <= NATIVE_TOPK_MAX]
    if native:
        sub = rows if len(native) == len(rows) else rows[native]
        found = largest_logits_rows(np.ascontiguousarray(sub), [samplers[r].candidate_count(V) for r in native])
        for r, (ids, vals) in zip(native, found):
            out[r] = samplers[r]._from_candidates(ids, vals)
    for r in pending:
        if out[r] is None:
            ids, vals = largest_logits(rows[r], samplers[r].candidate_count(V))
            out[r] = samplers[r]._from_candidates(ids, vals)
    for r, before in raw.items():
        samplers[r].probs.append(token_probs(before, int(out[r]), samplers[r].params.logprobs))
    return [int(t) for t in out]


_CAND_PARAMS = np.dtype([("temperature", "f8"), ("top_p", "f8"), ("min_p", "f8"), ("repeat", "f8"), ("presence", "f8"),
                         ("frequency", "f8"), ("top_k", "i4"), ("penalize", "i4"), ("n_bias", "i4"), ("bias_ids", "u8"),
                         ("bias_vals", "u8")], align=True)            # ChainParams of csrc/sampler_core.cpp
_CAND_FN = None


def _sample_candidates_native(samplers: Sequence["Sampler"], cand_ids: np.ndarray, cand_vals: np.ndarray,
                              windows: Sequence[Sequence[int]]) -> List[int]:
    """``sample_candidates`` for rows with the usual parameters, whole in the native core
    (``airun_sample_candidates`` of csrc/sampler_core.cpp), rows side by side on threads."""
    global _CAND_FN
    if _CAND_FN is None:
        from ..csrc import build
        assert _CAND_PARAMS.itemsize == ctypes.sizeof(_ChainParams)
        f = build.load("sampler_core").airun_sample_candidates
        f.restype = ctypes.c_int
        f.argtypes = [ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 7 + [ctypes.c_int]
        _CAND_FN = f
    n, C = cand_ids.shape
    ids = np.ascontiguousarray(cand_ids, dtype=np.int32)
    vals = np.ascontiguousarray(cand_vals, dtype=np.float32)
    params = np.empty(n, dtype=_CAND_PARAMS)
    states = np.empty(n, dtype=np.uint64)
    win_off = np.zeros(n + 1, dtype=np.int64)
    for r, s in enumerate(samplers):
        params[r] = s.packed_params()
        states[r] = s.rng.state
        win_off[r + 1] = win_off[r] + len(windows[r])
    window = np.fromiter(itertools.chain.from_iterable(windows), dtype=np.int64, count=int(win_off[n]))
    out = np.empty(n, dtype=np.int32)
    if _CAND_FN(n, C, ids.ctypes.data, vals.ctypes.data, window.ctypes.data, win_off.ctypes.data, params.ctypes.data,
                states.ctypes.data, out.ctypes.data, _TOPK_THREADS) != 0:
        raise ValueError("the native candidate chain refused its arguments")
    for r, s in enumerate(samplers):
        s.rng.state = int(states[r])
    return [int(t) for t in out]


def sample_candidates(samplers: Sequence["Sampler"], cand_ids: np.ndarray, cand_vals: np.ndarray,
                      windows: Sequence[Sequence[int]]) -> List[int]:
    """One token for every row from its largest raw logits instead of the whole row: ``cand_ids[r]`` / ``cand_vals[r]``
    are at least ``samplers[r].params.candidates_needed`` of them (any order; ids < 0 are padding), ``windows[r]`` the
    request's last ``repeat_last_n`` tokens.  The candidates, in ascending order of their ids, stand as a short row of
    their own, the window's tokens become positions in it (a token that is no candidate cannot be picked and is left
    out), and the row goes through ``sample_rows`` unchanged: same stages, same arithmetic, same use of the
    generator; equal values fall as in the whole row because positions keep the order of the ids."""
    n, C = cand_ids.shape
    if n and all(usual_chain(s.params, C) and not s.params.logit_bias for s in samplers):
        return _sample_candidates_native(samplers, cand_ids, cand_vals, windows)
    rows = np.full((n, C), -np.inf, dtype=np.float32)
    maps = []
    hist = []
    for r in range(n):
        ids = cand_ids[r]
        keep = np.nonzero(ids >= 0)[0]
        order = keep[np.argsort(ids[keep], kind="stable")]
        idmap = ids[order].astype(np.int64)
        rows[r, :len(order)] = cand_vals[r][order]
        maps.append(idmap)
        w = np.asarray(windows[r], dtype=np.int64)
        if w.size and idmap.size:
            pos = np.searchsorted(idmap, w)
            pos_ok = (pos < idmap.size)
            pos_ok[pos_ok] &= idmap[pos[pos_ok]] == w[pos_ok]
            hist.append(pos[pos_ok].tolist())
        else:
            hist.append([])
    picked = sample_rows(samplers, rows, hist)
    return [int(maps[r][t]) if 0 <= t < len(maps[r]) else 0 for r, t in enumerate(picked)]


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
