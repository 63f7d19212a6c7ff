"""The host sampling chain (no GPU): rules taken from the reference's sampler."""
import numpy as np
import pytest

from airun_b200.sampling.sampler import (Sampler, SamplingParams, XorShift64, apply_penalties, first_argmax)
import plain_qwen3 as P


def test_first_maximum_rule():
    assert first_argmax(np.array([1.0, 3.0, 3.0, 2.0], dtype=np.float32)) == 1
    assert first_argmax(np.array([np.nan, 1.0, np.nan], dtype=np.float32)) == 1
    assert first_argmax(np.full(5, -np.inf, dtype=np.float32)) == 0
    x = np.random.default_rng(0).normal(size=1000).astype(np.float32)
    assert first_argmax(x) == P.plain_argmax(x.tolist())


def test_generator_matches_the_plain_one():
    a, b = XorShift64(1234), P.PlainRng(1234)
    for _ in range(100):
        u = a.next_f32()
        assert u == b.next_f32() and 0.0 <= u < 1.0
    assert XorShift64(2).state == 3           # state is seed | 1


def test_defaults_are_the_reference_run_defaults():
    p = SamplingParams()
    assert (p.temperature, p.top_k, p.top_p, p.min_p, p.typical_p, p.repeat_penalty, p.repeat_last_n) == \
        (0.8, 40, 0.95, 0.05, 1.0, 1.1, 64)
    g = SamplingParams.greedy()
    assert g.is_pure_greedy and g.device_ok
    assert not SamplingParams().device_ok
    assert SamplingParams.temperature_only(0.7, 3).device_ok
    pen = SamplingParams.greedy()
    pen.repeat_penalty, pen.repeat_last_n = 1.3, 8
    assert not pen.is_pure_greedy


def test_seed_reproducibility_and_greedy_at_zero():
    logits = np.random.default_rng(1).normal(size=500).astype(np.float32) * 3
    a = [Sampler(SamplingParams(seed=42)).sample(logits.copy(), []) for _ in range(3)]
    assert a[0] == a[1] == a[2]
    s1, s2 = Sampler(SamplingParams(seed=42)), Sampler(SamplingParams(seed=42))
    assert [s1.sample(logits.copy(), []) for _ in range(20)] == [s2.sample(logits.copy(), []) for _ in range(20)]
    assert Sampler(SamplingParams.greedy()).sample(logits.copy(), []) == int(np.argmax(logits))


def test_penalties_once_per_distinct_token():
    logits = np.array([2.0, -2.0, 1.0, 0.5], dtype=np.float32)
    apply_penalties(logits, [0, 0, 1, 0], last_n=64, repeat=2.0, presence=0.5, frequency=0.25)
    assert logits[0] == pytest.approx(2.0 / 2.0 - (3 * 0.25 + 0.5))     # positive: divided once
    assert logits[1] == pytest.approx(-2.0 * 2.0 - (1 * 0.25 + 0.5))    # negative: multiplied
    assert logits[2] == 1.0 and logits[3] == 0.5
    logits = np.array([2.0, 1.0], dtype=np.float32)
    apply_penalties(logits, [0, 1, 1], last_n=2, repeat=2.0, presence=0.0, frequency=0.0)
    assert logits[0] == 2.0 and logits[1] == 0.5                          # token 0 is outside the window


def test_every_filter_keeps_at_least_one():
    logits = np.array([5.0, 4.9, 1.0, -3.0], dtype=np.float32)
    for kw in (dict(top_k=1), dict(top_p=1e-6), dict(min_p=1.0), dict(typical_p=1e-6), dict(top_n_sigma=1e-6)):
        p = SamplingParams.greedy()
        p.temperature, p.seed = 1.0, 5
        for k, v in kw.items():
            setattr(p, k, v)
        for _ in range(5):
            assert Sampler(p).sample(logits.copy(), []) in (0, 1)


def test_top_k_and_top_p_cut_the_tail():
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    p = SamplingParams.greedy()
    p.temperature, p.top_k, p.seed = 1.0, 2, 9
    s = Sampler(p)
    assert {s.sample(logits.copy(), []) for _ in range(200)} == {0, 1}
    p = SamplingParams.greedy()
    p.temperature, p.top_p, p.seed = 1.0, 0.8, 9          # 0.5 + 0.3 crosses 0.8: the crossing token stays
    s = Sampler(p)
    assert {s.sample(logits.copy(), []) for _ in range(200)} == {0, 1}


def test_temperature_draw_follows_the_distribution():
    probs = np.array([0.5, 0.25, 0.125, 0.125])
    logits = np.log(probs).astype(np.float32)
    s = Sampler(SamplingParams.temperature_only(1.0, seed=77))
    n = 8000
    counts = np.bincount([s.sample(logits.copy(), []) for _ in range(n)], minlength=4)
    chi2 = float(((counts - n * probs) ** 2 / (n * probs)).sum())
    assert chi2 < 16.3                                       # 3 degrees of freedom, p = 0.001
    cold = Sampler(SamplingParams.temperature_only(0.05, seed=77))
    assert all(cold.sample(logits.copy(), []) == 0 for _ in range(50))
