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


# ----------------------------------------------------------------------------- the further samplers
def _plain_dry(history, multiplier, base, allowed, last_n, breakers=()):
    """Token -> logit it loses, by trying every earlier occurrence of the newest token and
    comparing backwards one token at a time (crates/airun-core/src/sample.rs:598-637)."""
    n = len(history)
    lost = {}
    if n < 2 or history[-1] in breakers:
        return lost
    first = 0 if last_n == 0 else max(0, n - last_n)
    for j in range(first, n - 1):
        if history[j] != history[-1]:
            continue
        run = 0
        while j - run >= first and history[j - run] == history[n - 1 - run] and history[j - run] not in breakers:
            run += 1
        nxt = history[j + 1]
        if run >= allowed and nxt not in breakers:
            lost[nxt] = max(lost.get(nxt, 0.0), multiplier * base ** (run - allowed))
    return lost


def test_dry_punishes_the_token_that_would_extend_a_repeat():
    from airun_b200.sampling.sampler import apply_dry
    #          0  1  2  3  4  5  6  7  8
    history = [5, 6, 7, 8, 1, 5, 6, 7]                       # "5 6 7" again: 8 would repeat a run of three
    logits = np.zeros(10, dtype=np.float32)
    apply_dry(logits, history, multiplier=0.8, base=1.75, allowed_length=2, last_n=0)
    assert logits[8] == pytest.approx(-0.8 * 1.75 ** (3 - 2)) and np.count_nonzero(logits) == 1
    logits[:] = 0
    apply_dry(logits, history, 0.8, 1.75, allowed_length=4, last_n=0)      # a run of three is still allowed
    assert not logits.any()
    logits[:] = 0
    apply_dry(logits, history, 0.8, 1.75, 2, last_n=0, breakers=(6,))      # a breaker cuts the run to one token
    assert not logits.any()
    logits[:] = 0
    apply_dry(logits, history, 0.8, 1.75, 2, last_n=4)                     # the first "5 6 7" is outside the window
    assert not logits.any()
    rng = np.random.default_rng(3)
    for _ in range(200):                                      # against the plain restatement, small alphabets repeat a lot
        h = rng.integers(0, 4, size=int(rng.integers(0, 30))).tolist()
        allowed, last_n = int(rng.integers(1, 4)), int(rng.choice([0, 5, 12]))
        breakers = (3,) if rng.random() < 0.3 else ()
        logits = np.zeros(6, dtype=np.float32)
        apply_dry(logits, h, 0.7, 1.5, allowed, last_n, breakers)
        want = _plain_dry(h, 0.7, 1.5, allowed, last_n, breakers)
        for t in range(6):
            assert logits[t] == pytest.approx(-want.get(t, 0.0), rel=1e-5)
    p = SamplingParams.greedy()
    p.dry_multiplier = 5.0
    assert not p.is_pure_greedy and not p.device_ok
    logits = np.zeros(10, dtype=np.float32); logits[8] = 1.0; logits[2] = 0.5
    assert Sampler(p).sample(logits, history) == 2           # greedy would repeat; DRY moves it


def test_xtc_removes_the_top_choices_but_the_last_of_them():
    probs = np.array([0.4, 0.3, 0.2, 0.1])
    logits = np.log(probs).astype(np.float32)
    p = SamplingParams.temperature_only(1.0, seed=11)
    p.xtc_probability, p.xtc_threshold = 1.0, 0.25            # 0.4 and 0.3 are above: 0.4 goes, 0.3 stays
    assert not p.device_ok
    s = Sampler(p)
    seen = np.bincount([s.sample(logits.copy(), []) for _ in range(600)], minlength=4)
    assert seen[0] == 0 and all(seen[1:] > 0)
    p.xtc_threshold = 0.35                                    # one candidate above: nothing is removed
    s = Sampler(p)
    assert np.bincount([s.sample(logits.copy(), []) for _ in range(300)], minlength=4)[0] > 0
    p.xtc_probability, p.xtc_threshold = 0.5, 0.25            # the coin: about half of the draws keep token 0
    s = Sampler(p)
    seen = np.bincount([s.sample(logits.copy(), []) for _ in range(2000)], minlength=4)
    assert 0.12 < seen[0] / 2000 < 0.28                       # 0.5 * 0.4


def test_dynamic_temperature_moves_with_the_entropy():
    from airun_b200.sampling.sampler import dynamic_temperature
    flat = np.zeros(8, dtype=np.float32)                      # normalised entropy 1: the top of the range
    peaked = np.array([50.0] + [0.0] * 7, dtype=np.float32)   # entropy ~0: the bottom
    assert dynamic_temperature(flat, 1.0, 0.5, 1.0) == pytest.approx(1.5)
    assert dynamic_temperature(peaked, 1.0, 0.5, 1.0) == pytest.approx(0.5, abs=1e-3)
    assert dynamic_temperature(peaked, 0.3, 0.5, 1.0) == pytest.approx(1e-6, abs=1e-3)      # never below zero
    assert dynamic_temperature(flat, 0.8, 0.0, 1.0) == 0.8 and dynamic_temperature(flat[:1], 0.8, 0.5, 1.0) == 0.8
    two = np.log(np.array([0.75, 0.25])).astype(np.float32)
    h = -(0.75 * np.log(0.75) + 0.25 * np.log(0.25)) / np.log(2)
    assert dynamic_temperature(two, 1.0, 0.4, 2.0) == pytest.approx(0.6 + 0.8 * h ** 2, rel=1e-5)
    # in the chain: a peaked distribution is drawn colder than a flat one
    p = SamplingParams.temperature_only(1.0, seed=5)
    p.dynatemp_range = 0.9
    assert not p.device_ok
    logits = np.array([3.0, 0.0, 0.0, 0.0], dtype=np.float32)
    hot = Sampler(SamplingParams.temperature_only(1.0, seed=5))
    a = np.mean([Sampler.sample(hot, logits.copy(), []) == 0 for _ in range(1500)])
    dyn = Sampler(p)
    b = np.mean([dyn.sample(logits.copy(), []) == 0 for _ in range(1500)])
    assert b > a + 0.03


@pytest.mark.parametrize("version", [1, 2])
def test_mirostat_steers_the_surprise_with_tau(version):
    rng = np.random.default_rng(8)
    base = (rng.normal(size=2000) * 2.5).astype(np.float32)
    full = np.exp(base.astype(np.float64) - base.max())
    full /= full.sum()
    entropy = -np.sum(full * np.log2(full))                    # the mean surprise of untruncated draws: about 7.3 bits
    assert entropy > 6.5

    def mean_surprise(tau):
        p = SamplingParams.temperature_only(1.0, seed=21)
        p.mirostat, p.mirostat_tau, p.mirostat_eta = version, tau, 0.2
        assert not p.device_ok
        s = Sampler(p)
        assert s.mu == 2.0 * tau                               # starts at twice tau
        out = []
        for step in range(400):
            tok = s.sample(np.roll(base, step).copy(), [])
            out.append(-np.log2(np.roll(full, step)[tok]))
        return float(np.mean(out[100:]))

    low, mid, high = mean_surprise(1.0), mean_surprise(3.0), mean_surprise(5.0)
    assert low < mid - 0.4 and mid < high - 0.4 and high < entropy - 1.0
    p = SamplingParams.temperature_only(1.0, seed=21)
    p.mirostat, p.mirostat_tau, p.mirostat_eta = version, 3.0, 0.2
    # same seed, same tokens; and mirostat replaces top-k / top-p (they have no say)
    q = SamplingParams(temperature=1.0, seed=21, top_k=1, top_p=0.01, min_p=0.9, repeat_penalty=1.0)
    q.mirostat, q.mirostat_tau, q.mirostat_eta = version, 3.0, 0.2
    s1, s2 = Sampler(p), Sampler(q)
    assert [s1.sample(np.roll(base, i).copy(), []) for i in range(50)] == [s2.sample(np.roll(base, i).copy(), []) for i in range(50)]


def test_mirostat_2_keeps_tokens_whose_surprise_is_at_most_mu():
    probs = np.array([0.5, 0.25, 0.125, 0.0625, 0.0625])
    logits = np.log(probs).astype(np.float32)
    p = SamplingParams.temperature_only(1.0, seed=4)
    p.mirostat, p.mirostat_tau, p.mirostat_eta = 2, 1.0, 0.0   # mu stays 2: tokens with p >= 1/4
    s = Sampler(p)
    seen = np.bincount([s.sample(logits.copy(), []) for _ in range(400)], minlength=5)
    assert seen[0] > 0 and seen[1] > 0 and seen[2:].sum() == 0
    p.mirostat_tau = 0.1                                       # mu 0.2: nobody passes, the best stays
    s = Sampler(p)
    assert all(s.sample(logits.copy(), []) == 0 for _ in range(20))


# ----------------------------------------------------------------------------- the command line's options
def test_command_line_options_carry_the_reference_names_and_defaults():
    """``airun run`` (crates/airun-cli/src/run.rs:50-220), ``bench`` (bench.rs:11-92) and ``perplexity``
    (perplexity.rs:24-66): option names and defaults; parsing needs no GPU."""
    from airun_b200.cli import build_parser, parse_ids
    ap = build_parser()
    a = ap.parse_args(["run", "m", "-p", "1,2 3"])
    assert (a.predict, a.temp, a.top_k, a.top_p, a.min_p, a.typical_p, a.top_n_sigma) == (256, 0.8, 40, 0.95, 0.05, 1.0, 0.0)
    assert (a.repeat_penalty, a.presence_penalty, a.frequency_penalty, a.repeat_last_n, a.seed) == (1.1, 0.0, 0.0, 64, 0)
    assert a.ctx_size is None and a.batch_size == 512 and not a.stats and not a.quiet
    assert parse_ids(a.prompt) == [1, 2, 3]
    a = ap.parse_args(["run", "m", "-n", "8", "-c", "100", "-b", "32", "--temp", "0", "--seed", "7", "-q", "--stats"])
    assert (a.predict, a.ctx_size, a.batch_size, a.temp, a.seed, a.quiet, a.stats) == (8, 100, 32, 0.0, 7, True, True)
    b = ap.parse_args(["bench", "m"])
    assert (b.prefill, b.decode, b.decode_at, b.runs, b.warmup, b.temp) == ("128,512", 128, "16", 3, 1, 0.0)
    assert not b.forward_only and not b.random_tokens and not b.json and b.ctx_size is None
    b = ap.parse_args(["bench", "m", "--decode-at", "16,4096", "--random-tokens", "--forward-only", "-c", "8192", "--json"])
    assert b.decode_at == "16,4096" and b.random_tokens and b.forward_only and b.ctx_size == 8192 and b.json
    p = ap.parse_args(["perplexity", "m", "-f", "ids.txt"])
    assert (p.file, p.limit, p.chunk, p.batched, p.worst, p.ctx_size) == ("ids.txt", 0, 0, False, 0, 4096)
    p = ap.parse_args(["perplexity", "m", "--file", "x", "-n", "100", "--chunk", "64", "--batched", "--worst", "5", "-c", "512"])
    assert (p.limit, p.chunk, p.batched, p.worst, p.ctx_size) == (100, 64, True, 5, 512)
    s = ap.parse_args(["selftest", "--device", "0", "--verbose"])
    assert s.device == 0 and s.verbose
    with pytest.raises(SystemExit):
        parse_ids("  ")


# ----------------------------------------------------------------------------- the native top-k
def test_native_largest_logits_against_numpy():
    from airun_b200.sampling.sampler import largest_logits, largest_logits_rows
    rng = np.random.default_rng(12)
    for V, ks in ((1000, [1, 40, 999, 7]), (151936, [40, 1, 256]), (33, [33, 5])):
        rows = (rng.normal(size=(len(ks), V)) * 4).astype(np.float32)
        rows[0, rng.integers(0, V, size=5)] = np.nan              # NaN never wins
        if V > 100:
            rows[1, :50] = -np.inf
        got = largest_logits_rows(rows, ks)
        for r, k in enumerate(ks):
            ids, vals = got[r]
            want_ids, want_vals = largest_logits(rows[r], k)
            assert ids.shape == (k,) and np.array_equal(vals, want_vals)
            finite = np.isfinite(vals)                                        # random floats: no ties but among -inf
            assert np.array_equal(ids[finite], want_ids[finite])
            clean = np.where(np.isnan(rows[r]), -np.inf, rows[r])
            assert np.array_equal(clean[ids], vals) and np.all(vals[:-1] >= vals[1:]) and len(set(ids.tolist())) == k
            assert np.all(np.diff(ids[~finite]) > 0)                          # equal values by ascending id
    # a view with a row stride beyond its length, as a slice of a wider array is
    wide = (rng.normal(size=(3, 700))).astype(np.float32)
    view = wide[:, :500]
    for (ids, vals), row in zip(largest_logits_rows(view, [9, 9, 9]), view):
        assert np.array_equal(ids, largest_logits(row, 9)[0])
    with pytest.raises(ValueError):
        largest_logits_rows(wide[:, ::2], [3, 3, 3])
    with pytest.raises(ValueError):
        largest_logits_rows(view, [3, 3, 501])


def test_native_largest_logits_orders_equal_values_by_id():
    from airun_b200.sampling.sampler import largest_logits_rows
    row = np.array([[1.0, 5.0, 5.0, 0.0, 5.0, 1.0, 1.0, np.nan, 7.0]], dtype=np.float32)
    ids, vals = largest_logits_rows(row, [3])[0]
    assert ids.tolist() == [8, 1, 2] and vals.tolist() == [7.0, 5.0, 5.0]     # of three 5s the first two stay
    ids, _ = largest_logits_rows(row, [6])[0]
    assert ids.tolist() == [8, 1, 2, 4, 0, 5]
    flat = np.full((1, 50), -np.inf, dtype=np.float32)
    assert largest_logits_rows(flat, [4])[0][0].tolist() == [0, 1, 2, 3]


def test_rows_sampled_together_get_what_they_get_alone():
    from airun_b200.sampling.sampler import sample_rows
    rng = np.random.default_rng(13)
    V = 5000
    base = (rng.normal(size=(6, V)) * 3).astype(np.float32)
    hist = [rng.integers(0, V, size=30).tolist() for _ in range(6)]

    def make():
        ps = [SamplingParams(seed=3), SamplingParams.greedy(), SamplingParams(seed=4, top_k=0, min_p=0.02),
              SamplingParams(seed=5, top_k=5, dry_multiplier=0.8), SamplingParams(seed=6, mirostat=2),
              SamplingParams(seed=7, top_k=V + 10, xtc_probability=0.5)]
        return [Sampler(p) for p in ps]

    together, alone = make(), make()
    for step in range(12):
        rows = np.roll(base, step, axis=1).copy()
        got = sample_rows(together, rows, hist)
        want = [s.sample(np.roll(base[r], step).copy(), hist[r]) for r, s in enumerate(alone)]
        assert got == want
        assert got[1] == int(np.argmax(np.roll(base[1], step)))


def test_token_log_probabilities_come_from_the_raw_logits():
    """The reference's with_probs (crates/airun-core/src/sample.rs:128-140, :489-503): the sampled token's
    log-probability under softmax of the logits before bias, penalties or filters, and the n best."""
    from airun_b200.sampling.sampler import sample_rows, token_probs
    rng = np.random.default_rng(3)
    logits = (rng.normal(size=300) * 4).astype(np.float32)
    logits[5] = np.nan
    want = np.where(np.isnan(logits), -np.inf, logits).astype(np.float64)
    want = want - (want.max() + np.log(np.exp(want - want.max()).sum()))
    tp = token_probs(logits, 17, 4)
    assert tp.token == 17 and tp.logprob == pytest.approx(want[17], abs=1e-5)
    order = np.argsort(-want)[:4]
    assert [i for i, _ in tp.top] == order.tolist() and [l for _, l in tp.top] == pytest.approx(want[order].tolist(), abs=1e-5)
    assert token_probs(logits, 17, 0).top == [] and token_probs(logits, 5, 1).logprob == float("-inf")
    # in the chain: recorded per sampled token, from the logits as they came, not as the penalties left them
    p = SamplingParams(seed=2, repeat_penalty=5.0, logprobs=2)
    q = SamplingParams.greedy()
    q.logprobs = 0
    assert not p.device_ok and not q.device_ok and not q.is_pure_greedy and SamplingParams.greedy().device_ok
    sp, sq, plain = Sampler(p), Sampler(q), Sampler(SamplingParams(seed=2, repeat_penalty=5.0))
    hist = [int(np.argmax(want))] * 3
    for step in range(5):
        rows = np.stack([np.roll(logits, step), np.roll(logits, step)])
        toks = sample_rows([sp, sq], rows, [hist, hist])
        assert toks[0] == plain.sample(np.roll(logits, step).copy(), hist)       # recording changes no draw
        w = np.roll(want, step)
        assert sp.probs[step].token == toks[0] and sp.probs[step].logprob == pytest.approx(w[toks[0]], abs=1e-5)
        assert len(sp.probs[step].top) == 2 and sp.probs[step].top[0][0] == int(np.argmax(w))
        assert sq.probs[step].token == toks[1] == int(np.argmax(w)) and sq.probs[step].top == []
    assert len(sp.probs) == len(sq.probs) == 5 and plain.probs == []


# ----------------------------------------------------------------------------- the native usual-case chain
def _random_params(rng, V):
    p = SamplingParams(
        temperature=float(rng.choice([0.05, 0.5, 0.8, 1.0, 2.5])), top_k=int(rng.integers(1, min(V - 1, 60) + 1)),
        top_p=float(rng.choice([1.0, 0.95, 0.9, 0.5, 0.01])), min_p=float(rng.choice([0.0, 0.05, 0.3, 1.0])),
        repeat_penalty=float(rng.choice([1.0, 1.1, 1.5])), presence_penalty=float(rng.choice([0.0, 0.4])),
        frequency_penalty=float(rng.choice([0.0, 0.25])), repeat_last_n=int(rng.choice([0, 5, 64])),
        seed=int(rng.integers(1, 1 << 40)))
    if rng.random() < 0.3:
        p.logit_bias = ((int(rng.integers(0, V)), float(rng.normal() * 3)), (V + 5, 1.0), (int(rng.integers(0, V)), float("-inf")))
    return p


def test_native_chain_picks_what_the_python_chain_picks():
    """Rows with the usual parameters run in csrc/sampler_core.cpp; the Python chain is its plain twin:
    same token, same generator state afterwards, same logits left behind, over random parameters,
    histories (with ids outside the vocabulary), NaN and -inf logits, and equal logits at the cut."""
    from airun_b200.sampling.sampler import sample_rows, usual_chain
    rng = np.random.default_rng(21)
    checked = 0
    for trial in range(300):
        V = int(rng.choice([41, 64, 300, 5000]))
        R = int(rng.integers(1, 7))
        params = [_random_params(rng, V) for _ in range(R)]
        assert all(usual_chain(p, V) for p in params)
        a = [Sampler(p) for p in params]
        b = [Sampler(SamplingParams(**p.__dict__)) for p in params]
        hist = [rng.integers(-2, V + 3, size=int(rng.integers(0, 90))).tolist() for _ in range(R)]
        for step in range(4):
            rows = (rng.normal(size=(R, V)) * float(rng.choice([0.5, 3.0, 12.0]))).astype(np.float32)
            if rng.random() < 0.3:
                rows[0, rng.integers(0, V, size=3)] = np.nan
            if rng.random() < 0.2:
                rows[-1, :] = -np.inf
            if rng.random() < 0.3:
                rows[0, : V // 2] = np.float32(1.25)                 # many equal logits: ties at the cut
            ra, rb = rows.copy(), rows.copy()
            ta = sample_rows(a, ra, hist)
            tb = sample_rows(b, rb, hist, native=False)
            assert ta == tb, (trial, step, [p for p in params])
            assert [s.rng.state for s in a] == [s.rng.state for s in b]
            assert np.array_equal(ra, rb, equal_nan=True)
            for r in range(R):
                hist[r].append(ta[r])
            checked += R
    assert checked > 3000


def test_native_chain_is_left_to_python_for_everything_else():
    from airun_b200.sampling.sampler import usual_chain
    V = 1000
    assert usual_chain(SamplingParams(), V)
    for kw in (dict(temperature=0.0), dict(top_k=0), dict(top_k=V), dict(top_k=5000), dict(typical_p=0.9), dict(top_n_sigma=1.0),
               dict(dry_multiplier=0.5), dict(dynatemp_range=0.2), dict(xtc_probability=0.1), dict(mirostat=2), dict(logprobs=0)):
        assert not usual_chain(SamplingParams(**kw), V), kw


def test_the_chain_on_a_rows_largest_logits_picks_what_the_whole_row_picks():
    """Requests whose chain cuts to the k largest logits send only their k + n + 1 largest raw logits to the host (n:
    the tokens the penalties may lower).  ``sample_candidates`` must pick the token the whole row gives and leave the
    generator where the whole row leaves it: rows with many equal values, histories that hit the largest logits,
    every stage behind the cut (typical, min-p, top-p, XTC, dynamic temperature), greedy with penalties."""
    from airun_b200.sampling.sampler import Sampler, SamplingParams, sample_candidates, sample_rows
    rng = np.random.default_rng(0)
    V = 5000
    for trial in range(1, 240):
        p = SamplingParams(temperature=float(rng.choice([0.0, 0.7, 1.3])), top_k=int(rng.choice([1, 5, 40, 100])),
                           top_p=float(rng.choice([1.0, 0.9, 0.5])), min_p=float(rng.choice([0.0, 0.05, 0.3])),
                           repeat_penalty=float(rng.choice([1.0, 1.1, 1.5])), presence_penalty=float(rng.choice([0, 0.5])),
                           frequency_penalty=float(rng.choice([0, 0.2])), repeat_last_n=int(rng.choice([0, 16, 64])),
                           seed=trial, typical_p=float(rng.choice([1.0, 0.8])), xtc_probability=float(rng.choice([0.0, 0.5])),
                           dynatemp_range=float(rng.choice([0.0, 0.3])))
        need = p.candidates_needed(512)
        assert need == (1 if p.temperature <= 0 else p.top_k) + (p.repeat_last_n if p.penalizing else 0) + 1
        row = (rng.standard_normal(V) * 3).astype(np.float32)
        if trial % 3 == 0:
            row = np.round(row)                                   # many equal values, also at the cut
        hist = rng.integers(0, V, 200).tolist()
        hist[-30:] = rng.choice(np.argsort(-row, kind="stable")[:60], 30).tolist()     # the penalties hit the top
        a, b = Sampler(p), Sampler(p)
        want = sample_rows([a], row.copy().reshape(1, -1), [hist])[0]
        order = np.lexsort((np.arange(V), -row))[:need]           # what the device kernel sends: value down, id up
        order = order[rng.permutation(need)]                      # in any order
        window = hist[-p.repeat_last_n:] if p.penalizing else []
        got = sample_candidates([b], order.astype(np.int32).reshape(1, -1), row[order].reshape(1, -1), [window])[0]
        assert got == want and a.rng.state == b.rng.state, (trial, p)
    # what needs the whole row says so
    assert SamplingParams(logit_bias=((3, 1.0),)).candidates_needed(512) == 0
    assert SamplingParams(top_k=0).candidates_needed(512) == 0 and SamplingParams(mirostat=2).candidates_needed(512) == 0
    assert SamplingParams(logprobs=0).candidates_needed(512) == 0 and SamplingParams(top_k=500).candidates_needed(512) == 0
    assert SamplingParams().candidates_needed(512) == 40 + 64 + 1
