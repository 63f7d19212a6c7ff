"""The host sampling chain against the cases of the reference's own sampler tests.

The reference's sampler cannot be run here (Rust; no cargo or rustc), but its unit tests state
inputs and expected outputs in the open (crates/airun-core/src/sample.rs:846-1111).  Those pairs
are restated here as data and put to this package's chain; each test names the lines it comes
from.  No GPU."""
import numpy as np
import pytest

from airun_b200.sampling.sampler import (Sampler, SamplingParams, _typical, apply_dry, apply_penalties,
                                         apply_top_n_sigma)


def f32(values):
    return np.array(values, dtype=np.float32)


def test_greedy_picks_the_maximum():                                     # sample.rs:846-850
    assert Sampler(SamplingParams.greedy()).sample(f32([0.1, 5.0, 0.3, 2.0]), []) == 1


def test_dry_case():                                                     # sample.rs:853-871
    history = [1, 2, 3, 9, 1, 2]                                         # 3 would repeat "1 2 3"; 4 would not
    logits = np.zeros(10, dtype=np.float32)
    apply_dry(logits, history, multiplier=1.0, base=1.75, allowed_length=2, last_n=0)
    assert logits[3] < 0.0 and logits[4] == 0.0
    logits = np.zeros(10, dtype=np.float32)
    apply_dry(logits, history, 1.0, 1.75, 2, 0, breakers=(2,))           # a breaker inside the repeat ends it
    assert logits[3] == 0.0


@pytest.mark.parametrize("version", [1, 2])
def test_mirostat_samples_from_the_head_and_adapts(version):             # sample.rs:905-918
    p = SamplingParams.greedy()
    p.temperature, p.mirostat, p.seed = 1.0, version, 9
    s = Sampler(p)
    mu0 = s.mu
    base = f32([-i * 0.05 for i in range(1000)])
    for _ in range(20):
        assert 0 <= s.sample(base.copy(), []) < 1000
    assert s.mu != mu0


def test_top_k_of_one_is_deterministic():                                # sample.rs:921-937
    s = Sampler(SamplingParams(temperature=1.0, top_k=1, top_p=1.0, min_p=0.0, repeat_penalty=1.0, repeat_last_n=0, seed=42))
    assert all(s.sample(f32([0.1, 5.0, 0.3, 2.0]), []) == 1 for _ in range(20))


def test_a_fixed_seed_reproduces_the_same_sequence():                    # sample.rs:940-955
    def run():
        s = Sampler(SamplingParams(seed=12345))
        return [s.sample(f32([1.0, 1.2, 0.9, 1.1, 0.8, 1.05]), []) for _ in range(16)]
    assert run() == run()


def penalties(logits, history, last_n, repeat, presence, frequency):
    x = f32(logits)
    apply_penalties(x, history, last_n, repeat, presence, frequency)
    return x.tolist()


def test_penalty_cases():
    assert penalties([2.0, -2.0, 1.0], [0, 1], 8, 2.0, 0.0, 0.0) == [1.0, -4.0, 1.0]        # sample.rs:958-964
    assert penalties([2.0, 2.0], [0, 1], 1, 2.0, 0.0, 0.0) == [2.0, 1.0]                     # :967-973, the window
    assert penalties([5.0, 5.0, 5.0], [0, 0, 0], 8, 1.0, 0.0, 1.0)[0] == 2.0                 # :978-990
    assert penalties([5.0, 5.0, 5.0], [1], 8, 1.0, 0.0, 1.0) == [5.0, 4.0, 5.0]              # nothing left over from the call before
    history = [0, 0, 1, 0]                                                                   # :993-1008
    assert penalties([5.0, 5.0, 5.0], history, 8, 1.0, 0.5, 0.0) == [4.5, 4.5, 5.0]          # presence is flat
    assert penalties([5.0, 5.0, 5.0], history, 8, 1.0, 0.0, 0.5) == [3.5, 4.5, 5.0]          # frequency counts
    assert penalties([8.0], [0, 0, 0], 8, 2.0, 0.0, 0.0) == [4.0]                            # :1011-1017, once per token


def test_logit_bias_can_ban_and_promote():                               # sample.rs:1020-1030
    p = SamplingParams.greedy()
    p.logit_bias = ((1, float("-inf")), (3, 100.0))
    assert Sampler(p).sample(f32([0.1, 5.0, 0.3, 2.0]), []) == 3


def test_top_n_sigma_cases():
    logits = np.zeros(64, dtype=np.float32)                              # sample.rs:1033-1041
    logits[7] = 20.0
    apply_top_n_sigma(logits, 1.0)
    assert logits[7] == 20.0 and all(l == -np.inf for i, l in enumerate(logits) if i != 7)
    flat = np.ones(32, dtype=np.float32)                                 # :1044-1050: zero spread filters nothing
    apply_top_n_sigma(flat, 1.0)
    assert (flat == 1.0).all()


def test_typical_p_can_drop_the_most_likely_token():                     # sample.rs:1053-1078
    ids = np.arange(32)
    probs = f32([0.5, 0.2] + [0.01] * 30)
    got_ids, got_probs = _typical(ids, probs, 0.15)
    assert got_ids.tolist() == [1] and got_probs.tolist() == [np.float32(0.2)]            # the peak is not the typical token
    got_ids, got_probs = _typical(ids, probs, 0.5)
    assert got_ids.tolist() == [0, 1] and got_probs.tolist() == [np.float32(0.5), np.float32(0.2)]   # back in probability order


def test_every_filter_keeps_at_least_one_candidate():                    # sample.rs:1081-1110
    for kw in (dict(min_p=0.99), dict(top_p=0.0), dict(typical_p=0.0),
               dict(top_k=0, min_p=1.0, typical_p=0.01, top_p=0.01)):
        s = Sampler(SamplingParams(seed=7, **kw))
        assert 0 <= s.sample(np.ones(64, dtype=np.float32), []) < 64
