"""A model large enough to reach the kernels the tiny configurations never touch inside the
engine (head size 128 on tcgen05 attention and TMA decode attention, many-tile persistent
products, split-K decode products): its bfloat16 path against its own float32 path, and its
execution modes against one another."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import plain_qwen3 as P                                   # noqa: E402
from helpers import assert_close, bf16_noise, plain_random_weights   # noqa: E402

pytestmark = pytest.mark.gpu

MID = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=20000, hidden_size=1024,
           num_hidden_layers=3, num_attention_heads=16, num_key_value_heads=4, head_dim=128,
           intermediate_size=2816, max_position_embeddings=4096, rms_norm_eps=1e-6, rope_theta=1000000.0,
           tie_word_embeddings=False)


def logits_of(eng, plan):
    """plan: list of steps, each a list of (rid, tokens); every token's logits are wanted.
    Returns {rid: [T, V] float32}."""
    from airun_b200 import StepEntry
    got = {}
    for step in plan:
        for rid, _ in step:
            if rid not in eng.manager.requests:
                eng.manager.add_request(rid)
        out = eng.runner.step([StepEntry(rid, toks, tuple(range(len(toks)))) for rid, toks in step]).float().cpu().numpy()
        r = 0
        for rid, toks in step:
            got.setdefault(rid, []).append(out[r:r + len(toks)])
            r += len(toks)
    eng.runner.raise_on_device_error()
    for rid in list(eng.manager.requests):
        eng.manager.free_request(rid)
    return {rid: np.concatenate(v) for rid, v in got.items()}


def cosine(a, b):
    return float((a * b).sum() / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30))


@pytest.fixture(scope="module")
def engines():
    import airun_b200
    cfg = airun_b200.Qwen3Config.from_dict(MID)
    out = {}
    for dt in ("float32", "bfloat16"):
        out[dt] = airun_b200.Engine.from_config(cfg, seed=3, dtype=dt, page_size=16, cache_tokens=4096,
                                                max_batch_tokens=1024, max_requests=8, max_context=2048)
    return out


@pytest.fixture(scope="module")
def plain_mid():
    """The plain implementation on the weights ``Engine.from_config(MID, seed=3)`` fills the device with
    (made again on the CPU from the seed), for two sequences: without rounding and with the bfloat16
    path's rounding places."""
    W = plain_random_weights(MID, 3)
    g = np.random.default_rng(5)
    seqs = {"a": [int(t) for t in g.integers(0, MID["vocab_size"], size=700)],
            "b": [int(t) for t in g.integers(0, MID["vocab_size"], size=333)]}
    exact = {r: P.plain_forward(MID, W, s, torch.float32).numpy() for r, s in seqs.items()}
    rounded = {r: P.plain_forward(MID, W, s, torch.float32, round_to=torch.bfloat16).numpy() for r, s in seqs.items()}
    return seqs, exact, rounded


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_and_cut_against_the_plain_implementation(engines, plain_mid, dtype):
    """Head size 128 on the tcgen05 attention and the TMA decode attention, persistent many-tile
    products and split-K decode products, inside the engine, against the plain implementation: each
    request whole, then cut into portions beside the other request and single tokens from graphs."""
    seqs, exact, rounded = plain_mid
    a, b = seqs["a"], seqs["b"]
    want = exact if dtype == "float32" else rounded
    whole = logits_of(engines[dtype], [[("a", a)], [("b", b)]])
    cut = [[("a", a[:300])], [("a", a[300:302]), ("b", b[:129])], [("a", a[302:650]), ("b", b[129:300])]]
    cut += [[("a", [a[650 + i]]), ("b", [b[300 + i]])] for i in range(33)]
    cut += [[("a", a[683:])]]
    mixed = logits_of(engines[dtype], cut)
    for rid in ("a", "b"):
        noise = bf16_noise(rounded[rid], exact[rid])
        assert_close(whole[rid], want[rid], dtype, f"mid {dtype} whole {rid}", noise)
        assert_close(mixed[rid], want[rid], dtype, f"mid {dtype} cut {rid}", noise)


def test_forks_against_the_plain_implementation(engines):
    """Four requests forked from one 1,300-token prompt and decoded side by side (the shared pages are
    read once per step for all of them), each against the plain implementation on prompt + its tail."""
    from airun_b200 import StepEntry
    W = plain_random_weights(MID, 3)
    g = np.random.default_rng(21)
    n_prompt = 1100
    prompt = [int(t) for t in g.integers(0, MID["vocab_size"], size=n_prompt)]
    tails = [[int(t) for t in g.integers(0, MID["vocab_size"], size=6)] for _ in range(4)]
    eng = engines["bfloat16"]
    m = eng.manager
    m.add_request("p")
    eng.runner.step([StepEntry("p", prompt[:700], ())])
    eng.runner.step([StepEntry("p", prompt[700:], ())])
    rids = ["p", "f1", "f2", "f3"]
    for r in rids[1:]:
        eng.storage.run_copies(m.fork("p", r))
    rows = [eng.runner.step([StepEntry(r, [tails[i][k]], (0,)) for i, r in enumerate(rids)]).float().cpu().numpy()
            for k in range(6)]
    eng.runner.raise_on_device_error()
    assert any(isinstance(k, tuple) and k[0] == "shared" for k in eng.runner.graphs), "the shared-prefix path never ran"
    for r in rids:
        m.free_request(r)
    got = np.stack(rows)                                          # [step, request, V]
    for i in (3,):
        seq = prompt + tails[i]
        exact = P.plain_forward(MID, W, seq, torch.float32).numpy()[n_prompt:]
        rounded = P.plain_forward(MID, W, seq, torch.float32, round_to=torch.bfloat16).numpy()[n_prompt:]
        assert_close(got[:, i], rounded, "bfloat16", f"fork {i}", bf16_noise(rounded, exact))


def test_bfloat16_path_agrees_with_the_float32_path_and_with_itself(engines):
    g = np.random.default_rng(5)
    a = [int(t) for t in g.integers(0, MID["vocab_size"], size=700)]
    b = [int(t) for t in g.integers(0, MID["vocab_size"], size=333)]
    whole = [[("a", a)], [("b", b)]]
    ref = logits_of(engines["float32"], whole)
    bf = logits_of(engines["bfloat16"], whole)
    for rid in ("a", "b"):
        # the reference's own whole-model criterion for a reduced-precision path: cosine > 0.999 and
        # the same argmax (crates/airun-core/tests/prefill.rs:45-46); here for every position
        cos = [cosine(ref[rid][t], bf[rid][t]) for t in range(ref[rid].shape[0])]
        assert min(cos) > 0.999, (rid, min(cos), int(np.argmin(cos)))
        same = np.mean(ref[rid].argmax(-1) == bf[rid].argmax(-1))
        assert same > 0.97, (rid, same)
    # the same tokens cut differently: portions of changing size, then single tokens (graph replay),
    # side by side with the other request
    cut = [[("a", a[:300])], [("a", a[300:302]), ("b", b[:129])], [("a", a[302:650]), ("b", b[129:300])]]
    cut += [[("a", [a[650 + i]]), ("b", [b[300 + i]])] for i in range(33)]
    cut += [[("a", a[683:])]]
    mixed = logits_of(engines["bfloat16"], cut)
    noise = {rid: float(np.abs(bf[rid] - ref[rid]).max()) for rid in ref}
    for rid in ("a", "b"):
        err = float(np.abs(mixed[rid] - bf[rid]).max())
        # cutting the sequence differently moves the logits no more than bfloat16 itself does
        assert err <= noise[rid] + 1e-3, (rid, err, noise[rid])
    mixed32 = logits_of(engines["float32"], cut)
    for rid in ("a", "b"):
        scale = float(np.abs(ref[rid]).max())
        assert float(np.abs(mixed32[rid] - ref[rid]).max()) <= 2e-4 * scale + 2e-5, rid


def test_greedy_generation_in_a_batch_picks_defensible_tokens(engines):
    """Random weights give nearly flat logits, so a near-tie may flip with the batch size (other tile
    shapes, other slice counts) and the texts then part for good.  What must hold: in float32 the
    batch and the lone run agree token for token; in bfloat16 every token the batched run chose is,
    when the lone run scores the same context, within twice the bfloat16 noise of its best token."""
    import airun_b200
    from airun_b200 import StepEntry
    g = np.random.default_rng(6)
    prompts = [[int(t) for t in g.integers(0, MID["vocab_size"], size=n)] for n in (40, 300, 7, 129)]
    greedy = airun_b200.SamplingParams.greedy()
    e32, e16 = engines["float32"], engines["bfloat16"]
    together32 = e32.generate(prompts, greedy, max_new_tokens=24)
    assert e32.generate(prompts[1], greedy, max_new_tokens=24).token_ids == together32[1].token_ids
    together = e16.generate(prompts, greedy, max_new_tokens=24)
    for i in (1, 3):
        seq = prompts[i] + together[i].token_ids
        n = len(prompts[i])
        want = tuple(range(n - 1, len(seq) - 1))                 # the positions that chose the 24 tokens
        outs = {}
        for name, eng in (("b", e16), ("f", e32)):
            eng.manager.add_request("solo")
            outs[name] = eng.runner.step([StepEntry("solo", seq, want)]).float().cpu().numpy()
            eng.manager.free_request("solo")
        noise = float(np.abs(outs["b"] - outs["f"]).max())
        for t, tok in enumerate(together[i].token_ids):
            gap = float(outs["b"][t].max() - outs["b"][t][tok])
            assert gap <= 2 * noise + 1e-3, (i, t, gap, noise)
    assert e16.manager.free_pages() == {gr.gid: e16.manager.num_pages for gr in e16.manager.paged}


def test_folded_norms_give_the_same_logits(engines):
    """RMSNorm folded into the products around it (off by default) against the separate kernels."""
    from airun_b200.kernels import fast
    eng = engines["bfloat16"]
    g = np.random.default_rng(9)
    a = [int(t) for t in g.integers(0, MID["vocab_size"], size=400)]
    b = [int(t) for t in g.integers(0, MID["vocab_size"], size=37)]
    plan = [[("a", a[:390]), ("b", b[:30])]] + [[("a", [a[390 + i]]), ("b", [b[30 + i]])] for i in range(7)]
    plain = logits_of(eng, plan)
    ref = logits_of(engines["float32"], plan)
    old = fast.NORM_FUSION
    fast.NORM_FUSION = True
    saved = (dict(eng.runner.graphs), set(eng.runner._warm_buckets))
    eng.runner.graphs.clear()
    eng.runner._warm_buckets.clear()                 # graphs captured without the fusion must not be replayed
    try:
        fused = logits_of(eng, plan)
    finally:
        fast.NORM_FUSION = old
        eng.runner.graphs.clear()
        eng.runner._warm_buckets.clear()
        eng.runner.graphs.update(saved[0])
        eng.runner._warm_buckets.update(saved[1])
    for rid in ("a", "b"):
        noise = float(np.abs(plain[rid] - ref[rid]).max())
        assert float(np.abs(fused[rid] - plain[rid]).max()) <= noise + 1e-3, rid
        assert float(np.abs(fused[rid] - plain[rid]).max()) > 0.0      # it really took the other path


def test_long_context_in_portions_then_decoding():
    """Five thousand tokens in portions of 1024, then single tokens: block tables of hundreds of
    pages, positions in the thousands, many key tiles and several key slices per token."""
    import airun_b200
    cfg = airun_b200.Qwen3Config.from_dict(dict(MID, num_hidden_layers=2, vocab_size=5000))
    g = np.random.default_rng(11)
    seq = [int(t) for t in g.integers(0, 5000, size=5030)]
    want_at = [1023, 2047, 4095, 4999]                        # ends of portions, the page edge at 4096
    outs = {}
    for dt in ("float32", "bfloat16"):
        eng = airun_b200.Engine.from_config(cfg, seed=4, dtype=dt, page_size=16, cache_tokens=5120,
                                            max_batch_tokens=1024, max_requests=2, max_context=5120)
        from airun_b200 import StepEntry
        eng.manager.add_request("r")
        rows = []
        for p0 in range(0, 5000, 1024):
            part = seq[p0:min(p0 + 1024, 5000)]
            want = tuple(w - p0 for w in want_at if p0 <= w < p0 + len(part))
            out = eng.runner.step([StepEntry("r", part, want)])
            if want:
                rows.append(out.float().cpu().numpy())
        for t in seq[5000:]:
            rows.append(eng.runner.step([StepEntry("r", [t], (0,))]).float().cpu().numpy())
        eng.runner.raise_on_device_error()
        outs[dt] = np.concatenate(rows)
        del eng
        torch.cuda.empty_cache()
    assert outs["float32"].shape == (len(want_at) + 30, 5000)
    for i in range(outs["float32"].shape[0]):
        assert cosine(outs["float32"][i], outs["bfloat16"][i]) > 0.999, i
    assert np.mean(outs["float32"].argmax(-1) == outs["bfloat16"].argmax(-1)) > 0.9


def test_layers_of_the_8b_size_bfloat16_agrees_with_float32():
    """Two layers with the sizes of the benchmark's model (hidden 4096, 32/8 heads of 128,
    intermediate 12288, vocabulary 151936): a 200-token prompt in two portions, then eight single
    tokens, the bfloat16 path against the float32 path on the same weights."""
    import airun_b200
    from airun_b200 import StepEntry
    cfg = airun_b200.Qwen3Config.from_dict(dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
        num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
        max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False))
    g = np.random.default_rng(12)
    seq = [int(t) for t in g.integers(0, 151936, size=208)]
    outs = {}
    for dt in ("float32", "bfloat16"):
        eng = airun_b200.Engine.from_config(cfg, seed=6, dtype=dt, page_size=16, cache_tokens=512,
                                            max_batch_tokens=256, max_requests=2, max_context=512)
        eng.manager.add_request("r")
        rows = [eng.runner.step([StepEntry("r", seq[:130], (0, 64, 129))]).float().cpu().numpy(),
                eng.runner.step([StepEntry("r", seq[130:200], (69,))]).float().cpu().numpy()]
        for t in seq[200:]:
            rows.append(eng.runner.step([StepEntry("r", [t], (0,))]).float().cpu().numpy())
        eng.runner.raise_on_device_error()
        outs[dt] = np.concatenate(rows)
        del eng
        torch.cuda.empty_cache()
    assert outs["float32"].shape == (12, 151936)
    for i in range(12):
        assert cosine(outs["float32"][i], outs["bfloat16"][i]) > 0.999, i
        # the token the bfloat16 path picks is, on the float32 path, within bfloat16's own noise of the best
        pick = int(outs["bfloat16"][i].argmax())
        noise = float(np.abs(outs["float32"][i] - outs["bfloat16"][i]).max())
        assert outs["float32"][i].max() - outs["float32"][i][pick] <= 2 * noise, i


def test_forked_requests_read_their_shared_prompt_once(engines):
    """Four requests forked from one 1,300-token prompt decode side by side: the step's attention reads
    the pages they share once for all of them (a graph of its own).  The logits must be those of the
    same step with that path switched off, up to the order of sums."""
    from airun_b200 import StepEntry
    eng = engines["bfloat16"]
    g = np.random.default_rng(21)
    prompt = [int(t) for t in g.integers(0, MID["vocab_size"], size=1300)]
    tails = [[int(t) for t in g.integers(0, MID["vocab_size"], size=14)] for _ in range(4)]
    outs = {}
    for shared_path in (True, False):
        eng.runner.SHARED_PREFIX_MIN = 1024 if shared_path else 1 << 30
        m = eng.manager
        m.add_request("p")
        eng.runner.step([StepEntry("p", prompt[:700], ())])
        eng.runner.step([StepEntry("p", prompt[700:], ())])
        for i in range(1, 4):
            eng.storage.run_copies(m.fork("p", f"f{i}"))
        rids = ["p", "f1", "f2", "f3"]
        rows = []
        for k in range(14):
            if k == 9:                                    # one of them leaves: three go on sharing
                m.free_request("f2")
                rids.remove("f2")
            idx = [("p", "f1", "f2", "f3").index(r) for r in rids]
            out = eng.runner.step([StepEntry(r, [tails[i][k]], (0,)) for r, i in zip(rids, idx)])
            rows.append(out.float().cpu().numpy())
        eng.runner.raise_on_device_error()
        outs[shared_path] = np.concatenate(rows)
        if shared_path:
            assert any(isinstance(k, tuple) and k[0] == "shared" for k in eng.runner.graphs), "the shared-prefix path never ran"
        for r in rids:
            m.free_request(r)
        m.check_invariants()
    eng.runner.SHARED_PREFIX_MIN = 1024
    a, b = outs[True], outs[False]
    assert a.shape == b.shape and np.isfinite(a).all()
    scale = float(np.abs(b).max())
    assert float(np.abs(a - b).max()) <= 0.02 * scale, float(np.abs(a - b).max()) / scale
    for i in range(a.shape[0]):
        assert cosine(a[i], b[i]) > 0.9999, i
