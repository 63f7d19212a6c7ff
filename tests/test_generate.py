"""Generation through the Python entry point and the command line, on the GPU."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from helpers import ROOT, TINY, make_model_folder, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen_models")
    return {n: make_model_folder(n, str(root)) for n in TINY}


@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_matches_the_plain_implementation(name, folders):
    import airun_b200
    cfg, W = P.read_model_folder(folders[name])
    prompts = [random_tokens(n, cfg["vocab_size"], 50 + i) for i, n in enumerate((5, 17, 33))]
    want = [P.plain_greedy_generate(cfg, W, p, 16) for p in prompts]
    eng = airun_b200.Engine.from_folder(folders[name], dtype="float32", page_size=TINY[name]["page_size"],
                                        cache_tokens=512, max_batch_tokens=24, max_requests=4)
    got = eng.generate(prompts, airun_b200.SamplingParams.greedy(), max_new_tokens=16)
    assert [g.token_ids for g in got] == want
    assert all(g.finish_reason == "MaxTokens" for g in got)
    one = eng.generate(prompts[1], airun_b200.SamplingParams.greedy(), max_new_tokens=16)
    assert one.token_ids == want[1]                      # alone or in a batch: the same tokens
    assert eng.manager.free_pages() == {g.gid: eng.manager.num_pages for g in eng.manager.paged}


def test_generation_survives_preemption(folders):
    """A pool too small for all requests at once: some are preempted and recomputed, and
    every request still gets the tokens it gets when it runs alone."""
    import airun_b200
    name = "B"
    cfg, W = P.read_model_folder(folders[name])
    prompts = [random_tokens(n, cfg["vocab_size"], 80 + i) for i, n in enumerate((30, 26, 22, 18))]
    want = [P.plain_greedy_generate(cfg, W, p, 12) for p in prompts]
    eng = airun_b200.Engine.from_folder(folders[name], dtype="float32", page_size=8, num_pages=14,
                                        max_batch_tokens=32, max_requests=4, max_context=112)
    got = eng.generate(prompts, airun_b200.SamplingParams.greedy(), max_new_tokens=12)
    assert [g.token_ids for g in got] == want
    assert eng.scheduler.stats["preemptions"] >= 1
    eng.manager.check_invariants()


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(folders):
    import airun_b200
    name = "B"
    cfg, _ = P.read_model_folder(folders[name])
    prompts = [random_tokens(n, cfg["vocab_size"], 90 + i) for i, n in enumerate((70, 12, 9))]
    eng = airun_b200.Engine.from_folder(folders[name], dtype="float32", page_size=8, cache_tokens=1024,
                                        max_batch_tokens=24, max_requests=4)
    params = [airun_b200.SamplingParams.temperature_only(0.8, seed=100 + i) for i in range(3)]
    a = eng.generate(prompts, params, max_new_tokens=10)
    b = eng.generate(prompts, params, max_new_tokens=10)
    assert [x.token_ids for x in a] == [x.token_ids for x in b]
    alone = eng.generate(prompts[0], params[0], max_new_tokens=10)
    assert alone.token_ids == a[0].token_ids
    other = eng.generate(prompts[0], airun_b200.SamplingParams.temperature_only(0.8, seed=999), max_new_tokens=10)
    assert len(other.token_ids) == 10
    full = airun_b200.SamplingParams(seed=5)              # the whole chain runs on the host
    c = eng.generate(prompts[1], full, max_new_tokens=8)
    d = eng.generate(prompts[1], airun_b200.SamplingParams(seed=5), max_new_tokens=8)
    assert c.token_ids == d.token_ids and len(c.token_ids) == 8


def test_rows_sent_to_the_host_as_their_largest_logits_give_the_tokens_of_whole_rows(folders, monkeypatch):
    """A request whose chain cuts to its k largest logits travels to the host as k + n + 1 candidates found on the
    device; ``AIRUN_NARROW_ROWS=0`` sends whole rows instead.  Both must generate the same tokens: default parameters
    (top-k 40 with the repetition penalty over 64 tokens), greedy with penalties, a row beside device-sampled rows."""
    import airun_b200
    name = "B"
    cfg, _ = P.read_model_folder(folders[name])
    prompts = [random_tokens(n, cfg["vocab_size"], 190 + i) for i, n in enumerate((40, 12, 9, 30))]
    params = [airun_b200.SamplingParams(seed=7), airun_b200.SamplingParams(temperature=0.0, top_k=0, repeat_penalty=1.3, seed=1),
              airun_b200.SamplingParams.greedy(), airun_b200.SamplingParams(seed=9, top_k=5, min_p=0.0, top_p=0.8, xtc_probability=0.3)]
    out = {}
    for narrow in ("1", "0"):
        monkeypatch.setenv("AIRUN_NARROW_ROWS", narrow)
        eng = airun_b200.Engine.from_folder(folders[name], dtype="float32", page_size=8, cache_tokens=2048,
                                            max_batch_tokens=64, max_requests=4)
        assert eng._narrow_rows == (narrow == "1")
        res = eng.generate(prompts, [airun_b200.SamplingParams(**{**p.__dict__}) for p in params], max_new_tokens=24)
        out[narrow] = [r.token_ids for r in res]
        assert (eng._cand_bufs is not None) == (narrow == "1")
    assert out["1"] == out["0"] and all(len(t) == 24 for t in out["1"])
    # the way out when the kernel cannot vouch for a list (a second copy, of the whole row) gives the same tokens too
    monkeypatch.setenv("AIRUN_NARROW_ROWS", "1")
    eng = airun_b200.Engine.from_folder(folders[name], dtype="float32", page_size=8, cache_tokens=2048,
                                        max_batch_tokens=64, max_requests=4)
    eng._distrust_candidates = True
    res = eng.generate(prompts, [airun_b200.SamplingParams(**{**p.__dict__}) for p in params], max_new_tokens=24)
    assert [r.token_ids for r in res] == out["0"]


def test_end_token_stops_and_is_not_emitted(folders):
    import airun_b200
    cfg, W = P.read_model_folder(folders["B"])
    prompt = random_tokens(15, cfg["vocab_size"], 7)
    want = P.plain_greedy_generate(cfg, W, prompt, 8)
    eng = airun_b200.Engine.from_folder(folders["B"], dtype="float32", page_size=8, cache_tokens=256,
                                        max_batch_tokens=64, max_requests=2)
    stop = want[3]
    first = want.index(stop)
    got = eng.generate(prompt, airun_b200.SamplingParams.greedy(), max_new_tokens=8, eog_tokens=[stop])
    assert got.token_ids == want[:first] and got.finish_reason == "EndOfGeneration"


def test_command_line(folders, tmp_path):
    cfg, W = P.read_model_folder(folders["A"])
    prompt = random_tokens(9, cfg["vocab_size"], 3)
    want = P.plain_greedy_generate(cfg, W, prompt, 6)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "airun"), "run", folders["A"],
                          "-p", ",".join(map(str, prompt)), "-n", "6", "--temp", "0", "--repeat-penalty", "1.0",
                          "--dtype", "float32", "--cache-tokens", "256", "-q"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert [int(t) for t in out.stdout.strip().split(",")] == want


def test_smoke_entry():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as g
    g.smoke()


def test_perplexity_and_bench_subcommands(folders, tmp_path):
    """Token by token (the decode kernels) and in chunks (the prefill kernels) the loss agrees, and it
    is the plain implementation's (the reference's check: crates/airun-cli/src/perplexity.rs:9-11)."""
    import math
    import re
    cfg, W = P.read_model_folder(folders["C"])
    ids = random_tokens(90, cfg["vocab_size"], 21)
    def plain_loss(seq, first):
        logp = torch.log_softmax(P.plain_forward(cfg, W, seq, torch.float32).double(), dim=-1)
        return [-float(logp[r, seq[r + 1]]) for r in range(first, len(seq) - 1)]

    whole = plain_loss(ids, 0)
    chunks = [x for c in range(90 // 24) for x in plain_loss(ids[c * 24:(c + 1) * 24], 12)]   # second halves, fresh contexts
    f = tmp_path / "ids.txt"
    f.write_text(" ".join(map(str, ids)))
    for flags, want in (([], whole), (["--chunk", "24"], chunks), (["--chunk", "24", "--batched", "--worst", "2"], chunks)):
        out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "airun"), "perplexity", folders["C"],
                              "--file", str(f), "--dtype", "float32"] + flags, capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, out.stderr
        assert int(re.search(r"(\d+) tokens scored", out.stdout).group(1)) == len(want)
        assert abs(float(re.search(r"mean loss\s+([0-9.]+)", out.stdout).group(1)) - sum(want) / len(want)) < 2e-4
        assert ("worst-predicted" in out.stdout) == ("--worst" in flags)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "airun"), "bench", folders["C"], "--prefill", "33,64",
                          "--decode", "8", "--decode-at", "20", "--parallel", "2", "--runs", "2", "--temp", "0.7", "--json"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    import json
    rep = json.loads(out.stdout.strip().splitlines()[-1])
    assert set(rep["prefill"]) == {"33", "64"} and rep["decode"]["tokens_per_s"] > 0 and rep["decode"]["parallel"] == 2
    # several depths, random prompts, forwards only (the reference's options of the same names,
    # crates/airun-cli/src/bench.rs:23-27, 41-43, 73-77), and draws at a temperature
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "airun"), "bench", folders["C"], "--prefill", "16",
                          "--decode", "4", "--decode-at", "12,30", "--random-tokens", "--forward-only", "--runs", "1",
                          "--warmup", "0", "--json"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    rep = json.loads(out.stdout.strip().splitlines()[-1])
    assert set(rep["decode_at"]) == {"12", "30"} and all(v["tokens_per_s"] > 0 for v in rep["decode_at"].values())
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "airun"), "bench", folders["C"], "--prefill", "16",
                          "--decode", "4", "--temp", "0.7", "--runs", "1", "--warmup", "0", "-c", "8"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode != 0 and "--ctx-size" in out.stderr


@pytest.mark.parametrize("name", ["A", "B"])
def test_forked_requests_read_the_parents_pages_and_decode_on_their_own(name, folders):
    """A request is forked while it decodes (its last page partly filled): parent and children go on
    side by side and each gets the tokens the plain implementation gets for the same sequence."""
    import airun_b200
    cfg, W = P.read_model_folder(folders[name])
    ps = TINY[name]["page_size"]
    prompt = random_tokens(2 * ps + 3, cfg["vocab_size"], 130)
    want = P.plain_greedy_generate(cfg, W, prompt, 14)
    eng = airun_b200.Engine.from_folder(folders[name], dtype="float32", page_size=ps, cache_tokens=40 * ps,
                                        max_batch_tokens=24, max_requests=4)
    parent = eng.add_request(prompt, airun_b200.SamplingParams.greedy(), max_new_tokens=14)
    while len(parent.output) < 4:
        eng.run_step()
    free_before = eng.manager.free_pages()[0]
    kids = [eng.fork_request(parent, max_new_tokens=10) for _ in range(2)]
    # two whole pages are shared, each child took one page for the partly filled one
    assert eng.manager.free_pages()[0] == free_before - 2
    eng.manager.check_invariants()
    # a third child continues with another token than the parent sampled
    other = (parent.output[-1] + 1) % cfg["vocab_size"]
    odd = eng.fork_request(parent, max_new_tokens=6)
    odd.prompt[-1] = other
    want_odd = P.plain_greedy_generate(cfg, W, prompt + parent.output[:3] + [other], 6)
    while eng.has_work():
        eng.run_step()
        eng.manager.check_invariants()
    assert parent.output == want
    for k in kids:
        assert k.output == want[4:14]
    assert odd.output == want_odd
    assert eng.manager.free_pages() == {g.gid: eng.manager.num_pages for g in eng.manager.paged}


def test_cutting_a_request_back_and_going_on(folders):
    """The step function after ``truncate``: tokens past the cut are gone, the rest is still there,
    also when the cut falls inside a page that a fork shares."""
    from airun_b200.engine.step import StepEntry
    import airun_b200
    name = "B"
    cfg, W = P.read_model_folder(folders[name])
    V = cfg["vocab_size"]
    eng = airun_b200.Engine.from_folder(folders[name], dtype="float32", page_size=8, cache_tokens=256,
                                        max_batch_tokens=64, max_requests=4)
    first = random_tokens(29, V, 140)
    tail_a, tail_b = random_tokens(9, V, 141), random_tokens(7, V, 142)
    run, mgr = eng.runner, eng.manager
    mgr.add_request("a")
    run.step([StepEntry("a", first, ())])
    eng.storage.run_copies(mgr.fork("a", "b"))
    eng.storage.run_copies(mgr.truncate("b", 13))          # inside shared page 1
    eng.storage.run_copies(mgr.truncate("a", 24))          # at a page's edge
    mgr.check_invariants()
    got = run.step([StepEntry("a", tail_a, tuple(range(9))), StepEntry("b", tail_b, tuple(range(7)))]).cpu().numpy()
    want_a = P.plain_forward(cfg, W, first[:24] + tail_a).numpy()[24:]
    want_b = P.plain_forward(cfg, W, first[:13] + tail_b).numpy()[13:]
    from helpers import assert_close
    assert_close(got[:9], want_a, "float32", "request cut at a page's edge")
    assert_close(got[9:], want_b, "float32", "fork cut inside a shared page")


def test_selftest_subcommand_passes():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "airun"), "selftest", "--verbose"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "FAIL" not in r.stdout and "checks passed" in r.stdout


def test_next_step_laid_out_ahead_is_dropped_when_the_batch_changes(folders):
    """While a decode step runs, the engine lays out the next one.  A request that ends on an end
    token, one that is cancelled and one that arrives in between each make that lay-out stale; every
    request must still get the tokens it gets alone."""
    import airun_b200
    name = "A"
    cfg, W = P.read_model_folder(folders[name])
    prompts = [random_tokens(n, cfg["vocab_size"], 150 + i) for i, n in enumerate((9, 14, 20, 6))]
    want = [P.plain_greedy_generate(cfg, W, p, 24) for p in prompts]
    eog = want[1][7]                                    # request 1 meets its end token at its 8th token
    cut = want[1].index(eog)
    eng = airun_b200.Engine.from_folder(folders[name], dtype="float32", page_size=16, cache_tokens=1024,
                                        max_batch_tokens=32, max_requests=4)
    greedy = airun_b200.SamplingParams.greedy
    reqs = [eng.add_request(prompts[0], greedy(), max_new_tokens=24),
            eng.add_request(prompts[1], greedy(), max_new_tokens=24, eog_tokens=[eog]),
            eng.add_request(prompts[2], greedy(), max_new_tokens=24)]
    used_ahead = 0
    late = None
    while eng.has_work():
        if eng._ahead is not None:
            used_ahead += 1
        if late is None and len(reqs[0].output) == 12:
            late = eng.add_request(prompts[3], greedy(), max_new_tokens=24)      # arrives while others decode
        if len(reqs[2].output) == 15:
            reqs[2].cancelled = True
        eng.run_step()
        eng.manager.check_invariants()
    assert used_ahead > 5, "the look-ahead path never ran"
    assert reqs[0].output == want[0] and late.output == want[3]
    assert reqs[1].output == want[1][:cut] and reqs[1].finished.value == "EndOfGeneration"
    assert reqs[2].output == want[2][:len(reqs[2].output)] and reqs[2].finished.value == "Cancelled"
    assert eng.manager.free_pages() == {g.gid: eng.manager.num_pages for g in eng.manager.paged}


@pytest.mark.parametrize("seed,name,dtype", [(1, "B", "float32"), (2, "B", "float32"), (3, "B", "bfloat16"),
                                             (4, "D", "bfloat16")])
def test_random_arrivals_forks_and_cancellations_under_a_small_pool(seed, name, dtype, folders):
    """Forty requests arrive at random moments into an engine whose pool holds two or three of them:
    portions, preemption and recomputation, forks that share pages, cancellations, end tokens, the
    look-ahead path, graph replays.  In float32 every token every request ever gets must be the token the
    plain implementation gets for the same sequence; in bfloat16 (B: the mma.sync attention at head size
    32; D: the tcgen05 and TMA attention at head size 128) every token must be, for the plain implementation
    that rounds where the engine does, within twice that rounding's own effect of its best token.  In the
    end every page is back."""
    import random
    import airun_b200
    cfg, W = P.read_model_folder(folders[name])
    V = cfg["vocab_size"]
    rng = random.Random(seed)
    ps = TINY[name]["page_size"]
    eng = airun_b200.Engine.from_folder(folders[name], dtype=dtype, page_size=ps, num_pages=22 * 8 // ps,
                                        max_batch_tokens=48, max_requests=6, max_context=120)
    greedy = airun_b200.SamplingParams.greedy
    plain_cache = {}

    def plain(prompt, n):
        key = tuple(prompt)
        if key not in plain_cache or len(plain_cache[key]) < n:
            plain_cache[key] = P.plain_greedy_generate(cfg, W, list(prompt), n)
        return plain_cache[key][:n]

    pending = [random_tokens(rng.randint(3, 60), V, 1000 * seed + i) for i in range(40)]
    live = []                    # (request, prompt it started from, tokens wanted)
    done = []
    steps = 0
    while pending or eng.has_work():
        if pending and rng.random() < 0.35:
            p = pending.pop()
            n = rng.randint(1, 24)
            eog = ()
            if rng.random() < 0.3:                          # ends early on one of its own tokens
                eog = (plain(p, n)[rng.randrange(n)],)
            live.append((eng.add_request(p, greedy(), max_new_tokens=n, eog_tokens=eog), p, n))
        running = [t for t in live if t[0] in eng.scheduler.running and t[0].output and t[0].finished is None]
        if running and rng.random() < 0.08 and eng.manager.has_free_slot():
            parent, pp, pn = rng.choice(running)
            if parent.num_computed == parent.num_tokens - 1:
                try:
                    child = eng.fork_request(parent, max_new_tokens=rng.randint(1, 10))
                    live.append((child, list(child.prompt), child.max_new_tokens))
                except Exception as e:                       # out of pages or slots: the fork is refused whole
                    assert type(e).__name__ in ("OutOfPages", "CacheError"), e
        if running and rng.random() < 0.04:
            rng.choice(running)[0].cancelled = True
        if eng.has_work():
            eng.run_step()
            steps += 1
            eng.manager.check_invariants()
        assert steps < 5000, "the engine does not come to an end"
    assert eng.scheduler.stats["preemptions"] > 0, "the pool was meant to be too small"
    for req, prompt, n in live:
        assert req.finished is not None
        if req.finished.value == "Refused":
            continue
        got = req.output
        if req.finished.value == "MaxTokens":
            assert len(got) == n
        if dtype == "float32":
            want = plain(prompt, n)
            assert got == want[:len(got)], (req.rid, req.finished, len(prompt))
            if req.finished.value == "EndOfGeneration":
                assert want[len(got)] in req.eog_tokens
            continue
        # one pass over prompt + output scores every choice (position len(prompt) - 1 + t chose token t)
        seq = list(prompt) + list(got)
        rounded = P.plain_forward(cfg, W, seq, torch.float32, round_to=torch.bfloat16)
        exact = P.plain_forward(cfg, W, seq, torch.float32)
        noise = (rounded - exact).abs().max(dim=-1).values
        first = len(prompt) - 1
        for t, tok in enumerate(got):
            row = rounded[first + t]
            assert float(row.max() - row[tok]) <= 2 * float(noise[first + t]) + 1e-3, (req.rid, t, req.finished)
        if req.finished.value == "EndOfGeneration":
            row = rounded[first + len(got)]
            assert min(float(row.max() - row[e]) for e in req.eog_tokens) <= 2 * float(noise[first + len(got)]) + 1e-3
    assert eng.manager.free_pages() == {g.gid: eng.manager.num_pages for g in eng.manager.paged}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_more_than_a_hundred_requests(dtype, folders):
    """One step of 128 single tokens, then one of 100 single tokens beside a prompt portion, through the
    step function (batch sizes above every other test's, the largest graph bucket), each row against the
    plain implementation on its own sequence."""
    import airun_b200
    from airun_b200 import StepEntry
    from helpers import assert_close, bf16_noise
    name = "B"
    cfg, W = P.read_model_folder(folders[name])
    V = cfg["vocab_size"]
    eng = airun_b200.Engine.from_folder(folders[name], dtype=dtype, page_size=8, cache_tokens=128 * 40 + 256,
                                        max_batch_tokens=256, max_requests=130, max_context=64)
    assert eng.runner.graph_buckets[-1] >= 128
    seqs = [random_tokens(3 + (7 * i) % 28, V, 5000 + i) for i in range(128)]
    long_one = random_tokens(61, V, 6000)
    for i in range(128):
        eng.manager.add_request(i)
    eng.manager.add_request("p")
    # prompts, all but the last two tokens of each, in steps of up to 256 tokens
    batch, count = [], 0
    for i, s in enumerate(seqs):
        if count + len(s) - 2 > 256 or len(batch) == 130:
            eng.runner.step(batch)
            batch, count = [], 0
        batch.append(StepEntry(i, s[:-2], ()))
        count += len(s) - 2
    eng.runner.step(batch)
    got = {}
    for rep in range(2):                                   # twice: the first step of a size runs kernel by kernel, the second is captured
        a = eng.runner.step([StepEntry(i, [seqs[i][-2]], (0,)) for i in range(128)]).float().cpu().numpy()
        for i in range(128):
            eng.manager.truncate(i, len(seqs[i]) - 2)
        got["a"] = a
    a = eng.runner.step([StepEntry(i, [seqs[i][-2]], (0,)) for i in range(128)]).float().cpu().numpy()
    b = eng.runner.step([StepEntry(i, [seqs[i][-1]], (0,)) for i in range(100)]
                        + [StepEntry("p", long_one, (0, 60))]).float().cpu().numpy()
    eng.runner.raise_on_device_error()
    for i in list(range(0, 128, 9)) + [127]:
        exact = P.plain_forward(cfg, W, seqs[i], torch.float32).numpy()
        want = exact if dtype == "float32" else P.plain_forward(cfg, W, seqs[i], torch.float32, round_to=torch.bfloat16).numpy()
        noise = bf16_noise(want, exact)
        assert_close(a[i:i + 1], want[-2:-1], dtype, f"128 rows, request {i}", noise[-2:-1])
        if i < 100:
            assert_close(b[i:i + 1], want[-1:], dtype, f"100 rows + a portion, request {i}", noise[-1:])
    exact = P.plain_forward(cfg, W, long_one, torch.float32).numpy()
    want = exact if dtype == "float32" else P.plain_forward(cfg, W, long_one, torch.float32, round_to=torch.bfloat16).numpy()
    assert_close(b[100:], want[[0, 60]], dtype, "the portion beside 100 single tokens", bf16_noise(want, exact)[[0, 60]])


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("A", "bfloat16")])
def test_turns_of_a_conversation_start_from_the_kept_cache(name, dtype, folders):
    """With ``prefix_cache`` a finished request's pages are kept; a prompt that begins like it (the
    next turn of a conversation: the first prompt, its answer and more) starts from them.  The tokens
    are the ones the plain implementation gets for the whole prompt, in a pool so small that kept
    caches must give way, and beside a request that shares nothing."""
    import airun_b200
    cfg, W = P.read_model_folder(folders[name])
    V, ps = cfg["vocab_size"], TINY[name]["page_size"]
    eng = airun_b200.Engine.from_folder(folders[name], dtype=dtype, page_size=ps, num_pages={"A": 10, "B": 17}[name],
                                        max_batch_tokens=32, max_requests=4, max_context=128, prefix_cache=True)
    greedy = airun_b200.SamplingParams.greedy()

    def agree(prompt, got, what):
        if dtype == "float32":
            assert got == P.plain_greedy_generate(cfg, W, prompt, len(got)), what
        else:
            # bfloat16: a near-tie may flip with the kernels a token went through (a portion's, a single
            # token's).  Every token chosen must be, for the plain implementation that rounds where the
            # engine does, within twice that rounding's own effect on the logits of its best token.
            seq = list(prompt)
            for t in got:
                rounded = P.plain_forward(cfg, W, seq, torch.float32, round_to=torch.bfloat16)[-1]
                exact = P.plain_forward(cfg, W, seq, torch.float32)[-1]
                noise = float((rounded - exact).abs().max())
                assert float(rounded.max() - rounded[t]) <= 2 * noise + 1e-3, what
                seq.append(t)

    turn1 = random_tokens(3 * ps + 5, V, 300)
    out1 = eng.generate(turn1, greedy, max_new_tokens=9).token_ids
    agree(turn1, out1, "first turn")
    assert len(eng.scheduler.kept) == 1
    turn2 = turn1 + out1 + random_tokens(11, V, 301)
    other = random_tokens(2 * ps + 3, V, 302)
    res = eng.generate([turn2, other], greedy, max_new_tokens=7)
    agree(turn2, res[0].token_ids, "second turn, from the kept cache")
    agree(other, res[1].token_ids, "a request that shares nothing")
    st = eng.scheduler.stats
    assert st["prefix_hits"] == 1 and st["prefix_tokens"] == len(turn1) + len(out1) - 1
    # the same prompt again: all but its last token comes from the cache
    again = eng.generate(turn2, greedy, max_new_tokens=7).token_ids
    agree(turn2, again, "the same prompt again")
    assert st["prefix_hits"] == 2 and st["prefix_tokens"] == len(turn1) + len(out1) - 1 + len(turn2) - 1
    # a prompt that diverges inside a page, while the pool is too small for every kept cache
    turn3 = turn2[:2 * ps + 3] + random_tokens(40, V, 303)
    out3 = eng.generate(turn3, greedy, max_new_tokens=6).token_ids
    agree(turn3, out3, "third prompt, cut inside a shared page")
    assert st["prefix_hits"] == 3 and st["prefix_evictions"] >= 1
    eng.manager.check_invariants()
    while eng.scheduler._drop_kept():
        pass
    assert eng.manager.free_pages() == {g.gid: eng.manager.num_pages for g in eng.manager.paged}
