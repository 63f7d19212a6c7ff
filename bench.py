#!/usr/bin/env python3
"""Benchmark: decode tokens a second of the Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context C]

A step is one decode step of a batch of requests whose contexts stand at
``context`` tokens.  Weights are random N(0, 0.02); the caches are filled with
random keys and values (synthetic data) so that no time goes to prefilling them.
Prints ONE JSON line: ``value`` is the device-timed decode rate of the step
function, ``e2e`` the rate through the Python entry point (scheduler, sampling,
host tokens in and out; ``sampled_with_reference_defaults`` inside it: the same with the reference's default
sampling parameters instead of greedy picks), ``prefill`` a 2,048-token prompt in one step,
``roofline`` the bytes a decode step must read over its time, ``points`` the
decode rate at batch 1 and 64.  ``--workload serve`` and ``--workload long`` run
two further workloads end to end (continuous batching of 128 requests on the
Qwen3-1.7B shape; a 32,768-token prompt on the Qwen3-32B shape) and print a line
of their own.

Every decode point is the median of several repeats of ``--steps`` steps (at least 192 timed steps
together); between repeats the requests are cut back to where they began, so the contexts stay
just below ``--context``.  The bytes of the roofline are counted at the contexts that ran.  After
the timing, one step is run both from its CUDA graph and kernel by kernel and the two sets of
logits are compared, so the number belongs to a step that computes the right thing.

``--impl reference``: the reference is a Rust workspace and cannot be installed here (no cargo),
but its CUDA kernels compile unmodified for sm_100.  When ``baseline/_ref`` holds that library
(``python baseline/reference_kernels.py --build <reference checkout>``) the arm runs the same
decode step and prefill on the reference's own kernels through their C entry points, in the
order its runtime calls them, and says so in ``reference_class``; otherwise it prints why it is
unavailable.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, max_position_embeddings=40960, rms_norm_eps=1e-6,
                rope_theta=1000000.0, tie_word_embeddings=False)
QWEN3_1_7B = dict(QWEN3_8B, hidden_size=2048, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                  intermediate_size=6144, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                 intermediate_size=25600, tie_word_embeddings=False)
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                        bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                        source="measured")
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, period_ms: int = 50):
        self.lines, self.proc, self.period_ms = [], None, period_ms
        self.marks = []                         # (name, first sample index, last sample index)

    def region(self, name):
        """with sampler.region("b8"): ... remembers which samples fell into the block."""
        sampler = self

        class _R:
            def __enter__(self):
                self.i0 = len(sampler.lines)

            def __exit__(self, *exc):
                sampler.marks.append((name, self.i0, len(sampler.lines)))
        return _R()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons, at = [], 0, set(), {}
        for i, l in enumerate(self.lines):
            parts = [x.strip() for x in l.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(int(parts[0]))
                at[i] = int(parts[0])
                mx = max(mx, int(parts[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        out = dict(sm_mhz=int(statistics.median(sm)) if sm else None, sm_max_mhz=mx or None,
                   reasons=sorted(reasons), samples=len(sm), period_ms=self.period_ms)
        for name, i0, i1 in self.marks:
            got = [at[i] for i in range(i0, i1) if i in at]
            out[f"sm_mhz_{name}"] = int(statistics.median(got)) if got else None
            out[f"samples_{name}"] = len(got)
        return out


def decode_bytes(cfg, n_layers, batch, context, esz=2):
    """Bytes one decode step has to read: every weight it uses once (the embedding rows
    of the batch, not the table) and the cache of the live requests."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * H * I
    weights = (n_layers * per_layer + V * H) * esz + batch * H * esz
    norms = (n_layers * (2 * H + 2 * cfg.head_dim) + H) * 4
    kv = batch * context * 2 * cfg.kv_dim * esz * n_layers
    return weights + norms + kv


def prefill_flops(cfg, n_layers, T):
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * H * I
    gemm = 2.0 * T * n_layers * per_layer + 2.0 * V * H
    attn = n_layers * cfg.num_attention_heads * 4.0 * cfg.head_dim * T * (T + 1) / 2
    return gemm + attn


def fill_contexts(eng, rids, context, seed=0):
    """Gives every request ``context`` tokens of random keys and values without running the model."""
    import torch
    g = torch.Generator(device=eng.device)
    g.manual_seed(seed)
    for rid in rids:
        if rid not in eng.manager.requests:
            eng.manager.add_request(rid)
        eng.manager.reserve(rid, context)
        eng.manager.commit(rid, context)
    for pool in eng.storage.paged:
        for layer in range(pool.shape[0]):
            pool[layer].copy_(torch.randn(pool[layer].shape, generator=g, device=eng.device, dtype=torch.float32)
                              .mul_(0.5).to(pool.dtype))


def repeats_for(steps: int) -> int:
    """Repeats of ``steps`` timed steps: three at least, and 192 timed steps together."""
    return max(3, -(-192 // max(steps, 1)))


def time_decode(eng, batch, context, steps, warmup, tag, check=False):
    """Device time of ``steps`` decode steps of ``batch`` requests whose contexts end just below
    ``context``: the median of ``repeats_for(steps)`` repeats, each bracketed by CUDA events; the
    requests are cut back to their first length between repeats.  Returns (ms per step, kernel
    launches of one repeat, mean context of the timed steps, ms of every repeat)."""
    import torch
    from airun_b200 import StepEntry
    from airun_b200.kernels import ops
    rids = [f"{tag}{i}" for i in range(batch)]
    start = context - steps - 1
    fill_contexts(eng, rids, start)
    V = eng.config.vocab_size
    toks = torch.randint(0, V, (steps + 1, batch), generator=torch.Generator().manual_seed(1)).tolist()
    picked = torch.zeros(batch, dtype=torch.int32, device=eng.device)

    def one(i):
        logits = eng.runner.step([StepEntry(r, [toks[i][j]], (0,)) for j, r in enumerate(rids)])
        ops.sample(logits, picked)
        return logits

    def rewind():
        for r in rids:
            eng.manager.truncate(r, start)

    for i in range(warmup):
        if i and i % steps == 0:
            rewind()
        one(i % steps)
    rewind()
    times, launches = [], 0
    for _ in range(repeats_for(steps)):
        torch.cuda.synchronize()
        l0 = ops.LAUNCHES[0] + getattr(eng.runner, "graph_launches", 0)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(steps):
            one(i)
        ev1.record()
        torch.cuda.synchronize()
        launches = ops.LAUNCHES[0] + getattr(eng.runner, "graph_launches", 0) - l0
        times.append(ev0.elapsed_time(ev1) / steps)
        rewind()
    eng.runner.raise_on_device_error()
    if check:
        check_step(eng, rids, toks[0], start)
    for r in rids:
        eng.manager.free_request(r)
    # contexts of the timed steps: start + 1 .. start + steps keys
    return statistics.median(times), launches, start + (steps + 1) / 2.0, times


def check_step(eng, rids, tokens, start):
    """The step that was timed, once from its CUDA graph and once kernel by kernel: finite logits,
    the same picks, the same values up to the rounding of another split of the keys."""
    import torch
    from airun_b200 import StepEntry
    entries = [StepEntry(r, [tokens[j]], (0,)) for j, r in enumerate(rids)]
    a = eng.runner.step(entries).clone()
    for r in rids:
        eng.manager.truncate(r, start)
    graphs = eng.runner.use_graphs
    eng.runner.use_graphs = False
    try:
        b = eng.runner.step(entries).clone()
    finally:
        eng.runner.use_graphs = graphs
    for r in rids:
        eng.manager.truncate(r, start)
    torch.cuda.synchronize()
    if not (torch.isfinite(a).all() and torch.isfinite(b).all()):
        raise RuntimeError("the timed decode step gave non-finite logits")
    scale = float(b.abs().max())
    err = float((a - b).abs().max())
    if err > 0.02 * scale:
        raise RuntimeError(f"the timed decode step differs from its kernel-by-kernel run: {err:.4g} of {scale:.4g}")
    return err / max(scale, 1e-30)


def time_e2e(eng, batch, context, steps, warmup, sampled=False):
    """The same decode through the Python entry point: requests live in the scheduler, every step
    copies the step's inputs from pinned host memory and reads the sampled tokens back.  Median of
    three repeats of ``steps`` steps by the host clock.  ``sampled``: the requests sample with the
    reference's default parameters (temperature 0.8, top-k 40, top-p 0.95, min-p 0.05, repetition penalty 1.1
    over 64 tokens) instead of greedily, which brings the host's sampling chain into every step."""
    import torch
    from airun_b200 import SamplingParams
    from airun_b200.engine.scheduler import Request
    rids = [f"{'s' if sampled else 'e'}{i}" for i in range(batch)]
    reps = 3
    start = context - reps * steps - warmup - 1
    fill_contexts(eng, rids, start - 1)
    g = torch.Generator().manual_seed(2)
    reqs = []
    for rid in rids:
        prompt = torch.randint(0, eng.config.vocab_size, (start,), generator=g).tolist()
        r = Request(rid, prompt, SamplingParams(seed=len(reqs) + 1) if sampled else SamplingParams.greedy(), reps * steps + warmup + 8)
        r.num_computed = start - 1                # its cache stands one token short of the prompt
        eng.scheduler.running.append(r)
        reqs.append(r)
    for _ in range(warmup):
        eng.run_step()
    times = []
    gap0 = eng.stats.host_gap_ms
    for _ in range(reps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            eng.run_step()
        torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) * 1e3 / steps)
    time_e2e.host_gap_ms = (eng.stats.host_gap_ms - gap0) / (reps * steps)
    assert all(len(r.output) == reps * steps + warmup for r in reqs), "the entry point did not decode every step"
    for r in reqs:
        eng.scheduler._finish(r, "bench")
    h2d = eng.runner.meta_host.numel() * 4 + eng._small_host.numel() * 4
    d2h = eng._picked_host.numel() * 4
    return statistics.median(times), h2d, d2h


def time_prefill(eng, T, runs=3):
    import torch
    from airun_b200 import StepEntry
    toks = torch.randint(0, eng.config.vocab_size, (T,), generator=torch.Generator().manual_seed(3)).tolist()
    times = []
    for i in range(runs + 1):
        rid = f"p{i}"
        eng.manager.add_request(rid)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        eng.runner.step([StepEntry(rid, toks, (T - 1,))])
        ev1.record()
        torch.cuda.synchronize()
        times.append(ev0.elapsed_time(ev1))
        eng.manager.free_request(rid)
    eng.runner.raise_on_device_error()
    return statistics.median(times[1:])


def workload_serve(a) -> int:
    """Continuous batching: 128 requests at once, prompt lengths uniform in [64, 2048], 256 new
    tokens each, a step budget of 512 tokens (Qwen3-1.7B shape).  Runs the whole workload three times
    through the Python entry point and times the third run: a step shape is launched kernel by kernel the
    first time it is seen and captured the second time, so a shape that a run meets once is only replayed
    from its graph in the third."""
    import torch
    from airun_b200 import Engine, EngineOptions, Qwen3Config, SamplingParams
    d = dict(QWEN3_1_7B)
    if a.layers:
        d["num_hidden_layers"] = a.layers
    cfg = Qwen3Config.from_dict(d)
    n_req, new = a.requests, a.new_tokens
    eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
        dtype=a.dtype, page_size=16, cache_tokens=n_req * (2048 + new + 16) + 4096, max_batch_tokens=a.budget,
        max_requests=n_req, max_context=2048 + new + 16))
    g = torch.Generator().manual_seed(4)
    lens = torch.randint(64, 2049, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    res = {}
    for run in range(3):
        sampler = ClockSampler()
        sampler.start()
        steps0 = eng.stats.steps
        reqs = [eng.add_request(p, SamplingParams.greedy(), max_new_tokens=new) for p in prompts]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        steps = 0
        gap0 = eng.stats.host_gap_ms
        while eng.has_work():
            eng.run_step()
            steps += 1
        torch.cuda.synchronize()
        sec = time.perf_counter() - t0
        # from reading a step's tokens to having launched the next step: the GPU may idle that long
        gap_sec = (eng.stats.host_gap_ms - gap0) / 1e3
        clocks = sampler.stop()
        gen = sum(len(r.output) for r in reqs)
        assert gen == n_req * new, "a request ended early"
        res = {"workload": "serve", "model": "Qwen3-1.7B shape, random weights", "layers": cfg.num_hidden_layers,
               "layers_full": 28, "requests": n_req, "prompt_tokens": sum(lens), "generated_tokens": gen,
               "step_budget": a.budget, "seconds": round(sec, 3), "steps": steps,
               "ms_per_step": round(sec * 1e3 / steps, 3),
               "total_tokens_per_s": round((sum(lens) + gen) / sec, 1), "decode_tokens_per_s": round(gen / sec, 1),
               "host_gap_seconds": round(gap_sec, 3), "host_share_at_most": round(gap_sec / sec, 4),
               "preemptions": eng.scheduler.stats["preemptions"], "dtype": a.dtype, "clocks": clocks}
    print(json.dumps(res))
    return 0


def workload_long(a) -> int:
    """Long context: one 32,768-token prompt in portions of 2,048, then 512 tokens decoded alone, then
    15 forks of the request (reading the same prompt pages: 16 private caches would not fit beside
    the weights; attention reads those pages once per step for all 16) and 512 tokens decoded by all
    16 (Qwen3-32B shape)."""
    import torch
    from airun_b200 import Engine, EngineOptions, Qwen3Config, SamplingParams
    d = dict(QWEN3_32B)
    if a.layers:
        d["num_hidden_layers"] = a.layers
    cfg = Qwen3Config.from_dict(d)
    T, new, forks = a.prompt, a.new_tokens, a.forks
    eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
        dtype=a.dtype, page_size=16, cache_tokens=T + (forks + 2) * (2 * new + 32) + 4096,
        max_batch_tokens=2048, max_requests=forks + 1, max_context=T + 2 * new + 32))
    L = cfg.num_hidden_layers
    pk = peaks()
    esz = 2 if a.dtype == "bfloat16" else 4
    prompt = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(5)).tolist()
    # warm-up: a short request through the same kernels (prefill portion, decode graph)
    eng.generate(prompt[:4096], SamplingParams.greedy(), max_new_tokens=8)
    sampler = ClockSampler()
    sampler.start()
    parent = eng.add_request(prompt, SamplingParams.greedy(), max_new_tokens=2 * new + 1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while not parent.output:
        eng.run_step()
    torch.cuda.synchronize()
    t_pre = time.perf_counter() - t0
    t0 = time.perf_counter()
    while len(parent.output) < 1 + new:
        eng.run_step()
    torch.cuda.synchronize()
    t_b1 = time.perf_counter() - t0
    kids = [eng.fork_request(parent, max_new_tokens=new) for _ in range(forks)]
    eng.run_step()                                   # the forks' first step is not a pure decode step
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_steps = 0
    while len(kids[0].output) < new:
        eng.run_step()
        n_steps += 1
    torch.cuda.synchronize()
    t_bn = time.perf_counter() - t0
    clocks = sampler.stop()
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * H * I
    flops = 2.0 * T * L * per_layer + L * cfg.num_attention_heads * 4.0 * cfg.head_dim * T * (T + 1) / 2
    b1_bytes = decode_bytes(cfg, L, 1, T + new // 2, esz)
    bn_bytes = decode_bytes(cfg, L, forks + 1, T + new + new // 2, esz)
    once_bytes = decode_bytes(cfg, L, 1, T, esz) + (forks + 1) * (new + new // 2) * 2 * cfg.kv_dim * esz * L
    print(json.dumps({
        "workload": "long", "model": "Qwen3-32B shape, random weights", "layers": L, "layers_full": 64,
        "prompt_tokens": T, "portion": 2048, "dtype": a.dtype, "peaks": pk["source"],
        "prefill": {"seconds": round(t_pre, 3), "tokens_per_s": round(T / t_pre, 1),
                    "frac_of_bf16_peak": round(flops / t_pre / (pk["bf16_tflops"] * 1e12), 4)},
        "decode_b1": {"tokens": new, "tokens_per_s": round(new / t_b1, 2), "ms_per_step": round(t_b1 * 1e3 / new, 3),
                      "hbm_frac": round(b1_bytes / (t_b1 / new) / 1e9 / pk["hbm_gbs"], 4)},
        f"decode_b{forks + 1}": {"tokens": n_steps * (forks + 1), "tokens_per_s": round(n_steps * (forks + 1) / t_bn, 2),
                                 "ms_per_step": round(t_bn * 1e3 / n_steps, 3), "shared_prompt_pages": True,
                                 "hbm_frac_if_every_request_reads_the_prompt":
                                     round(bn_bytes / (t_bn / n_steps) / 1e9 / pk["hbm_gbs"], 4),
                                 "hbm_frac_prompt_read_once":
                                     round(once_bytes / (t_bn / n_steps) / 1e9 / pk["hbm_gbs"], 4)},
        "clocks": clocks}))
    return 0


REFERENCE_CLASS = "reference kernels through their C ABI; host loop restated, Rust runtime not buildable"


def workload_ablate(a) -> int:
    """What each kind of kernel adds to the decode step: the step is captured and timed again with one kind left out.

    The logits of such a step are wrong on purpose; only its time is read.  The difference to the whole step is the
    kind's marginal cost on the step's critical path, which is what a faster kernel could win back: it is smaller than
    the kernel's own duration where the next kernel's prologue overlaps it (programmatic dependent launch).
    ``rmsnorm_as_empty_kernel`` puts a kernel that does next to nothing in the norm's place: what one more
    launch boundary costs.  One JSON line per kind.
    """
    import torch
    from airun_b200 import Engine, EngineOptions, Qwen3Config
    from airun_b200.kernels import fast, ops
    d = dict(QWEN3_8B)
    if a.layers:
        d["num_hidden_layers"] = a.layers
    cfg = Qwen3Config.from_dict(d)
    L = cfg.num_hidden_layers
    eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
        dtype="bfloat16", page_size=16, cache_tokens=64 * a.context + 4096, max_batch_tokens=2048, max_requests=64,
        max_context=a.context))
    qkv_rows = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    kinds = {(qkv_rows, cfg.hidden_size): "product_qkv",
             (2 * cfg.intermediate_size, cfg.hidden_size): "product_gate_up",
             (cfg.hidden_size, cfg.intermediate_size): "product_down",
             (cfg.vocab_size, cfg.hidden_size): "product_head"}
    kinds.setdefault((cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim), "product_o")
    skip: set = set()
    gemm, rms, post, att = fast.gemm_tcgen05, ops.rmsnorm, ops.qkv_post, fast.attn_decode
    src, rows, dst = (torch.zeros(8, 64, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda"),
                      torch.zeros(8, 64, device="cuda"))

    def gemm_or_not(x, w, *args, **kw):
        return None if kinds.get(tuple(w.shape)) in skip else gemm(x, w, *args, **kw)

    def rms_or_not(*args, **kw):
        if "rmsnorm" in skip:
            return None
        if "rmsnorm_as_empty_kernel" in skip:
            return ops.gather_rows(src, rows, dst)
        return rms(*args, **kw)

    fast.gemm_tcgen05 = gemm_or_not
    ops.rmsnorm = rms_or_not
    ops.qkv_post = lambda *args, **kw: None if "qkv_post" in skip else post(*args, **kw)
    fast.attn_decode = lambda *args, **kw: None if "attention" in skip else att(*args, **kw)
    base = {}
    try:
        for kind in [None, "rmsnorm", "rmsnorm_as_empty_kernel", "qkv_post", "attention", *sorted(set(kinds.values()))]:
            skip.clear()
            if kind:
                skip.add(kind)
            eng.runner.graphs.clear()
            eng.runner._warm_buckets.clear()
            res = {}
            for b in (8, 1, 64):
                ms, _, _, _ = time_decode(eng, b, a.context, a.steps, a.warmup, f"ab{b}_")
                res[f"b{b}"] = round(ms, 4)
                if kind is None:
                    base[b] = ms
            line = {"workload": "ablate", "left_out": kind, "layers": L, "context": a.context, "ms_per_step": res}
            if kind:
                per = 1 if kind == "product_head" else L
                line["marginal_us_each" if kind == "product_head" else "marginal_us_per_layer"] = {
                    f"b{b}": round((base[b] - res[f"b{b}"]) * 1e3 / per, 2) for b in (8, 1, 64)}
            print(json.dumps(line), flush=True)
    finally:
        fast.gemm_tcgen05, ops.rmsnorm, ops.qkv_post, fast.attn_decode = gemm, rms, post, att
    return 0


def reference_arm(a) -> int:
    """The same metric on the reference's own CUDA kernels (compiled unmodified for sm_100), called
    through their C entry points in the order the reference's runtime calls them
    (baseline/reference_kernels.py).  The decode step is captured into a CUDA graph as the reference
    captures its own; no scheduler, sampler or host transfer of the reference runs, so there is no
    end-to-end figure."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_kernels as rk
        if not rk.available():
            raise FileNotFoundError("baseline/_ref/libairun_ref_kernels.so has not been built")
        rk.load()
    except (OSError, ImportError) as e:
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (pip: 'not installable', no cargo or rustc in this image) "
                          f"and its CUDA kernels are not built here: {e}"}))
        return 0
    if a.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference arm here drives one GPU"}))
        return 0
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no GPU is visible to this process"}))
        return 0
    a.warmup = max(a.warmup, 3)
    cfg = dict(QWEN3_8B)
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    L, H, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["vocab_size"]
    nh, nkv, hd, I = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"]
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)

    def mat(r, c):
        return (0.02 * torch.randn(r, c, generator=g, device=dev, dtype=torch.float32)).to(torch.bfloat16)

    def vec(n):
        return 1.0 + 0.1 * torch.randn(n, generator=g, device=dev, dtype=torch.float32)

    W = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": vec(H), "lm_head.weight": mat(V, H)}
    for l in range(L):
        p = f"model.layers.{l}"
        W.update({f"{p}.input_layernorm.weight": vec(H), f"{p}.post_attention_layernorm.weight": vec(H),
                  f"{p}.self_attn.q_proj.weight": mat(nh * hd, H), f"{p}.self_attn.k_proj.weight": mat(nkv * hd, H),
                  f"{p}.self_attn.v_proj.weight": mat(nkv * hd, H), f"{p}.self_attn.o_proj.weight": mat(H, nh * hd),
                  f"{p}.self_attn.q_norm.weight": vec(hd), f"{p}.self_attn.k_norm.weight": vec(hd),
                  f"{p}.mlp.gate_proj.weight": mat(I, H), f"{p}.mlp.up_proj.weight": mat(I, H),
                  f"{p}.mlp.down_proj.weight": mat(H, I)})
    slots = max(64, a.batch) if not a.skip_points else a.batch
    dec = rk.ReferenceDecoder(cfg, W, ctx=a.context, slots=slots, max_batch=512, logit_rows=max(64, a.batch))
    for s_ in range(slots):                          # random keys and values, as in the other arm
        dec.kc[s_].normal_(0.0, 0.5, generator=g)
        dec.vc[s_].normal_(0.0, 0.5, generator=g)
    pk = peaks()
    sampler = ClockSampler()
    sampler.start()

    def time_rows(batch, steps):
        start = a.context - steps - 1
        rows = list(range(batch))
        dec.prepare_rows(rows)
        toks = torch.randint(0, V, (steps + 1, batch), generator=torch.Generator().manual_seed(1)).to(dev, torch.int32)
        pos = torch.zeros(batch, dtype=torch.int32, device=dev)
        graph = None

        def one(i):
            dec.tokens[:batch].copy_(toks[i])
            dec.positions[:batch].copy_(pos)
            pos.add_(1)
            if graph is None:
                dec.launch_rows()
            else:
                graph.replay()

        pos.fill_(start)
        one(0)                                          # loads and configures every kernel
        torch.cuda.synchronize()
        try:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                dec.launch_rows()
            graph = gr
        except Exception as e:                          # the reference falls back the same way (runtime.rs:3096-3103)
            print(f"note: the reference arm's decode runs without a CUDA graph: {e}", file=sys.stderr)
            torch.cuda.synchronize()
        for i in range(a.warmup):
            pos.fill_(start + (i % steps))
            one(i % steps)
        times = []
        for _ in range(repeats_for(steps)):
            pos.fill_(start)
            torch.cuda.synchronize()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for i in range(steps):
                one(i)
            ev1.record()
            torch.cuda.synchronize()
            times.append(ev0.elapsed_time(ev1) / steps)
        if not torch.isfinite(dec.logits[:batch]).all():
            raise RuntimeError("the reference arm's decode step gave non-finite logits")
        return statistics.median(times), start + (steps + 1) / 2.0, graph is not None

    esz = 2
    cfgo = QwenShape(cfg)
    with sampler.region("b%d" % a.batch):
        ms, mean_ctx, graphed = time_rows(a.batch, a.steps)
    value = a.batch / (ms / 1e3)
    gbs = decode_bytes(cfgo, L, a.batch, mean_ctx, esz) / (ms / 1e3) / 1e9
    points, detail = {}, {}
    if not a.skip_points:
        for b in (1, 64):
            with sampler.region(f"b{b}"):
                pms, pctx, _ = time_rows(b, max(4, a.steps // 2))
            points[f"decode_b{b}"] = round(b / (pms / 1e3), 2)
            detail[f"decode_b{b}"] = {"tok_s": round(b / (pms / 1e3), 2), "ms_per_step": round(pms, 4), "hbm_frac": round(
                decode_bytes(cfgo, L, b, pctx, esz) / (pms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
    T = 2048
    ptoks = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(3)).tolist()
    ptimes = []
    with sampler.region("prefill"):
        for i in range(3):
            dec.n_past[0] = 0
            torch.cuda.synchronize()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            dec.forward(0, ptoks)                         # portions of 512 tokens, the reference's default batch
            ev1.record()
            torch.cuda.synchronize()
            ptimes.append(ev0.elapsed_time(ev1))
    pre_ms = statistics.median(ptimes[1:])
    clocks = sampler.stop()
    flops = prefill_flops(cfgo, L, T)
    out = {
        "metric": "Qwen3-8B decode tok/s @ batch 1/8/64; prefill tok/s @ 2048 tok; % roofline",
        "value": round(value, 2), "unit": "tokens/s", "value_of": f"decode tok/s at batch {a.batch}, context {a.context}",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4), "repeats": repeats_for(a.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference", "reference_class": REFERENCE_CLASS,
        "config": {"model": "Qwen3-8B shape, random weights", "layers": L, "layers_full": QWEN3_8B["num_hidden_layers"],
                   "hidden": H, "heads": nh, "kv_heads": nkv, "head_dim": hd, "intermediate": I, "vocab": V,
                   "global_batch": a.batch, "seq_len": a.context, "kv_cache": "float16, contiguous per slot",
                   "activations": "float32", "decode_graph": graphed, "prefill_portion": 512,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (weights and cache are read once per step)",
                   "peaks": pk["source"]},
        "e2e": None, "gpu_launches": 0,
        "prefill": {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4), "mean_context": round(mean_ctx, 1)},
        "points": points, "points_detail": detail, "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


class QwenShape:
    """The sizes ``decode_bytes`` and ``prefill_flops`` read, from a config dictionary."""

    def __init__(self, d):
        self.hidden_size, self.intermediate_size, self.vocab_size = d["hidden_size"], d["intermediate_size"], d["vocab_size"]
        self.num_attention_heads, self.head_dim = d["num_attention_heads"], d["head_dim"]
        self.q_dim = d["num_attention_heads"] * d["head_dim"]
        self.kv_dim = d["num_key_value_heads"] * d["head_dim"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=None, help="layers to build (default: all 36)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--decode-only", action="store_true", help="time the decode step only (for profiling runs)")
    ap.add_argument("--prefill-only", action="store_true", help="time the 2,048-token prompt only (for profiling runs)")
    ap.add_argument("--workload", default="decode", choices=("decode", "serve", "long", "ablate"),
                    help="decode: the headline line; serve: 128 requests continuously batched (Qwen3-1.7B shape); "
                         "long: a 32,768-token prompt, then decoding alone and as 16 forks (Qwen3-32B shape); "
                         "ablate: the decode step timed with one kind of kernel left out at a time")
    ap.add_argument("--requests", type=int, default=128, help="serve: requests")
    ap.add_argument("--new-tokens", type=int, default=None, help="serve / long: tokens decoded per request")
    ap.add_argument("--budget", type=int, default=512, help="serve: tokens per step")
    ap.add_argument("--prompt", type=int, default=32768, help="long: prompt length")
    ap.add_argument("--forks", type=int, default=15, help="long: forks of the request for the batched decode")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {a.gpus} is not supported (the engine is single-GPU)")
        return 2
    a.warmup = max(a.warmup, 3)
    if a.workload == "serve":
        a.new_tokens = a.new_tokens or 256
        return workload_serve(a)
    if a.workload == "long":
        a.new_tokens = a.new_tokens or 512
        return workload_long(a)
    if a.workload == "ablate":
        return workload_ablate(a)

    import torch
    from airun_b200 import Engine, EngineOptions, Qwen3Config
    d = dict(QWEN3_8B)
    full_layers = d["num_hidden_layers"]
    if a.layers:
        d["num_hidden_layers"] = a.layers
    cfg = Qwen3Config.from_dict(d)
    L = cfg.num_hidden_layers
    pk = peaks()
    max_batch = a.batch if (a.decode_only or a.skip_points or a.prefill_only) else max(64, a.batch)
    cache_tokens = max_batch * a.context + 4096
    cache_gb = cache_tokens * full_layers * 2 * cfg.num_key_value_heads * cfg.head_dim * (2 if a.dtype == "bfloat16" else 4) / 1e9
    if cache_gb > 140.0:
        print(f"bench.py: a cache of {cache_tokens} tokens ({cache_gb:.0f} GB) does not fit beside the weights; "
              f"lower --batch or --context" + ("" if max_batch == a.batch else " or pass --skip-points"))
        return 2
    eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
        dtype=a.dtype, page_size=16, cache_tokens=cache_tokens, max_batch_tokens=2048,
        max_requests=max_batch, max_context=a.context))
    esz = 2 if a.dtype == "bfloat16" else 4

    if a.prefill_only:
        pre_ms = time_prefill(eng, 2048)
        print(json.dumps({"prefill_only": True, "tokens": 2048, "ms": round(pre_ms, 3),
                          "value": round(2048 / (pre_ms / 1e3), 1), "layers": L}))
        return 0
    sampler = ClockSampler()
    sampler.start()
    with sampler.region(f"b{a.batch}"):
        ms, launches, mean_ctx, reps = time_decode(eng, a.batch, a.context, a.steps, a.warmup, "d", check=True)
    value = a.batch / (ms / 1e3)

    if a.decode_only:
        sampler.stop()
        print(json.dumps({"decode_only": True, "ms_per_step": round(ms, 4), "value": round(value, 2),
                          "layers": L, "batch": a.batch, "context": a.context, "mean_context": round(mean_ctx, 1),
                          "hbm_frac": round(decode_bytes(cfg, L, a.batch, mean_ctx, esz) / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}))
        return 0
    with sampler.region("e2e"):
        e2e_ms, h2d, d2h = time_e2e(eng, a.batch, a.context, a.steps, a.warmup)
        e2e_gap = getattr(time_e2e, "host_gap_ms", 0.0)
        e2e_sampled_ms, _, _ = time_e2e(eng, a.batch, a.context, a.steps, a.warmup, sampled=True)
    points, detail = {}, {}
    if not a.skip_points:
        for b in (1, 64):
            with sampler.region(f"b{b}"):
                pms, _, pctx, _ = time_decode(eng, b, a.context, a.steps, a.warmup, f"b{b}_", check=True)
            points[f"decode_b{b}"] = round(b / (pms / 1e3), 2)
            detail[f"decode_b{b}"] = {"tok_s": round(b / (pms / 1e3), 2), "ms_per_step": round(pms, 4), "hbm_frac": round(
                decode_bytes(cfg, L, b, pctx, esz) / (pms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
    T = 2048
    with sampler.region("prefill"):
        pre_ms = time_prefill(eng, T)
    clocks = sampler.stop()
    flops = prefill_flops(cfg, L, T)
    pre = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3), "frac": None}
    if a.dtype == "bfloat16":
        pre["frac"] = pre["frac_burst"] = round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)
        pre["frac_sustained"] = round(flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
    gbs = decode_bytes(cfg, L, a.batch, mean_ctx, esz) / (ms / 1e3) / 1e9
    out = {
        "metric": "Qwen3-8B decode tok/s @ batch 1/8/64; prefill tok/s @ 2048 tok; % roofline",
        "value": round(value, 2), "unit": "tokens/s", "value_of": f"decode tok/s at batch {a.batch}, context {a.context}",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4),
        "repeats": len(reps), "ms_per_step_repeats": [round(t, 4) for t in reps],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if a.dtype == "bfloat16" else "fp32", "data": "synthetic", "impl": "ours",
        "config": {"model": "Qwen3-8B shape, random weights", "layers": L, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": a.batch, "seq_len": a.context, "page_size": 16, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights and cache are read once per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(a.batch / (e2e_ms / 1e3), 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "host_gap_ms_per_step": round(e2e_gap, 4),
                "sampled_with_reference_defaults": {"value": round(a.batch / (e2e_sampled_ms / 1e3), 2),
                                                    "ms_per_step": round(e2e_sampled_ms, 4)}},
        "gpu_launches": launches,
        "prefill": pre,
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4), "mean_context": round(mean_ctx, 1)},
        "points": points, "points_detail": detail,
        "checked": "each timed decode step: finite logits, graph replay against a kernel-by-kernel run",
        "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
