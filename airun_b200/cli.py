"""Command line in the manner of the reference's ``airun run``.

Option names, meanings and defaults follow crates/airun-cli/src/run.rs:50-220:
``-n/--predict`` 256, ``-c/--ctx-size``, ``-b/--batch-size``, ``--temp`` 0.8,
``--top-k`` 40, ``--top-p`` 0.95, ``--min-p`` 0.05, ``--typical-p`` 1.0,
``--top-n-sigma`` 0, ``--repeat-penalty`` 1.1, ``--presence-penalty`` 0,
``--frequency-penalty`` 0, ``--repeat-last-n`` 64, ``--seed`` 0 (0 = from the
clock), ``--stats``, ``-q/--quiet``.  The model is a folder with config.json
and model.safetensors; the prompt is a list of token ids (``-p 1,2,3``, a file,
or standard input), since the engine works on token ids.  ``--dtype`` takes the
place of ``--kv-type``: the cache is kept in the compute type.

Subcommands: ``run`` (generate), ``bench`` (prefill and decode rates of a model
folder, median of runs, in the manner of crates/airun-cli/src/bench.rs:11-92),
``perplexity`` (loss and top-1 of a token file; ``--chunk``, ``--batched``,
``--limit``, ``--worst`` as in crates/airun-cli/src/perplexity.rs:97-222), ``init`` (random-weights mode: write
a model folder from a config.json and a seed), ``inspect`` (describe a model
folder: configuration, tensors, whether it can be loaded; ``--tensors``,
``--json``, ``--values TENSOR --count N`` as crates/airun-cli/src/inspect.rs:10-36),
``selftest``.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import time
from typing import List, Optional


def parse_ids(text: str) -> List[int]:
    ids = [int(t) for t in re.split(r"[\s,]+", text.strip()) if t]
    if not ids:
        raise SystemExit("the prompt holds no token ids")
    return ids


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="airun", description="airun_b200: Qwen3 inference on one B200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    run = sub.add_parser("run", help="generate from a prompt of token ids")
    run.add_argument("model", help="folder with config.json and model.safetensors")
    run.add_argument("-p", "--prompt", help="token ids separated by commas or spaces; standard input when omitted")
    run.add_argument("--prompt-file", help="file holding the token ids")
    run.add_argument("-n", "--predict", type=int, default=256, help="tokens to generate")
    run.add_argument("-c", "--ctx-size", type=int, default=None, help="longest context of a request")
    run.add_argument("-b", "--batch-size", type=int, default=512, help="token budget of one step")
    run.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    run.add_argument("--page-size", type=int, default=16)
    run.add_argument("--cache-tokens", type=int, default=None, help="tokens the cache holds (default: what fits)")
    run.add_argument("--parallel", type=int, default=8, help="requests live at a time")
    run.add_argument("--temp", type=float, default=0.8)
    run.add_argument("--top-k", type=int, default=40)
    run.add_argument("--top-p", type=float, default=0.95)
    run.add_argument("--min-p", type=float, default=0.05)
    run.add_argument("--typical-p", type=float, default=1.0)
    run.add_argument("--top-n-sigma", type=float, default=0.0)
    run.add_argument("--repeat-penalty", type=float, default=1.1)
    run.add_argument("--presence-penalty", type=float, default=0.0)
    run.add_argument("--frequency-penalty", type=float, default=0.0)
    run.add_argument("--repeat-last-n", type=int, default=64)
    run.add_argument("--seed", type=int, default=0)
    run.add_argument("--eog", default="", help="token ids that end generation")
    run.add_argument("--stats", action="store_true", help="print timing to stderr")
    run.add_argument("-q", "--quiet", action="store_true", help="print only the generated ids")

    be = sub.add_parser("bench", help="prefill and decode tokens a second of a model folder")
    be.add_argument("model")
    be.add_argument("--prefill", default="128,512", help="prompt lengths to time, comma separated")
    be.add_argument("--decode", type=int, default=128, help="tokens to decode per run")
    be.add_argument("--decode-at", default="16", help="context depths at which decoding is timed, comma separated")
    be.add_argument("-c", "--ctx-size", type=int, default=None, help="longest context of a request (default: what the runs need)")
    be.add_argument("--random-tokens", action="store_true",
                    help="prompts of fixed-seed random ids instead of one repeated token")
    be.add_argument("--forward-only", action="store_true",
                    help="time exactly N forward steps on fixed tokens, without sampling")
    be.add_argument("--temp", type=float, default=0.0, help="temperature of the decode runs; 0 is greedy")
    be.add_argument("--parallel", type=int, default=1, help="requests decoding side by side")
    be.add_argument("--runs", type=int, default=3)
    be.add_argument("--warmup", type=int, default=1)
    be.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    be.add_argument("-b", "--batch-size", type=int, default=2048)
    be.add_argument("--json", action="store_true")

    pp = sub.add_parser("perplexity", help="loss and top-1 accuracy over a file of token ids")
    pp.add_argument("model")
    pp.add_argument("-f", "--file", "--tokens-file", dest="file", help="file of token ids to score")
    pp.add_argument("-n", "--limit", type=int, default=0, help="stop after this many tokens; 0 scores everything")
    pp.add_argument("--chunk", type=int, default=0,
                    help="split the ids into passes of this many tokens, each from an empty context, and count "
                         "only the predictions of a pass's second half; 0: one pass over everything")
    pp.add_argument("--batched", action="store_true",
                    help="with --chunk: feed each pass in one step (the prefill kernels) instead of one token "
                         "at a time (the decode kernels)")
    pp.add_argument("--worst", type=int, default=0, help="print this many tokens with the highest loss")
    pp.add_argument("-c", "--ctx-size", type=int, default=4096, help="context length in tokens")
    pp.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")

    init = sub.add_parser("init", help="write a model folder with seeded random weights")
    init.add_argument("config", help="a config.json of the architecture")
    init.add_argument("out", help="folder to write")
    init.add_argument("--seed", type=int, default=1)

    ins = sub.add_parser("inspect", help="describe a model folder: configuration, tensors, whether it can be loaded")
    ins.add_argument("model")
    ins.add_argument("--tensors", action="store_true", help="list every tensor with its shape, type and size")
    ins.add_argument("--json", action="store_true", help="machine-readable JSON instead of a report")
    ins.add_argument("--values", metavar="TENSOR", help="print a tensor's first values and summary statistics")
    ins.add_argument("--count", type=int, default=16, help="how many values --values prints")

    gp = sub.add_parser("gpu", help="the CUDA devices the engine can see and whether it can run on them")
    gp.add_argument("--json", action="store_true", help="machine-readable JSON instead of a report")

    st = sub.add_parser("selftest", help="every kernel against a plain reference of the same operation")
    st.add_argument("--device", type=int, default=0)
    st.add_argument("--verbose", action="store_true")
    return ap


def cmd_run(a) -> int:
    from . import Engine, EngineOptions, SamplingParams
    if a.prompt is not None:
        prompt = parse_ids(a.prompt)
    elif a.prompt_file:
        with open(a.prompt_file) as f:
            prompt = parse_ids(f.read())
    else:
        prompt = parse_ids(sys.stdin.read())
    t0 = time.perf_counter()
    eng = Engine.from_folder(a.model, EngineOptions(
        dtype=a.dtype, page_size=a.page_size, cache_tokens=a.cache_tokens, max_batch_tokens=a.batch_size,
        max_requests=a.parallel, max_context=a.ctx_size))
    load_s = time.perf_counter() - t0
    if not a.quiet:
        print(f"[airun] {eng.config.summary()}; context {eng.max_context}, "
              f"{eng.manager.num_pages} pages of {eng.manager.page_size}", file=sys.stderr)
    params = SamplingParams(temperature=a.temp, top_k=a.top_k, top_p=a.top_p, min_p=a.min_p,
                            typical_p=a.typical_p, top_n_sigma=a.top_n_sigma, repeat_penalty=a.repeat_penalty,
                            presence_penalty=a.presence_penalty, frequency_penalty=a.frequency_penalty,
                            repeat_last_n=a.repeat_last_n, seed=a.seed)
    eog = parse_ids(a.eog) if a.eog.strip() else []

    def on_token(req, tok):
        if not a.quiet:
            print(tok, end=" ", flush=True)

    res = eng.generate(prompt, params, max_new_tokens=a.predict, eog_tokens=eog, on_token=on_token)
    if a.quiet:
        print(",".join(str(t) for t in res.token_ids))
    else:
        print()
    if a.stats or not a.quiet:
        s = eng.stats
        print(f"[airun] prompt {s.prompt_tokens} tokens in {s.prefill_ms:.1f} ms ({s.prefill_tps:.1f} tok/s), "
              f"generated {s.generated_tokens} in {s.decode_ms:.1f} ms ({s.decode_tps:.1f} tok/s), "
              f"stop: {res.finish_reason}, load {load_s:.1f} s", file=sys.stderr)
    return 0


def _random_ids(n: int, vocab: int, seed: int = 0x2545F4914F6CDD1D) -> List[int]:
    """A fixed-seed xorshift id stream, as the reference's bench --random-tokens
    (crates/airun-cli/src/bench.rs:177-187)."""
    x, out = seed, []
    for _ in range(n):
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        out.append(x % vocab)
    return out


def cmd_bench(a) -> int:
    import statistics
    import torch
    from . import Engine, EngineOptions, StepEntry
    from .kernels import ops
    lengths = [int(x) for x in a.prefill.split(",") if x]
    depths = [int(x) for x in str(a.decode_at).split(",") if x] or [16]
    need = max(lengths + [d + a.decode + 1 for d in depths]) + 64
    if a.ctx_size is not None:
        if a.ctx_size < need - 64:
            raise SystemExit(f"--ctx-size {a.ctx_size} is shorter than the longest run ({need - 64} tokens)")
        need = max(need, a.ctx_size)
    n_par = max(a.parallel, 1)
    eng = Engine.from_folder(a.model, EngineOptions(dtype=a.dtype, cache_tokens=need * n_par + 64,
                                                     max_batch_tokens=max(a.batch_size, 16), max_requests=n_par,
                                                     max_context=need))
    V = eng.config.vocab_size
    picked = torch.zeros(n_par, dtype=torch.int32, device=eng.device)
    temps = torch.full((n_par,), float(a.temp), dtype=torch.float32, device=eng.device) if a.temp > 0 else None
    # Prompts: one repeated token (the reference's default, crates/airun-cli/src/bench.rs:163-169; there
    # is no tokenizer here, so the filler is id 1) or a fixed-seed random stream (bench.rs:177-187).
    filler = 1 % V

    def prompt_ids(n, seed=0x9E3779B97F4A7C15):
        return _random_ids(n, V, seed) if a.random_tokens else [filler] * n

    def timed(fn):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    def prefill(rid, toks):
        eng.manager.add_request(rid)
        for p0 in range(0, len(toks), a.batch_size):
            part = toks[p0:p0 + a.batch_size]
            last = p0 + len(part) == len(toks)
            eng.runner.step([StepEntry(rid, part, (len(part) - 1,) if last else ())])

    report = {"prefill": {}, "decode": {}}
    for n in lengths:
        toks = prompt_ids(n)
        ms = []
        for r in range(a.warmup + a.runs):
            t = timed(lambda: prefill("p", toks))
            eng.manager.free_request("p")
            if r >= a.warmup:
                ms.append(t)
        report["prefill"][n] = dict(tokens_per_s=n / (statistics.median(ms) / 1e3), ms=ms)
    rids = [f"d{i}" for i in range(n_par)]
    report["decode_at"] = {}
    for depth in depths:
        ms = []
        for r in range(a.warmup + a.runs):
            for i, rid in enumerate(rids):
                prefill(rid, prompt_ids(depth, seed=1234 + i))
            fixed = prompt_ids(a.decode * len(rids), seed=99)
            gen = torch.Generator(device="cpu").manual_seed(7)

            def decode():
                # --forward-only: fixed tokens, no sampling.  Otherwise every step's tokens are the ones
                # the step before picked (first maximum, or a draw at --temp), read back like a generation.
                cur = fixed[:len(rids)]
                for s in range(a.decode):
                    if a.forward_only:
                        cur = fixed[s * len(rids):(s + 1) * len(rids)]
                    logits = eng.runner.step([StepEntry(rid, [int(cur[i])], (0,)) for i, rid in enumerate(rids)])
                    if not a.forward_only:
                        u = torch.rand(len(rids), generator=gen).to(eng.device) if temps is not None else None
                        ops.sample(logits, picked, temps, u)
                        cur = picked[:len(rids)].tolist()

            t = timed(decode)
            for rid in rids:
                eng.manager.free_request(rid)
            if r >= a.warmup:
                ms.append(t)
        report["decode_at"][depth] = dict(tokens_per_s=a.decode * len(rids) / (statistics.median(ms) / 1e3), depth=depth,
                                          parallel=len(rids), ms=ms)
    report["decode"] = report["decode_at"][depths[0]]
    eng.runner.raise_on_device_error()
    if a.json:
        print(json.dumps(report))
    else:
        for n, v in report["prefill"].items():
            print(f"prefill {n:6d} tokens: {v['tokens_per_s']:10.1f} tok/s (median of {len(v['ms'])})")
        for d in report["decode_at"].values():
            print(f"decode {a.decode} tokens at depth {d['depth']} x {d['parallel']}: {d['tokens_per_s']:10.1f} tok/s")
    return 0


def cmd_perplexity(a) -> int:
    """Scores a file of token ids as the reference's ``airun perplexity`` scores a text
    (crates/airun-cli/src/perplexity.rs:97-222): one pass over everything, token by token, or with
    ``--chunk N`` passes of N tokens that each start from an empty context and count only the
    predictions of their second half; ``--batched`` feeds a pass in one step (the kernels of prompt
    portions) instead of one token at a time (the decode kernels).  The two agree to rounding."""
    import math
    import torch
    from . import Engine, EngineOptions, StepEntry
    if not a.file:
        raise SystemExit("perplexity needs --file with the token ids to score (the engine has no tokenizer)")
    with open(a.file) as f:
        ids = parse_ids(f.read())
    if len(ids) < 2:
        raise SystemExit(f"need at least two tokens to score; the file holds {len(ids)}")
    scored = len(ids) if a.limit <= 0 else min(a.limit, len(ids))
    if a.batched and a.chunk <= 0:
        raise SystemExit("--batched needs --chunk")
    if a.chunk > 0:
        if a.chunk < 4 or a.chunk > scored:
            raise SystemExit(f"--chunk {a.chunk} needs at least 4 tokens and at most the file's {scored}")
        passes = [(c * a.chunk, (c + 1) * a.chunk, a.chunk // 2) for c in range(scored // a.chunk)]
    else:
        passes = [(0, scored, 0)]
    longest = max(e - s0 for s0, e, _ in passes)
    if longest + 1 >= a.ctx_size:
        raise SystemExit(f"a pass is {longest} tokens but the context is {a.ctx_size}; raise --ctx-size")
    eng = Engine.from_folder(a.model, EngineOptions(dtype=a.dtype, cache_tokens=longest + 64, max_requests=1,
                                                     max_batch_tokens=max(longest if a.batched else 1, 16),
                                                     max_context=longest + 64))
    losses = []                                    # (position, token, loss)
    total, top1 = 0.0, 0

    def score(logits_row, pos):
        nonlocal total, top1
        logp = torch.log_softmax(logits_row.double(), dim=-1)
        nll = -float(logp[ids[pos]])
        top1 += int(int(torch.argmax(logits_row)) == ids[pos])
        total += nll
        losses.append((pos, ids[pos], nll))

    for start, end, first in passes:
        slot = eng.manager.add_request("t").slot   # an empty context for every pass
        eng.storage.zero_state_slot(slot)
        if a.batched:
            rows = [r for r in range(end - start) if r >= first and r + 1 < end - start]
            logits = eng.runner.step([StepEntry("t", ids[start:end], tuple(rows))])
            host = logits.float().cpu() if logits is not None else None
            for k, r in enumerate(rows):
                score(host[k], start + r + 1)
        else:
            for i in range(start, end - 1):
                wanted = i - start >= first
                logits = eng.runner.step([StepEntry("t", [ids[i]], (0,) if wanted else ())])
                if wanted:
                    score(logits.float().cpu()[0], i + 1)
        eng.manager.free_request("t")
        if len(passes) > 1:
            print(f"[{len(losses) // max(end - start - 1 - first, 1)}]{math.exp(total / max(len(losses), 1)):.4f},",
                  end="", file=sys.stderr, flush=True)
    if len(passes) > 1:
        print(file=sys.stderr)
    eng.runner.raise_on_device_error()
    n = len(losses)
    mean = total / n
    print(f"\n{n} tokens scored\n  mean loss   {mean:.4f} nats/token\n  perplexity  {math.exp(mean):.2f}\n"
          f"  top-1       {100.0 * top1 / n:.1f}% ({top1}/{n})")
    if a.worst > 0:
        print("\nworst-predicted tokens:")
        for pos, tok, nll in sorted(losses, key=lambda t: -t[2])[:a.worst]:
            print(f"  pos {pos:>4}  loss {nll:>8.3f}  token {tok}")
    return 0


def cmd_init(a) -> int:
    import torch
    from .config import architecture_name, lookup_architecture
    from .weights import write_model_folder
    with open(a.config) as f:
        d = json.load(f)
    config_cls, builder = lookup_architecture(architecture_name(d))
    config = config_cls.from_dict(d)
    model = builder(config, torch.float32, "cpu")
    write_model_folder(a.out, config, model.weight_specs(), a.seed)
    print(f"wrote {a.out}: {config.summary()}")
    return 0


def _human_bytes(n: int) -> str:
    for unit in ("B", "KiB", "MiB", "GiB"):
        if n < 1024 or unit == "GiB":
            return f"{n} B" if unit == "B" else f"{n:.2f} {unit}"
        n /= 1024.0
    return f"{n:.2f} GiB"


def cmd_inspect(a) -> int:
    """Describes a model folder in the manner of the reference's ``airun inspect``
    (crates/airun-cli/src/inspect.rs:10-36: ``--tensors``, ``--json``, ``--values TENSOR --count N``):
    the configuration, the tensors of its safetensors files, and whether they are what the
    architecture wants (the error a load would raise, without loading anything).  Needs no GPU."""
    import torch
    from .config import architecture_name, load_config, lookup_architecture, read_config_json
    from .weights import WeightError, check_source, open_model_folder
    config = load_config(a.model)
    src = open_model_folder(a.model)
    try:
        if a.values:
            if a.values not in src.names():
                raise SystemExit(f"no tensor named {a.values!r} in {a.model} (see --tensors)")
            t = src.read(a.values)
            flat = t.reshape(-1)
            head = flat[:max(a.count, 0)].tolist()
            print(f"{a.values}  {str(t.dtype).replace('torch.', '')}  {list(t.shape)}")
            print("first values: " + " ".join(f"{v:.6g}" for v in head))
            if flat.numel() and t.dtype.is_floating_point:
                d = flat.double()
                print(f"min {float(d.min()):.6g}  max {float(d.max()):.6g}  mean {float(d.mean()):.6g}  "
                      f"std {float(d.std(unbiased=False)):.6g}  non-finite {int((~torch.isfinite(d)).sum())}")
            return 0
        tensors = []
        for name in sorted(src.names()):
            dt, shape = src.info(name)
            n = 1
            for k in shape:
                n *= int(k)
            tensors.append(dict(name=name, dtype=str(dt).replace("torch.", ""), shape=list(shape),
                                bytes=n * torch.empty(0, dtype=dt).element_size()))
        _, builder = lookup_architecture(architecture_name(read_config_json(a.model)))
        model = builder(config, torch.float32, "meta")
        problem = None
        try:
            check_source(model.weight_specs(), src, model.ignorable_tensors())
        except WeightError as e:
            problem = str(e)
    finally:
        src.close()
    total = sum(t["bytes"] for t in tensors)
    by_type = {}
    for t in tensors:
        by_type[t["dtype"]] = by_type.get(t["dtype"], 0) + t["bytes"]
    if a.json:
        out = dict(folder=a.model, architecture=config.architecture, config=config.to_dict(), summary=config.summary(),
                   tensor_count=len(tensors), tensor_bytes=total, bytes_by_dtype=by_type, loadable=problem is None,
                   problem=problem)
        if a.tensors:
            out["tensors"] = tensors
        print(json.dumps(out))
        return 0 if problem is None else 1
    print(f"folder    {a.model}")
    print(f"model     {config.summary()}")
    print(f"tensors   {len(tensors)}, {_human_bytes(total)} (" +
          ", ".join(f"{k} {_human_bytes(v)}" for k, v in sorted(by_type.items())) + ")")
    print("weights   " + ("every tensor the architecture wants is there, with the right shape" if problem is None
                          else "NOT loadable:"))
    if problem is not None:
        print(problem)
    if a.tensors:
        width = max((len(t["name"]) for t in tensors), default=4)
        for t in tensors:
            print(f"  {t['name']:<{width}}  {t['dtype']:<9} {str(t['shape']):<20} {_human_bytes(t['bytes'])}")
    return 0 if problem is None else 1


def cmd_gpu(a) -> int:
    """The reference's ``airun gpu`` (crates/airun-cli/src/gpu.rs:8-95): the CUDA devices in CUDA's own
    order, their architecture, memory and size, and whether this engine runs on them (its kernels
    are built for sm_100a only).  It reads; it changes no setting of any device."""
    import torch
    devices = []
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for i in range(n):
        pr = torch.cuda.get_device_properties(i)
        try:
            free, total = torch.cuda.mem_get_info(i)
        except RuntimeError:
            free, total = 0, int(pr.total_memory)
        devices.append(dict(ordinal=i, name=pr.name, compute_capability=f"{pr.major}.{pr.minor}",
                            supported=(pr.major, pr.minor) == (10, 0), free_bytes=int(free), total_bytes=int(total),
                            sm_count=int(pr.multi_processor_count),
                            threads_per_sm=int(getattr(pr, "max_threads_per_multi_processor", 0)),
                            l2_bytes=int(getattr(pr, "L2_cache_size", 0))))
    if a.json:
        print(json.dumps(dict(cuda_runtime=torch.version.cuda, devices=devices)))
        return 0
    print(f"CUDA runtime {torch.version.cuda} (the one PyTorch was built with)")
    if not devices:
        print("\nNo CUDA device found.")
        print("  - Check that an NVIDIA GPU is present and `nvidia-smi` works.")
        print("  - airun_b200 has no CPU path: it needs a B200 (sm_100a).")
        return 0
    print(f"\n{len(devices)} CUDA device(s). Ordinals below are CUDA's, which need not match nvidia-smi's order.\n")
    for d in devices:
        print(f"GPU {d['ordinal']} - {d['name']}" + ("" if d["supported"] else "  [UNSUPPORTED: the kernels are built for sm_100a]"))
        print(f"  arch          compute {d['compute_capability']}")
        print(f"  memory        {_human_bytes(d['free_bytes'])} free of {_human_bytes(d['total_bytes'])}")
        print(f"  compute       {d['sm_count']} SMs, {d['threads_per_sm']} threads/SM, {_human_bytes(d['l2_bytes'])} L2")
    return 0


def cmd_selftest(a) -> int:
    """The reference's ``airun selftest --device N --verbose`` (crates/airun-cli/src/selftest.rs:13-22)."""
    from . import selftest
    return selftest.run(a.device, a.verbose)


def main(argv: Optional[List[str]] = None) -> int:
    a = build_parser().parse_args(argv)
    return {"run": cmd_run, "bench": cmd_bench, "perplexity": cmd_perplexity, "init": cmd_init,
            "inspect": cmd_inspect, "gpu": cmd_gpu, "selftest": cmd_selftest}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
