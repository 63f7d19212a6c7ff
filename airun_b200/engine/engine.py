"""The engine: a model folder (or a configuration and a seed) in, tokens out.

``Engine`` owns the model, the cache manager with its device storage, the step
function and a scheduler, and offers ``generate`` (token ids in, token ids
out), ``add_request`` / ``run_step`` for callers that drive the loop
themselves, and ``runner.step`` for raw logits.  The reference's Rust API is
``loader::load`` followed by ``Runtime::generate``
(crates/airun-core/src/loader.rs:216, crates/airun-core/src/runtime.rs:4903-5089);
its per-run statistics (prompt / generated counts, prefill and decode
milliseconds, stop reason) are ``GenerationStats`` (runtime.rs:5130-5165).
"""
from __future__ import annotations

import itertools
import os
import time
from dataclasses import dataclass
from typing import Hashable, List, Optional, Sequence, Union

import numpy as np
import torch

from ..cache.manager import CacheManager, CacheStorage
from ..config.base import ModelConfig, architecture_name, lookup_architecture, read_config_json
from ..kernels import ops
from ..sampling.sampler import SamplingParams, sample_candidates, sample_rows
from ..weights.loader import open_model_folder
from .scheduler import FinishReason, Request, Scheduler
from .step import StepEntry, StepRunner

# AIRUN_SCHED_TIMING=1 prints the host time of every scheduler step (the reference's switch of the
# same name, crates/airun-cli/src/sched.rs:345-348).
SCHED_TIMING = __import__("os").environ.get("AIRUN_SCHED_TIMING", "") not in ("", "0")

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


@dataclass
class EngineOptions:
    dtype: Union[str, torch.dtype] = "bfloat16"
    device: str = "cuda:0"
    page_size: int = 16
    num_pages: Optional[int] = None          # pages per cache group; None: from cache_tokens
    cache_tokens: Optional[int] = None       # tokens the cache holds; None: from memory_fraction
    memory_fraction: float = 0.85            # of the memory free after loading the weights
    max_batch_tokens: int = 2048             # token budget of one step (the reference's -b/--batch-size)
    max_requests: int = 64                   # requests live at a time (the reference's --parallel slots)
    max_context: Optional[int] = None        # longest request (the reference's -c/--ctx-size)
    prefix_cache: bool = False               # keep finished requests' caches for prompts that begin alike


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    steps: int = 0
    preemptions: int = 0
    host_gap_ms: float = 0.0       # time from reading a step's result to having launched the next step: the GPU
                                   # may idle for as long (an upper bound on what the host costs)

    @property
    def prefill_tps(self) -> float:
        return self.prompt_tokens / (self.prefill_ms / 1e3) if self.prefill_ms > 0 else 0.0

    @property
    def decode_tps(self) -> float:
        return self.generated_tokens / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0


@dataclass
class GenerationResult:
    token_ids: List[int]
    finish_reason: str
    prompt_tokens: int
    logprobs: Optional[list] = None          # TokenProbs per sampled token when SamplingParams.logprobs is set


class Engine:
    def __init__(self, config: ModelConfig, model, options: EngineOptions):
        self.config, self.model, self.options = config, model, options
        self.device = model.device
        self.dtype = model.dtype
        o = options
        specs, cache_from = model.cache_specs()
        ps = o.page_size
        if o.num_pages is not None:
            num_pages = int(o.num_pages)
        else:
            tokens = o.cache_tokens if o.cache_tokens is not None else self._tokens_that_fit(specs, cache_from, o)
            num_pages = max(1, (int(tokens) + ps - 1) // ps)
        self.max_context = int(o.max_context or min(num_pages * ps,
                                                    max(getattr(config, "max_position_embeddings", 4096), 1)))
        self.max_context = min(self.max_context, num_pages * ps)
        self.manager = CacheManager(specs, cache_from, ps, num_pages, o.max_requests,
                                    max_blocks=(self.max_context + ps - 1) // ps)
        self.storage = CacheStorage(self.manager, self.dtype, self.device)
        self.runner = StepRunner(model, self.manager, self.storage, o.max_batch_tokens,
                                 min(o.max_requests, o.max_batch_tokens), self.max_context)
        self.scheduler = Scheduler(self.manager, o.max_batch_tokens, self.runner.R_max, self.max_context,
                                   prefix_cache=o.prefix_cache, run_copies=self.storage.run_copies)
        self._ids = itertools.count()
        R = self.runner.R_max
        self._small_host = torch.zeros(2 * R, dtype=torch.float32, pin_memory=self.device.type == "cuda")
        self._small_dev = torch.zeros(2 * R, dtype=torch.float32, device=self.device)
        self._picked_dev = torch.zeros(R + 1, dtype=torch.int32, device=self.device)
        self._picked_host = torch.zeros(R + 1, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        self.stats = GenerationStats()
        self._ahead = None        # (requests, prepared step): the next decode step, laid out while this one runs
        self._host_rows = None    # buffers for the logits rows the host samples
        self._cand_bufs = None    # buffers for the largest logits of the rows whose chain cuts to them anyway
        # AIRUN_NARROW_ROWS=0: every row the host samples travels whole (the plain way; tests compare the two)
        self._narrow_rows = os.environ.get("AIRUN_NARROW_ROWS", "1") != "0"
        self._distrust_candidates = False   # tests: treat every list of largest logits as one the kernel could not vouch for
        self._result_read_at = None

    # ------------------------------------------------------------ construction
    @staticmethod
    def _tokens_that_fit(specs, cache_from, o: EngineOptions) -> int:
        """Tokens of cache the free memory holds: ``memory_fraction`` of it, less the fixed-size state of
        ``max_requests`` requests, over the bytes a token takes in all paged layers."""
        from ..parts.base import PagedKVSpec, StateSpec
        dt = _DTYPES[o.dtype]
        esz = 2 if dt == torch.bfloat16 else 4
        per_token = sum(2 * s.num_kv_heads * s.head_dim * esz
                        for s, src in zip(specs, cache_from) if isinstance(s, PagedKVSpec) and src is None)
        if per_token == 0:
            return o.page_size
        state = 0
        for s, src in zip(specs, cache_from):
            if isinstance(s, StateSpec) and src is None:
                n = torch.empty((), dtype=s.dtype).element_size()
                for d in s.shape:
                    n *= int(d)
                state += n * o.max_requests
        free, _ = torch.cuda.mem_get_info(torch.device(o.device))
        return max(o.page_size, (int(free * o.memory_fraction) - state) // per_token)

    @classmethod
    def from_folder(cls, model_dir: str, options: Optional[EngineOptions] = None, **kw) -> "Engine":
        """Loads config.json and model.safetensors of ``model_dir``."""
        options = options or EngineOptions(**kw)
        cls._require_gpu(options)
        d = read_config_json(model_dir)
        config_cls, builder = lookup_architecture(architecture_name(d))
        config = config_cls.from_dict(d)
        model = builder(config, _DTYPES[options.dtype], options.device)
        src = open_model_folder(model_dir)
        try:
            model.load(src)
        finally:
            src.close()
        return cls(config, model, options)

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int, options: Optional[EngineOptions] = None, **kw) -> "Engine":
        """Random-weights mode: seeded weights made on the device, no files."""
        options = options or EngineOptions(**kw)
        cls._require_gpu(options)
        _, builder = lookup_architecture(config.architecture)
        model = builder(config, _DTYPES[options.dtype], options.device)
        model.load_random(seed)
        return cls(config, model, options)

    @staticmethod
    def _require_gpu(options: EngineOptions) -> None:
        if options.dtype not in _DTYPES:
            raise ValueError(f"dtype {options.dtype!r}: the engine computes in bfloat16 or float32")
        if not torch.cuda.is_available():
            raise RuntimeError("airun_b200 runs on a CUDA GPU (sm_100a); none is visible and there is no CPU path")

    # ------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    max_new_tokens: int = 256, eog_tokens: Sequence[int] = (), rid: Hashable = None) -> Request:
        rid = next(self._ids) if rid is None else rid
        V = self.config.vocab_size
        bad = [t for t in prompt if not (0 <= int(t) < V)]
        if bad:
            raise ValueError(f"prompt holds token ids outside [0, {V}): {bad[:5]}")
        req = Request(rid, [int(t) for t in prompt], params or SamplingParams(), int(max_new_tokens),
                      tuple(int(t) for t in eog_tokens))
        self.scheduler.add(req)
        return req

    def fork_request(self, parent: Request, params: Optional[SamplingParams] = None,
                     max_new_tokens: Optional[int] = None, rid: Hashable = None) -> Request:
        """A new request that continues ``parent``'s tokens so far with its own sampling, reading
        the parent's cache pages instead of computing them again (only a partly filled last page
        is copied).  Raises ``OutOfPages`` / ``CacheError`` if a page or a request slot is short."""
        rid = next(self._ids) if rid is None else rid
        child = Request(rid, list(parent.tokens), params or SamplingParams(**{**parent.params.__dict__}),
                        int(max_new_tokens if max_new_tokens is not None else parent.max_new_tokens),
                        parent.eog_tokens)
        self.storage.run_copies(self.scheduler.fork(parent, child))
        return child

    def cancel(self, req: Request) -> None:
        """Ends ``req`` with ``Cancelled`` at the next step's planning (its pages are given back then);
        a request that is still waiting never starts."""
        req.cancelled = True

    def clear_prefix_cache(self) -> int:
        """Gives back the pages of every kept cache (``EngineOptions.prefix_cache``); returns how many
        caches were dropped."""
        n = 0
        while self.scheduler._drop_kept():
            n += 1
        return n

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def run_step(self) -> List[Request]:
        """One scheduler step: plan, run, sample.  Returns the requests that finished."""
        t_start = time.perf_counter() if SCHED_TIMING else 0.0
        ahead, self._ahead = self._ahead, None
        finished: List[Request] = []
        plan, prep = None, None
        if ahead is not None:
            plan, prep, sampled = ahead
            finished += plan.finished
            self.stats.preemptions += len(plan.preempted)
            if any(r.finished is not None or r.cancelled for r in sampled):
                plan, prep = None, None      # a request it counted on is gone: plan again (what it admitted stays)
        if plan is None:
            plan = self.scheduler.plan()
            finished += plan.finished
            self.stats.preemptions += len(plan.preempted)
        if not plan.entries:
            return finished
        entries = []
        wanting: List[Request] = []
        for e in plan.entries:
            toks = e.request.token_slice(e.start, e.count)
            entries.append(StepEntry(e.request.rid, toks, (e.count - 1,) if e.wants_logits else ()))
            if e.wants_logits:
                wanting.append(e.request)
        if prep is not None:
            logits = self.runner.launch_prepared(prep, [t for e in entries for t in e.tokens])
        else:
            logits = self.runner.step(entries, checked=True)
        if self._result_read_at is not None:
            self.stats.host_gap_ms += (time.perf_counter() - self._result_read_at) * 1e3
            self._result_read_at = None
        self.scheduler.advance(plan)
        if wanting:
            tokens = self._sample(logits, wanting, look_ahead=True)
            for req, tok in zip(wanting, tokens):
                if self.scheduler.accept(req, tok) is not None:
                    finished.append(req)
        self.stats.steps += 1
        if not self.scheduler.has_work():
            self._result_read_at = None                    # idle from here on: what follows is not a gap between steps
        if SCHED_TIMING:
            import sys
            print(f"[airun_b200] step {self.stats.steps}: {len(plan.entries)} requests, "
                  f"{sum(e.count for e in plan.entries)} tokens{' (laid out ahead)' if prep is not None else ''}, "
                  f"{(time.perf_counter() - t_start) * 1e3:.3f} ms", file=sys.stderr)
        return finished

    # While the GPU runs a step, the host plans and lays out the next one (admission, portions, pages,
    # positions, block tables, their copy to the device): all of it but the values of the tokens being
    # sampled right now, which it only has when it has read this step's result.  A request whose token on
    # its way is certainly its last (its length or the context ends there) is left out of that plan; it
    # keeps its pages and slot until the token has been read.  The others are taken to go on; it is only
    # done when pages are plentiful, so that the plan cannot end or preempt anybody, and if one of them
    # ends all the same (an end token, a cancellation), the plan's batch is dropped and the step is
    # planned again.
    _PLACEHOLDER = 0

    def _prepare_ahead(self, sampled: List[Request]) -> None:
        sch = self.scheduler
        going: List[Request] = []
        ending: List[Request] = []
        for r in sampled:
            if r.cancelled or r.num_computed != r.num_tokens:
                return
            last = len(r.output) + 1 >= r.max_new_tokens or r.num_tokens + 2 > self.max_context
            (ending if last else going).append(r)
        ps = self.manager.page_size
        margin = len(sch.running) + len(sch.waiting) + self.options.max_batch_tokens // ps + 2
        if any(g.allocator.num_free < margin for g in self.manager.paged):
            return
        for r in going:
            r.output.append(self._PLACEHOLDER)             # stands for the token on its way
        for r in ending:
            r.ending = True
        prep = None
        try:
            plan = sch.plan()
            if plan.entries and not plan.preempted:
                entries = [StepEntry(e.request.rid, e.request.token_slice(e.start, e.count),
                                     (e.count - 1,) if e.wants_logits else ()) for e in plan.entries]
                try:
                    prep = self.runner.prepare_step(entries)
                except Exception:                          # noqa: BLE001 - e.g. out of pages: the ordinary path decides
                    prep = None
        finally:
            for r in going:
                r.output.pop()
            for r in ending:
                r.ending = False
        self._ahead = (plan, prep, list(going))

    def _sample(self, logits: torch.Tensor, reqs: List[Request], look_ahead: bool = False) -> List[int]:
        n = len(reqs)
        R = self.runner.R_max
        host = self._small_host.numpy()
        for i, r in enumerate(reqs):
            p = r.params
            dev = r.sampler.device_ok
            host[i] = p.temperature if (dev and p.temperature > 0.0) else 0.0
            host[R + i] = r.sampler.next_uniform() if (dev and p.temperature > 0.0) else 0.0
        self._small_dev.copy_(self._small_host, non_blocking=True)
        ops.sample(logits, self._picked_dev, self._small_dev[:R], self._small_dev[R:])
        self._picked_dev[R:R + 1].copy_(self.runner.err)
        self._picked_host.copy_(self._picked_dev, non_blocking=True)
        # Rows the device kernel cannot pick alone: those whose chain cuts to its k largest logits anyway send only
        # their largest logits to the host (found on the device), the others their whole row.
        cand_rows, host_rows, n_cand = [], [], 0
        for i, r in enumerate(reqs):
            if r.sampler.device_ok:
                continue
            need = r.sampler.candidates_needed if self._narrow_rows else 0
            if need > 0:
                cand_rows.append(i)
                n_cand = max(n_cand, need)
            else:
                host_rows.append(i)
        cands = self._candidates_to_host(logits, cand_rows, n_cand) if cand_rows else None
        rows_host = self._rows_to_host(logits, host_rows) if host_rows else None
        if look_ahead and not host_rows and self._ahead is None:
            self._prepare_ahead(reqs)                      # the GPU is busy: plan and lay out the next step meanwhile
        torch.cuda.current_stream().synchronize()
        self._result_read_at = time.perf_counter()
        picked = self._picked_host.numpy()
        if picked[R]:
            self.runner.err.zero_()
            raise RuntimeError("a kernel reported: " + ops.describe_device_error(int(picked[R])))
        out = [int(picked[i]) for i in range(n)]
        if cand_rows:
            ids, vals, flags = cands
            unsure = [i for j, i in enumerate(cand_rows) if flags[j] or self._distrust_candidates]
            if unsure:                                      # the kernel could not vouch for these lists: whole rows
                more = self._rows_to_host(logits, unsure)
                torch.cuda.current_stream().synchronize()
                for i, tok in zip(unsure, sample_rows([reqs[i].sampler for i in unsure], more, [reqs[i].tokens for i in unsure])):
                    out[i] = tok
            sure = [j for j, i in enumerate(cand_rows) if not (flags[j] or self._distrust_candidates)]
            if sure:
                rq = [reqs[cand_rows[j]] for j in sure]
                windows = [r.token_slice(max(0, r.num_tokens - r.params.repeat_last_n), min(r.num_tokens, r.params.repeat_last_n))
                           if r.params.penalizing else [] for r in rq]
                for j, tok in zip(sure, sample_candidates([r.sampler for r in rq], ids[sure], vals[sure], windows)):
                    out[cand_rows[j]] = tok
        if host_rows:
            picked_host = sample_rows([reqs[i].sampler for i in host_rows], rows_host, [reqs[i].tokens for i in host_rows])
            for i, tok in zip(host_rows, picked_host):
                out[i] = tok
        return out

    def _candidates_to_host(self, logits: torch.Tensor, rows: List[int], n_cand: int):
        """The ``n_cand`` largest logits of each of ``rows`` with their ids, found by the engine's own kernel and
        copied to pinned memory (queued; the caller synchronises the stream): ids, values, flags as numpy views."""
        n, cap = len(rows), self.runner.R_max
        if self._cand_bufs is None:
            C = ops.LARGEST_LOGITS_MAX
            self._cand_bufs = (torch.empty(cap, dtype=torch.int32, pin_memory=True),
                               torch.empty(cap, dtype=torch.int32, device=self.device),
                               torch.empty(cap * C, dtype=torch.int32, device=self.device),
                               torch.empty(cap * C, dtype=torch.float32, device=self.device),
                               torch.empty(cap, dtype=torch.int32, device=self.device),
                               torch.empty(cap * C, dtype=torch.int32, pin_memory=True),
                               torch.empty(cap * C, dtype=torch.float32, pin_memory=True),
                               torch.empty(cap, dtype=torch.int32, pin_memory=True))
        idx_host, idx_dev, ids_dev, vals_dev, flags_dev, ids_host, vals_host, flags_host = self._cand_bufs
        idx_host[:n] = torch.as_tensor(rows, dtype=torch.int32)
        idx_dev[:n].copy_(idx_host[:n], non_blocking=True)
        ops.largest_logits(logits, idx_dev, n, n_cand, ids_dev, vals_dev, flags_dev)
        ids_host[:n * n_cand].copy_(ids_dev[:n * n_cand], non_blocking=True)
        vals_host[:n * n_cand].copy_(vals_dev[:n * n_cand], non_blocking=True)
        flags_host[:n].copy_(flags_dev[:n], non_blocking=True)
        return (ids_host[:n * n_cand].numpy().reshape(n, n_cand), vals_host[:n * n_cand].numpy().reshape(n, n_cand),
                flags_host[:n].numpy())

    def _rows_to_host(self, logits: torch.Tensor, rows: List[int]) -> np.ndarray:
        """The logits of the rows the host samples: gathered by the engine's own kernel into one buffer
        and copied to pinned memory in one transfer (queued; the caller synchronises the stream)."""
        n, V = len(rows), logits.shape[1]
        if self._host_rows is None or self._host_rows[0].shape[0] < n:
            cap = max(n, min(self.runner.R_max, 8))
            self._host_rows = (torch.empty((cap, V), dtype=torch.float32, device=self.device),
                               torch.empty((cap, V), dtype=torch.float32, pin_memory=True),
                               torch.empty(cap, dtype=torch.int32, pin_memory=True),
                               torch.empty(cap, dtype=torch.int32, device=self.device))
        dev, host, idx_host, idx_dev = self._host_rows
        idx_host[:n] = torch.as_tensor(rows, dtype=torch.int32)
        idx_dev[:n].copy_(idx_host[:n], non_blocking=True)
        ops.gather_rows(logits, idx_dev[:n], dev)
        host[:n].copy_(dev[:n], non_blocking=True)
        return host[:n].numpy()

    # ------------------------------------------------------------ generation
    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]],
                 params: Union[None, SamplingParams, Sequence[SamplingParams]] = None,
                 max_new_tokens: int = 256, eog_tokens: Sequence[int] = (),
                 on_token=None) -> Union[GenerationResult, List[GenerationResult]]:
        """Generates for one prompt (a list of ids) or several (a list of lists)."""
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple, np.ndarray))
        plist = [prompts] if single else list(prompts)
        if isinstance(params, SamplingParams) or params is None:
            params_list = [params] * len(plist)
        else:
            params_list = list(params)
        reqs = []
        for p, sp in zip(plist, params_list):
            if sp is not None and len(plist) > 1:
                sp = SamplingParams(**{**sp.__dict__})          # one generator per request
            reqs.append(self.add_request(p, sp, max_new_tokens, eog_tokens))
        self.stats = GenerationStats(prompt_tokens=sum(len(p) for p in plist))
        emitted = {id(r): 0 for r in reqs}
        t0 = time.perf_counter()
        t_first = None
        while any(r.finished is None for r in reqs):
            if not self.has_work():
                break
            self.run_step()
            if t_first is None and all(r.output or r.finished for r in reqs):
                t_first = time.perf_counter()
            if on_token is not None:
                for r in reqs:
                    while emitted[id(r)] < len(r.output):
                        on_token(r, r.output[emitted[id(r)]])
                        emitted[id(r)] += 1
        t1 = time.perf_counter()
        t_first = t_first or t1
        self.stats.prefill_ms = (t_first - t0) * 1e3
        self.stats.decode_ms = (t1 - t_first) * 1e3
        self.stats.generated_tokens = sum(len(r.output) for r in reqs)
        res = [GenerationResult(list(r.output), (r.finished or FinishReason.CANCELLED).value, len(r.prompt),
                                list(r.sampler.probs) if r.params.logprobs is not None else None)
               for r in reqs]
        return res[0] if single else res
