"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees.

The reference's scheduler keeps a FIFO of jobs, admits one waiting job per loop
iteration when a slot is free, prefills it alone and whole, and otherwise
decodes one token for every active request (crates/airun-cli/src/sched.rs:82-213,
:485-508); its finish reasons are MaxTokens, EndOfGeneration (the end token is
not emitted), Cancelled and ContextFull (sched.rs:511-539,
crates/airun-core/src/runtime.rs:5099-5108, :5020-5023).  It can never run out
of cache at run time because every slot owns a full context.  Here the cache is
paged, so each step is planned under two limits, a token budget and the free
pages:

1. Every running request comes first, in admission order: one token if it is
   decoding, else the next portion of its prompt, as large as budget and free
   pages allow (a portion may be as small as one token).
2. If a decoding request cannot get the page it needs, the most recently
   admitted running request is preempted: its pages are given back and it
   returns to the FRONT of the waiting queue, to be recomputed later from its
   prompt plus the tokens it has produced.  A request that is alone and still
   cannot get a page ends with ContextFull.
3. Then waiting requests are admitted first-in first-out while budget, request
   slots and pages for at least part of the prompt remain.
A prompt longer than the whole pool or the context limit is refused at submission.

Prefix reuse (off unless asked for).  The reference keeps every slot's token history and starts a
new turn from the longest common prefix of that history and the new prompt, at most all but the
prompt's last token so that one token is always computed for its logits
(crates/airun-core/src/runtime.rs:3256-3264, :2680-2681), and picks the slot with the longest
such prefix (crates/airun-cli/src/sched.rs:381-388).  Here a finished request's pages are kept
under a private name with the tokens they hold; a new request is forked from the kept cache with
the longest common prefix (a page or more) and cut back to that prefix, so whole pages are shared
and never written, and only the page the cut falls into is copied.  Kept caches are the first to
go when pages or request slots run short, the one unused longest first, before anybody is
preempted.  Models with fixed-size state or windows cannot be cut back and take no part.

The scheduler is host-side only; it decides, the step function runs.
"""
from __future__ import annotations

import itertools
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Deque, Dict, Hashable, List, Optional, Tuple

from ..cache.manager import CacheError, CacheManager, CopyPlan, OutOfPages, OutOfSlots
from ..sampling.sampler import Sampler, SamplingParams


class FinishReason(str, Enum):
    MAX_TOKENS = "MaxTokens"
    END_OF_GENERATION = "EndOfGeneration"
    CANCELLED = "Cancelled"
    CONTEXT_FULL = "ContextFull"
    REFUSED = "Refused"


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    params: SamplingParams
    max_new_tokens: int
    eog_tokens: Tuple[int, ...] = ()
    output: List[int] = field(default_factory=list)
    num_computed: int = 0            # tokens whose keys and values are in the cache
    finished: Optional[FinishReason] = None
    cancelled: bool = False
    preemptions: int = 0
    sampler: Optional[Sampler] = None
    ending: bool = False             # the token being sampled right now is its last: a plan made meanwhile leaves it out

    def __post_init__(self):
        if self.sampler is None:
            self.sampler = Sampler(self.params)

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def token_slice(self, start: int, count: int) -> List[int]:
        """tokens[start:start+count] without building the whole list."""
        np_ = len(self.prompt)
        end = start + count
        if end <= np_:
            return self.prompt[start:end]
        if start >= np_:
            return self.output[start - np_:end - np_]
        return self.prompt[start:] + self.output[:end - np_]

    @property
    def decoding(self) -> bool:
        return self.num_computed >= len(self.prompt) and self.num_tokens - self.num_computed == 1


@dataclass
class PlannedEntry:
    request: Request
    start: int                       # first token (index into request.tokens) run this step
    count: int
    wants_logits: bool               # the portion ends at the newest token: sample after it


@dataclass
class Plan:
    entries: List[PlannedEntry]
    preempted: List[Request]
    finished: List[Request]          # requests ended while planning (ContextFull)


class Scheduler:
    def __init__(self, manager: CacheManager, max_batch_tokens: int, max_batch_reqs: int, max_context: int,
                 prefix_cache: bool = False, run_copies=None):
        """``prefix_cache``: keep the caches of finished requests for later prompts that begin alike.
        ``run_copies``: called with the CopyPlan of every reuse as soon as it is decided (the engine
        queues the page copies on its stream, ahead of the step that reads them)."""
        self.manager = manager
        self.max_batch_tokens, self.max_batch_reqs, self.max_context = max_batch_tokens, max_batch_reqs, max_context
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []        # in admission order
        self.stats = dict(steps=0, preemptions=0, admitted=0, refused=0, prefix_hits=0, prefix_tokens=0,
                          prefix_evictions=0)
        self.prefix_cache = bool(prefix_cache) and manager.can_rewind
        self.run_copies = run_copies
        self.kept: "OrderedDict[Hashable, List[int]]" = OrderedDict()   # kept cache -> its tokens, least recently used first
        self._kept_ids = itertools.count()

    # ------------------------------------------------------------ submission
    def add(self, req: Request) -> None:
        capacity = self.manager.max_tokens_possible()
        if len(req.prompt) == 0:
            req.finished = FinishReason.REFUSED
        elif (req.rid in self.manager.requests or any(r.rid == req.rid for r in self.waiting)
              or any(r.rid == req.rid for r in self.running)):
            # a second request under a live id would wedge the queue at admission
            req.finished = FinishReason.REFUSED
        elif len(req.prompt) + 1 > min(capacity, self.max_context):
            req.finished = FinishReason.REFUSED
        if req.finished is not None:
            self.stats["refused"] += 1
            return
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def fork(self, parent: Request, child: Request):
        """``child`` (whose prompt must be the parent's tokens so far) starts from the parent's
        cache instead of computing it again: whole pages are shared.  Returns the device copies
        the caller has to run before the next step."""
        if parent not in self.running or parent.finished is not None:
            raise ValueError("only a running request can be forked")
        if child.prompt != parent.tokens:
            raise ValueError("a fork continues the parent's tokens; its prompt must equal them")
        if child.rid in self.manager.requests or any(r.rid == child.rid for r in self.waiting):
            raise ValueError(f"request id {child.rid!r} is in use")
        while True:
            try:
                copies = self.manager.fork(parent.rid, child.rid)
                break
            except (OutOfPages, OutOfSlots):              # a shortage: kept caches give way to a fork as well
                if not self._drop_kept():
                    raise
        child.num_computed = parent.num_computed
        self.running.append(child)
        self.stats["admitted"] += 1
        return copies

    # ------------------------------------------------------------ kept caches of finished requests
    def _keep(self, req: Request) -> bool:
        """Keeps the cache of a request that ends instead of freeing it; False if it is not worth it."""
        if not self.prefix_cache or req.num_computed < self.manager.page_size:
            return False
        name = ("kept", next(self._kept_ids))
        self.manager.rename(req.rid, name)
        self.manager.truncate(name, req.num_computed)      # pages taken ahead for a token that never came
        self.kept[name] = req.tokens[:req.num_computed]
        return True

    def _drop_kept(self, spare: Hashable = None) -> bool:
        """Frees the kept cache that went unused longest (never ``spare``); False if none is left."""
        name = next((k for k in self.kept if k != spare), None)
        if name is None:
            return False
        del self.kept[name]
        self.manager.free_request(name)
        self.stats["prefix_evictions"] += 1
        return True

    def _start_from_kept(self, req: Request) -> bool:
        """Makes ``req`` a live request that starts from the kept cache sharing the longest prefix with
        its tokens (a page or more, never the last token).  False: nothing to reuse, ``req`` is not live."""
        toks = req.tokens
        limit = len(toks) - 1
        best, best_n = None, 0
        for name, have in self.kept.items():
            n, m = 0, min(limit, len(have))
            if m <= best_n:
                continue
            while n < m and have[n] == toks[n]:
                n += 1
            if n > best_n:
                best, best_n = name, n
        if best is None or best_n < self.manager.page_size:
            return False
        while True:
            # the fork wants a page for a partly filled last page, the cut one for a shared page it
            # falls into: other kept caches give way to that, the one unused longest first
            try:
                forked = self.manager.fork(best, req.rid)
            except (OutOfPages, OutOfSlots):
                if self._drop_kept(spare=best):
                    continue
                return False
            try:
                cut = self.manager.truncate(req.rid, best_n)
                break
            except OutOfPages:
                self.manager.free_request(req.rid)
                if not self._drop_kept(spare=best):
                    return False
        # a copy the fork asked for is moot if the cut gave its page back
        held = {gid: set(self.manager.block_table(req.rid, gid)) for gid in {g for g, _, _ in forked.pages}}
        pages = [c for c in forked.pages if c[2] in held[c[0]]] + cut.pages
        if pages and self.run_copies is not None:
            self.run_copies(CopyPlan(pages))
        self.kept.move_to_end(best)
        req.num_computed = best_n
        self.stats["prefix_hits"] += 1
        self.stats["prefix_tokens"] += best_n
        return True

    # ------------------------------------------------------------ planning
    def _need_if_fits(self, req: Request, n: int, planned: Dict[int, int]) -> Optional[Dict[int, int]]:
        """Pages ``n`` more tokens of ``req`` would take, or None if they are not free.  Kept caches
        are given up, the one unused longest first, for as long as that can make them fit."""
        need = self.manager.pages_needed(req.rid, n)
        while True:
            free = self.manager.free_pages()
            if all(k + planned.get(gid, 0) <= free[gid] for gid, k in need.items()):
                return need
            if not self._drop_kept():
                return None

    def _pages_fit(self, req: Request, n: int, planned: Dict[int, int]) -> bool:
        return self._need_if_fits(req, n, planned) is not None

    @staticmethod
    def _note_need(need: Dict[int, int], planned: Dict[int, int]) -> None:
        for gid, k in need.items():
            if k:
                planned[gid] = planned.get(gid, 0) + k

    def _note(self, req: Request, n: int, planned: Dict[int, int]) -> None:
        self._note_need(self.manager.pages_needed(req.rid, n), planned)

    def _largest_portion(self, req: Request, want: int, planned: Dict[int, int]) -> Tuple[int, Dict[int, int]]:
        """Largest n <= want whose pages are free now (0 if not even one token fits), and its pages."""
        need = self._need_if_fits(req, want, planned)
        if need is not None:
            return want, need
        lo, hi, lo_need = 0, want, {}            # fits(lo) holds, fits(hi) fails
        while hi - lo > 1:
            mid = (lo + hi) // 2
            need = self._need_if_fits(req, mid, planned)
            if need is not None:
                lo, lo_need = mid, need
            else:
                hi = mid
        return lo, lo_need

    def _preempt(self, victim: Request) -> None:
        self.manager.free_request(victim.rid)
        victim.num_computed = 0
        victim.preemptions += 1
        self.running.remove(victim)
        self.waiting.appendleft(victim)
        self.stats["preemptions"] += 1

    def _finish(self, req: Request, reason: FinishReason) -> None:
        req.finished = reason
        if req in self.running:
            self.running.remove(req)
            if not self._keep(req):
                self.manager.free_request(req.rid)

    def plan(self) -> Plan:
        fast = self._plan_steady_decode()
        if fast is not None:
            self.stats["steps"] += 1
            return fast
        preempted: List[Request] = []
        finished: List[Request] = []
        for req in [r for r in self.running if r.cancelled]:
            self._finish(req, FinishReason.CANCELLED)
            finished.append(req)

        while True:
            entries, stuck = self._plan_running()
            if stuck is None:
                break
            # ``stuck`` cannot get a page.  Give back the newest running request's pages.
            victim = self.running[-1]
            if len(self.running) == 1:
                self._finish(victim, FinishReason.CONTEXT_FULL)
                finished.append(victim)
            else:
                self._preempt(victim)
                preempted.append(victim)

        budget = self.max_batch_tokens - sum(e.count for e in entries)
        planned: Dict[int, int] = {}
        for e in entries:
            self._note(e.request, e.count, planned)
        while (self.waiting and budget > 0 and len(entries) < self.max_batch_reqs
               and (self.manager.has_free_slot() or self._drop_kept()) and not preempted):
            req = self.waiting[0]
            if req.finished is not None:                  # ended while it waited (after a preemption)
                self.waiting.popleft()
                continue
            if req.cancelled:
                self.waiting.popleft()
                req.finished = FinishReason.CANCELLED
                finished.append(req)
                continue
            if not (self.kept and self._start_from_kept(req)):
                self.manager.add_request(req.rid)
            want = min(req.num_tokens - req.num_computed, budget)
            if not self._pages_fit(req, want, planned):
                self.manager.free_request(req.rid)
                req.num_computed = 0
                if not self.running:
                    # nothing else holds pages, so this request can never start
                    self.waiting.popleft()
                    req.finished = FinishReason.CONTEXT_FULL
                    finished.append(req)
                    continue
                break
            self.waiting.popleft()
            self.running.append(req)
            self.stats["admitted"] += 1
            entries.append(PlannedEntry(req, req.num_computed, want, req.num_computed + want == req.num_tokens))
            self._note(req, want, planned)
            budget -= want
        self.stats["steps"] += 1
        return Plan(entries, preempted, finished)

    def _plan_steady_decode(self) -> Optional[Plan]:
        """The common step while generating: nobody waits, nobody is cancelled, every running request
        brings one token, and even if each needed a new page in every group the pages are there.
        The general planner would decide the same; this only skips its bookkeeping."""
        running = self.running
        n = len(running)
        if self.waiting or n == 0 or n > self.max_batch_reqs or n > self.max_batch_tokens:
            return None
        for g in self.manager.paged:
            if g.allocator.num_free < n:
                return None
        entries = []
        for req in running:
            if req.ending:
                continue
            if req.cancelled or req.num_computed < len(req.prompt) or req.num_tokens - req.num_computed != 1:
                return None
            entries.append(PlannedEntry(req, req.num_computed, 1, True))
        return Plan(entries, [], [])

    def _plan_running(self) -> Tuple[List[PlannedEntry], Optional[Request]]:
        """Portions for the running requests, in admission order.  Returns the
        entries and, if the step cannot go on as it is, the request that is stuck:
        a decoding request without a page, or, when nothing at all could be planned,
        the first request that is waiting for pages."""
        budget = self.max_batch_tokens
        entries: List[PlannedEntry] = []
        planned: Dict[int, int] = {}
        starved: Optional[Request] = None
        for req in self.running:
            if budget <= 0 or len(entries) >= self.max_batch_reqs:
                break
            if req.ending:
                continue
            want = min(req.num_tokens - req.num_computed, budget)
            n, need = self._largest_portion(req, want, planned)
            if n == 0:
                if req.decoding:
                    return entries, req
                starved = starved or req
                continue
            entries.append(PlannedEntry(req, req.num_computed, n, req.num_computed + n == req.num_tokens))
            self._note_need(need, planned)
            budget -= n
        if not entries and starved is not None:
            return entries, starved
        return entries, None

    # ------------------------------------------------------------ after the step
    def advance(self, plan: Plan) -> None:
        """The step ran: the planned tokens are in the cache."""
        for e in plan.entries:
            e.request.num_computed += e.count

    def accept(self, req: Request, token: int) -> Optional[FinishReason]:
        """Takes the token sampled for ``req``; returns the finish reason if it ends."""
        if req.cancelled:
            reason = FinishReason.CANCELLED
        elif token in req.eog_tokens:
            reason = FinishReason.END_OF_GENERATION     # the end token is not emitted
        else:
            req.output.append(int(token))
            if len(req.output) >= req.max_new_tokens:
                reason = FinishReason.MAX_TOKENS
            elif req.num_tokens >= self.max_context:
                reason = FinishReason.CONTEXT_FULL
            else:
                return None
        self._finish(req, reason)
        return reason
