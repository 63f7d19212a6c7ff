"""The cache manager: pages of keys and values with a block table per request,
and slots for per-request state of fixed size.

The reference gives every conversation slot one contiguous full-context cache
per layer (crates/airun-core/src/runtime.rs:1033-1037, :2865-2871) and reaches
the rows of a batch through a device table of pointers rewritten before each
step (runtime.rs:3152-3173); its fixed-size per-slot state is the delta-net
layers' ``LayerState`` (runtime.rs:26-41).  Here the same two needs are met
with pages:

* The cache owners of the execution order are put into *groups*: owners whose
  cache spec is equal (same KV heads, head size and window) share one page
  pool and one block table per request, so a page id is valid in every layer of
  its group.  One layer's pages are ``[num_pages, 2 (K,V), kv_heads, page_size,
  head_dim]``.
* A request's block table in a group is the list of its page ids by block
  (position // page_size).  Pages are taken from a LIFO free list before a step
  runs the tokens that need them, and given back when the request ends or, in a
  group with a window, when every key of the page lies behind the window of all
  tokens still to come; a freed page is the next one handed out.
* Pages may be shared: ``fork`` gives a child request the parent's pages with one more holder
  each, and ``truncate`` moves a request's end back.  A page that more than one table holds is
  never written: the page a request writes next is its own, which ``fork`` and ``truncate`` see
  to by handing out a fresh page and telling the caller which page to copy into it.  (The
  reference rewinds a slot by moving its cursor, crates/airun-core/src/runtime.rs:3280-3308, and
  reuses the common prefix of a slot's history, runtime.rs:3256-3273; with pages the same prefix
  can serve several live requests at once.)
* State groups hold ``[max_requests, *shape]`` per owner; a request gets a slot
  at admission (the caller zero-fills it) and returns it at the end.

All bookkeeping is host-side and needs no GPU; ``CacheStorage`` owns the
device tensors.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import PagedKVSpec, StateSpec


class OutOfPages(RuntimeError):
    """Not enough free pages; nothing was taken."""


class CacheError(RuntimeError):
    """Misuse of the manager (unknown request, double free, ...)."""


class PageAllocator:
    """Free list of page ids with a holder count per page."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() hands out page 0 first
        self._holders = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._holders[p] != 0:
                raise CacheError(f"page {p} was on the free list while held")
            self._holders[p] = 1
        return out

    def share(self, page: int) -> None:
        if self._holders[page] <= 0:
            raise CacheError(f"page {page} is not held and cannot be shared")
        self._holders[page] += 1

    def give_back(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise CacheError(f"page {page} is outside the pool")
        if self._holders[page] <= 0:
            raise CacheError(f"page {page} is freed twice")
        self._holders[page] -= 1
        if self._holders[page] == 0:
            self._free.append(page)

    def holders(self, page: int) -> int:
        return self._holders[page]


@dataclass
class PagedGroup:
    gid: int
    spec: PagedKVSpec
    owners: List[int]                 # entries of the execution order that own a cache in this group
    page_size: int
    allocator: PageAllocator

    @property
    def window(self) -> int:
        return self.spec.window


@dataclass
class StateGroup:
    gid: int
    spec: StateSpec
    owners: List[int]


@dataclass
class RequestCache:
    rid: Hashable
    slot: int
    num_tokens: int = 0                                  # tokens whose cache content is final
    reserved: int = 0                                    # tokens pages are held for (>= num_tokens)
    blocks: Dict[int, List[int]] = field(default_factory=dict)   # gid -> page id per block, -1 = given back


@dataclass
class CopyPlan:
    """Device copies that make a fork or a cut-back true: whole pages ``(gid, src, dst)`` in every
    layer of their group, and the state of request slot ``state[0]`` into slot ``state[1]``."""
    pages: List[Tuple[int, int, int]] = field(default_factory=list)
    state: Optional[Tuple[int, int]] = None


@dataclass(frozen=True)
class CacheBinding:
    """Where one entry of the execution order finds its cache."""
    kind: str            # "paged" | "state" | "none"
    gid: int
    index: int           # row of the group's tensor
    shared: bool         # True: reads another entry's cache and writes nothing


class CacheManager:
    def __init__(self, specs: Sequence[object], cache_from: Sequence[Optional[int]],
                 page_size: int, num_pages: int, max_requests: int, max_blocks: Optional[int] = None):
        """``specs[i]`` is the cache spec of entry i of the execution order (or None),
        ``cache_from[i]`` the entry whose cache entry i reads instead of its own."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.paged: List[PagedGroup] = []
        self.state: List[StateGroup] = []
        self.bindings: List[CacheBinding] = []
        for i, (spec, src) in enumerate(zip(specs, cache_from)):
            if src is not None:
                if not (0 <= src < i) or cache_from[src] is not None:
                    raise ValueError(f"entry {i} reads the cache of entry {src}, which must be an earlier owner")
                if specs[src] != spec:
                    raise ValueError(f"entry {i} cannot read the cache of entry {src}: their cache specs differ")
                b = self.bindings[src]
                self.bindings.append(CacheBinding(b.kind, b.gid, b.index, True))
            elif spec is None:
                self.bindings.append(CacheBinding("none", -1, -1, False))
            elif isinstance(spec, PagedKVSpec):
                g = next((g for g in self.paged if g.spec == spec), None)
                if g is None:
                    g = PagedGroup(len(self.paged), spec, [], page_size, PageAllocator(num_pages))
                    self.paged.append(g)
                g.owners.append(i)
                self.bindings.append(CacheBinding("paged", g.gid, len(g.owners) - 1, False))
            elif isinstance(spec, StateSpec):
                g = next((g for g in self.state if g.spec == spec), None)
                if g is None:
                    g = StateGroup(len(self.state), spec, [])
                    self.state.append(g)
                g.owners.append(i)
                self.bindings.append(CacheBinding("state", g.gid, len(g.owners) - 1, False))
            else:
                raise TypeError(f"entry {i} has an unknown cache spec {spec!r}")
        self.requests: Dict[Hashable, RequestCache] = {}
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        # Host mirror of every request's block table, one row per request slot, so that a step
        # gathers the rows of its batch with one array operation instead of a loop over requests.
        self.max_blocks = int(max_blocks) if max_blocks else num_pages
        self.tables = [np.full((max_requests, self.max_blocks), -1, dtype=np.int32) for _ in self.paged]

    # ------------------------------------------------------------ requests
    def add_request(self, rid: Hashable) -> RequestCache:
        if rid in self.requests:
            raise CacheError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are in use")
        rc = RequestCache(rid, self._free_slots.pop(), blocks={g.gid: [] for g in self.paged})
        self.requests[rid] = rc
        return rc

    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def get(self, rid: Hashable) -> RequestCache:
        try:
            return self.requests[rid]
        except KeyError:
            raise CacheError(f"request {rid!r} is not live") from None

    def _blocks_for(self, n_tokens: int) -> int:
        return (n_tokens + self.page_size - 1) // self.page_size

    def pages_needed(self, rid: Hashable, n_new: int) -> Dict[int, int]:
        """Pages each paged group would have to hand out to hold ``n_new`` more tokens."""
        rc = self.get(rid)
        want = self._blocks_for(rc.num_tokens + n_new)
        return {g.gid: max(0, want - len(rc.blocks[g.gid])) for g in self.paged}

    def can_reserve(self, rid: Hashable, n_new: int, already: Optional[Dict[int, int]] = None) -> bool:
        need = self.pages_needed(rid, n_new)
        return all(need[g.gid] + (already or {}).get(g.gid, 0) <= g.allocator.num_free for g in self.paged)

    def reserve(self, rid: Hashable, n_new: int, need: Optional[Dict[int, int]] = None) -> None:
        """Takes the pages for the next ``n_new`` tokens in every group, or none at all.
        ``need`` may carry the result of ``pages_needed(rid, n_new)`` if the caller has it."""
        rc = self.get(rid)
        if need is None:
            need = self.pages_needed(rid, n_new)
        for g in self.paged:
            if need[g.gid] > g.allocator.num_free:
                raise OutOfPages(f"request {rid!r} needs {need[g.gid]} pages in group {g.gid}, "
                                 f"{g.allocator.num_free} free")
        for g in self.paged:
            if need[g.gid]:
                blocks = rc.blocks[g.gid]
                first = len(blocks)
                blocks.extend(g.allocator.take(need[g.gid]))
                if len(blocks) <= self.max_blocks:
                    self.tables[g.gid][rc.slot, first:len(blocks)] = blocks[first:]
        rc.reserved = max(rc.reserved, rc.num_tokens + n_new)

    def commit(self, rid: Hashable, n_new: int) -> None:
        """The step wrote ``n_new`` tokens; pages a window has passed are given back."""
        rc = self.get(rid)
        if rc.num_tokens + n_new > rc.reserved:
            raise CacheError(f"request {rid!r}: {n_new} tokens committed beyond the reserved pages")
        rc.num_tokens += n_new
        for g in self.paged:
            if g.window > 0:
                # the next query sits at position num_tokens and sees keys j > num_tokens - window
                last_dead = rc.num_tokens - g.window
                blocks = rc.blocks[g.gid]
                b = 0
                while b < len(blocks) and (b + 1) * self.page_size - 1 <= last_dead:
                    if blocks[b] >= 0:
                        g.allocator.give_back(blocks[b])
                        blocks[b] = -1
                        if b < self.max_blocks:
                            self.tables[g.gid][rc.slot, b] = -1
                    b += 1

    def free_request(self, rid: Hashable) -> None:
        rc = self.requests.pop(rid, None)
        if rc is None:
            raise CacheError(f"request {rid!r} is freed twice or was never added")
        for g in self.paged:
            for p in rc.blocks[g.gid]:
                if p >= 0:
                    g.allocator.give_back(p)
            self.tables[g.gid][rc.slot, :min(len(rc.blocks[g.gid]), self.max_blocks)] = -1
        self._free_slots.append(rc.slot)

    # ------------------------------------------------------------ sharing and rewinding
    def fork(self, parent: Hashable, child: Hashable) -> "CopyPlan":
        """Makes ``child`` a live request holding the same ``num_tokens`` tokens as ``parent``.
        Whole pages are shared (one more holder); a last page that is only partly filled is the
        place both would write next, so the child gets a fresh one.  Returns the copies the caller
        has to run on the device before the child's first step: pages ``(gid, src, dst)`` and the
        state slot.  Takes everything or, if pages or slots are short, nothing."""
        prc = self.get(parent)
        if child in self.requests:
            raise CacheError(f"request {child!r} is already live")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are in use")
        n = prc.num_tokens
        full, part = divmod(n, self.page_size)
        for g in self.paged:
            if part and prc.blocks[g.gid][full] >= 0 and g.allocator.num_free < 1:
                raise OutOfPages(f"forking {parent!r} needs a page in group {g.gid}, none is free")
        crc = RequestCache(child, self._free_slots.pop(), num_tokens=n, reserved=n,
                           blocks={g.gid: [] for g in self.paged})
        plan = CopyPlan(state=(prc.slot, crc.slot) if self.state else None)
        for g in self.paged:
            src = prc.blocks[g.gid]
            blocks = list(src[:full])
            for p in blocks:
                if p >= 0:
                    g.allocator.share(p)
            if part:
                if src[full] >= 0:
                    new = g.allocator.take(1)[0]
                    plan.pages.append((g.gid, src[full], new))
                    blocks.append(new)
                else:
                    blocks.append(-1)
            crc.blocks[g.gid] = blocks
            self.tables[g.gid][crc.slot, :min(len(blocks), self.max_blocks)] = blocks[:self.max_blocks]
        self.requests[child] = crc
        return plan

    def truncate(self, rid: Hashable, n_tokens: int) -> "CopyPlan":
        """Moves the end of ``rid`` back to ``n_tokens``: pages wholly past it are given back, and
        if the page that is written next has other holders the request gets a copy of its own
        (returned for the caller to run on the device).  Fixed-size state cannot be moved back, and
        neither can a window whose pages are gone."""
        rc = self.get(rid)
        if not (0 <= n_tokens <= rc.num_tokens):
            raise CacheError(f"request {rid!r} holds {rc.num_tokens} tokens and cannot be cut to {n_tokens}")
        if n_tokens == rc.num_tokens and rc.reserved == rc.num_tokens:
            return CopyPlan()
        if self.state and n_tokens < rc.num_tokens:
            raise CacheError("a request with fixed-size state cannot be moved back, only restarted")
        full, part = divmod(n_tokens, self.page_size)
        for g in self.paged:
            blocks = rc.blocks[g.gid]
            if g.window > 0 and n_tokens > 0:
                first_needed = max(0, n_tokens - g.window + 1) // self.page_size
                if first_needed < len(blocks) and blocks[first_needed] < 0:
                    raise CacheError(f"request {rid!r}: the window's pages before token {n_tokens} were given back")
            if part and blocks[full] >= 0 and g.allocator.holders(blocks[full]) > 1 and g.allocator.num_free < 1:
                raise OutOfPages(f"cutting {rid!r} inside a shared page needs a page in group {g.gid}")
        plan = CopyPlan()
        keep = full + (1 if part else 0)
        for g in self.paged:
            blocks = rc.blocks[g.gid]
            for p in blocks[keep:]:
                if p >= 0:
                    g.allocator.give_back(p)
            self.tables[g.gid][rc.slot, keep:min(len(blocks), self.max_blocks)] = -1
            del blocks[keep:]
            if part and blocks[full] >= 0 and g.allocator.holders(blocks[full]) > 1:
                new = g.allocator.take(1)[0]
                plan.pages.append((g.gid, blocks[full], new))
                g.allocator.give_back(blocks[full])
                blocks[full] = new
                if full < self.max_blocks:
                    self.tables[g.gid][rc.slot, full] = new
        rc.num_tokens = rc.reserved = n_tokens
        return plan

    # ------------------------------------------------------------ views
    def block_table(self, rid: Hashable, gid: int) -> List[int]:
        return self.get(rid).blocks[gid]

    def free_pages(self) -> Dict[int, int]:
        return {g.gid: g.allocator.num_free for g in self.paged}

    def max_tokens_possible(self) -> int:
        """Tokens one request alone could hold in the smallest pool."""
        return self.num_pages * self.page_size

    def check_invariants(self) -> None:
        """No page lost, none held twice: every page is either free or in exactly
        ``holders`` block tables."""
        for g in self.paged:
            seen: Dict[int, int] = {}
            for rc in self.requests.values():
                for p in rc.blocks[g.gid]:
                    if p >= 0:
                        seen[p] = seen.get(p, 0) + 1
            free = g.allocator._free
            if len(set(free)) != len(free):
                raise CacheError(f"group {g.gid}: a page is on the free list twice")
            for p in free:
                if p in seen:
                    raise CacheError(f"group {g.gid}: page {p} is both free and held")
            for p, n in seen.items():
                if g.allocator.holders(p) != n:
                    raise CacheError(f"group {g.gid}: page {p} is in {n} tables but has "
                                     f"{g.allocator.holders(p)} holders")
            if len(free) + len(seen) != g.allocator.num_pages:
                raise CacheError(f"group {g.gid}: {g.allocator.num_pages - len(free) - len(seen)} pages are lost")
            for rc in self.requests.values():
                b = rc.num_tokens // self.page_size
                blocks = rc.blocks[g.gid]
                for p in blocks[b:]:
                    if p >= 0 and g.allocator.holders(p) != 1:
                        raise CacheError(f"group {g.gid}: request {rc.rid!r} would write page {p}, which "
                                         f"{g.allocator.holders(p)} tables hold")
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a request slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a request slot is lost")


class CacheStorage:
    """Device tensors behind a :class:`CacheManager`."""

    def __init__(self, manager: CacheManager, dtype: torch.dtype, device):
        self.manager = manager
        self.paged = [torch.zeros((len(g.owners), manager.num_pages, 2, g.spec.num_kv_heads,
                                   manager.page_size, g.spec.head_dim), dtype=dtype, device=device)
                      for g in manager.paged]
        self.state = [torch.zeros((len(g.owners), manager.max_requests) + tuple(g.spec.shape),
                                  dtype=g.spec.dtype, device=device) for g in manager.state]

    def zero_state_slot(self, slot: int) -> None:
        for t in self.state:
            t[:, slot].zero_()

    def run_copies(self, plan: CopyPlan) -> None:
        """Runs the copies of a fork or cut-back on the current stream."""
        for gid, src, dst in plan.pages:
            self.paged[gid][:, dst].copy_(self.paged[gid][:, src])
        if plan.state is not None:
            for t in self.state:
                t[:, plan.state[1]].copy_(t[:, plan.state[0]])

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.paged + self.state)
