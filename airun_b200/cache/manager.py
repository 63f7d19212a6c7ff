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

All bookkeeping is host-side and needs no GPU; it is done by the native core
(``csrc/host_core.cpp``, compiled with the C++ compiler at first use), of which the
classes here are thin views that map request ids to slots and status codes to
exceptions.  ``CacheStorage`` owns the device tensors.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int32, c_longlong, c_void_p

import numpy as np
import torch

from ..csrc import build

from ..parts.base import PagedKVSpec, StateSpec


class OutOfPages(RuntimeError):
    """Not enough free pages; nothing was taken."""


class CacheError(RuntimeError):
    """Misuse of the manager (unknown request, double free, ...)."""


class OutOfSlots(CacheError):
    """Every request slot is in use; nothing was taken.  A shortage like OutOfPages, not a misuse."""


_LIB = None


def _lib():
    """The native host core, loaded (and compiled) once."""
    global _LIB
    if _LIB is not None:
        return _LIB
    lib = build.load("host_core")
    P, I, L = c_void_p, c_int, c_longlong
    IP, LP = POINTER(c_int), POINTER(c_longlong)
    sigs = {
        "airun_pool_create": (P, [I]), "airun_pool_destroy": (None, [P]), "airun_pool_error": (c_char_p, [P]),
        "airun_pool_num_pages": (I, [P]), "airun_pool_num_free": (I, [P]), "airun_pool_take": (I, [P, I, IP]),
        "airun_pool_share": (I, [P, I]), "airun_pool_give_back": (I, [P, I]), "airun_pool_holders": (I, [P, I]),
        "airun_pool_free_list": (I, [P, IP, I]),
        "airun_cache_create": (P, [I, IP, I, I, I, I, I]), "airun_cache_destroy": (None, [P]),
        "airun_cache_error": (c_char_p, [P]), "airun_cache_pool": (P, [P, I]),
        "airun_cache_table": (POINTER(c_int32), [P, I]), "airun_cache_has_free_slot": (I, [P]),
        "airun_cache_num_live": (I, [P]), "airun_cache_add": (I, [P]), "airun_cache_free": (I, [P, I]),
        "airun_cache_num_tokens": (L, [P, I]), "airun_cache_reserved": (L, [P, I]),
        "airun_cache_num_blocks": (I, [P, I, I]), "airun_cache_blocks": (I, [P, I, I, IP, I]),
        "airun_cache_pages_needed": (I, [P, I, L, IP]), "airun_cache_reserve_many": (I, [P, I, IP, LP]),
        "airun_cache_commit_many": (I, [P, I, IP, LP]), "airun_cache_fork": (I, [P, I, IP, IP, IP]),
        "airun_cache_truncate": (I, [P, I, L, IP, IP]), "airun_cache_check": (I, [P]),
        "airun_cache_build_batch": (I, [P, I, IP, IP, c_void_p, IP, IP, c_void_p, LP, I, I, I, I, LP]),
    }
    for name, (res, args) in sigs.items():
        f = getattr(lib, name)
        f.restype, f.argtypes = res, args
    _LIB = lib
    return lib


def _raise(status: int, text: bytes, who: str = "") -> None:
    msg = (who + ": " if who else "") + text.decode()
    raise (OutOfPages if status == 1 else CacheError)(msg)


def _ints(values) -> ctypes.Array:
    return (c_int * len(values))(*values)


def _longs(values) -> ctypes.Array:
    return (c_longlong * len(values))(*values)


class PageAllocator:
    """Free list of page ids with a holder count per page (a view of the native pool: its own,
    or the pool of a cache group)."""

    def __init__(self, num_pages: int, _borrowed: Optional[int] = None):
        self._lib = _lib()
        self._own = _borrowed is None
        if self._own:
            if num_pages <= 0:
                raise ValueError("a page pool needs at least one page")
            self._h = self._lib.airun_pool_create(int(num_pages))
        else:
            self._h = _borrowed
        self.num_pages = int(num_pages)

    def __del__(self):
        if getattr(self, "_own", False) and self._h:
            self._lib.airun_pool_destroy(self._h)
            self._h = None

    def _check(self, status: int) -> None:
        if status:
            _raise(status, self._lib.airun_pool_error(self._h))

    @property
    def num_free(self) -> int:
        return self._lib.airun_pool_num_free(self._h)

    def take(self, n: int) -> List[int]:
        out = (c_int * max(n, 1))()
        self._check(self._lib.airun_pool_take(self._h, int(n), out))
        return list(out[:n])

    def share(self, page: int) -> None:
        self._check(self._lib.airun_pool_share(self._h, int(page)))

    def give_back(self, page: int) -> None:
        self._check(self._lib.airun_pool_give_back(self._h, int(page)))

    def holders(self, page: int) -> int:
        return self._lib.airun_pool_holders(self._h, int(page))

    def free_list(self) -> List[int]:
        """The free pages, the next one to be handed out last."""
        out = (c_int * self.num_pages)()
        n = self._lib.airun_pool_free_list(self._h, out, self.num_pages)
        return list(out[:n])


@dataclass
class PagedGroup:
    gid: int
    spec: PagedKVSpec
    owners: List[int]                 # entries of the execution order that own a cache in this group
    page_size: int
    allocator: Optional[PageAllocator] = None

    @property
    def window(self) -> int:
        return self.spec.window


@dataclass
class StateGroup:
    gid: int
    spec: StateSpec
    owners: List[int]


class RequestCache:
    """A live request as the manager sees it: its slot, and views of its counters and pages."""

    __slots__ = ("rid", "slot", "_m")

    def __init__(self, rid: Hashable, slot: int, manager: "CacheManager"):
        self.rid, self.slot, self._m = rid, slot, manager

    @property
    def num_tokens(self) -> int:                   # tokens whose cache content is final
        return self._m._lib.airun_cache_num_tokens(self._m._h, self.slot)

    @property
    def reserved(self) -> int:                     # tokens pages are held for (>= num_tokens)
        return self._m._lib.airun_cache_reserved(self._m._h, self.slot)

    @property
    def blocks(self) -> Dict[int, List[int]]:      # gid -> page id per block, -1 = given back
        return {g.gid: self._m._blocks(self.slot, g.gid) for g in self._m.paged}


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
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
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
                    g = PagedGroup(len(self.paged), spec, [], page_size)
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
        self.max_blocks = int(max_blocks) if max_blocks else num_pages
        self._lib = _lib()
        n = len(self.paged)
        self._h = self._lib.airun_cache_create(n, _ints([g.window for g in self.paged] or [0]), page_size, num_pages,
                                               max_requests, self.max_blocks, 1 if self.state else 0)
        if not self._h:
            raise ValueError("the cache core refuses these sizes")
        for g in self.paged:
            g.allocator = PageAllocator(num_pages, _borrowed=self._lib.airun_cache_pool(self._h, g.gid))
        # The core's mirror of every request's block table, one row per request slot: a step
        # copies the rows of its batch from here.
        self.tables = [np.ctypeslib.as_array(self._lib.airun_cache_table(self._h, g.gid),
                                             shape=(max_requests, self.max_blocks)) for g in self.paged]
        self.requests: Dict[Hashable, RequestCache] = {}
        self._need = (c_int * max(n, 1))()
        self._copies = (c_int * (3 * max(n, 1)))()

    def __del__(self):
        if getattr(self, "_h", None):
            self.tables = []
            self._lib.airun_cache_destroy(self._h)
            self._h = None

    def _check(self, status: int, rid: Hashable = None) -> None:
        if status:
            _raise(status, self._lib.airun_cache_error(self._h), f"request {rid!r}" if rid is not None else "")

    # ------------------------------------------------------------ requests
    def add_request(self, rid: Hashable) -> RequestCache:
        if rid in self.requests:
            raise CacheError(f"request {rid!r} is already live")
        slot = self._lib.airun_cache_add(self._h)
        if slot < 0:
            raise OutOfSlots(f"all {self.max_requests} request slots are in use")
        rc = RequestCache(rid, slot, self)
        self.requests[rid] = rc
        return rc

    def has_free_slot(self) -> bool:
        return bool(self._lib.airun_cache_has_free_slot(self._h))

    def get(self, rid: Hashable) -> RequestCache:
        try:
            return self.requests[rid]
        except KeyError:
            raise CacheError(f"request {rid!r} is not live") from None

    def pages_needed(self, rid: Hashable, n_new: int) -> Dict[int, int]:
        """Pages each paged group would have to hand out to hold ``n_new`` more tokens."""
        self._check(self._lib.airun_cache_pages_needed(self._h, self.get(rid).slot, int(n_new), self._need), rid)
        return {g.gid: self._need[g.gid] for g in self.paged}

    def can_reserve(self, rid: Hashable, n_new: int, already: Optional[Dict[int, int]] = None) -> bool:
        need = self.pages_needed(rid, n_new)
        return all(need[g.gid] + (already or {}).get(g.gid, 0) <= g.allocator.num_free for g in self.paged)

    def reserve(self, rid: Hashable, n_new: int, need: Optional[Dict[int, int]] = None) -> None:
        """Takes the pages for the next ``n_new`` tokens in every group, or none at all."""
        self.reserve_many([rid], [n_new])

    def reserve_many(self, rids: Sequence[Hashable], n_new: Sequence[int]) -> None:
        """Takes the pages for the next tokens of all listed requests, or of none."""
        slots = [self.get(r).slot for r in rids]
        self._check(self._lib.airun_cache_reserve_many(self._h, len(slots), _ints(slots), _longs(list(n_new))),
                    rids[0] if len(rids) == 1 else None)

    def commit(self, rid: Hashable, n_new: int) -> None:
        """The step wrote ``n_new`` tokens; pages a window has passed are given back."""
        self.commit_many([rid], [n_new])

    def commit_many(self, rids: Sequence[Hashable], n_new: Sequence[int]) -> None:
        slots = [self.get(r).slot for r in rids]
        self._check(self._lib.airun_cache_commit_many(self._h, len(slots), _ints(slots), _longs(list(n_new))),
                    rids[0] if len(rids) == 1 else None)

    def free_request(self, rid: Hashable) -> None:
        rc = self.requests.pop(rid, None)
        if rc is None:
            raise CacheError(f"request {rid!r} is freed twice or was never added")
        self._check(self._lib.airun_cache_free(self._h, rc.slot), rid)

    def rename(self, old: Hashable, new: Hashable) -> None:
        """The live request ``old`` is known as ``new`` from now on (its slot, tokens and pages stay):
        how a finished request's cache is kept under a name no later request can collide with."""
        if new in self.requests:
            raise CacheError(f"request {new!r} is already live")
        rc = self.get(old)
        del self.requests[old]
        rc.rid = new
        self.requests[new] = rc

    @property
    def can_rewind(self) -> bool:
        """Whether ``truncate`` can move any request back: no fixed-size state and no window whose
        pages are given back behind it."""
        return not self.state and all(g.window == 0 for g in self.paged)

    # ------------------------------------------------------------ sharing and rewinding
    def _plan(self, n: int, state: Optional[Tuple[int, int]] = None) -> CopyPlan:
        c = self._copies
        return CopyPlan([(c[3 * i], c[3 * i + 1], c[3 * i + 2]) for i in range(n)], state)

    def fork(self, parent: Hashable, child: Hashable) -> CopyPlan:
        """Makes ``child`` a live request holding the same ``num_tokens`` tokens as ``parent``.
        Whole pages are shared (one more holder); a last page that is only partly filled is the
        place both would write next, so the child gets a fresh one.  Returns the copies the caller
        has to run on the device before the child's first step: pages ``(gid, src, dst)`` and the
        state slot.  Takes everything or, if pages or slots are short, nothing."""
        prc = self.get(parent)
        if child in self.requests:
            raise CacheError(f"request {child!r} is already live")
        if not self.has_free_slot():
            raise OutOfSlots(f"all {self.max_requests} request slots are in use")
        slot, n = c_int(-1), c_int(0)
        self._check(self._lib.airun_cache_fork(self._h, prc.slot, ctypes.byref(slot), self._copies, ctypes.byref(n)),
                    parent)
        self.requests[child] = RequestCache(child, slot.value, self)
        return self._plan(n.value, (prc.slot, slot.value) if self.state else None)

    def truncate(self, rid: Hashable, n_tokens: int) -> CopyPlan:
        """Moves the end of ``rid`` back to ``n_tokens``: pages wholly past it are given back, and
        if the page that is written next has other holders the request gets a copy of its own
        (returned for the caller to run on the device).  Fixed-size state cannot be moved back, and
        neither can a window whose pages are gone."""
        n = c_int(0)
        self._check(self._lib.airun_cache_truncate(self._h, self.get(rid).slot, int(n_tokens), self._copies,
                                                   ctypes.byref(n)), rid)
        return self._plan(n.value)

    # ------------------------------------------------------------ the batch of a step
    def build_batch(self, rids: Sequence[Hashable], qlens: Sequence[int], tokens: np.ndarray,
                    want_counts: Sequence[int], want: Sequence[int], base_ptr: int, offsets: ctypes.Array,
                    max_reqs: int, bt_cols: int, pad_to: int, pad_want: int) -> tuple:
        """Lays the batch of a step into the staging buffer at ``base_ptr`` (see csrc/host_core.cpp).
        Returns (tokens, wanted rows, longest context, longest portion, slots, shared prefix per group)."""
        slots = [self.requests[r].slot for r in rids]
        out = (c_longlong * (4 + max(len(self.paged), 1)))()
        self._check(self._lib.airun_cache_build_batch(
            self._h, len(slots), _ints(slots), _ints(list(qlens)), tokens.ctypes.data, _ints(list(want_counts) or [0]),
            _ints(list(want) or [0]), base_ptr, offsets, max_reqs, bt_cols, pad_to, pad_want, out))
        return out[0], out[1], out[2], out[3], slots, [out[4 + g.gid] for g in self.paged]

    # ------------------------------------------------------------ views
    def _blocks(self, slot: int, gid: int) -> List[int]:
        n = self._lib.airun_cache_num_blocks(self._h, slot, gid)
        out = (c_int * max(n, 1))()
        self._lib.airun_cache_blocks(self._h, slot, gid, out, n)
        return list(out[:n])

    def block_table(self, rid: Hashable, gid: int) -> List[int]:
        return self._blocks(self.get(rid).slot, gid)

    def free_pages(self) -> Dict[int, int]:
        return {g.gid: g.allocator.num_free for g in self.paged}

    def max_tokens_possible(self) -> int:
        """Tokens one request alone could hold in the smallest pool."""
        return self.num_pages * self.page_size

    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held; every page is in exactly
        ``holders`` block tables; the page a request writes next has no other holder; no request
        slot lost or held twice."""
        self._check(self._lib.airun_cache_check(self._h))
        if len(self.requests) != self._lib.airun_cache_num_live(self._h) or \
                len({rc.slot for rc in self.requests.values()}) != len(self.requests):
            raise CacheError("the request ids and the core's slots do not match")


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
        """Runs the copies of a fork or cut-back on the current stream, in the order of the plan: the
        pages of a cache group go in one kernel launch (all owner layers at once) as long as no copy
        reads or overwrites a page an earlier copy of the same launch writes (a copy of a copy: the
        partly filled page a fork copied, cut back again); such a copy starts the next launch."""
        batches: List[Tuple[int, List[Tuple[int, int]]]] = []
        for gid, src, dst in plan.pages:
            if batches and batches[-1][0] == gid:
                written = {d for _, d in batches[-1][1]}
                read = {s_ for s_, _ in batches[-1][1]}
                if src not in written and dst not in written and dst not in read:
                    batches[-1][1].append((src, dst))
                    continue
            batches.append((gid, [(src, dst)]))
        for gid, pairs in batches:
            pool = self.paged[gid]
            if pool.is_cuda:
                from ..kernels import ops
                ops.copy_pages(pool, torch.tensor(pairs, dtype=torch.int32).to(pool.device, non_blocking=True))
            else:
                for src, dst in pairs:
                    pool[:, dst].copy_(pool[:, src])
        if plan.state is not None:
            for t in self.state:
                t[:, plan.state[1]].copy_(t[:, plan.state[0]])

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.paged + self.state)
