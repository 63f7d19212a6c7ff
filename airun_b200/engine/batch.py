"""What one step hands to the model: the flat batch of tokens with their
request, position and cache addresses, plus scratch memory.

A batch is a flat list of T rows; the rows of one request are contiguous and in
position order.  Any mix of prompt portions and single decoded tokens is just a
list of (request, tokens) entries.  The reference's passes are either n tokens
of one sequence or one token for each of n slots
(crates/airun-core/src/runtime.rs:2046-2100, :3050-3147); here both are the
same thing.
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


class Workspace:
    """Bump allocator over device memory, rewound at the start of each use.

    The same sequence of requests returns the same addresses, which CUDA graph
    replay relies on.  Memory is obtained in chunks and never returned."""

    ALIGN = 256

    def __init__(self, device, chunk_bytes: int = 64 << 20):
        self.device, self.chunk_bytes = device, chunk_bytes
        self.chunks: List[torch.Tensor] = []
        self.ci, self.off = 0, 0

    def reset(self) -> None:
        self.ci, self.off = 0, 0

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = max(n * esz, 1)
        need = (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        while True:
            if self.ci >= len(self.chunks):
                self.chunks.append(torch.empty(max(self.chunk_bytes, need), dtype=torch.uint8, device=self.device))
            c = self.chunks[self.ci]
            if self.off + need <= c.numel():
                t = c[self.off:self.off + n * esz].view(dtype).view(*shape)
                self.off += need
                return t
            self.ci += 1
            self.off = 0

    def bytes(self) -> int:
        return sum(c.numel() for c in self.chunks)


class WeightStream:
    """The weight matrices of one pass over the model, in the order the pass reads them, and how far ahead
    of the product now running the L2 cache has been asked for them.

    A decode step is bound by streaming the weights from memory, and at every boundary between two kernels
    the stream would pause: the kernel in front has issued its last loads, the next one has not started.
    Kernels therefore ask the L2 cache for the first megabytes of the weights that come NEXT (a kernel
    parameter: pointer and bytes; csrc/common.cuh ``l2_prefetch_slice``).  This class hands those ranges
    out on the host while the step's kernels are launched (or captured into a graph: the ranges are the same
    for every replay): ``consume(w)`` when a product over ``w`` is launched, ``claim(n)`` for the next ``n``
    bytes nobody has asked for yet, never more than ``max_ahead`` bytes beyond the product now running (what
    the cache can hold beside the step's other traffic).  After the last matrix the first one follows: the
    next step's.  The reference keeps its weights streaming the same way across kernels of a decode step by
    launching the next kernel early (its graphs; crates/airun-core/src/runtime.rs:2285-2311); it has no L2
    prefetch."""

    def __init__(self, tensors: List[torch.Tensor], max_ahead: int = 48 << 20):
        self.ptrs = [t.data_ptr() for t in tensors]
        self.sizes = [t.numel() * t.element_size() for t in tensors]
        self.starts = [0]
        for n in self.sizes:
            self.starts.append(self.starts[-1] + n)
        self.total = self.starts[-1]
        self.where: Dict[int, List[int]] = {}
        for i, ptr in enumerate(self.ptrs):
            self.where.setdefault(ptr, []).append(i)
        self.max_ahead = int(max_ahead)
        # positions in the endless stream matrix 0, 1, ..., last, 0, 1, ...: bytes from the start of this pass
        self.front = 0                    # first byte nobody has asked for
        self.reset()

    def reset(self) -> None:
        """A new pass begins.  What the pass before asked for beyond its own end are this pass's first bytes."""
        self.front = self.front - self.total if self.front > self.total > 0 else 0
        self.cur_start = -1               # where the matrix of the product now running starts
        self.cur_end = 0                  # and ends

    def consume(self, w: torch.Tensor) -> None:
        """A product over ``w`` is being launched (matrices unknown to the stream are ignored)."""
        places = self.where.get(w.data_ptr())
        if not places:
            return
        starts = [self.starts[i] for i in places] + [self.total + self.starts[places[0]]]
        start = next(s for s in starts if s > self.cur_start)
        i = places[starts.index(start) % len(places)]
        self.cur_start, self.cur_end = start, start + self.sizes[i]
        self.front = max(self.front, self.cur_end)

    def claim(self, nbytes: int):
        """(address, bytes) of the next range to ask for, or (0, 0): at most ``nbytes``, inside one matrix,
        a multiple of 256 bytes, and within ``max_ahead`` of the end of the matrix now being read."""
        if self.total <= 0:
            return 0, 0
        for _ in range(2):
            room = self.max_ahead - (self.front - self.cur_end)
            rem = self.front % self.total
            i = bisect.bisect_right(self.starts, rem) - 1
            off = rem - self.starts[i]
            left = self.sizes[i] - off
            take = min(int(nbytes), left, room) // 256 * 256
            if take > 0:
                self.front += take
                return self.ptrs[i] + off, take
            if left >= 256 or room < 256:
                return 0, 0
            self.front += left            # a ragged end of less than 256 bytes: on to the next matrix
        return 0, 0


@dataclass
class CacheView:
    """The cache of one entry of the execution order, as its mixer sees it."""
    kind: str                                   # "paged" | "state" | "none"
    shared: bool = False                        # reads another entry's cache, writes nothing
    pool: Optional[torch.Tensor] = None         # [pages, 2, kv_heads, page_size, head_dim]
    block_table: Optional[torch.Tensor] = None  # int32 [R, max_blocks]
    page_size: int = 0
    state: Optional[torch.Tensor] = None        # [max_requests, *shape]
    gid: int = -1
    shared_prefix: Optional[torch.Tensor] = None   # int32 [1] on the device: tokens at the start of every request of
                                                   # the batch that lie in the very same pages (0: none, or not known)


@dataclass
class StepContext:
    num_tokens: int
    num_reqs: int
    token_ids: torch.Tensor          # int32 [T]
    positions: torch.Tensor          # int32 [T]
    req_of_token: torch.Tensor       # int32 [T], row of the block tables
    cu_tokens: torch.Tensor          # int32 [R + 1], first row of each request
    context_lens: torch.Tensor       # int32 [R], tokens in the cache after this step
    state_slots: torch.Tensor        # int32 [R]
    err: torch.Tensor                # int32 [1], device-side error bits
    ws: Workspace = None
    ws_pair: tuple = ()
    ws_main: Workspace = None
    caches: List[CacheView] = field(default_factory=list)
    # host-side copies for planning launches
    query_lens: List[int] = field(default_factory=list)
    context_lens_host: List[int] = field(default_factory=list)
    state_slots_host: List[int] = field(default_factory=list)
    max_query_len: int = 0
    max_context_len: int = 0
    decode_only: bool = False
    extras: Dict[str, object] = field(default_factory=dict)
    weights: Optional[WeightStream] = None     # set by the model for steps of few tokens (see WeightStream)

    def prefetch(self, nbytes: int):
        """(address, bytes) of weights a kernel launched now should ask into L2, or (0, 0)."""
        return self.weights.claim(nbytes) if self.weights is not None else (0, 0)
