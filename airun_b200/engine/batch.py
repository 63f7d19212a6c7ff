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
