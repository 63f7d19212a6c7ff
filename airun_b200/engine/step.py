"""The step function: one batch of (request, its next tokens) through the model.

``StepRunner.step(entries)`` takes a list of ``StepEntry(rid, tokens, want)``:
portions of prompts beside single decoded tokens, cut anywhere.  It takes the
pages the new tokens need, runs only the tokens it is given, as one batch, from
the cache that earlier steps left, writes their keys and values, and returns the
float32 logits at the wanted places, in the order of the entries and of
``want``.  It is policy-free: the scheduler and the trace replay both drive it.

The reference's equivalents are ``Runtime::step`` for n tokens of one sequence
and ``decode_rows`` for one token of each of n slots
(crates/airun-core/src/runtime.rs:2046-2100, :3050-3147); a non-final prompt
chunk returns nothing and does not synchronise (runtime.rs:2032-2037).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, CacheStorage, OutOfPages
from ..kernels import ops
from .batch import CacheView, StepContext, Workspace
from .model import DecoderModel


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among ``tokens`` whose logits are wanted


class StepError(RuntimeError):
    pass


class StepRunner:
    def __init__(self, model: DecoderModel, manager: CacheManager, storage: CacheStorage,
                 max_batch_tokens: int, max_batch_reqs: int, max_context: int):
        self.model, self.manager, self.storage = model, manager, storage
        self.device = model.device
        self.T_max, self.R_max = int(max_batch_tokens), int(max_batch_reqs)
        self.max_context = int(max_context)
        self.max_blocks = (self.max_context + manager.page_size - 1) // manager.page_size
        n_groups = len(manager.paged)
        # one pinned staging buffer, one device mirror, fixed offsets
        sizes = [("token_ids", self.T_max), ("positions", self.T_max), ("req_of_token", self.T_max),
                 ("want_rows", self.T_max), ("cu_tokens", self.R_max + 1), ("context_lens", self.R_max),
                 ("state_slots", self.R_max)]
        sizes += [(f"bt{g}", self.R_max * self.max_blocks) for g in range(n_groups)]
        sizes += [(f"shared{g}", 1) for g in range(n_groups)]      # tokens at the start that all requests share
        self.offsets: Dict[str, tuple] = {}
        off = 0
        for name, n in sizes:
            self.offsets[name] = (off, n)
            off += (n + 63) // 64 * 64
        # a ring of pinned staging buffers: the host may run ahead of the copies of earlier steps
        self._ring = []
        for _ in range(4):
            h = torch.zeros(off, dtype=torch.int32, pin_memory=self.device.type == "cuda")
            self._ring.append((h, h.numpy(), torch.cuda.Event() if self.device.type == "cuda" else None))
        self._ring_i = 0
        self.meta_host, self.meta_np, self._meta_event = self._ring[0]
        self._ring_used = [False] * 4
        self.meta_dev = torch.zeros(off, dtype=torch.int32, device=self.device)
        names = ["token_ids", "positions", "req_of_token", "want_rows", "cu_tokens", "context_lens", "state_slots"]
        names += [f"bt{g}" for g in range(n_groups)] + [f"shared{g}" for g in range(n_groups)]
        self._offs = (ctypes.c_longlong * len(names))(*[self.offsets[n][0] for n in names])
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.ws_main = Workspace(self.device)
        self.ws_pair = (Workspace(self.device), Workspace(self.device))
        self.steps_run = 0
        # CUDA graphs of decode-only steps, one per batch-size bucket
        self.use_graphs = bool(getattr(model, "graph_safe", lambda: True)())
        self.graph_buckets = [b for b in (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256) if b <= self.R_max]
        if self.graph_buckets and self.graph_buckets[-1] < self.R_max and self.R_max <= 512:
            self.graph_buckets.append(self.R_max)
        self.graphs: Dict[object, tuple] = {}
        self._warm_buckets = set()
        self.graph_launches = 0
        # ... and of any other step (prompt portions, several wanted places) of a model whose parts
        # read the batch's layout on the device: one graph per (padded tokens, padded wanted rows)
        self.mixed_graphs = bool(getattr(model, "device_driven", lambda: False)())
        self.max_mixed_graphs = 96
        self.token_buckets = sorted({b for k in range(3, 24) for b in (1 << k, 3 << (k - 1)) if b <= self.T_max}
                                    | {self.T_max})
        self.want_buckets = sorted({4 ** k for k in range(12) if 4 ** k < self.T_max} | {self.T_max})
        self.row_buckets = sorted({8 * 4 ** k for k in range(8) if 8 * 4 ** k < self.R_max} | {self.R_max})
        self.portion_buckets = sorted({4 ** k for k in range(8) if 4 ** k < self.R_max} | {self.R_max})
        self.want_arange = torch.arange(max(self.R_max, 1), dtype=torch.int32, device=self.device)

    def _view(self, name: str, dev: bool = True):
        off, n = self.offsets[name]
        return (self.meta_dev if dev else self.meta_np)[off:off + n]

    def _cache_views(self) -> List[CacheView]:
        views = []
        for b in self.manager.bindings:
            if b.kind == "paged":
                bt = self._view(f"bt{b.gid}").view(self.R_max, self.max_blocks)
                views.append(CacheView("paged", b.shared, self.storage.paged[b.gid][b.index], bt,
                                       self.manager.page_size, gid=b.gid, shared_prefix=self._view(f"shared{b.gid}")))
            elif b.kind == "state":
                views.append(CacheView("state", b.shared, state=self.storage.state[b.gid][b.index], gid=b.gid))
            else:
                views.append(CacheView("none"))
        return views

    def check_entries(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.R_max:
            raise StepError(f"{len(entries)} requests in one step, the runner was made for {self.R_max}")
        total = sum(len(e.tokens) for e in entries)
        if total > self.T_max:
            raise StepError(f"{total} tokens in one step, the runner was made for {self.T_max}")
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.rid!r} brings no tokens")
            rc = self.manager.get(e.rid)
            if rc.num_tokens + len(e.tokens) > self.max_context:
                raise StepError(f"request {e.rid!r} would reach {rc.num_tokens + len(e.tokens)} tokens, "
                                f"the context limit is {self.max_context}")
            for w in e.want:
                if not (0 <= w < len(e.tokens)):
                    raise StepError(f"request {e.rid!r} wants place {w} of {len(e.tokens)} tokens")

    def reserve(self, entries: Sequence[StepEntry]) -> None:
        """Takes the pages of all entries, or of none."""
        self.manager.reserve_many([e.rid for e in entries], [len(e.tokens) for e in entries])
        self._start_requests(entries)

    def _start_requests(self, entries: Sequence[StepEntry]) -> None:
        """A request whose first tokens arrive starts from zero state: its slot of every fixed-size state
        tensor is cleared before the step runs (the slot may have served another request before).  The
        step function owns this rule, so no caller has to know it; a forked request arrives with tokens
        and keeps the copy of its parent's state."""
        if self.storage.state:
            for e in entries:
                rc = self.manager.get(e.rid)
                if rc.num_tokens == 0:
                    self.storage.zero_state_slot(rc.slot)

    def build_context(self, entries: Sequence[StepEntry], pad_to: int = 0, pad_want: int = 0) -> tuple:
        """Fills the staging buffer and returns (StepContext, n_want).  With ``pad_to`` the
        batch is padded with rows that belong to no request (request -1, position -1), which
        every kernel skips, and with requests that bring no tokens; that is how a captured graph
        of a fixed size runs a smaller batch.  ``pad_want`` pads the wanted rows with row 0.
        The arrays are laid out by the native core (csrc/host_core.cpp: build_batch)."""
        m = self.manager
        self._ring_i = (self._ring_i + 1) % len(self._ring)
        self.meta_host, self.meta_np, self._meta_event = self._ring[self._ring_i]
        if self._ring_used[self._ring_i] and self._meta_event is not None:
            self._meta_event.synchronize()      # the copy that last read this buffer is done
        R = len(entries)
        qlens = [len(e.tokens) for e in entries]
        if max(qlens) == 1:
            toks = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=R)
        else:
            toks = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        want = [w for e in entries for w in e.want]
        t, n_want, max_ctx, max_q, slots, shared = m.build_batch(
            [e.rid for e in entries], qlens, toks, [len(e.want) for e in entries], want,
            self.meta_host.data_ptr(), self._offs, self.R_max, self.max_blocks, pad_to, pad_want)
        clens = self._view("context_lens", dev=False)[:R].tolist()
        t = max(t, pad_to)
        self.meta_dev.copy_(self.meta_host, non_blocking=True)
        if self._meta_event is not None:
            self._meta_event.record()
            self._ring_used[self._ring_i] = True
        ctx = StepContext(
            num_tokens=t, num_reqs=self.R_max if pad_to else len(entries),
            token_ids=self._view("token_ids"), positions=self._view("positions"),
            req_of_token=self._view("req_of_token"), cu_tokens=self._view("cu_tokens"),
            context_lens=self._view("context_lens"), state_slots=self._view("state_slots"),
            err=self.err, ws_pair=self.ws_pair, ws_main=self.ws_main, caches=self._cache_views(),
            query_lens=qlens, context_lens_host=clens, state_slots_host=slots,
            max_query_len=max_q, max_context_len=max_ctx,
            decode_only=max_q == 1)
        ctx.extras["shared_prefix_host"] = shared
        return ctx, n_want

    def step(self, entries: Sequence[StepEntry], checked: bool = False) -> Optional[torch.Tensor]:
        """Runs the entries as one batch; returns float32 logits [wanted, vocab] on
        the device (valid until the next step) or None when nothing is wanted.
        ``checked``: the caller (the scheduler) has made the entries itself and vouches for them."""
        if not checked:
            self.check_entries(entries)
        self.reserve(entries)
        if self.use_graphs and self.device.type == "cuda" and all(
                len(e.tokens) == 1 and tuple(e.want) == (0,) for e in entries):
            logits = self._decode_step_graphed(entries)
        elif self.use_graphs and self.mixed_graphs and self.device.type == "cuda":
            logits = self._mixed_step_graphed(entries)
        else:
            ctx, n_want = self.build_context(entries)
            logits = self.model.forward(ctx, self._view("want_rows"), n_want)
        self.manager.commit_many([e.rid for e in entries], [len(e.tokens) for e in entries])
        self.steps_run += 1
        return logits

    # ---- a step in two halves: what does not depend on the newest tokens, and the rest
    def prepare_step(self, entries: Sequence[StepEntry]) -> Optional[dict]:
        """The part of a step that does not need the values of its tokens: pages, the batch's layout,
        its copy to the device, which queues up behind whatever the stream is running.  Tokens not
        known yet may hold any valid id; ``launch_prepared`` brings the real ones and replays the
        step's graph.  None when the step's shape has no captured graph yet (it then goes the ordinary
        way); raises OutOfPages like ``step``."""
        if not self.use_graphs or self.device.type != "cuda":
            return None
        rids, counts = [e.rid for e in entries], [len(e.tokens) for e in entries]
        if all(c == 1 and tuple(e.want) == (0,) for c, e in zip(counts, entries)):
            n = len(entries)
            bucket = next((b for b in self.graph_buckets if b >= n), None)
            if bucket is None or (bucket not in self.graphs and ("shared", bucket) not in self.graphs):
                return None
            self.manager.reserve_many(rids, counts)
            self._start_requests(entries)
            ctx, _ = self.build_context(entries, pad_to=bucket)
            key, n_want = self._decode_key(ctx, bucket), n
        else:
            if not self.mixed_graphs:
                return None
            key, tb, wb, _, _, n_want = self._mixed_key(entries)
            if key not in self.graphs:
                return None
            self.manager.reserve_many(rids, counts)
            self._start_requests(entries)
            self.build_context(entries, pad_to=tb, pad_want=wb)
        if key not in self.graphs:
            return None                 # (the pages are taken and the lay-out is unused: the ordinary path redoes it)
        return dict(rids=rids, counts=counts, key=key, slot=self._ring_i, n_want=n_want)

    def launch_prepared(self, prep: dict, tokens) -> Optional[torch.Tensor]:
        """Second half of ``prepare_step``: all the step's tokens (one flat sequence) go to the device
        and the graph is replayed.  Nothing may have touched the runner or these requests in between."""
        n = len(tokens)
        off, _ = self.offsets["token_ids"]
        host, host_np, event = self._ring[prep["slot"]]
        host_np[off:off + n] = tokens
        self.meta_dev[off:off + n].copy_(host[off:off + n], non_blocking=True)
        if event is not None:
            event.record()
        graph, out, kernels = self.graphs[prep["key"]]
        graph.replay()
        self.graph_launches += kernels
        self.manager.commit_many(prep["rids"], prep["counts"])
        self.steps_run += 1
        return out[:prep["n_want"]] if prep["n_want"] else None

    SHARED_PREFIX_MIN = 1024       # tokens all requests of a decode step must share before it pays to read them once

    def _decode_key(self, ctx, bucket: int):
        """The graph a step of single tokens runs from: the plain one of its batch-size bucket, or,
        when the requests of the batch begin with the same pages (forks of one request), the one
        whose attention reads that shared prefix once for all of them."""
        ctx.extras["planning_context_len"] = self.max_context
        shared = ctx.extras.get("shared_prefix_host") or [0]
        if self.mixed_graphs and max(shared) >= self.SHARED_PREFIX_MIN:
            ctx.extras["use_shared_prefix"] = True
            return ("shared", bucket)
        return bucket

    def _decode_step_graphed(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """A step of single decoded tokens, all of whose logits are wanted, replayed from a
        CUDA graph of the next larger captured batch size.  The reference captures its decode
        step the same way, with token, position and cache addresses read from device buffers
        that outlive the replays (crates/airun-core/src/runtime.rs:2285-2359).  Here the graph
        reads the step's metadata from the runner's fixed device buffer; the number of key
        slices of the attention kernel is fixed at capture for the longest allowed context."""
        n = len(entries)
        bucket = next((b for b in self.graph_buckets if b >= n), None)
        if bucket is None:
            ctx, n_want = self.build_context(entries)
            return self.model.forward(ctx, self._view("want_rows"), n_want)
        ctx, n_want = self.build_context(entries, pad_to=bucket)
        return self._run_graphed(self._decode_key(ctx, bucket), ctx, self.want_arange, bucket)[:n]

    def _run_graphed(self, key, ctx, want_rows: torch.Tensor, n_want: int) -> Optional[torch.Tensor]:
        """Runs the padded batch of ``ctx``: kernel by kernel the first time a step of this shape comes
        (that loads and configures every kernel the graph will hold), captured the second time
        (capturing runs nothing) and replayed from then on."""
        entry = self.graphs.get(key)
        if entry is None:
            if key not in self._warm_buckets:
                self._warm_buckets.add(key)
                return self.model.forward(ctx, want_rows, n_want)
            torch.cuda.current_stream().synchronize()
            before = ops.LAUNCHES[0]
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self.model.forward(ctx, want_rows, n_want)
            entry = (graph, out, ops.LAUNCHES[0] - before)
            ops.LAUNCHES[0] = before
            self.graphs[key] = entry
        graph, out, kernels = entry
        graph.replay()
        self.graph_launches += kernels
        return out

    def _mixed_key(self, entries: Sequence[StepEntry]):
        """(graph key, padded tokens, padded wanted rows, row bucket index, portion bucket, wanted rows)."""
        T = W = singles = portions = 0
        for e in entries:
            n = len(e.tokens)
            T += n
            W += len(e.want)
            if n == 1:
                singles += 1
            else:
                portions += 1
        tb = next((b for b in self.token_buckets if b >= T), None)
        wb = next((b for b in self.want_buckets if b >= W), None) if W else 0
        ri = next((i for i, b in enumerate(self.row_buckets) if b >= singles), None) if singles else -1
        pb = next((b for b in self.portion_buckets if b >= portions), None) if portions else 0
        return ("mixed", tb, wb, ri, pb), tb, wb, ri, pb, W

    def _mixed_step_graphed(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Any other step, replayed from a CUDA graph of the next larger captured shape: tokens,
        wanted rows, single-token requests and requests with a portion, each rounded up to a bucket.
        The batch is padded; which rows are portions and which single tokens, how the portions are
        cut into tiles and how many slices a decoded token's keys get is worked out on the device
        (kernels/fast.py, ``device_plan``), so one graph serves every batch of its shape.  Shapes
        beyond the buckets, or more shapes than ``max_mixed_graphs``, run kernel by kernel."""
        key, tb, wb, ri, pb, W = self._mixed_key(entries)
        if None in key or (key not in self.graphs and key not in self._warm_buckets
                           and len(self._warm_buckets) >= self.max_mixed_graphs + len(self.graph_buckets)):
            ctx, n_want = self.build_context(entries)
            return self.model.forward(ctx, self._view("want_rows"), n_want)
        ctx, n_want = self.build_context(entries, pad_to=tb, pad_want=wb)
        ctx.decode_only = False
        # what the graph is made for: at most this many single tokens (and more than the bucket
        # below holds) and at most this many portions
        ctx.extras["device_plan"] = dict(
            max_rows=self.row_buckets[ri] if ri >= 0 else 0,
            min_rows=(self.row_buckets[ri - 1] + 1 if ri > 0 else 1) if ri >= 0 else 0,
            max_portions=pb)
        ctx.extras["planning_context_len"] = self.max_context
        out = self._run_graphed(key, ctx, self._view("want_rows"), wb)
        return out[:W] if W else None

    def device_error(self) -> int:
        """Error bits the kernels have set since the last call (synchronises)."""
        bits = int(self.err.item())
        if bits:
            self.err.zero_()
        return bits

    def raise_on_device_error(self) -> None:
        bits = self.device_error()
        if bits:
            raise StepError("a kernel reported: " + ops.describe_device_error(bits))
