"""Model + cache + step function behind one small interface: feed tokens, get logits.

This is the layer the scheduler drives and the trace replay drives directly.  A request
is opened the first time it brings tokens, its pages are reserved before the step and the
step's tokens are recorded after it; ``end`` gives everything back.
"""

from __future__ import annotations

import gc
from collections import OrderedDict
from typing import Hashable, Optional, Sequence

import torch

from ..cache.manager import CacheManager, OutOfPages
from ..cache.storage import CacheStorage
from ..kernels import ops
from .batch import BatchContext, Entry
from .model import load_model


class DeviceStatusError(RuntimeError):
    pass


class StepGraphs:
    """CUDA graphs of steps whose shape comes again.  What a graph fixes is the shape of the launches:
    tokens, requests, how many of them bring a single token, the longest portion, the number of
    wanted logits and the context bucket of 1024 tokens (it sets the row pitch of the block tables and
    the number of key ranges the decode attention uses).  Everything else - token ids, positions,
    lengths, tables, which rows are wanted - is data in a fixed buffer that each step's batch is
    copied into before the replay.

    Decode-only steps (every request brings one token and wants its logits) are recorded the first
    time their shape appears; other shapes (full-size prompt portions, which a long prompt repeats)
    when they appear a second time, so that one-off shapes are never recorded; at most MAX_GRAPHS are
    kept, the least recently replayed one making room.  The first step of a
    shape always runs kernel by kernel: it is this step's result, and first-use set-up must not
    happen inside a capture.  The graphs share one memory pool: only one of them runs at a time."""

    BUCKET = 1024
    MAX_GRAPHS = 96

    def __init__(self, session: "Session"):
        self.session = session
        self.graphs = OrderedDict()  # least recently replayed first
        self.seen = {}
        self.pool = None
        self.replays = 0

    @staticmethod
    def decode_only(entries: Sequence[Entry]) -> bool:
        return all(len(e.tokens) == 1 and tuple(e.want) == (0,) for e in entries)

    def run(self, entries: Sequence[Entry], ahead: int = 0, token_source: Optional[torch.Tensor] = None) -> torch.Tensor:
        s = self.session
        longest = max(s.manager.length(e.request) + len(e.tokens) for e in entries) + ahead
        bucket = -(-longest // self.BUCKET) * self.BUCKET
        stride = -(-bucket // s.manager.page_size)
        lens = [len(e.tokens) for e in entries]
        key = (sum(lens), len(entries), sum(1 for n in lens if n == 1), max(lens),
               sum(len(e.want) for e in entries), bucket,
               tuple(sorted((name, len(rows[0]) if rows and not isinstance(rows[0], int) else 1)
                            for name, rows in (entries[0].extra or {}).items())))
        slot = self.graphs.get(key)
        if slot is not None:
            self.graphs.move_to_end(key)
            ctx, graph, logits = slot
            ctx.build(entries, s.vocab_size, table_stride=stride, keep_buffer=True, ahead=ahead)
            if token_source is not None:
                ctx.token_ids.copy_(token_source)
            graph.replay()
            self.replays += 1
            s.last_context, s.last_graph = ctx, (graph, logits)
            return logits
        ctx = BatchContext(s.manager, s.storage, s.rt).build(entries, s.vocab_size, table_stride=stride, ahead=ahead)
        if token_source is not None:
            ctx.token_ids.copy_(token_source)
        ctx.max_kv_len = bucket  # the split count recorded in a graph is the bucket's
        eager = s.model.step(ctx)
        s.last_context, s.last_graph = ctx, None
        self.seen[key] = self.seen.get(key, 0) + 1
        if len(self.seen) > 4096:
            self.seen.clear()
        wanted = self.decode_only(entries) or self.seen[key] >= 2
        if not wanted:
            return eager
        while len(self.graphs) >= self.MAX_GRAPHS:  # the shape that has not come for the longest time makes room
            self.graphs.popitem(last=False)
        graph = torch.cuda.CUDAGraph()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
            self.capture_stream = torch.cuda.Stream(device=s.rt.device)
        # Recorded with capture_begin / capture_end on a stream of the engine's own rather than through
        # torch.cuda.graph(), which synchronises the device, runs the garbage collector and empties the
        # allocator's cache every time (tens of milliseconds, and the steps after it pay for new allocations).
        # No garbage collection while recording: the collector may destroy an older engine's graphs, and
        # destroying a graph is a CUDA call that invalidates a capture in progress.
        collecting = gc.isenabled()
        gc.disable()
        current = torch.cuda.current_stream(s.rt.device)
        self.capture_stream.wait_stream(current)
        try:
            with torch.cuda.stream(self.capture_stream):
                graph.capture_begin(pool=self.pool)
                try:
                    logits = s.model.step(ctx)
                finally:
                    graph.capture_end()
        finally:
            if collecting:
                gc.enable()
        current.wait_stream(self.capture_stream)
        self.graphs[key] = (ctx, graph, logits)
        s.last_graph = (graph, logits)
        return eager


class Session:
    def __init__(self, model_dir: str, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                 num_pages: Optional[int] = None, cache_tokens: Optional[int] = None, max_seqs: int = 32,
                 max_step_tokens: int = 3000, poison_freed_pages: bool = False, cuda_graphs: bool = True,
                 random_weights: Optional[int] = None):
        """``num_pages`` pages per group, or ``cache_tokens`` (rounded up to whole pages).
        ``random_weights``: a seed; the folder then needs only config.json (weights drawn on the device).
        ``cuda_graphs``: replay steps whose shape repeats (decode steps, full-size prompt portions) from
        captured graphs instead of launching kernel by kernel."""
        if num_pages is None:
            if cache_tokens is None:
                raise ValueError("give num_pages or cache_tokens")
            num_pages = -(-int(cache_tokens) // page_size)
        self.model, self.config, self.rt = load_model(model_dir, dtype, device, max_step_tokens, max_seqs,
                                                     random_weights=random_weights)
        layout = self.model.cache_layout()
        self.manager = CacheManager(layout, page_size, num_pages, max_seqs)
        self.storage = CacheStorage(layout, page_size, max_seqs, self.rt.device, self.rt.dtype)
        self.vocab_size = self.model.spec.vocab_size
        self.max_positions = self.model.spec.max_positions
        self.manager.on_open = self.storage.clear_slot
        self.poison_freed_pages = poison_freed_pages
        if poison_freed_pages:
            self.manager.freed_log = []
        self.last_context: Optional[BatchContext] = None
        self.step_graphs = StepGraphs(self) if cuda_graphs and self.model.graph_capturable else None
        self.last_graph = None

    # ------------------------------------------------------------------ requests
    def open(self, request: Hashable) -> None:
        self.manager.open(request)

    def length(self, request: Hashable) -> int:
        return self.manager.length(request)

    def end(self, request: Hashable) -> None:
        self.manager.close(request)
        self._poison()

    def _poison(self) -> None:
        if self.poison_freed_pages and self.manager.freed_log:
            self.storage.poison(self.manager.freed_log)
            self.manager.freed_log.clear()

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: Sequence[Entry]) -> None:
        """Opens new requests and reserves pages for every entry; raises OutOfPages with nothing
        taken for the entry that does not fit (entries before it keep their pages)."""
        seen = set()
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if e.request not in self.manager:
                self.open(e.request)
            new_length = self.manager.length(e.request) + len(e.tokens)
            if new_length > self.max_positions:
                raise ValueError(f"request {e.request!r} would reach {new_length} tokens, "
                                 f"the model's max_position_embeddings is {self.max_positions}")
            self.manager.reserve(e.request, new_length)

    def step(self, entries: Sequence[Entry]) -> torch.Tensor:
        """Runs the entries as one batch.  Returns float32 logits [sum(len(want)), vocab] on the
        device, in the order of the entries and of their ``want``."""
        entries = [e if isinstance(e, Entry) else Entry(*e) for e in entries]
        if not entries:
            return torch.empty(0, self.vocab_size, dtype=torch.float32, device=self.rt.device)
        self.prepare(entries)
        logits = self._run(entries)
        for e in entries:
            self.manager.advance(e.request, self.manager.length(e.request) + len(e.tokens))
        self._poison()
        return logits

    def step_reserved(self, entries: Sequence[Entry], ahead: int = 0,
                      token_source: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The step for a caller (the scheduler) that has opened the requests and reserved their
        pages itself and will record the progress itself: builds the batch and runs it.
        ``ahead``: an earlier step, still running, will have added this many tokens to every request
        of this one by the time it runs; ``token_source``: int32 on the device, one per row: the token
        ids of this step (those that the earlier step is about to sample), copied in on the stream."""
        return self._run(entries, ahead, token_source)

    def _run(self, entries: Sequence[Entry], ahead: int = 0, token_source: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.step_graphs is not None:
            return self.step_graphs.run(entries, ahead, token_source)
        ctx = BatchContext(self.manager, self.storage, self.rt).build(entries, self.vocab_size, ahead=ahead)
        if token_source is not None:
            ctx.token_ids.copy_(token_source)
        self.last_context, self.last_graph = ctx, None
        return self.model.step(ctx)

    def rerun_last(self) -> torch.Tensor:
        """Runs the last step's batch again as it ran (graph replay or plain launches); the
        cache is left as it was, since the same keys and values are written again.  For timing."""
        if self.last_graph is not None:
            graph, logits = self.last_graph
            graph.replay()
            return logits
        return self.model.step(self.last_context)

    def launches_per_decode_step(self, ctx: BatchContext) -> int:
        """Launches of this engine's own kernels in one step of ``ctx`` (counted by running it once
        kernel by kernel; library matrix products are not counted)."""
        before = ops.launch_count()
        self.model.step(ctx)
        return ops.launch_count() - before

    def after_step(self) -> None:
        self._poison()

    def check_status(self) -> None:
        """Reads the device status word (synchronises) and raises if a kernel flagged bad table data."""
        self.raise_on_status(int(self.rt.status.item()))

    def raise_on_status(self, word: int) -> None:
        """``word``: the status word as the caller has just read it from the device."""
        if word:
            self.rt.status.zero_()
            raise DeviceStatusError(f"a kernel reported: {ops.describe_status(word)}")
