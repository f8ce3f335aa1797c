"""Model + cache + step function behind one small interface: feed tokens, get logits.

This is the layer the scheduler drives and the trace replay drives directly.  A request
is opened the first time it brings tokens, its pages are reserved before the step and the
step's tokens are recorded after it; ``end`` gives everything back.
"""

from __future__ import annotations

from typing import Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager, OutOfPages
from ..cache.storage import CacheStorage
from ..kernels import ops
from .batch import BatchContext, Entry
from .model import load_model


class DeviceStatusError(RuntimeError):
    pass


class Session:
    def __init__(self, model_dir: str, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                 num_pages: Optional[int] = None, cache_tokens: Optional[int] = None, max_seqs: int = 32,
                 max_step_tokens: int = 3000, poison_freed_pages: bool = False):
        """``num_pages`` pages per group, or ``cache_tokens`` (rounded up to whole pages)."""
        if num_pages is None:
            if cache_tokens is None:
                raise ValueError("give num_pages or cache_tokens")
            num_pages = -(-int(cache_tokens) // page_size)
        self.model, self.config, self.rt = load_model(model_dir, dtype, device, max_step_tokens, max_seqs)
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
        ctx = BatchContext(self.manager, self.storage, self.rt).build(entries, self.vocab_size)
        self.last_context = ctx
        logits = self.model.step(ctx)
        for e in entries:
            self.manager.advance(e.request, self.manager.length(e.request) + len(e.tokens))
        self._poison()
        return logits

    def step_reserved(self, entries: Sequence[Entry]) -> torch.Tensor:
        """The step for a caller (the scheduler) that has opened the requests and reserved their
        pages itself and will record the progress itself: builds the batch and runs it."""
        ctx = BatchContext(self.manager, self.storage, self.rt).build(entries, self.vocab_size)
        self.last_context = ctx
        return self.model.step(ctx)

    def after_step(self) -> None:
        self._poison()

    def check_status_word_async(self) -> None:
        """Checks the status word when the caller has just synchronised anyway (a token read)."""
        self.check_status()

    def check_status(self) -> None:
        """Reads the device status word (synchronises) and raises if a kernel flagged bad table data."""
        word = int(self.rt.status.item())
        if word:
            self.rt.status.zero_()
            raise DeviceStatusError(f"a kernel reported: {ops.describe_status(word)}")
