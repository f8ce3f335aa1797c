"""Builds the device-side description of one step's batch.

A batch is a list of entries (request, its next tokens, which of them want logits).  Rows
that bring a single token are placed first (the decode kernels take that range), the
rest after them; the wanted logits keep the order in which the caller gave the entries.
All integer arrays go to the device in one copy from pinned memory (the reference builds a
tensor per array, each with a copy of its own: inference/model_worker.py:177-210).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..parts.base import Runtime, StepContext


@dataclass
class Entry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()  # indices into ``tokens`` whose logits are asked for
    # per-token integers that a part of the model defines for itself (positions on several axes, segment
    # ids, ...): name -> one int, or one row of ints, per token; they reach the parts as ``ctx.extra[name]``
    extra: Optional[Dict[str, Sequence]] = None


class BatchContext(StepContext):
    def __init__(self, manager: CacheManager, storage: CacheStorage, rt: Runtime):
        self.manager, self.storage, self.rt = manager, storage, rt
        self._tables: List[torch.Tensor] = []
        self._extra_layout: List = []
        self.extra: Dict[str, torch.Tensor] = {}
        self._head_views = None
        self._cuts = None
        self.requests: List[Hashable] = []

    def _decode_only_rebuild(self, entries: Sequence[Entry], vocab_size: int, table_stride: Optional[int],
                             ahead: int = 0) -> bool:
        """The common step of a running engine in as little Python as possible: the same requests as the
        last build in the same order, one token each, each wanting its logits, no block table changed.
        Writes tokens, positions and lengths into the pinned buffer and copies them; False if the step is
        not of that kind (nothing has been touched then)."""
        m, B = self.manager, len(entries)
        if (self._cuts[:7] != [B, B, B, B + 1, B, B, B] or self._extra_layout
                or (table_stride is not None and self._fixed_stride != table_stride)):
            return False
        tokens, starts, versions = [], [], []
        for e, request in zip(entries, self.requests):
            if e.request != request or len(e.tokens) != 1 or tuple(e.want) != (0,) or e.extra:
                return False
            t = int(e.tokens[0])
            if not 0 <= t < vocab_size:
                raise ValueError(f"request {e.request!r}: token id {t} is outside the vocabulary of {vocab_size}")
            length, _, version = m.row_state(request)
            tokens.append(t)
            starts.append(length + ahead)
            versions.append(version)
        if versions != self._versions:
            return False
        lens = [n + 1 for n in starts]
        # order of the buffer: tokens, positions, tok_seq, q_start, kv_len, slots, logit_rows; the rows'
        # numbers (tok_seq, q_start, slots, logit_rows) are those of the last build
        if self._head_views is None or self._head_views[0] != 7 * B + 1:
            n = 7 * B + 1
            self._head_views = (n, self._host.numpy()[:n], self._host[:n], self._dev[:n])
        _, host_np, host_head, dev_head = self._head_views
        self._copied.synchronize()
        host_np[:B] = tokens
        host_np[B:2 * B] = starts
        host_np[4 * B + 1:5 * B + 1] = lens
        dev_head.copy_(host_head, non_blocking=True)
        self._copied.record()
        self.q_lens, self.kv_lens = [1] * B, lens
        self.num_tokens = self.num_seqs = self.num_decode = B
        self.max_q_len, self.max_kv_len = 1, max(lens)
        self.h2d_bytes = (7 * B + 1) * 4
        return True

    @staticmethod
    def _extra_of(entries: Sequence[Entry], order: Sequence[int]):
        """The entries' ``extra`` arrays in the batch's row order: (all values flat, [(name, width)])."""
        names = sorted(entries[0].extra or {})
        flat: List[int] = []
        layout = []
        for e in entries:
            if sorted(e.extra or {}) != names:
                raise ValueError(f"request {e.request!r} brings the per-token arrays {sorted(e.extra or {})}, "
                                 f"others of the step bring {names}")
        for name in names:
            width = None
            for orig in order:
                e = entries[orig]
                rows = e.extra[name]
                if len(rows) != len(e.tokens):
                    raise ValueError(f"request {e.request!r}: '{name}' has {len(rows)} rows for {len(e.tokens)} tokens")
                for r in rows:
                    vals = [int(r)] if isinstance(r, int) else [int(x) for x in r]
                    if width is None:
                        width = len(vals)
                    if len(vals) != width or width == 0:
                        raise ValueError(f"request {e.request!r}: rows of '{name}' differ in width")
                    flat.extend(vals)
            layout.append((name, width))
        return flat, layout

    def pages(self, cache_id: int):
        return self.storage.planes(cache_id), self._tables[self.storage.group_of(cache_id)]

    def state(self, cache_id: int):
        return self.storage.states[cache_id]

    def build(self, entries: Sequence[Entry], vocab_size: int, table_stride: Optional[int] = None,
              keep_buffer: bool = False, ahead: int = 0) -> "BatchContext":
        """``entries``: each request at most once, every request open with pages reserved for
        its new length.  Fills every field of StepContext.

        ``table_stride`` fixes the row pitch of the block tables (else the longest table of the
        batch decides).  With ``keep_buffer`` the device arrays are written into the buffer of the
        previous build, which must have had the same layout (same counts of tokens, rows, wanted
        logits and the same stride): this is what lets a captured CUDA graph be replayed on new data.
        ``ahead``: tokens of every request that an earlier step, still running, will have added by the
        time this one runs: positions and lengths count them in."""
        m = self.manager
        if (keep_buffer and self._cuts is not None and len(entries) == len(self.requests)
                and self._decode_only_rebuild(entries, vocab_size, table_stride, ahead)):
            return self
        order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))
        row_of = {orig: row for row, orig in enumerate(order)}
        tokens: List[int] = []
        positions: List[int] = []
        tok_seq: List[int] = []
        q_start = [0]
        kv_len: List[int] = []
        slots: List[int] = []
        self.q_lens, self.kv_lens = [], []
        self.requests = []
        for row, orig in enumerate(order):
            e = entries[orig]
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request!r} brings no tokens")
            start = m.length(e.request) + ahead
            for t in e.tokens:
                if not 0 <= int(t) < vocab_size:
                    raise ValueError(f"request {e.request!r}: token id {t} is outside the vocabulary of {vocab_size}")
            tokens.extend(int(t) for t in e.tokens)
            positions.extend(range(start, start + n))
            tok_seq.extend([row] * n)
            q_start.append(q_start[-1] + n)
            kv_len.append(start + n)
            slots.append(m.slot(e.request))
            self.q_lens.append(n)
            self.kv_lens.append(start + n)
            self.requests.append(e.request)
        logit_rows: List[int] = []
        for orig, e in enumerate(entries):
            base = q_start[row_of[orig]]
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
                logit_rows.append(base + int(w))
        extra_flat, extra_layout = self._extra_of(entries, order)
        T, B, R = len(tokens), len(order), len(logit_rows)
        if T > self.rt.max_tokens:
            raise ValueError(f"a step of {T} tokens exceeds the {self.rt.max_tokens} the engine was sized for")
        if B > self.rt.max_seqs:
            raise ValueError(f"a step of {B} requests exceeds the {self.rt.max_seqs} the engine was sized for")
        n_groups = len(m.layout.groups)
        head = tokens + positions + tok_seq + q_start + kv_len + slots + logit_rows + extra_flat
        versions = [m.table_version(r) for r in self.requests]
        self.num_tokens, self.num_seqs = T, B
        self.max_q_len, self.max_kv_len = max(self.q_lens), max(self.kv_lens)
        self.num_decode = sum(1 for n in self.q_lens if n == 1)
        if (keep_buffer and getattr(self, "_cuts", None) is not None and self._cuts[:7] == [T, T, T, B + 1, B, B, R]
                and self._extra_layout == extra_layout
                and self._versions == versions and (table_stride is None or self._fixed_stride == table_stride)):
            # same requests, no block table changed since the last build: only the short arrays travel
            n_head = len(head)
            if self._head_views is None or self._head_views[0] != n_head:
                self._head_views = (n_head, self._host.numpy()[:n_head], self._host[:n_head], self._dev[:n_head])
            _, host_np, host_head, dev_head = self._head_views
            self._copied.synchronize()
            host_np[:] = head  # straight into the pinned buffer
            dev_head.copy_(host_head, non_blocking=True)
            self._copied.record()
            self.h2d_bytes = n_head * 4
            return self
        strides = []
        flat_tables: List[int] = []
        for g in range(n_groups):
            rows = [m.table(g, self.requests[row]) for row in range(B)]
            stride = max(1, max(len(r) for r in rows))
            if table_stride is not None:
                if stride > table_stride:
                    raise ValueError(f"a block table of {stride} pages does not fit the fixed stride {table_stride}")
                stride = table_stride
            strides.append(stride)
            for r in rows:
                flat_tables.extend(r)
                flat_tables.extend([-1] * (stride - len(r)))
        flat = head + flat_tables
        self._versions, self._fixed_stride = versions, table_stride
        cuts = [T, T, T, B + 1, B, B, R] + [T * w for _, w in extra_layout] + [B * s for s in strides]
        if keep_buffer and getattr(self, "_cuts", None) == cuts:
            self._copied.synchronize()  # the previous copy out of the pinned buffer has finished
            self._host.copy_(torch.tensor(flat, dtype=torch.int32))
            self._dev.copy_(self._host, non_blocking=True)
            self._copied.record()
            self.h2d_bytes = self._host.numel() * 4
            return self
        if keep_buffer and getattr(self, "_cuts", None) is not None:
            raise ValueError("this batch does not have the layout of the buffer it was asked to reuse")
        host = torch.tensor(flat, dtype=torch.int32).pin_memory()
        dev = host.to(self.rt.device, non_blocking=True)
        self._host, self._dev, self._cuts, self._extra_layout = host, dev, cuts, extra_layout
        self._head_views = None
        self._copied = torch.cuda.Event()
        self._copied.record()
        views = torch.split(dev, cuts)
        (self.token_ids, self.positions, self.tok_seq, self.q_start, self.kv_len, self.slot_ids,
         self.logit_rows) = views[:7]
        n_extra = len(extra_layout)
        self.extra = {name: views[7 + i].view(T, w) for i, (name, w) in enumerate(extra_layout)}
        self._tables = [views[7 + n_extra + g].view(B, strides[g]) for g in range(n_groups)]
        self.h2d_bytes = host.numel() * 4
        return self
