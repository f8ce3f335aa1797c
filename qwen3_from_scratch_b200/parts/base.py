"""Interfaces of the parts a model is put together from.

A *part* is built from explicit sizes and constants (never from a model
configuration object), says which tensors it needs by name (``weight_specs``),
receives them on the device (``setup``) and then runs on activations.  The
kinds of part and what each must offer:

``Norm``
    ``add_norm(stream, delta) -> normed``: adds ``delta`` (or nothing) into the
    float32 residual stream and returns the normed activations in the compute
    dtype; ``norm_rows(stream, delta, rows) -> normed`` does the same for chosen
    rows without changing the stream; ``forward(x)`` norms a plain tensor.
``PositionEncoding``
    ``apply(x[T, heads, D], positions[T]) -> x'``; optionally
    ``fused_rotary() -> (inv_freq, rotary_dim)`` when it is a rotate-half rotary
    encoding that the attention kernels can apply themselves.
``Mixer``
    ``cache_spec()`` (pages of keys/values, a fixed-size state, or none) and
    ``forward(x[T, width], ctx, cache_id, write_cache) -> y[T, width]``.
``FeedForward``
    ``forward(x[T, width]) -> y[T, width]``.
``Block``
    ``forward(stream, pending, ctx, cache_id, write_cache) -> pending'``: the
    arrangement of norms, mixer and feed-forward around the residual stream.
    ``pending`` is a sub-layer output not yet added to the stream (the next norm
    adds it, which saves one pass over the activations).

No part knows which model it is in: the model specification (``ModelSpec``)
chooses parts and their parameters layer by layer and lists the order in which
layers run.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Union

import torch

# ---------------------------------------------------------------------- weights


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part needs from the model folder.

    kind:
      ``matrix``  operand of a matrix product: kept as stored (bfloat16 stays
                  bfloat16, a tensor stored in float32 stays float32 and its
                  product runs in float32); in a float32 run everything is
                  widened to float32.
      ``vector``  small parameter read by float32 arithmetic (norm weights):
                  held in float32 on the device whatever it was stored as.
      ``index``   integer table: held as int32.
    init: how the random-weights writer fills it (``normal``: N(0, 0.02);
      ``one_plus_normal``: 1 + N(0, 0.1); ``zeros``).
    """

    name: str
    shape: Tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"


# ---------------------------------------------------------------------- cache needs


@dataclass(frozen=True)
class CachePlane:
    """One array of a paged cache: for every token ``heads`` vectors of ``width`` values.
    ``dtype``: ``"compute"`` (the engine's dtype) or ``"float32"``."""

    name: str
    heads: int
    width: int
    dtype: str = "compute"


@dataclass(frozen=True)
class PagedCacheSpec:
    """Pages with one slot per token, in one or more named planes (keys and values of attention; one
    latent vector per token; keys and values of different widths; ...).  A plane's pages are one tensor
    ``[num_pages, heads, page_size, width]``; all planes of a cache share the page ids.
    ``window`` = how many of the latest tokens a query still reads (None: all of them); pages a window
    has passed are given back."""

    planes: Tuple[CachePlane, ...]
    window: Optional[int] = None

    def bytes_per_token(self, compute_itemsize: int) -> int:
        return sum(p.heads * p.width * (4 if p.dtype == "float32" else compute_itemsize) for p in self.planes)


def KVCacheSpec(num_kv_heads: int, head_dim: int, window: Optional[int] = None) -> PagedCacheSpec:
    """The usual attention cache: planes ``k`` and ``v`` of ``num_kv_heads`` vectors of ``head_dim`` per token."""
    return PagedCacheSpec((CachePlane("k", int(num_kv_heads), int(head_dim)),
                           CachePlane("v", int(num_kv_heads), int(head_dim))), window)


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size per request (a recurrent mixer's), kept in a slot while the request lives.
    ``dtype``: ``"float32"`` or ``"compute"``."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


CacheSpec = Union[PagedCacheSpec, StateSpec, None]

# ---------------------------------------------------------------------- runtime


@dataclass
class Runtime:
    """What a part may rely on at run time: device, compute dtype, the largest step, the status word."""

    device: torch.device
    dtype: torch.dtype
    max_tokens: int
    max_seqs: int
    status: torch.Tensor = None  # int32[1] on the device; kernels OR error bits into it
    mailbox: torch.Tensor = None  # int32[1 + max_seqs]: the status word, then a step's sampled tokens

    def __post_init__(self):
        if self.status is None:
            # the status word and the sampled tokens lie side by side, so that one read brings both
            self.mailbox = torch.zeros(1 + max(1, self.max_seqs), dtype=torch.int32, device=self.device)
            self.status = self.mailbox[:1]

    def empty(self, *shape: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(*shape, dtype=dtype or self.dtype, device=self.device)

    def shared(self, tag: str, *shape: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """A scratch buffer that every part asking with the same tag, shape and dtype gets.
        Layers run one after the other, so the buffers of one role (the normed activations,
        the merged QKV product, ...) can be the same memory in every layer.  A tag's buffer
        must be consumed before the same role writes it again."""
        if not hasattr(self, "_shared"):
            self._shared = {}
        key = (tag, tuple(shape), dtype or self.dtype)
        if key not in self._shared:
            self._shared[key] = self.empty(*shape, dtype=dtype)
        return self._shared[key]


class StepContext:
    """Everything the parts need to know about the batch of one step.

    Device tensors (int32): ``token_ids[T]``, ``positions[T]`` (absolute position of each
    token in its request), ``tok_seq[T]`` (row of the batch each token belongs to),
    ``q_start[B + 1]`` (token offsets of the rows), ``kv_len[B]`` (tokens of each request
    after this step), ``slot_ids[B]`` (state slot of each request), ``logit_rows[R]``.
    Host mirrors: ``q_lens``, ``kv_lens``, ``max_q_len``, ``max_kv_len``, ``num_decode``
    (rows that bring exactly one token come first in the batch).
    ``pages(cache_id)`` gives ``({plane name: pages}, block_table)`` of a cache of pages,
    ``kv(cache_id)`` the same as ``(k_pages, v_pages, block_table)`` for a cache with planes ``k`` and
    ``v``, and ``state(cache_id)`` the ``[slots, *shape]`` tensor of a cache of fixed-size state.
    ``extra``: per-token integer arrays that the caller sent along with the tokens (``Entry.extra``),
    by name, int32 ``[T, width]`` on the device: positions on several axes, segment ids, whatever a part
    of the model defines for itself; ``positions`` (``start + i``) is always there.
    """

    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    tok_seq: torch.Tensor
    q_start: torch.Tensor
    kv_len: torch.Tensor
    slot_ids: torch.Tensor
    logit_rows: torch.Tensor
    q_lens: List[int]
    kv_lens: List[int]
    max_q_len: int
    max_kv_len: int
    num_decode: int

    def shared_in_step(self, key, make):
        """What ``make()`` returns, computed once per step: parts of different layers that need the
        same derived data of the batch (a table of angles for the step's positions, ...) ask with
        the same key.  ``Model.step`` empties ``per_step`` before the first layer runs."""
        store = self.__dict__.setdefault("per_step", {})
        if key not in store:
            store[key] = make()
        return store[key]

    def pages(self, cache_id: int):  # pragma: no cover - interface
        raise NotImplementedError

    def kv(self, cache_id: int):
        planes, table = self.pages(cache_id)
        return planes["k"], planes["v"], table

    extra: Dict[str, torch.Tensor] = {}

    def state(self, cache_id: int):  # pragma: no cover - interface
        raise NotImplementedError


# ---------------------------------------------------------------------- a norm that is not computed


STREAM_SUMSQ = "stream.sumsq"  # key in StepContext.per_step: StreamStats of the stream as it stands
NEXT_NORM_WEIGHT = "stream.next_norm_weight"  # key in StepContext.per_step: weight of the next block's first norm


@dataclass
class StreamStats:
    """What the projection that last added into the residual stream left about the stream's rows:
    ``sumsq[p, t]`` for ``p < parts`` are partial sums of squares of row ``t``; ``scaled``, if given, is
    the rows times ``scaled_for`` (a norm's weight), rounded once to bfloat16."""

    sumsq: torch.Tensor
    parts: int
    scaled: Optional[torch.Tensor] = None
    scaled_for: Optional[torch.Tensor] = None


@dataclass
class StreamNorm:
    """RMSNorm of the residual stream, not computed: a projection that takes it (``Linear``, for a few
    rows) runs on ``scaled``, the stream times the norm's ``weight`` in bfloat16 as the projection before
    left it, and multiplies its result by each row's 1 / rms (from ``sumsq``), so that no norm kernel runs."""

    stream: torch.Tensor
    weight: torch.Tensor
    eps: float
    sumsq: torch.Tensor
    parts: int
    scaled: torch.Tensor

    @property
    def shape(self):
        return self.stream.shape

    @property
    def dtype(self):
        return torch.bfloat16


# ---------------------------------------------------------------------- parts


class Part:
    """Base of all parts.  ``name`` is the prefix of its tensors in the model folder.

    ``graph_capturable``: the part's work is only kernel launches on the current stream, with
    no read of device data on the host and no state kept on the host, so a step can be captured
    in a CUDA graph and replayed.  Parts that do not say so keep the model on plain launches."""

    graph_capturable = False

    def __init__(self, name: str = ""):
        self.name = name

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        """Takes its tensors (already on the device) and allocates what it reuses every step."""
        self.rt = rt


class Norm(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, stream: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def norm_rows(self, stream: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def fused_rotary(self) -> Optional[Tuple[torch.Tensor, int]]:
        """(inv_freq, rotary_dim) if the encoding is a rotate-half rotation by position * inv_freq
        that the fused kernel can apply, else None (``apply`` is then used)."""
        return None

    def step_table(self, ctx: "StepContext") -> Optional[torch.Tensor]:
        """With ``fused_rotary``: float32 [T, rotary_dim] cosines then sines of the step's tokens,
        shared by all layers of the step, or None (the fused kernel then computes the angles)."""
        return None


class Mixer(Part):
    def cache_spec(self) -> CacheSpec:
        """What the mixer keeps per request: ``PagedCacheSpec`` (``KVCacheSpec(...)`` for keys and values),
        ``StateSpec``, or None."""
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_id: Optional[int], write_cache: bool) -> torch.Tensor:
        raise NotImplementedError

    #: a mixer (or feed-forward) that sets this also has ``can_fuse_stream(rows)``; where that is true its
    #: ``forward`` takes a ``StreamNorm`` for ``x`` and ``into_stream=stream`` (with ``next_norm_weight``, the
    #: weight of the norm that will read the stream next, or None), adds its output into the stream itself and
    #: returns the ``StreamStats`` of the stream's new rows instead of the output
    fuses_stream = False


class FeedForward(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    fuses_stream = False  # see Mixer.fuses_stream


class Block(Part):
    mixer: Mixer

    #: a block that sets this leaves ``ctx.per_step[STREAM_SUMSQ]`` describing the stream as it returns it
    #: (and returns no pending output); after any other block the model drops the entry
    keeps_stream_stats = False

    def forward(self, stream: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache_id: Optional[int], write_cache: bool) -> Optional[torch.Tensor]:
        raise NotImplementedError


# ---------------------------------------------------------------------- model specification


@dataclass(frozen=True)
class PartSpec:
    """Which registered part, with which parameters (sizes, constants, nested PartSpecs)."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run layer ``layer`` on cache ``cache``.

    A layer may appear in several calls (shared weights), each with a cache of its own,
    or with ``write_cache=False`` on a cache that an earlier call filled (shared keys/values).
    """

    layer: int
    cache: Optional[int]
    write_cache: bool = True


@dataclass
class ModelSpec:
    """A whole model as data: parts by layer, and the order in which layers run."""

    embedding: Tuple[str, PartSpec]  # every part comes as (tensor-name prefix, spec)
    layers: List[Tuple[str, PartSpec]]
    order: List[LayerCall]
    final_norm: Tuple[str, PartSpec]
    head: Tuple[str, PartSpec]
    vocab_size: int
    max_positions: int
    ignorable_weights: Tuple[str, ...] = ()
    eos_token_id: Optional[int] = None
