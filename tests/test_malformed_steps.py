"""A malformed step is refused on the host, before anything is copied or launched: the same request twice,
a wanted place outside the portion, an empty portion, a token id outside the vocabulary, more tokens or
requests than the engine was sized for, a block table longer than the fixed row pitch.  The batch builder
needs no GPU for these checks (they come before its first device call)."""

from types import SimpleNamespace

import pytest

from qwen3_from_scratch_b200.cache.manager import CacheManager, layout_of
from qwen3_from_scratch_b200.engine.batch import BatchContext, Entry
from qwen3_from_scratch_b200.parts.base import KVCacheSpec

VOCAB = 100


def context(max_tokens=64, max_seqs=4, pages=32):
    manager = CacheManager(layout_of({0: KVCacheSpec(2, 16), 1: KVCacheSpec(2, 16)}), page_size=4, num_pages=pages,
                           max_seqs=8)
    rt = SimpleNamespace(max_tokens=max_tokens, max_seqs=max_seqs, device="cpu")
    return manager, BatchContext(manager, storage=None, rt=rt)


def opened(manager, name, tokens):
    manager.open(name)
    manager.reserve(name, tokens)
    return name


def test_a_wanted_place_outside_the_portion():
    manager, ctx = context()
    opened(manager, "a", 5)
    for want in ([5], [-1], [0, 7]):
        with pytest.raises(ValueError, match="wanted place"):
            ctx.build([Entry("a", [1, 2, 3, 4, 5], want)], VOCAB)


def test_an_empty_portion_and_a_token_outside_the_vocabulary():
    manager, ctx = context()
    opened(manager, "a", 3)
    with pytest.raises(ValueError, match="brings no tokens"):
        ctx.build([Entry("a", [], ())], VOCAB)
    for bad in (VOCAB, -1, 10 ** 9):
        with pytest.raises(ValueError, match="outside the vocabulary"):
            ctx.build([Entry("a", [1, bad, 2], ())], VOCAB)


def test_more_tokens_or_requests_than_the_engine_was_sized_for():
    manager, ctx = context(max_tokens=8, max_seqs=2)
    for name in "abc":
        opened(manager, name, 6)
    with pytest.raises(ValueError, match="exceeds the 8"):
        ctx.build([Entry("a", [1] * 6, ()), Entry("b", [1] * 3, ())], VOCAB)
    with pytest.raises(ValueError, match="exceeds the 2"):
        ctx.build([Entry("a", [1], ()), Entry("b", [1], ()), Entry("c", [1], ())], VOCAB)


def test_a_block_table_longer_than_the_fixed_row_pitch():
    manager, ctx = context()
    opened(manager, "a", 20)  # five pages of four tokens
    with pytest.raises(ValueError, match="does not fit the fixed stride 4"):
        ctx.build([Entry("a", [1] * 20, ())], VOCAB, table_stride=4)


def test_a_request_that_is_not_open():
    manager, ctx = context()
    with pytest.raises(KeyError):
        ctx.build([Entry("nobody", [1], (0,))], VOCAB)
