"""The engine against the plain implementation under every way of cutting the work,
in float32 and in bfloat16, on the tiny configurations."""

import pytest
import torch

from conftest import TINY, random_tokens
from harness import Replayer, assert_close, plain_logits

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
LENGTHS = {"a": [5, 17, 31, 70, 131], "b": [1, 9, 33, 64, 100], "c": [3, 50, 97, 160], "d": [20, 150, 33, 300],
           "e": [2, 25, 49, 120]}
PAGE = {"a": 4, "b": 8, "c": 16, "d": 16, "e": 8}


def sequences(key):
    vocab = TINY[key][0]["vocab_size"]
    return {f"{key}{i}": random_tokens(vocab, n, 100 + i) for i, n in enumerate(LENGTHS[key])}


_plain_cache = {}


def oracle(folder, key):
    if key not in _plain_cache:
        _plain_cache[key] = plain_logits(folder, sequences(key))
    return _plain_cache[key]


def make_session(folder, dtype, key, cache_tokens=2048, **kw):
    from qwen3_from_scratch_b200.engine.session import Session
    return Session(folder, dtype=dtype, page_size=PAGE[key], cache_tokens=cache_tokens, max_seqs=8,
                   max_step_tokens=1024, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", list(TINY))
def test_each_request_alone_and_whole(tiny_folders, key, dtype):
    seqs = sequences(key)
    session = make_session(tiny_folders[key], dtype, key)
    rep = Replayer(session, seqs)
    for req, ids in seqs.items():
        rep.step([(req, len(ids))])
    session.manager.check()
    assert not session.manager.live_requests()
    assert_close(rep.result(), oracle(tiny_folders[key], key), dtype, "whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", list(TINY))
def test_prefill_then_last_32_one_by_one(tiny_folders, key, dtype):
    seqs = sequences(key)
    session = make_session(tiny_folders[key], dtype, key)
    rep = Replayer(session, seqs)
    for req, ids in seqs.items():
        head = max(0, len(ids) - 32)
        if head:
            rep.step([(req, head)])
        while rep.remaining(req):
            rep.step([(req, 1)])
    assert_close(rep.result(), oracle(tiny_folders[key], key), dtype, "prefill+decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", list(TINY))
def test_portions_of_changing_size(tiny_folders, key, dtype):
    seqs = sequences(key)
    session = make_session(tiny_folders[key], dtype, key)
    rep = Replayer(session, seqs)
    sizes = [16, 7, 5, 3, 2, 2, 11, 1, 2, 29]
    for req in seqs:
        i = 0
        while rep.remaining(req):
            rep.step([(req, sizes[i % len(sizes)])])
            i += 1
    assert_close(rep.result(), oracle(tiny_folders[key], key), dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", list(TINY))
def test_mixed_batches_with_page_reuse(tiny_folders, key, dtype):
    """Up to four live requests, portions of some beside single tokens of others, in a pool so
    small that pages are given back and used again; freed pages are filled with NaN."""
    seqs = sequences(key)
    page = PAGE[key]
    lengths = sorted((len(s) for s in seqs.values()), reverse=True)
    # room for the largest requests that are ever live together, rounded up to pages, nothing more
    cache_tokens = sum(-(-n // page) * page for n in lengths[:3]) + page
    session = make_session(tiny_folders[key], dtype, key, cache_tokens=cache_tokens, poison_freed_pages=True)
    rep = Replayer(session, seqs)
    waiting = list(seqs)
    live = []
    total_pages = -(-cache_tokens // page)
    pages_of = {r: -(-len(ids) // page) for r, ids in seqs.items()}
    portion = [13, 2, 6, 1, 9, 3]
    tick = 0
    while waiting or live:
        # admit while the whole of every live request still fits (so no step can run out of pages)
        while waiting and len(live) < 4 and sum(pages_of[r] for r in live) + pages_of[waiting[0]] <= total_pages:
            live.append(waiting.pop(0))
        assert live, "the pool is too small for the next request alone"
        step = []
        for j, req in enumerate(live):
            # the oldest live request decodes token by token, the others bring portions
            n = 1 if (j == 0 and rep.fed[req] > 0) else portion[(tick + j) % len(portion)]
            step.append((req, n))
        rep.step(step)
        session.manager.check()
        live = [r for r in live if rep.remaining(r)]
        tick += 1
    assert not session.manager.live_requests()
    assert_close(rep.result(), oracle(tiny_folders[key], key), dtype, "mixed")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_the_first_token(tiny_folders, dtype):
    """One token at a time from position 0 for several hundred steps (tiny A and its page of 4)."""
    key = "a"
    vocab = TINY[key][0]["vocab_size"]
    seqs = {"long": random_tokens(vocab, 300, 7)}
    session = make_session(tiny_folders[key], dtype, key)
    rep = Replayer(session, seqs)
    while rep.remaining("long"):
        rep.step([("long", 1)])
    want = plain_logits(tiny_folders[key], seqs)
    assert_close(rep.result(), want, dtype, "long decode")


def test_float32_cuts_give_identical_bits(tiny_folders):
    """In float32 every kernel sums in an order that does not depend on the batch, so whole
    prompts, portions and single tokens agree exactly, not only within a tolerance."""
    key = "b"
    seqs = sequences(key)
    results = []
    for sizes in ([1000], [16, 7, 5, 3, 2, 2], [1]):
        session = make_session(tiny_folders[key], "float32", key)
        rep = Replayer(session, seqs)
        for req in seqs:
            i = 0
            while rep.remaining(req):
                rep.step([(req, sizes[i % len(sizes)])])
                i += 1
        results.append(rep.result())
    for other in results[1:]:
        for req in seqs:
            assert torch.equal(results[0][req], other[req]), f"request {req} differs between cuts"
