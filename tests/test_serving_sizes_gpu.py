"""Schedules through the scheduler in bfloat16 at the head size and page size the serving kernels are made
for (tiny D: heads of 128, pages of 16): the TMA decode attention that takes the raw projection, the products
that add into the stream and apply the norm, the tcgen05 portion attention and gate/up product.  Requests of
different lengths that finish at different steps, arrive while others decode, are preempted and recomputed,
and decode twelve to sixteen at a time beside a prompt portion.

bfloat16 may pick the runner-up where the plain logits nearly tie, so ids are checked against the plain
implementation token by token along the engine's own path (the chosen token's logit within 2e-2 of the
scale below the best), and two runs of the engine are compared up to the first such near tie.
"""

import pytest
import torch

import plain_qwen3 as plain
from conftest import TINY, random_tokens

pytestmark = pytest.mark.gpu

KEY, PAGE = "d", 16
VOCAB = TINY[KEY][0]["vocab_size"]
NEAR = 2e-2


def plain_path(cfg, w, prompt, output):
    """For each generated token: (how far below the best plain logit it lies, the margin between the two best
    plain logits), both relative to the largest |logit| of that position."""
    ids = list(prompt) + list(output)
    logits = plain.forward_logits(cfg, w, ids[:-1])[len(prompt) - 1:]
    out = []
    for row, token in zip(logits, output):
        scale = float(row.abs().max())
        top = torch.topk(row, 2).values
        out.append((float(top[0] - row[token]) / scale, float(top[0] - top[1]) / scale))
    return out


def assert_follows_plain(cfg, w, prompts, outputs, what):
    for i, (p, o) in enumerate(zip(prompts, outputs)):
        for step, (gap, _) in enumerate(plain_path(cfg, w, p, o)):
            assert gap <= NEAR, f"{what}: request {i}, token {step}: the plain logits rule it out (gap {gap:.3g})"


def assert_same_up_to_near_ties(cfg, w, prompts, a, b, what):
    for i, (p, x, y) in enumerate(zip(prompts, a, b)):
        margins = [m for _, m in plain_path(cfg, w, p, x)]
        for step, (s, t) in enumerate(zip(x, y)):
            if s != t:
                assert margins[step] <= 2 * NEAR, f"{what}: request {i} differs at token {step} without a near tie"
                break


def test_requests_of_many_lengths_with_lookahead_and_graphs(tiny_folders):
    """Five requests with different prompt lengths and token limits, one ending on an end-of-sequence
    token, two arriving while the others decode: the engine as it serves (CUDA graphs, steps launched
    ahead) against the engine with neither, and both against the plain implementation."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    from qwen3_from_scratch_b200.engine.request import RequestStatus, SamplingParams
    folder = tiny_folders[KEY]
    cfg, w = plain.read_model_folder(folder)
    prompts = [random_tokens(VOCAB, n, 160 + i) for i, n in enumerate([7, 150, 33, 290, 64])]
    limits = [40, 9, 31, 24, 50]
    runs = []
    for fast in (False, True):
        engine = SyncEngine(folder, dtype="bfloat16", block_size=PAGE, num_pages=96, max_num_seqs=4,
                            max_num_tokens=192, chunked_prefill_size=128, cuda_graphs=fast, lookahead=fast)
        # an id that the first request is known to produce (from the first run): it ends there in both
        engine.eos_token_id = None if not runs else runs[0][0][0][14]
        params = [SamplingParams(max_new_tokens=n, ignore_eos=i != 0) for i, n in enumerate(limits)]
        reqs = [engine.add_request(p, params=q) for p, q in zip(prompts[:3], params[:3])]
        steps = 0
        while any(r.status != RequestStatus.FINISHED for r in reqs):
            engine.step()
            steps += 1
            if steps == 7:
                reqs += [engine.add_request(p, params=q) for p, q in zip(prompts[3:], params[3:])]
        engine.drain()
        engine.session.manager.check()
        assert not engine.session.manager.live_requests()
        runs.append(([list(r.output) for r in reqs], [r.finish_reason for r in reqs], engine))
    (slow_ids, slow_why, _), (fast_ids, fast_why, fast_engine) = runs
    assert fast_engine.num_ahead > 10 and fast_engine.session.step_graphs.replays > 20
    assert_follows_plain(cfg, w, prompts, slow_ids, "plain launches")
    assert_follows_plain(cfg, w, prompts, fast_ids, "graphs and lookahead")
    eos = slow_ids[0][14]
    stop = slow_ids[0].index(eos)
    if fast_ids[0][:stop + 1] == slow_ids[0][:stop + 1]:
        assert fast_why[0] == "eos" and len(fast_ids[0]) == stop + 1
    assert fast_why[1:] == slow_why[1:] == ["length"] * 4
    assert_same_up_to_near_ties(cfg, w, prompts[1:], slow_ids[1:], fast_ids[1:], "graphs and lookahead against neither")


def test_preemption_and_page_reuse_at_the_serving_head_size(tiny_folders):
    """A pool too small for all requests at once: some are preempted, their pages go to others and they are
    recomputed over prompt + generated tokens; each still produces what the plain logits allow."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    folder = tiny_folders[KEY]
    cfg, w = plain.read_model_folder(folder)
    prompts = [random_tokens(VOCAB, n, 180 + i) for i, n in enumerate([120, 100, 90, 130])]
    alone = SyncEngine(folder, dtype="bfloat16", block_size=PAGE, num_pages=64, max_num_seqs=4, max_num_tokens=256)
    want = [alone.generate(p, max_new_tokens=48, ignore_eos=True) for p in prompts]
    # 4 requests end at 138 to 178 tokens = 9 to 12 pages each, 42 together; the pool has 30
    tight = SyncEngine(folder, dtype="bfloat16", block_size=PAGE, num_pages=30, max_num_seqs=4, max_num_tokens=256)
    results, _ = tight.batch_generate(prompts, max_new_tokens=48, ignore_eos=True)
    assert tight.scheduler.num_preemptions > 0
    got = [r.token_ids for r in results]
    assert all(len(g) == 48 for g in got)
    assert_follows_plain(cfg, w, prompts, got, "with preemption")
    assert_same_up_to_near_ties(cfg, w, prompts, want, got, "preempted against alone")
    tight.session.manager.check()
    assert not tight.session.manager.live_requests()


def test_twelve_to_sixteen_requests_decode_together_beside_a_portion(tiny_folders):
    """``max_num_seqs=16``: sixteen requests decode together (the second token tile of the few-rows products),
    some finish so that fifteen down to twelve remain, and a new request's prompt portions run beside them."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    from qwen3_from_scratch_b200.engine.request import RequestStatus, SamplingParams
    folder = tiny_folders[KEY]
    cfg, w = plain.read_model_folder(folder)
    prompts = [random_tokens(VOCAB, 20 + 3 * i, 200 + i) for i in range(16)] + [random_tokens(VOCAB, 200, 230)]
    limits = [16 + (i % 5) * 4 for i in range(16)] + [10]
    engine = SyncEngine(folder, dtype="bfloat16", block_size=PAGE, num_pages=160, max_num_seqs=16,
                        max_num_tokens=96, chunked_prefill_size=64)
    reqs = [engine.add_request(p, params=SamplingParams(max_new_tokens=n, ignore_eos=True))
            for p, n in zip(prompts[:16], limits[:16])]
    seen_rows, beside = set(), 0
    added = False
    while any(r.status != RequestStatus.FINISHED for r in reqs):
        plan = engine.step()
        decoding = sum(1 for s in plan if s.num_tokens == 1)
        seen_rows.add(decoding)
        if any(s.num_tokens > 1 for s in plan) and decoding > 8:
            beside += 1
        if not added and all(r.is_decoding for r in reqs[:16]) and min(len(r.output) for r in reqs[:16]) >= 11:
            # one request is about to finish: its slot goes to the late request, whose portions run beside the rest
            reqs.append(engine.add_request(prompts[16], params=SamplingParams(max_new_tokens=limits[16], ignore_eos=True)))
            added = True
    engine.drain()
    assert 16 in seen_rows and any(12 <= n <= 15 for n in seen_rows), sorted(seen_rows)
    assert added and beside >= 2, "no prompt portion ran beside more than eight decoding requests"
    assert_follows_plain(cfg, w, prompts, [list(r.output) for r in reqs], "sixteen together")
    engine.session.manager.check()
    assert not engine.session.manager.live_requests()


def test_a_step_of_more_than_a_thousand_rows_beside_decoding_requests(tiny_folders):
    """Four prompts of 300 tokens arrive while two requests decode and are run in one step of 1,202 rows: at
    this many rows the QKV projection (with head norm, rotation and page write in its epilogue) and the gate/up
    product (with SwiGLU) are the ones that pairs of CTAs compute with the paired tensor-core instruction."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    from qwen3_from_scratch_b200.engine.request import RequestStatus, SamplingParams
    from qwen3_from_scratch_b200.kernels import ops
    folder = tiny_folders[KEY]
    cfg, w = plain.read_model_folder(folder)
    prompts = [random_tokens(VOCAB, n, 300 + i) for i, n in enumerate([40, 25, 300, 300, 300, 300])]
    engine = SyncEngine(folder, dtype="bfloat16", block_size=PAGE, num_pages=160, max_num_seqs=8,
                        max_num_tokens=2048, chunked_prefill_size=2048)
    weights = engine.session.model.layers[0]
    assert ops.gemm_tc_qkv_pays(1202, weights.mixer.qkv.weight) == "pair"
    assert ops.gemm_tc_swiglu_pays(1202, weights.feed_forward.gate_up.weight) == "pair"
    reqs = [engine.add_request(p, params=SamplingParams(max_new_tokens=24, ignore_eos=True)) for p in prompts[:2]]
    while not all(r.is_decoding for r in reqs) or min(len(r.output) for r in reqs) < 3:
        engine.step()
    reqs += [engine.add_request(p, params=SamplingParams(max_new_tokens=12, ignore_eos=True)) for p in prompts[2:]]
    largest = 0
    while any(r.status != RequestStatus.FINISHED for r in reqs):
        plan = engine.step()
        largest = max(largest, sum(s.num_tokens for s in plan))
    engine.drain()
    assert largest == 1202, f"the largest step had {largest} rows"
    assert_follows_plain(cfg, w, prompts, [list(r.output) for r in reqs], "a step of 1,202 rows")
    engine.session.manager.check()
    assert not engine.session.manager.live_requests()
