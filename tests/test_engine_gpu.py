"""Generation through the Python entry point and the command line, and trace replay as a program."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import ROOT, TINY, random_tokens

pytestmark = pytest.mark.gpu


def greedy_by_plain(folder, prompt, n):
    cfg, w = plain.read_model_folder(folder)
    ids = list(prompt)
    margins = []
    for _ in range(n):
        logits = plain.forward_logits(cfg, w, ids)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        ids.append(plain.greedy_token(logits))
    return ids[len(prompt):], margins


@pytest.mark.parametrize("key,page", [("a", 4), ("b", 8)])
def test_greedy_generation_equals_the_plain_implementation(tiny_folders, key, page):
    """float32 end to end: two tiny workloads (prompts of 5/17/31 and 1/9/33/64/100 tokens,
    16 greedy tokens each) through batch_generate with chunked prompts and continuous batching."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    folder = tiny_folders[key]
    vocab = TINY[key][0]["vocab_size"]
    lengths = [5, 17, 31] if key == "a" else [1, 9, 33, 64, 100]
    # prompts whose plain top-2 logits stay apart at every step, so that equality of ids is a fair demand
    prompts, expected = [], []
    for i, n in enumerate(lengths):
        for seed in range(1 + 100 * i, 100 + 100 * i):
            prompt = random_tokens(vocab, n, seed)
            want, margins = greedy_by_plain(folder, prompt, 16)
            if min(margins) > 1e-3:
                break
        prompts.append(prompt)
        expected.append(want)
    engine = SyncEngine(folder, dtype="float32", block_size=page, num_pages=128, max_num_seqs=4,
                        max_num_tokens=48, chunked_prefill_size=16)
    results, batch = engine.batch_generate(prompts, max_new_tokens=16, ignore_eos=True)
    assert batch.num_requests == len(prompts) and batch.total_tokens == 16 * len(prompts)
    for want, r in zip(expected, results):
        assert r.finish_reason == "length"
        assert r.token_ids == want
    engine.session.manager.check()
    assert engine.session.manager.free_slots() == 4


@pytest.mark.parametrize("key,page,length", [("a", 4, 17), ("d", 16, 150)])
def test_bfloat16_generation_follows_plain_within_near_ties(tiny_folders, key, page, length):
    """Through the engine as it serves (graphs, lookahead); "d" has the head size of the serving kernels, so
    its prompt runs on the tcgen05 kernels and its decode steps without norm and qkv_post kernels."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    folder = tiny_folders[key]
    cfg, w = plain.read_model_folder(folder)
    prompt = random_tokens(TINY[key][0]["vocab_size"], length, 2)
    engine = SyncEngine(folder, dtype="bfloat16", block_size=page, num_pages=64, max_num_seqs=2,
                        max_num_tokens=max(32, length))
    got = engine.generate(prompt, max_new_tokens=12, ignore_eos=True)
    ids = list(prompt)
    for token in got:
        logits = plain.forward_logits(cfg, w, ids)[-1]
        gap = float(logits.max() - logits[token])
        assert gap <= 2e-2 * float(logits.abs().max()), "bfloat16 picked a token the plain logits rule out"
        ids.append(token)


def test_temperature_and_top_k_match_plain_with_the_same_generator(tiny_folders):
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    from qwen3_from_scratch_b200.engine.request import SamplingParams
    folder = tiny_folders["b"]
    cfg, w = plain.read_model_folder(folder)
    prompts = [random_tokens(384, n, 3 + i) for i, n in enumerate([9, 33])]
    params = [SamplingParams(temperature=0.7, max_new_tokens=10, seed=42, ignore_eos=True),
              SamplingParams(temperature=1.1, top_k=20, max_new_tokens=10, seed=42, ignore_eos=True)]
    engine = SyncEngine(folder, dtype="float32", block_size=8, num_pages=64, max_num_seqs=4, max_num_tokens=32,
                        chunked_prefill_size=16)
    reqs = [engine.add_request(p, params=q) for p, q in zip(prompts, params)]
    while any(r.finish_reason is None for r in reqs):
        engine.step()
    for req, prompt, p in zip(reqs, prompts, params):
        ids = list(prompt)
        for token in req.output:
            logits = plain.forward_logits(cfg, w, ids)[-1]
            want = plain.sample_token(logits, p.temperature, p.top_k, p.seed, req.key, len(ids))
            assert token == want
            ids.append(token)
        assert len(set(req.output)) > 1  # it is sampling, not a constant


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portion_graphs_give_what_plain_launches_give(tiny_folders, dtype):
    """Equal prompt portions: from the third on they are replayed from a graph recorded at the second.
    The logits of every portion against the same portions launched kernel by kernel, for two
    requests whose portions alternate (so a graph is replayed on another request's tables)."""
    from qwen3_from_scratch_b200.engine.session import Session
    folder = tiny_folders["c"]
    prompts = {"x": random_tokens(331, 6 * 24, 7), "y": random_tokens(331, 5 * 24 + 9, 8)}
    outs = []
    for graphs in (True, False):
        session = Session(folder, dtype=dtype, page_size=8, num_pages=64, max_seqs=4, max_step_tokens=64,
                          cuda_graphs=graphs)
        got = []
        at = {"x": 0, "y": 0}
        while any(at[r] < len(prompts[r]) for r in prompts):
            for r in prompts:
                piece = prompts[r][at[r]:at[r] + 24]
                if piece:
                    got.append(session.step([(r, piece, (len(piece) - 1,))]).float().cpu())
                    at[r] += len(piece)
        outs.append(torch.cat(got))
        if graphs:
            assert session.step_graphs.replays >= 7
    if dtype == "float32":
        assert torch.equal(outs[0], outs[1])
    else:
        assert torch.allclose(outs[0], outs[1], atol=1e-5, rtol=0)  # the same kernels in the same order


def test_decoding_across_context_buckets_with_lookahead(tiny_folders):
    """The context bucket of the graphs made small, so that decoding crosses it again and again (a new
    table pitch and a new graph each time) with steps launched ahead; against plain launches, no lookahead."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    folder = tiny_folders["b"]
    prompts = [random_tokens(384, n, 80 + i) for i, n in enumerate([5, 40, 23])]
    outs = []
    for fast in (True, False):
        engine = SyncEngine(folder, dtype="float32", block_size=8, num_pages=96, max_num_seqs=4, max_num_tokens=64,
                            cuda_graphs=fast, lookahead=fast)
        if fast:
            engine.session.step_graphs.BUCKET = 32
        results, _ = engine.batch_generate(prompts, max_new_tokens=150, ignore_eos=True)
        outs.append([r.token_ids for r in results])
        if fast:
            assert engine.num_ahead > 100 and len(engine.session.step_graphs.graphs) >= 5
        engine.session.manager.check()
    assert outs[0] == outs[1]


def test_graphs_beyond_the_limit_make_room(tiny_folders):
    """More step shapes than graphs are kept: the least recently replayed one is dropped and recorded
    again when its shape comes back; the logits stay those of plain launches."""
    from qwen3_from_scratch_b200.engine.session import Session
    folder = tiny_folders["a"]
    prompts = {r: random_tokens(256, 6 + i, 70 + i) for i, r in enumerate("pqrs")}
    outs = []
    for graphs in (True, False):
        session = Session(folder, dtype="float32", page_size=4, num_pages=64, max_seqs=4, max_step_tokens=64,
                          cuda_graphs=graphs)
        if graphs:
            session.step_graphs.MAX_GRAPHS = 2
        got = [session.step([(r, ids, (len(ids) - 1,)) for r, ids in prompts.items()]).cpu()]
        token = 5
        for live in (4, 3, 2, 1, 2, 3, 4, 1, 4):  # decode steps of changing width: four shapes, room for two
            for _ in range(2):
                token = (token * 7 + 3) % 256
                got.append(session.step([(r, [token], (0,)) for r in "pqrs"[:live]]).cpu())
        outs.append(torch.cat(got))
        if graphs:
            assert len(session.step_graphs.graphs) == 2 and session.step_graphs.replays >= 9
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_gives_what_plain_launches_give(tiny_folders, dtype):
    """Decode steps replayed from CUDA graphs against the same steps launched kernel by kernel."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    folder = tiny_folders["b"]
    prompts = [random_tokens(384, n, 40 + i) for i, n in enumerate([3, 21, 40])]
    outs = []
    for graphs in (True, False):
        engine = SyncEngine(folder, dtype=dtype, block_size=8, num_pages=64, max_num_seqs=4, max_num_tokens=64,
                            cuda_graphs=graphs)
        results, _ = engine.batch_generate(prompts, max_new_tokens=40, ignore_eos=True)
        outs.append([r.token_ids for r in results])
        if graphs:
            assert engine.session.step_graphs.replays > 30
        else:
            assert engine.session.step_graphs is None
    assert outs[0] == outs[1]


def test_eos_stops_a_request(tiny_folders):
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    folder = tiny_folders["a"]
    prompt = random_tokens(256, 9, 5)
    want, _ = greedy_by_plain(folder, prompt, 6)
    engine = SyncEngine(folder, dtype="float32", block_size=4, num_pages=32, max_num_seqs=2, max_num_tokens=32,
                        eos_token_id=want[3])
    chunks = list(engine.generate_stream(prompt, max_new_tokens=20))
    stop = want.index(want[3])
    assert [c.token_id for c in chunks] == want[:stop + 1]
    assert chunks[-1].metrics.token_count == stop + 1 and chunks[-1].metrics.ttft > 0
    assert not engine.session.manager.live_requests()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lookahead_changes_nothing_but_the_timing(tiny_folders, dtype):
    """Steps launched before the tokens of the step before them have been read: requests that stop at
    different lengths, one that stops at an end-of-sequence token (it has then been run one token too
    far, which is dropped), requests that arrive while others decode, sampling with a temperature.
    The same ids and finish reasons as with every step planned after the last was read."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    from qwen3_from_scratch_b200.engine.request import RequestStatus, SamplingParams
    folder = tiny_folders["b"]
    prompts = [random_tokens(384, n, 60 + i) for i, n in enumerate([7, 19, 3, 30, 11])]
    limits = [25, 9, 31, 14, 20]
    outcomes = []
    for lookahead in (False, True):
        engine = SyncEngine(folder, dtype=dtype, block_size=8, num_pages=96, max_num_seqs=4, max_num_tokens=64,
                            lookahead=lookahead)
        if lookahead:  # an id that the first request is known to produce: it ends there
            engine.eos_token_id = outcomes[0][0][0][12]
        else:
            engine.eos_token_id = None
        params = [SamplingParams(max_new_tokens=n, temperature=0.7 if i == 3 else 0.0, top_k=5 if i == 3 else 0, seed=11,
                                 ignore_eos=i != 0) for i, n in enumerate(limits)]
        reqs = [engine.add_request(p, params=q) for p, q in zip(prompts[:3], params[:3])]
        steps = 0
        while any(r.status != RequestStatus.FINISHED for r in reqs):
            engine.step()
            steps += 1
            if steps == 6:  # two more arrive while the first three decode
                reqs += [engine.add_request(p, params=q) for p, q in zip(prompts[3:], params[3:])]
            for i, r in enumerate(reqs):
                r.key = 1000 + i  # the random stream of a request is keyed by this: the same in both engines
        engine.drain()
        outcomes.append(([list(r.output) for r in reqs], [r.finish_reason for r in reqs], engine.num_ahead))
        engine.session.manager.check()
        assert not engine.session.manager.live_requests()
    (ids0, why0, ahead0), (ids1, why1, ahead1) = outcomes
    assert ahead0 == 0 and ahead1 > 10
    stop = ids0[0].index(ids0[0][12])  # where the chosen id first appears
    assert ids1[0] == ids0[0][:stop + 1] and why1[0] == "eos"
    assert ids1[1:] == ids0[1:] and why1[1:] == why0[1:]


def test_preemption_keeps_the_result(tiny_folders):
    """A pool too small for all requests at once: some are preempted and recomputed, and every
    request still produces what it produces alone."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    folder = tiny_folders["a"]
    prompts = [random_tokens(256, n, 20 + i) for i, n in enumerate([30, 28, 26, 31])]
    alone = SyncEngine(folder, dtype="float32", block_size=4, num_pages=64, max_num_seqs=4, max_num_tokens=64)
    want = [alone.generate(p, max_new_tokens=24, ignore_eos=True) for p in prompts]
    tight = SyncEngine(folder, dtype="float32", block_size=4, num_pages=36, max_num_seqs=4, max_num_tokens=64)
    results, _ = tight.batch_generate(prompts, max_new_tokens=24, ignore_eos=True)
    assert tight.scheduler.num_preemptions > 0
    assert [r.token_ids for r in results] == want
    tight.session.manager.check()


def test_request_that_cannot_fit_is_refused(tiny_folders):
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    engine = SyncEngine(tiny_folders["a"], dtype="float32", block_size=4, num_pages=8, max_num_seqs=2,
                        max_num_tokens=32)
    with pytest.raises(ValueError, match="can never fit"):
        engine.add_request([1] * 30, max_new_tokens=10)
    with pytest.raises(ValueError, match="tokenizer"):
        engine.add_request("text without a tokenizer")


def test_a_kernel_that_gave_up_a_wait_raises_and_the_engine_carries_on(tiny_folders):
    """The time-out bit of the status word reaches the caller as ``DeviceStatusError``; after it the same
    session runs other requests correctly (nothing was left held on the device)."""
    from harness import Replayer, assert_close, plain_logits
    from qwen3_from_scratch_b200.engine.session import DeviceStatusError, Session
    from qwen3_from_scratch_b200.kernels import ops
    folder = tiny_folders["d"]
    vocab = TINY["d"][0]["vocab_size"]
    session = Session(folder, dtype="bfloat16", page_size=16, cache_tokens=1024, max_seqs=4, max_step_tokens=512,
                      cuda_graphs=False)
    doomed = random_tokens(vocab, 300, 41)
    try:
        ops.set_wait_test(limit=1 << 14, drop_copy=1)
        session.step([("doomed", doomed, [len(doomed) - 1])])
        with pytest.raises(DeviceStatusError, match="wait"):
            session.check_status()
    finally:
        ops.set_wait_test()
    session.end("doomed")
    seqs = {"after": random_tokens(vocab, 280, 42)}
    rep = Replayer(session, seqs)
    rep.step([("after", 200)])
    while rep.remaining("after"):
        rep.step([("after", 1)])
    assert_close(rep.result(), plain_logits(folder, seqs), "bfloat16", "after a time-out")


def run_trace(folder, dtype, steps, out, max_tokens, extra=()):
    env = dict(os.environ)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", out, "--max-tokens", str(max_tokens), *extra]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tiny_folders, tmp_path, dtype):
    """The program itself: portions, a request left out of a step, ends, wanted places, files."""
    folder = tiny_folders["c"]
    vocab = TINY["c"][0]["vocab_size"]
    a, b = random_tokens(vocab, 70, 31), random_tokens(vocab, 50, 32)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:2], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[40:41], "want": [0]},
                                {"id": "b", "tokens": b[2:50], "want": [47, 0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[41:70], "want": list(range(29))}], "end": ["a"]},
    ]
    out = str(tmp_path / "out")
    run_trace(folder, dtype, steps, out, max_tokens=128 + 64, extra=["--poison-freed-pages"])
    assert sorted(os.listdir(out)) == ["0.f32", "2.f32", "3.f32"]
    cfg, w = plain.read_model_folder(folder)
    la, lb = plain.forward_logits(cfg, w, a), plain.forward_logits(cfg, w, b)
    tol = {"float32": 1e-5, "bfloat16": 2e-2}[dtype]

    def check(step, rows):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4")).view(len(rows), vocab)
        want = torch.stack(rows)
        assert float((got - want).abs().max()) <= tol * float(want.abs().max())

    check(0, [la[0], la[39]])
    check(2, [la[40], lb[49], lb[2]])
    check(3, [la[41 + i] for i in range(29)])


def test_command_line_generates(tiny_folders):
    folder = tiny_folders["a"]
    prompt = random_tokens(256, 5, 1)
    want, _ = greedy_by_plain(folder, prompt, 6)
    cmd = [sys.executable, "-m", "qwen3_from_scratch_b200", "generate", "--model", folder, "--dtype", "float32",
           "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--ignore-eos",
           "--block-size", "4", "--num-pages", "32", "--max-num-seqs", "2", "--max-num-tokens", "32"]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    record = json.loads(proc.stdout.splitlines()[0])
    assert record["token_ids"] == want and record["finish_reason"] == "length"
